"""Paged attention layer (GQA / MHA / MQA) and its per-step metadata.

Batch layout of one step: the first ``num_decodes`` tokens are single-token decode
requests, followed by the tokens of ``num_prefills`` requests with more than one
scheduled token (prefill chunks, speculative verification).  The reference orders
its MLA batches the same way (vllm_gcu/attention/backends/mla_v1_fusion.py:126-138).

KV cache of a layer: one tensor ``[2, num_blocks, block_size, kv_heads, head_dim]``
(the "flash" layout of csrc/src/reshape_and_cache_flash.cpp:23).

GPU path per layer: one fused RoPE + cache-write kernel, then the split-KV decode
kernel on the decode rows and the varlen paged-prefill kernel on the rest.  CPU path:
the torch reference of the same ops.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import cuda as C
from ..ops import ref
from .basic import RMSNorm, RotaryEmbedding


@dataclass
class AttentionMetadata:
    num_tokens: int                      # tokens in the step (incl. graph padding)
    num_decodes: int                     # leading single-token requests
    num_prefills: int                    # following multi-token requests
    num_decode_tokens: int               # == num_decodes (kept for clarity)
    positions: torch.Tensor              # [T] int64
    slot_mapping: torch.Tensor           # [T] int64, -1 = padding
    block_tables: torch.Tensor           # [B, max_blocks] int32
    seq_lens: torch.Tensor               # [B] int32, kv length after this step
    cu_q_prefill: Optional[torch.Tensor] = None   # [num_prefills + 1] int32, relative
    num_q_tiles: int = 0                 # sum ceil(q_len / 64) over prefills (host value)
    num_q_tiles_128: Optional[int] = None  # the same for 128-row tiles (tcgen05 kernel)
    max_seq_len: int = 0
    decode_splits: int = 1
    decode_workspace: Optional[tuple[torch.Tensor, torch.Tensor]] = None
    sample_indices: Optional[torch.Tensor] = None  # rows of the hidden states to sample from
    # host copies (CPU reference path, drafters)
    q_lens_cpu: list[int] = field(default_factory=list)
    seq_lens_cpu: list[int] = field(default_factory=list)
    # speculative decoding: every request with q_len > 1 verifies draft tokens
    is_dummy: bool = False
    # multimodal rotary embedding: (t, h, w) position of every token, ``[3, T]``; the cos / sin
    # rows gathered per section are cached here by the first layer of a step
    mrope_positions: Optional[torch.Tensor] = None
    mrope_cos_sin: Optional[torch.Tensor] = None
    # shared-prefix (cascade) attention: every request of the step starts with the same
    # ``common_prefix_len`` cached tokens (a multiple of the block size; 0 = off) and
    # ``cu_q_all`` holds the query offsets of all requests, decodes included
    common_prefix_len: int = 0
    cu_q_all: Optional[torch.Tensor] = None


def cascade_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      block_tables: torch.Tensor, cu_q: torch.Tensor, seq_lens: torch.Tensor,
                      scale: float, common_prefix_len: int, q_lens_cpu: list[int],
                      native: bool) -> torch.Tensor:
    """Attention of a batch whose requests all start with the same ``common_prefix_len``
    cached tokens: one pass of all query tokens over the shared prefix (read once instead of
    once per request, no causal mask: every query lies behind it), one causal pass per request
    over its own suffix, merged by their log-sum-exp values.  q ``[T, Hq, D]``; ``cu_q`` /
    ``seq_lens`` / ``block_tables`` describe all requests (the reference's cascade path,
    vllm_gcu/v1/attention/flash_attn.py:97-177)."""
    bs = k_cache.shape[1]
    assert common_prefix_len > 0 and common_prefix_len % bs == 0
    T = q.shape[0]
    nb = common_prefix_len // bs
    dev = q.device
    one_cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    one_len = torch.tensor([common_prefix_len], dtype=torch.int32, device=dev)
    suffix_lens = (seq_lens - common_prefix_len).to(torch.int32)
    suffix_bt = block_tables[:, nb:].contiguous()
    if native:
        p_out, p_lse = C.varlen_prefill(q, k_cache, v_cache, block_tables[:1, :nb].contiguous(),
                                        one_cu, one_len, scale, -(-T // 64), causal=False,
                                        return_lse=True, num_q_tiles_128=-(-T // 128))
        s_out, s_lse = C.varlen_prefill(
            q, k_cache, v_cache, suffix_bt, cu_q, suffix_lens, scale,
            sum(-(-n // 64) for n in q_lens_cpu), return_lse=True,
            num_q_tiles_128=sum(-(-n // 128) for n in q_lens_cpu))
        out, _ = C.merge_attn_states(p_out, p_lse, s_out, s_lse, want_lse=False)
        return out
    p_out, p_lse = ref.varlen_prefill_attention(q, k_cache, v_cache, block_tables[:1, :nb],
                                                one_cu, one_len, scale, causal=False,
                                                return_lse=True)
    s_out, s_lse = ref.varlen_prefill_attention(q, k_cache, v_cache, suffix_bt, cu_q, suffix_lens,
                                                scale, return_lse=True)
    return ref.merge_attn_states(p_out, p_lse, s_out, s_lse)[0]


def allocate_kv_cache(num_layers: int, num_blocks: int, block_size: int, kv_heads: int,
                      head_dim: int, dtype: torch.dtype, device) -> list[torch.Tensor]:
    return [torch.zeros(2, num_blocks, block_size, kv_heads, head_dim, dtype=dtype, device=device)
            for _ in range(num_layers)]


def alibi_slopes(num_heads: int) -> torch.Tensor:
    """ALiBi slopes of all heads, fp32 ``[num_heads]``: a geometric sequence 2^(-8 i / n) for the
    largest power of two n <= num_heads, then every other term of the sequence for 2n (the
    published recipe; Baichuan-13B, BLOOM and MPT checkpoints assume it)."""
    import math
    n = 2 ** math.floor(math.log2(num_heads))
    base = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
    slopes = torch.pow(torch.tensor(base, dtype=torch.float32), torch.arange(1, n + 1))
    if n != num_heads:
        extra_base = 2.0 ** (-(2.0 ** -(math.log2(2 * n) - 3)))
        rem = min(n, num_heads - n)
        extra = torch.pow(torch.tensor(extra_base, dtype=torch.float32),
                          torch.arange(1, 1 + 2 * rem, 2))
        slopes = torch.cat([slopes, extra])
    return slopes.float()


class PagedAttention(nn.Module):
    def __init__(self, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 rotary: Optional[RotaryEmbedding], q_norm: Optional[RMSNorm] = None,
                 k_norm: Optional[RMSNorm] = None, sliding_window: int = 0,
                 alibi: Optional[torch.Tensor] = None):
        super().__init__()
        # ALiBi slopes of this rank's heads (fp32 [num_heads]); the kernels add
        # slope * (key position - query position) to the scores
        # (vllm_gcu/attention/ops/paged_attn.py:78-162 passes them to both attention ops)
        self.register_buffer("alibi", alibi, persistent=False)
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.scale = scale
        self.rotary = rotary
        self.q_norm, self.k_norm = q_norm, k_norm
        self.window = sliding_window
        self.mrope_section: Optional[list[int]] = None     # set by M-RoPE models (Qwen2.5-VL)
        # per-tensor scales of an fp8 / int8 KV cache (value = stored * scale); checkpoints may
        # provide them (``load_kv_cache_scales`` of the reference's quantised models,
        # vllm_gcu/models/deepseek_moe_quant.py:487), the default 1.0 suits fp8
        self.k_scale = 1.0
        self.v_scale = 1.0
        self._scale_t = None

    def forward(self, qkv: torch.Tensor, kv_cache: torch.Tensor, md: AttentionMetadata
                ) -> torch.Tensor:
        """qkv ``[T, (Hq + 2 Hkv) * D]`` -> ``[T, Hq * D]``."""
        T = qkv.shape[0]
        D, Hq, Hkv = self.head_dim, self.num_heads, self.num_kv_heads
        q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
        if kv_cache is None or md.is_dummy:
            # memory profile / keep-alive step of an idle rank: no cache, no attention
            return torch.zeros((T, Hq * D), dtype=qkv.dtype, device=qkv.device)
        if self.q_norm is not None:     # per-head QK RMSNorm (Qwen3)
            q = self.q_norm(q.reshape(T, Hq, D)).reshape(T, Hq * D)
            k = self.k_norm(k.reshape(T, Hkv, D)).reshape(T, Hkv * D)
        k_cache, v_cache = kv_cache[0], kv_cache[1]
        if ops.use_native(qkv) and qkv.dtype in (torch.bfloat16, torch.float16):
            return self._forward_cuda(q, k, v, k_cache, v_cache, md)
        return self._forward_ref(q, k, v, k_cache, v_cache, md)

    def _rope_inputs(self, md: AttentionMetadata, T: int):
        """(positions, cos/sin table) of this step; with M-RoPE the table rows are gathered
        per section once per step and the ordinary rotary kernel runs with positions 0..T-1
        (vllm_gcu/kernels/rotary_embedding.py:108-169)."""
        rot = self.rotary
        if rot is None:
            return None, None
        if md.mrope_positions is None or not self.mrope_section:
            return md.positions, rot.cos_sin_cache
        if md.mrope_cos_sin is None:
            from .basic import mrope_gather_cos_sin
            md.mrope_cos_sin = mrope_gather_cos_sin(
                rot.cos_sin_cache.float(), md.mrope_positions[:, :T], self.mrope_section)
            md.mrope_arange = torch.arange(T, device=md.mrope_cos_sin.device)
        return md.mrope_arange, md.mrope_cos_sin

    # -- GPU -----------------------------------------------------------------
    def _forward_cuda(self, q, k, v, k_cache, v_cache, md: AttentionMetadata) -> torch.Tensor:
        T = q.shape[0]
        D, Hq = self.head_dim, self.num_heads
        rot = self.rotary
        rope_pos, rope_table = self._rope_inputs(md, T)
        kvq = None
        ks_t = vs_t = None
        if k_cache.element_size() == 1:
            if k_cache.dtype == torch.int8 and self.k_scale == 1.0 and self.v_scale == 1.0:
                # no calibrated scales were loaded: a fixed step that keeps |x| < 8 in range
                self.k_scale = self.v_scale = 1.0 / 16.0
                import warnings
                warnings.warn("int8 KV cache without loaded k/v scales: using 1/16 for both; "
                              "load calibrated scales for accuracy", stacklevel=2)
            if self._scale_t is None or self._scale_t.device != q.device:
                self._scale_t = torch.tensor([self.k_scale, self.v_scale], dtype=torch.float32,
                                             device=q.device)
            ks_t, vs_t = self._scale_t[0:1], self._scale_t[1:2]
            kvq = (self.k_scale, self.v_scale, 0.0, 0.0)
        C.rope_cache_flash(q, k, v, rope_pos, rope_table,
                           rot.is_neox if rot is not None else True, D, md.slot_mapping,
                           k_cache, v_cache, ks_t, vs_t)
        out = torch.empty((T, Hq * D), dtype=q.dtype, device=q.device)
        nd = md.num_decode_tokens
        if (md.common_prefix_len > 0 and kvq is None and D in (64, 128) and not self.window
                and self.alibi is None):
            B = md.num_decodes + md.num_prefills
            n_real = sum(md.q_lens_cpu[:B])
            o = cascade_attention(q[:n_real].view(n_real, Hq, D), k_cache, v_cache,
                                  md.block_tables[:B], md.cu_q_all, md.seq_lens[:B], self.scale,
                                  md.common_prefix_len, md.q_lens_cpu[:B], native=True)
            out[:n_real] = o.reshape(n_real, Hq * D)
            return out
        if nd > 0:
            C.paged_decode(q[:nd].view(nd, Hq, D), k_cache, v_cache, md.block_tables[:nd],
                           md.seq_lens[:nd], self.scale, out=out[:nd].view(nd, Hq, D),
                           num_splits=md.decode_splits, workspace=md.decode_workspace,
                           kv_quant=kvq, alibi_slopes=self.alibi)
        if md.num_prefills > 0 and D not in (64, 128) and kvq is None:
            # head sizes the prefill kernels do not cover (Gemma-7B: 256): torch formulation
            npf = T - nd
            sl = slice(md.num_decodes, md.num_decodes + md.num_prefills)
            o = ref.varlen_prefill_attention(q[nd:].view(npf, Hq, D), k_cache, v_cache,
                                             md.block_tables[sl], md.cu_q_prefill,
                                             md.seq_lens[sl], self.scale, window=self.window,
                                             alibi_slopes=self.alibi)
            out[nd:] = o.reshape(npf, Hq * D)
        elif md.num_prefills > 0:
            npf = T - nd
            C.varlen_prefill(q[nd:].view(npf, Hq, D), k_cache, v_cache,
                             md.block_tables[md.num_decodes:md.num_decodes + md.num_prefills],
                             md.cu_q_prefill,
                             md.seq_lens[md.num_decodes:md.num_decodes + md.num_prefills],
                             self.scale, md.num_q_tiles, out=out[nd:].view(npf, Hq, D),
                             window=self.window, num_q_tiles_128=md.num_q_tiles_128,
                             kv_quant=kvq, alibi_slopes=self.alibi)
        return out

    # -- CPU reference ----------------------------------------------------------
    def _forward_ref(self, q, k, v, k_cache, v_cache, md: AttentionMetadata) -> torch.Tensor:
        T = q.shape[0]
        D, Hq, Hkv = self.head_dim, self.num_heads, self.num_kv_heads
        if self.rotary is not None:
            rope_pos, rope_table = self._rope_inputs(md, T)
            if rope_table is self.rotary.cos_sin_cache:
                q, k = self.rotary(md.positions, q, k)
            else:
                q, k = ref.rotary_embedding(rope_pos, q, k, D, rope_table, self.rotary.is_neox)
        ref.reshape_and_cache_flash(k.reshape(T, Hkv, D), v.reshape(T, Hkv, D), k_cache, v_cache,
                                    md.slot_mapping)
        B = md.num_decodes + md.num_prefills
        q_lens = [1] * md.num_decodes + list(md.q_lens_cpu[md.num_decodes:B])
        cu = torch.zeros(B + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(q_lens, dtype=torch.int32).cumsum(0)
        n_real = int(cu[-1])
        out = torch.zeros((T, Hq * D), dtype=q.dtype, device=q.device)
        if md.common_prefix_len > 0 and not self.window and self.alibi is None:
            o = cascade_attention(q[:n_real].reshape(n_real, Hq, D), k_cache, v_cache,
                                  md.block_tables[:B], cu, md.seq_lens[:B], self.scale,
                                  md.common_prefix_len, q_lens, native=False)
            out[:n_real] = o.reshape(n_real, Hq * D)
            return out
        o = ref.varlen_prefill_attention(q[:n_real].reshape(n_real, Hq, D), k_cache, v_cache,
                                         md.block_tables[:B], cu, md.seq_lens[:B], self.scale,
                                         window=self.window, alibi_slopes=self.alibi)
        out[:n_real] = o.reshape(n_real, Hq * D)
        return out
