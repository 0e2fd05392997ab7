"""DeepSeek-V2 / V3 / R1: multi-head latent attention (MLA) + grouped-routing MoE.

MLA keeps one latent row ``[kv_c (kv_lora_rank) | k_pe (rope)]`` per token in the paged
cache.  Queries are projected into the latent space ("absorbed" form, W_UK folded into the
query and W_UV applied to the attention output), so attention is multi-query over the
latent rows with a 576-wide key and a 512-wide value for DeepSeek-V3, as in the reference's
fused backend (vllm_gcu/attention/backends/mla_v1_fusion.py:83-242,
vllm_gcu/models/deepseek_v3/deepseek_v3_fusion.py:105-258):

1. ``qkv_a`` = merged ``q_a_proj`` + ``kv_a_proj_with_mqa`` (one GEMM);
2. one fused kernel splits the latent, applies RMSNorm to ``kv_c``, RoPE to ``q_pe`` / ``k_pe``
   and writes the latent row into the paged cache (``ops.cuda.mla_rope_cache``);
3. ``q_nope x W_UK`` -> latent query; attention over the cached latents; ``x W_UV``; ``o_proj``.

The attention core runs in the tcgen05 latent attention kernel (csrc/attention_mla.cu:
decode, multi-token verification and prefill chunks in one kernel) for bf16 caches and a
power-of-two head count up to 128; other layouts fall back to batched matrix products over
gathered latent rows (decode: one padded batch; prefill: per sequence).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..config import ModelConfig
from ..layers.attention import AttentionMetadata
from ..layers.basic import RMSNorm, build_cos_sin_cache, _yarn_mscale
from ..layers.linear import (ColumnParallelLinear, MergedReplicatedLinear, ReplicatedLinear,
                             RowParallelLinear)
from ..ops import cuda as C
from ..ops import ref
from ..parallel.state import tp_size
from .decoder import get_linear_method
from .moe_models import MoeDecoderLM


USE_MLA_KERNEL = True     # tcgen05 latent attention (csrc/attention_mla.cu) where the layout allows


def mla_attention_ref(q_full: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor,
                      q_lens: list[int], seq_lens: list[int], scale: float, L: int
                      ) -> torch.Tensor:
    """q_full ``[T, N, L + R]`` (latent query | rotated rope part); cache ``[blocks, bs, L + R]``.
    Returns the latent-space output ``[T, N, L]``.  Causal inside each request."""
    T, N, W = q_full.shape
    nb, bs, _ = cache.shape
    flat = cache.view(nb * bs, W)
    out = torch.zeros(T, N, L, dtype=q_full.dtype, device=q_full.device)
    t0 = 0
    for b, (ql, n) in enumerate(zip(q_lens, seq_lens)):
        if ql == 0 or n == 0:
            t0 += ql
            continue
        pos = torch.arange(n, device=cache.device)
        slots = block_tables[b, (pos // bs).long()].long() * bs + pos % bs
        kv = flat[slots].float()                               # [n, W]
        q = q_full[t0:t0 + ql].float()                         # [ql, N, W]
        s = torch.einsum("qhw,nw->hqn", q, kv) * scale
        qpos = torch.arange(n - ql, n, device=cache.device)[:, None]
        s = s.masked_fill((pos[None, :] > qpos)[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[t0:t0 + ql] = torch.einsum("hqn,nl->qhl", p, kv[:, :L]).to(out.dtype)
        t0 += ql
    return out


def mla_decode_batched(q_full: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor,
                       seq_lens: torch.Tensor, max_len: int, scale: float, L: int) -> torch.Tensor:
    """Decode-only fast path (one query per request): gathers the latent rows of the whole
    batch into a padded ``[B, max_len, W]`` tensor and runs two batched GEMMs."""
    B, N, W = q_full.shape
    nb, bs, _ = cache.shape
    pos = torch.arange(max_len, device=cache.device)
    blk = block_tables[:, : (max_len + bs - 1) // bs].long()
    slots = blk.gather(1, (pos // bs)[None].expand(B, -1)) * bs + (pos % bs)[None]
    mask = pos[None, :] < seq_lens[:, None]
    slots = torch.where(mask, slots, torch.zeros_like(slots))
    kv = cache.view(nb * bs, W)[slots]                         # [B, max_len, W]
    if kv.dtype != q_full.dtype:                               # fp8 latent cache (scale 1)
        kv = kv.to(q_full.dtype)
    s = torch.bmm(q_full, kv.transpose(1, 2)).float() * scale  # [B, N, max_len]
    s = s.masked_fill(~mask[:, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1).to(q_full.dtype)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.bmm(p, kv[..., :L])                           # [B, N, L]


class MLAAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device, prefix: str):
        super().__init__()
        self.cfg = cfg
        tp = tp_size()
        H = cfg.hidden_size
        self.N = cfg.num_attention_heads // tp
        self.L, self.R = cfg.kv_lora_rank, cfg.qk_rope_head_dim
        self.nope, self.vdim = cfg.qk_nope_head_dim, cfg.v_head_dim
        self.qk_dim = self.nope + self.R
        dt = cfg.dtype
        lm = lambda n: get_linear_method(cfg, prefix + "." + n)  # noqa: E731
        if cfg.q_lora_rank > 0:
            # q_a_proj and kv_a_proj_with_mqa read the same input: one merged GEMM
            self.qkv_a_proj = MergedReplicatedLinear(H, [cfg.q_lora_rank, self.L + self.R],
                                                     dtype=dt, device=device,
                                                     quant_method=lm("qkv_a_proj"),
                                                     prefix=prefix + ".qkv_a_proj")
            self.q_a_layernorm = RMSNorm(cfg.q_lora_rank, cfg.rms_norm_eps, dt, device)
            self.q_b_proj = ColumnParallelLinear(cfg.q_lora_rank,
                                                 cfg.num_attention_heads * self.qk_dim, dtype=dt,
                                                 device=device, quant_method=lm("q_b_proj"),
                                                 prefix=prefix + ".q_b_proj")
        else:
            self.q_proj = ColumnParallelLinear(H, cfg.num_attention_heads * self.qk_dim, dtype=dt,
                                               device=device, quant_method=lm("q_proj"),
                                               prefix=prefix + ".q_proj")
            self.kv_a_proj_with_mqa = ReplicatedLinear(H, self.L + self.R, dtype=dt, device=device,
                                                       quant_method=lm("kv_a_proj_with_mqa"),
                                                       prefix=prefix + ".kv_a_proj_with_mqa")
        self.kv_a_layernorm = RMSNorm(self.L, cfg.rms_norm_eps, dt, device)
        self.kv_b_proj = ColumnParallelLinear(self.L, cfg.num_attention_heads *
                                              (self.nope + self.vdim), dtype=dt, device=device,
                                              prefix=prefix + ".kv_b_proj")
        self.o_proj = RowParallelLinear(cfg.num_attention_heads * self.vdim, H, dtype=dt,
                                        device=device, quant_method=lm("o_proj"),
                                        prefix=prefix + ".o_proj")
        cache = build_cos_sin_cache(self.R, cfg.max_position_embeddings, cfg.rope_theta,
                                    cfg.rope_scaling)
        self.register_buffer("cos_sin_cache", cache.to(device=device, dtype=torch.float32),
                             persistent=False)
        self.scale = self.qk_dim ** -0.5
        rs = cfg.rope_scaling
        if rs and rs.get("mscale_all_dim"):
            m = _yarn_mscale(float(rs.get("factor", 1.0)), float(rs["mscale_all_dim"]))
            self.scale *= m * m
        self.w_uk_t: Optional[torch.Tensor] = None     # [N, nope, L]
        self.w_uv: Optional[torch.Tensor] = None       # [N, L, vdim]

    def finalize(self) -> None:
        """Splits ``kv_b_proj`` into the absorbed matrices W_UK^T and W_UV."""
        w = self.kv_b_proj.weight.data.view(self.N, self.nope + self.vdim, self.L)
        self.w_uk_t = w[:, : self.nope, :].contiguous()                     # [N, nope, L]
        self.w_uv = w[:, self.nope:, :].transpose(1, 2).contiguous()        # [N, L, vdim]

    def forward(self, x: torch.Tensor, kv_cache: Optional[torch.Tensor], md: AttentionMetadata
                ) -> torch.Tensor:
        T = x.shape[0]
        N, L, R = self.N, self.L, self.R
        if kv_cache is None or md.is_dummy:
            # idle data-parallel rank / memory profile: identical zero input for the MoE
            # (vllm_gcu/attention/backends/mla_v1_fusion.py:106-110)
            return self.o_proj(torch.zeros((T, N * self.vdim), dtype=x.dtype, device=x.device))
        if self.w_uk_t is None:
            self.finalize()
        cfg = self.cfg
        if cfg.q_lora_rank > 0:
            qkv_a = self.qkv_a_proj(x)
            q_c, kv = qkv_a.split([cfg.q_lora_rank, L + R], dim=-1)
            q = self.q_b_proj(self.q_a_layernorm(q_c.contiguous()))
        else:
            q = self.q_proj(x)
            kv = self.kv_a_proj_with_mqa(x)
        q = q.view(T, N, self.qk_dim)
        q_nope, q_pe = q[..., : self.nope], q[..., self.nope:]
        q_full = torch.empty((T, N, L + R), dtype=x.dtype, device=x.device)
        # latent query: q_nope x W_UK^T, written straight into the concatenated query
        q_full[..., :L].copy_(torch.bmm(q_nope.transpose(0, 1), self.w_uk_t).transpose(0, 1))
        if ops.use_native(x) and x.dtype in (torch.bfloat16, torch.float16):
            C.mla_rope_cache(q_pe, kv, md.positions, self.cos_sin_cache,
                             self.kv_a_layernorm.weight, cfg.rms_norm_eps, kv_cache,
                             md.slot_mapping, L, is_neox=cfg.rope_is_neox, q_out=q_full[..., L:])
        else:
            q_rot, _, _ = ref.mla_rope_cache(q_pe, kv, md.positions, self.cos_sin_cache,
                                             self.kv_a_layernorm.weight, cfg.rms_norm_eps,
                                             kv_cache, md.slot_mapping, L, cfg.rope_is_neox)
            q_full[..., L:] = q_rot
        nd = md.num_decode_tokens
        o_lat = torch.empty((T, N, L), dtype=x.dtype, device=x.device)
        B = md.num_decodes + md.num_prefills
        if (USE_MLA_KERNEL and ops.use_native(x)
                and C.mla_attention_supported(q_full, kv_cache, L)):
            # tcgen05 kernel: decode rows (one token per request), then the multi-token
            # requests (prefill chunks, draft verification) with their own offsets
            max_len = max(md.max_seq_len, 1)
            if nd > 0:
                C.mla_attention(q_full[:nd], kv_cache, md.block_tables[:nd], md.seq_lens[:nd],
                                None, nd, max_len, self.scale, out=o_lat[:nd])
            if md.num_prefills > 0:
                tq = 128 // N
                n_pf = sum(md.q_lens_cpu[md.num_decodes:B])
                tiles = sum(-(-q // tq) for q in md.q_lens_cpu[md.num_decodes:B])
                C.mla_attention(q_full[nd:nd + n_pf], kv_cache, md.block_tables[md.num_decodes:B],
                                md.seq_lens[md.num_decodes:B], md.cu_q_prefill, tiles, max_len,
                                self.scale, out=o_lat[nd:nd + n_pf])
                if nd + n_pf < T:
                    o_lat[nd + n_pf:] = 0
            elif nd < T:
                o_lat[nd:] = 0
            o = torch.bmm(o_lat.transpose(0, 1), self.w_uv).transpose(0, 1).reshape(
                T, N * self.vdim)
            return self.o_proj(o)
        if nd > 0 and x.is_cuda:
            o_lat[:nd] = mla_decode_batched(q_full[:nd], kv_cache, md.block_tables[:nd],
                                            md.seq_lens[:nd], max(md.max_seq_len, 1), self.scale,
                                            L)
            rest = range(md.num_decodes, B)
            t0 = nd
        else:
            rest = range(0, B)
            t0 = 0
        if len(rest) > 0:
            q_lens = [1] * md.num_decodes + list(md.q_lens_cpu[md.num_decodes:B])
            ql = [q_lens[i] for i in rest]
            sl = [md.seq_lens_cpu[i] for i in rest]
            n = sum(ql)
            o_lat[t0:t0 + n] = mla_attention_ref(q_full[t0:t0 + n], kv_cache,
                                                 md.block_tables[rest.start:rest.stop], ql, sl,
                                                 self.scale, L)
            if t0 + n < T:
                o_lat[t0 + n:] = 0
        o = torch.bmm(o_lat.transpose(0, 1), self.w_uv).transpose(0, 1).reshape(T, N * self.vdim)
        return self.o_proj(o)


class DeepseekV3ForCausalLM(MoeDecoderLM):
    """Checkpoint conventions handled here (deepseek_v3.py:1037-1173): ``q_a_proj`` and
    ``kv_a_proj_with_mqa`` load into the merged ``qkv_a_proj``; ``mlp.experts.N.*`` into the
    stacked expert tensors; ``mlp.shared_experts.*`` into the shared MLP; the trailing MTP
    layers (index >= num_hidden_layers) are skipped."""

    def map_weight_name(self, name: str):
        if self.cfg.q_lora_rank > 0:
            if ".self_attn.q_a_proj." in name:
                owner, _, pname = name.replace(".q_a_proj.", ".qkv_a_proj.").rpartition(".")
                return owner, pname, 0
            if ".self_attn.kv_a_proj_with_mqa." in name:
                owner, _, pname = name.replace(".kv_a_proj_with_mqa.",
                                               ".qkv_a_proj.").rpartition(".")
                return owner, pname, 1
        elif ".self_attn.q_proj." in name or ".self_attn.kv_a_proj_with_mqa." in name:
            # no query down-projection (DeepSeek-V2-Lite): q_proj is a layer of its own here,
            # not a shard of a fused qkv projection
            owner, _, pname = name.rpartition(".")
            return owner, pname, None
        return super().map_weight_name(name)

    def load_special(self, name, tensor, owners) -> bool:
        if name.startswith("model.layers."):
            idx = int(name.split(".")[2])
            if idx >= self.cfg.num_hidden_layers:
                return True      # multi-token-prediction layers belong to the drafter
        return super().load_special(name, tensor, owners)
