"""Attention backend that vLLM's own engine loads through the platform plugin.

``B200Platform.get_attn_backend_cls`` returns this backend for decoder attention with head
sizes 64 / 128 and a bf16 / fp16 KV cache; its ``forward`` runs this package's kernels:
``b200_rope_cache_flash`` (cache write), ``b200_paged_decode_tma`` / ``b200_paged_decode`` on the
decode rows and ``b200_fmha_prefill`` / ``b200_varlen_prefill`` on the rest.  The reference
selects its backends the same way (vllm_gcu/gcu.py:70-104) and implements them in
vllm_gcu/v1/attention/flash_attn.py.

Batch layout: the metadata builder asks vLLM to put single-token requests first
(``reorder_batch_threshold = 1``), which is the layout of this package's kernels (decodes,
then prefills).  KV cache: ``[2, num_blocks, block_size, kv_heads, head_size]``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Optional

import torch

from vllm.v1.attention.backend import (AttentionBackend, AttentionCGSupport, AttentionImpl,
                                       AttentionMetadataBuilder, AttentionType,
                                       CommonAttentionMetadata, MultipleOf)
from vllm.v1.attention.backends.utils import split_decodes_and_prefills

from ..ops import cuda as C

BACKEND_PATH = "vllm_gcu_b200.runtime.vllm_attention.B200AttentionBackend"


@dataclass
class B200AttentionMetadata:
    num_actual_tokens: int
    num_decodes: int
    num_prefills: int
    num_decode_tokens: int
    block_table: torch.Tensor            # [num_reqs, max_blocks] int32
    seq_lens: torch.Tensor               # [num_reqs] int32
    slot_mapping: torch.Tensor           # [num_actual_tokens] int64
    max_seq_len: int
    decode_splits: int = 1
    decode_workspace: Optional[tuple[torch.Tensor, torch.Tensor]] = None
    cu_q_prefill: Optional[torch.Tensor] = None     # [num_prefills + 1] int32, relative
    num_q_tiles: int = 0
    num_q_tiles_128: int = 0


class B200AttentionBackend(AttentionBackend):
    supported_dtypes: ClassVar[list[torch.dtype]] = [torch.float16, torch.bfloat16]
    supported_kv_cache_dtypes: ClassVar[list[str]] = ["auto", "float16", "bfloat16"]
    forward_includes_kv_cache_update: bool = False

    @staticmethod
    def get_supported_kernel_block_sizes():
        return [MultipleOf(16)]

    @staticmethod
    def get_name() -> str:
        return "CUSTOM"

    @staticmethod
    def get_impl_cls():
        return B200AttentionImpl

    @staticmethod
    def get_builder_cls():
        return B200AttentionMetadataBuilder

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> tuple[int, ...]:
        return (2, num_blocks, block_size, num_kv_heads, head_size)

    @classmethod
    def get_supported_head_sizes(cls) -> list[int]:
        return [64, 128]

    @classmethod
    def supports_head_size(cls, head_size: int) -> bool:
        return head_size in (64, 128)

    @classmethod
    def supports_attn_type(cls, attn_type: str) -> bool:
        return attn_type == AttentionType.DECODER

    @classmethod
    def supports_compute_capability(cls, capability) -> bool:
        return capability.major == 10


def accepts(cfg) -> bool:
    """Whether this backend covers an ``AttentionSelectorConfig`` of vLLM."""
    return (not cfg.use_mla and not cfg.has_sink and not cfg.use_sparse
            and not cfg.use_mm_prefix and not cfg.use_non_causal
            and cfg.attn_type == AttentionType.DECODER
            and cfg.head_size in (64, 128)
            and cfg.dtype in (torch.float16, torch.bfloat16)
            and (cfg.kv_cache_dtype in (None, "auto", "float16", "bfloat16"))
            and (cfg.block_size is None or cfg.block_size % 16 == 0))


class B200AttentionMetadataBuilder(AttentionMetadataBuilder[B200AttentionMetadata]):
    # decode-only batches replay from full CUDA graphs; mixed batches run piecewise / eagerly
    _cudagraph_support: ClassVar[AttentionCGSupport] = \
        AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE

    def __init__(self, kv_cache_spec, layer_names, vllm_config, device):
        super().__init__(kv_cache_spec, layer_names, vllm_config, device)
        self._init_reorder_batch_threshold(1)
        self.num_kv_heads = kv_cache_spec.num_kv_heads
        self.head_size = kv_cache_spec.head_size
        pc = vllm_config.parallel_config
        self.num_heads = vllm_config.model_config.get_num_attention_heads(pc)
        self.max_model_len = vllm_config.model_config.max_model_len
        max_seqs = vllm_config.scheduler_config.max_num_seqs
        ns = 32
        # split-KV partial results of the decode kernel (shared by all layers: they run
        # one after the other)
        self.workspace = (
            torch.empty(max_seqs * self.num_heads * ns * self.head_size // 8 + 1024,
                        dtype=torch.float32, device=device),
            torch.empty(max_seqs * self.num_heads * ns // 8 + 1024, dtype=torch.float32,
                        device=device))

    def _splits(self, batch: int, max_seq_len: int) -> int:
        s = C.decode_num_splits(batch, self.num_kv_heads, max_seq_len)
        while s > 1 and batch * self.num_heads * s * self.head_size > self.workspace[0].numel():
            s -= 1
        return s

    def build(self, common_prefix_len: int, common_attn_metadata: CommonAttentionMetadata,
              fast_build: bool = False) -> B200AttentionMetadata:
        cm = common_attn_metadata
        nd, npf, nd_tok, npf_tok = split_decodes_and_prefills(cm, decode_threshold=1)
        md = B200AttentionMetadata(
            num_actual_tokens=cm.num_actual_tokens, num_decodes=nd, num_prefills=npf,
            num_decode_tokens=nd_tok, block_table=cm.block_table_tensor,
            seq_lens=cm.seq_lens, slot_mapping=cm.slot_mapping, max_seq_len=cm.max_seq_len,
            decode_workspace=self.workspace)
        if nd:
            md.decode_splits = self._splits(nd, cm.max_seq_len)
        if npf:
            qs = cm.query_start_loc_cpu[nd:nd + npf + 1]
            q_lens = (qs[1:] - qs[:-1])
            md.num_q_tiles = int(((q_lens + 63) // 64).sum())
            md.num_q_tiles_128 = int(((q_lens + 127) // 128).sum())
            dev_qs = cm.query_start_loc[nd:nd + npf + 1]
            md.cu_q_prefill = (dev_qs - dev_qs[0]).to(torch.int32)
        return md

    def build_for_cudagraph_capture(self, common_attn_metadata: CommonAttentionMetadata
                                    ) -> B200AttentionMetadata:
        # the number of KV splits is baked into the captured launch: size it for the longest
        # sequence the model accepts
        md = self.build(0, common_attn_metadata)
        if md.num_decodes:
            md.decode_splits = self._splits(md.num_decodes, self.max_model_len)
        return md


class B200AttentionImpl(AttentionImpl[B200AttentionMetadata]):
    def __init__(self, num_heads: int, head_size: int, scale: float,
                 num_kv_heads: Optional[int] = None, alibi_slopes=None,
                 sliding_window: Optional[int] = None, kv_cache_dtype: str = "auto",
                 logits_soft_cap: Optional[float] = None,
                 attn_type: str = AttentionType.DECODER,
                 kv_sharing_target_layer_name: Optional[str] = None, **kw) -> None:
        if logits_soft_cap:
            raise NotImplementedError("logit soft caps are not supported by the B200 attention "
                                      "backend")
        # ALiBi slopes (one per head of this rank) go to the kernels as an fp32 vector
        self.alibi = None if alibi_slopes is None else \
            torch.as_tensor(alibi_slopes, dtype=torch.float32)
        if kv_sharing_target_layer_name is not None:
            raise NotImplementedError("KV sharing between layers is not supported")
        self.num_heads = num_heads
        self.head_size = head_size
        self.scale = float(scale)
        self.num_kv_heads = num_kv_heads or num_heads
        self.kv_cache_dtype = kv_cache_dtype
        self.window = int(sliding_window) if sliding_window else 0
        self.attn_type = attn_type

    def do_kv_cache_update(self, layer, key: torch.Tensor, value: torch.Tensor,
                           kv_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
        """Paged write of this step's keys / values (RoPE has been applied by the model)."""
        n = slot_mapping.shape[0]
        Hkv, D = self.num_kv_heads, self.head_size
        C.rope_cache_flash(None, key[:n].reshape(n, Hkv * D), value[:n].reshape(n, Hkv * D), None,
                           None, True, D, slot_mapping, kv_cache[0], kv_cache[1])

    def forward(self, layer, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                kv_cache: torch.Tensor, attn_metadata: Optional[B200AttentionMetadata],
                output: torch.Tensor, output_scale=None, output_block_scale=None) -> torch.Tensor:
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("fused output quantisation is not supported")
        if attn_metadata is None:            # memory-profiling run
            return output.fill_(0)
        md = attn_metadata
        Hq, D = self.num_heads, self.head_size
        T = md.num_actual_tokens
        q = query[:T].reshape(T, Hq, D)
        out = output[:T].view(T, Hq, D)
        k_cache, v_cache = kv_cache[0], kv_cache[1]
        if self.alibi is not None and self.alibi.device != q.device:
            self.alibi = self.alibi.to(q.device)
        nd = md.num_decode_tokens
        if nd > 0:
            C.paged_decode(q[:nd], k_cache, v_cache, md.block_table[:md.num_decodes],
                           md.seq_lens[:md.num_decodes], self.scale, out=out[:nd],
                           num_splits=md.decode_splits, workspace=md.decode_workspace,
                           alibi_slopes=self.alibi)
        if md.num_prefills > 0:
            lo, hi = md.num_decodes, md.num_decodes + md.num_prefills
            C.varlen_prefill(q[nd:], k_cache, v_cache, md.block_table[lo:hi], md.cu_q_prefill,
                             md.seq_lens[lo:hi], self.scale, md.num_q_tiles, out=out[nd:],
                             window=self.window, num_q_tiles_128=md.num_q_tiles_128,
                             alibi_slopes=self.alibi)
        return output
