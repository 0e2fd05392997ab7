"""Norm, rotary, embedding and LM-head layers."""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import cuda as C
from ..ops import ref
from ..parallel.communicator import get_comm
from ..parallel.state import tp_rank, tp_size


class RMSNorm(nn.Module):
    """``forward(x)`` or ``forward(x, residual)`` (fused add, residual updated in place on
    the GPU path); same contract as the reference's ``RMSNorm.forward_oot``
    (vllm_gcu/kernels/layernorm.py:10-41), including the empty-tensor guard."""

    def __init__(self, hidden_size: int, eps: float = 1e-6, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device),
                                   requires_grad=False)
        self.eps = eps

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        if x.numel() == 0:
            return x if residual is None else (x, residual)
        if ops.use_native(x) and x.dtype in (torch.bfloat16, torch.float16) \
                and x.shape[-1] % 8 == 0:
            if residual is None:
                return C.norm(x, self.weight, self.eps)
            out = C.norm(x, self.weight, self.eps, residual=residual)
            return out, residual
        if residual is None:
            return ref.rms_norm(x, self.weight, self.eps)
        return ref.fused_add_rms_norm(x, residual, self.weight, self.eps)

    def forward_quant(self, x: torch.Tensor, residual: Optional[torch.Tensor], mode: str,
                      scale: Optional[torch.Tensor] = None):
        """(Residual add +) RMSNorm + activation quantisation in one kernel, for a consumer
        GEMM with 8-bit activations (the fusions the reference's compile pass performs,
        vllm_gcu/compilation/fusion.py:889-1023).  GPU only.  Returns
        ``(x_q, x_scale, residual)``; ``x_scale`` is per row (``[T, 1]``), per 128-wide group
        (``[T, H / 128]``) or the static scale repeated per row."""
        out = C.norm(x, self.weight, self.eps, residual=residual, quant=mode, scale=scale)
        if isinstance(out, tuple):
            return out[0], out[1], residual
        return out, scale.reshape(1).expand(x.shape[0]).contiguous(), residual

    def load_weight(self, name: str, full: torch.Tensor, shard_id=None) -> None:
        self.weight.data.copy_(full)


def _yarn_find_correction_dim(num_rot, dim, base, max_pos):
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def _yarn_mscale(scale: float, mscale: float = 1.0) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


def build_cos_sin_cache(rot_dim: int, max_pos: int, base: float,
                        rope_scaling: Optional[dict]) -> torch.Tensor:
    """fp32 ``[max_pos, rot_dim]`` = ``[cos | sin]``; handles plain, linear, llama3 and
    YaRN / deepseek_yarn scaling (the variants used by the reference's models,
    vllm_gcu/kernels/rotary_embedding.py:67-106, deepseek_v3.py:393-411)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    mscale = 1.0
    t_scale = 1.0
    if rope_scaling:
        kind = rope_scaling.get("rope_type", rope_scaling.get("type", "default"))
        factor = float(rope_scaling.get("factor", 1.0))
        if kind == "linear":
            t_scale = factor
        elif kind == "llama3":
            lo = rope_scaling.get("low_freq_factor", 1.0)
            hi = rope_scaling.get("high_freq_factor", 4.0)
            orig = rope_scaling.get("original_max_position_embeddings", 8192)
            wavelen = 2 * math.pi / inv_freq
            smooth = ((orig / wavelen) - lo) / (hi - lo)
            scaled = torch.where(wavelen > orig / lo, inv_freq / factor, inv_freq)
            mid = (wavelen <= orig / lo) & (wavelen >= orig / hi)
            inv_freq = torch.where(mid, (1 - smooth) * inv_freq / factor + smooth * inv_freq,
                                   scaled)
        elif kind in ("yarn", "deepseek_yarn"):
            orig = rope_scaling.get("original_max_position_embeddings", 4096)
            beta_fast = rope_scaling.get("beta_fast", 32)
            beta_slow = rope_scaling.get("beta_slow", 1)
            low = max(math.floor(_yarn_find_correction_dim(beta_fast, rot_dim, base, orig)), 0)
            high = min(math.ceil(_yarn_find_correction_dim(beta_slow, rot_dim, base, orig)),
                       rot_dim - 1)
            ramp = ((torch.arange(rot_dim // 2, dtype=torch.float32) - low)
                    / max(high - low, 1e-3)).clamp(0, 1)
            mask = 1.0 - ramp
            inv_freq = inv_freq / factor * (1 - mask) + inv_freq * mask
            # magnitude of cos / sin: an explicit attention_factor, else the ratio of the two
            # mscale terms when the checkpoint gives both (DeepSeek-V2 / V3 configs, whose type
            # is plain "yarn"; the mscale_all_dim part goes into the softmax scale of the
            # attention layer instead), else the plain YaRN factor
            af = rope_scaling.get("attention_factor")
            ms, ms_all = rope_scaling.get("mscale"), rope_scaling.get("mscale_all_dim")
            if af is not None:
                mscale = float(af)
            elif kind == "deepseek_yarn" or (ms and ms_all):
                mscale = (_yarn_mscale(factor, float(ms if ms is not None else 1.0))
                          / _yarn_mscale(factor, float(ms_all or 0.0)))
            else:
                mscale = _yarn_mscale(factor)
    t = torch.arange(max_pos, dtype=torch.float32) / t_scale
    freqs = torch.outer(t, inv_freq)
    return torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1)


class RotaryEmbedding(nn.Module):
    def __init__(self, head_size: int, rot_dim: int, max_pos: int, base: float, is_neox: bool,
                 rope_scaling: Optional[dict] = None, dtype=torch.bfloat16, device=None,
                 keep_fp32: bool = False):
        super().__init__()
        self.head_size, self.rot_dim, self.is_neox = head_size, rot_dim, is_neox
        cache = build_cos_sin_cache(rot_dim, max_pos, base, rope_scaling)
        self.register_buffer("cos_sin_cache",
                             cache.to(device=device, dtype=torch.float32 if keep_fp32 else dtype),
                             persistent=False)

    def forward(self, positions, q, k=None):
        """In place on the GPU path (q ``[T, H*D]``, k ``[T, Hkv*D]``)."""
        if ops.use_native(q) and q.dtype in (torch.bfloat16, torch.float16):
            C.rope_cache_flash(q, k, None, positions, self.cos_sin_cache, self.is_neox,
                               self.head_size)
            return q, k
        return ref.rotary_embedding(positions, q, k, self.head_size, self.cos_sin_cache,
                                    self.is_neox)


def mrope_gather_cos_sin(cos_sin_cache: torch.Tensor, positions: torch.Tensor,
                         mrope_section: list[int]) -> torch.Tensor:
    """Multimodal RoPE: ``positions`` is ``[3, T]`` (t, h, w); the cache rows are gathered
    per section so the ordinary rotary kernel can run with ``positions = arange(T)``
    (vllm_gcu/kernels/rotary_embedding.py:108-169)."""
    rot = cos_sin_cache.shape[-1]
    half = rot // 2
    cs = cos_sin_cache[positions.long()]            # [3, T, rot]
    cos, sin = cs[..., :half], cs[..., half:]
    idx = []
    for i, n in enumerate(mrope_section):
        idx += [i] * n
    sel = torch.tensor(idx, device=positions.device)
    ar = torch.arange(half, device=positions.device)
    cos_g = cos[sel, :, ar].transpose(0, 1)         # [T, half]
    sin_g = sin[sel, :, ar].transpose(0, 1)
    return torch.cat([cos_g, sin_g], dim=-1).contiguous()


class VocabParallelEmbedding(nn.Module):
    def __init__(self, vocab_size: int, hidden_size: int, dtype=torch.bfloat16, device=None):
        super().__init__()
        tp = tp_size()
        self.vocab_size = vocab_size
        self.padded = -(-vocab_size // (tp * 64)) * (tp * 64)
        self.per_rank = self.padded // tp
        self.start = tp_rank() * self.per_rank
        self.weight = nn.Parameter(torch.zeros(self.per_rank, hidden_size, dtype=dtype,
                                               device=device), requires_grad=False)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if tp_size() == 1:
            return F.embedding(ids, self.weight)
        local = ids - self.start
        mask = (local >= 0) & (local < self.per_rank)
        out = F.embedding(local.clamp(0, self.per_rank - 1), self.weight)
        out = out * mask.unsqueeze(-1).to(out.dtype)
        return get_comm("tp").all_reduce(out)

    def load_weight(self, name: str, full: torch.Tensor, shard_id=None) -> None:
        end = min(self.start + self.per_rank, full.shape[0])
        n = max(0, end - self.start)
        if n > 0:
            self.weight.data[:n].copy_(full[self.start:end])


class ParallelLMHead(VocabParallelEmbedding):
    """Vocab-parallel output projection.  ``logits(hidden)`` returns the full-vocabulary
    logits on every rank (all-gather over TP); ``greedy(hidden)`` takes the cheaper route
    of per-shard (max, argmax) pairs (2 numbers per row per rank instead of V/tp)."""

    def _local_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        if ops.use_native(hidden) and hidden.dtype == torch.bfloat16:
            return C.gemm_bf16(hidden, self.weight)
        return F.linear(hidden, self.weight)

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        if tp_size() > 1 and ops.use_native(hidden) and hidden.dim() == 2:
            # GEMM whose epilogue writes this rank's vocabulary block into every peer
            fg = getattr(get_comm("tp"), "fused_gather", None)
            lg = fg.gemm_all_gather(hidden, self.weight) if fg is not None else None
            if lg is not None:
                return lg[..., : self.vocab_size]
        lg = self._local_logits(hidden)
        if tp_size() > 1:
            lg = get_comm("tp").all_gather(lg, dim=-1)
        return lg[..., : self.vocab_size]

    def greedy(self, hidden: torch.Tensor) -> torch.Tensor:
        lg = self._local_logits(hidden)
        valid = min(self.per_rank, max(0, self.vocab_size - self.start))
        lg = lg[..., :valid]
        if tp_size() == 1:
            return lg.argmax(-1)
        if valid == 0:
            # a vocabulary smaller than the padded shards leaves the last ranks without a real
            # column: they take part in the exchange with a value that never wins
            lg = lg.new_full((*lg.shape[:-1], 1), float("-inf"))
            valid = 1
        if ops.use_native(hidden) and lg.dim() == 2:
            fused = getattr(get_comm("tp"), "fused", None)
            ids = fused.greedy_argmax(lg, valid, self.start) if fused is not None else None
            if ids is not None:
                return ids
        val, idx = lg.float().max(-1)
        pair = torch.stack([val, (idx + self.start).float()], dim=-1)
        allp = get_comm("tp").all_gather(pair.unsqueeze(0), dim=0)    # [tp, B, 2]
        best = allp[..., 0].argmax(0)
        return allp[..., 1].gather(0, best.unsqueeze(0)).squeeze(0).long()
