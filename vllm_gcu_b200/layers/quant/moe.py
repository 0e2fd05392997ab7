"""Quantised checkpoints for mixture-of-experts layers.

The reference serves MoE models from AWQ / GPTQ (``moe_wna16_gcu``,
vllm_gcu/kernels/quantization/moe_wna16.py:26-643), fp8 block-scaled (fp8.py:215-380), int8
w8a8 (w8a8.py:174-342) and w4a8 (w4a8.py) expert tensors by re-arranging them at load time
and running a quantised grouped GEMM.  Here the expert tensors of those checkpoint formats
are read unchanged.  On a GPU, fp8 experts with 128 x 128 block scales and int8 / fp8 experts
with per-channel scales stay quantised and run through the grouped 8-bit tcgen05 GEMM
(``expert_storage``); AWQ / GPTQ experts stay packed 4 / 8-bit integers with their per-group
scales and run through the grouped de-quantising GEMM (``b200_gemm_wna16_grouped``); every
format on the CPU path (and shapes the kernels do not cover) is de-quantised **once at load
time** into the bf16 expert tensors of the bf16 grouped GEMM (bf16 footprint).
File formats and the routing / expert-parallel behaviour are the same either way.

``QuantExpertLoader`` collects the pieces of one expert projection (``qweight`` / ``qzeros``
/ ``scales`` / ``g_idx``, or ``weight`` / ``weight_scale`` / ``weight_scale_inv``) as the
checkpoint iterator yields them and hands the de-quantised matrix to
``FusedMoE.load_expert_weight`` when the set is complete.
"""
from __future__ import annotations

from typing import Optional

import torch

FP8 = torch.float8_e4m3fn

_PIECES = {
    "awq": ("qweight", "qzeros", "scales"),
    "gptq": ("qweight", "qzeros", "scales"),
    "fp8": ("weight",),           # + weight_scale or weight_scale_inv when present
    "w8a8": ("weight",),          # + weight_scale / out_scales
}


def dequant_fp8(weight: torch.Tensor, scale: Optional[torch.Tensor],
                block: Optional[list[int]], dtype: torch.dtype) -> torch.Tensor:
    w = weight.to(torch.float32)
    if scale is None:
        return w.to(dtype)
    s = scale.to(torch.float32)
    if block and s.dim() == 2:
        bn, bk = block
        s = s.repeat_interleave(bn, 0)[: w.shape[0]].repeat_interleave(bk, 1)[:, : w.shape[1]]
        return (w * s).to(dtype)
    if s.numel() == 1:
        return (w * s.reshape(())).to(dtype)
    return (w * s.reshape(-1, 1)).to(dtype)


def dequant_int8(weight: torch.Tensor, scale: Optional[torch.Tensor], dtype: torch.dtype
                 ) -> torch.Tensor:
    w = weight.to(torch.float32)
    if scale is not None:
        s = scale.to(torch.float32)
        w = w * (s.reshape(()) if s.numel() == 1 else s.reshape(-1, 1))
    return w.to(dtype)


def dequant_wna16(kind: str, bits: int, group: int, qweight: torch.Tensor, qzeros: torch.Tensor,
                  scales: torch.Tensor, dtype: torch.dtype, sym: bool = False) -> torch.Tensor:
    """AWQ / GPTQ tensors of one projection -> ``[N, K]`` weight."""
    from . import unpack_awq, unpack_gptq
    if kind == "awq":
        w, z = unpack_awq(qweight, qzeros)              # [K, N], [K/g, N]
        z = z.to(torch.float32)
    else:
        w, z = unpack_gptq(qweight, qzeros, bits)
        z = z.to(torch.float32)
        if sym:
            z = torch.full_like(z, float(1 << (bits - 1)))
    K = w.shape[0]
    g = group if group > 0 else K
    s = scales.to(torch.float32)                         # [K/g, N]
    zf = z.repeat_interleave(g, 0)[:K]
    sf = s.repeat_interleave(g, 0)[:K]
    return ((w.to(torch.float32) - zf) * sf).t().contiguous().to(dtype)


def unpack_wna16(kind: str, bits: int, qweight: torch.Tensor, qzeros: torch.Tensor,
                 scales: torch.Tensor, sym: bool = False):
    """AWQ / GPTQ tensors of one projection -> integers ``q [N, K]`` (uint8), ``scale
    [N, K/g]`` and ``zs = zero * scale [N, K/g]`` (the device layout of the de-quantising
    GEMMs before nibble packing): ``w = q * scale - zs``."""
    from . import unpack_awq, unpack_gptq
    if kind == "awq":
        w, z = unpack_awq(qweight, qzeros)              # [K, N], [K/g, N]
    else:
        w, z = unpack_gptq(qweight, qzeros, bits)
        if sym:
            z = torch.full_like(z, 1 << (bits - 1))
    sc = scales.t().contiguous()                         # [N, K/g]
    zs = (z.t().to(torch.float32) * sc.to(torch.float32)).to(sc.dtype).contiguous()
    return w.t().contiguous().to(torch.uint8), sc, zs


def expert_storage(quant_name: Optional[str], quant_cfg: Optional[dict]) -> Optional[str]:
    """How a GPU keeps the experts of a checkpoint format: ``"fp8_block"`` (fp8, 128 x 128
    scales), ``"fp8"`` / ``"int8"`` (one scale per output channel), ``"wna16"`` (AWQ / GPTQ
    integers with per-group scales, packed) or None (de-quantised to bf16 at load: act-order
    GPTQ, unknown block shapes)."""
    n = (quant_name or "").replace("_gcu", "")
    q = quant_cfg or {}
    method = {"compressed-tensors": "w8a8"}.get(q.get("quant_method", n), q.get("quant_method", n))
    if method == "fp8":
        block = q.get("weight_block_size")
        if block:
            return "fp8_block" if list(block) == [128, 128] else None
        return "fp8"
    if method == "w8a8":
        return "int8"
    if n in ("moe_wna16", "w4a8"):
        method = q.get("quant_method", "awq") if q.get("quant_method") in ("awq", "gptq") \
            else "awq"
    if method in ("awq", "gptq") and int(q.get("bits", q.get("w_bit", 4))) in (4, 8) \
            and not q.get("desc_act", False):
        return "wna16"
    return None


class QuantExpertLoader:
    """Buffers quantised expert tensors until a projection is complete."""

    def __init__(self, quant_name: str, quant_cfg: dict, dtype: torch.dtype):
        n = (quant_name or "").replace("_gcu", "")
        q = quant_cfg or {}
        method = q.get("quant_method", n)
        if n in ("moe_wna16", "w4a8"):
            method = q.get("quant_method", "awq")
        self.kind = {"compressed-tensors": "w8a8"}.get(method, method)
        if self.kind not in _PIECES:
            raise ValueError(f"no expert loader for quantization {quant_name!r}")
        self.bits = int(q.get("bits", q.get("w_bit", 4)))
        self.group = int(q.get("group_size", q.get("q_group_size", 128)))
        self.sym = bool(q.get("sym", False))
        self.block = q.get("weight_block_size")
        self.dtype = dtype
        self.pending: dict[tuple, dict[str, torch.Tensor]] = {}

    def add(self, moe, layer_key: str, expert: int, which: str, piece: str,
            tensor: torch.Tensor) -> None:
        """``piece`` is the tensor's suffix (``qweight``, ``scales``, ``weight_scale_inv``...)."""
        le = expert - moe.expert_start
        if le < 0 or le >= moe.local_experts:
            return                                        # the expert lives on another rank
        key = (layer_key, expert, which)
        d = self.pending.setdefault(key, {})
        d[piece] = tensor
        if piece == "g_idx":
            g = tensor.to(torch.int64)
            want = torch.arange(g.numel(), device=g.device) // max(self.group, 1)
            if self.group > 0 and not torch.equal(g, want):
                raise ValueError("GPTQ act-order (shuffled g_idx) is not supported")
        if not all(p in d for p in _PIECES[self.kind]):
            return
        if self.kind in ("awq", "gptq") and getattr(moe, "wna16", None):
            q, sc, zs = unpack_wna16(self.kind, self.bits, d["qweight"], d["qzeros"], d["scales"],
                                     self.sym)
            del self.pending[key]
            moe.load_expert_weight_wna16(expert, which, q, sc, zs)
            return
        if self.kind in ("awq", "gptq"):
            w = dequant_wna16(self.kind, self.bits, self.group, d["qweight"], d["qzeros"],
                              d["scales"], self.dtype, self.sym)
            del self.pending[key]
        else:
            # the scale may arrive after the weight: wait for it unless the format has none
            sc = d.get("weight_scale_inv", d.get("weight_scale", d.get("out_scales")))
            if sc is None and not d.get("_flushed"):
                return
            if (self.kind == "fp8" and getattr(moe, "fp8_block", False) and sc is not None
                    and sc.dim() == 2 and d["weight"].dtype == torch.float8_e4m3fn):
                # the experts stay fp8 with their block scales (grouped fp8 GEMM path)
                moe.load_expert_weight_fp8(expert, which, d["weight"], sc.to(torch.float32))
                del self.pending[key]
                return
            if getattr(moe, "q8_channel", False) and d["weight"].dtype == moe.w13.dtype and (
                    sc is None or sc.dim() <= 1 or sc.shape[-1] == 1):
                moe.load_expert_weight_q8(expert, which, d["weight"], sc)
                del self.pending[key]
                return
            w = (dequant_fp8(d["weight"], sc, self.block, self.dtype) if self.kind == "fp8"
                 else dequant_int8(d["weight"], sc, self.dtype))
            del self.pending[key]
        moe.load_expert_weight(expert, which, w)

    def flush(self, resolve) -> None:
        """Loads projections whose optional scale never came (unscaled fp8 / int8).
        ``resolve(layer_key)`` returns the FusedMoE module."""
        for (layer_key, expert, which), d in list(self.pending.items()):
            if "weight" in d and self.kind in ("fp8", "w8a8"):
                moe = resolve(layer_key)
                if getattr(moe, "q8_channel", False) and d["weight"].dtype == moe.w13.dtype:
                    moe.load_expert_weight_q8(expert, which, d["weight"], None)
                    del self.pending[(layer_key, expert, which)]
                    continue
                w = (dequant_fp8(d["weight"], None, self.block, self.dtype) if self.kind == "fp8"
                     else dequant_int8(d["weight"], None, self.dtype))
                moe.load_expert_weight(expert, which, w)
                del self.pending[(layer_key, expert, which)]
        if self.pending:
            missing = sorted(f"{k[0]}experts.{k[1]}.{k[2]}" for k in self.pending)[:4]
            raise ValueError(f"incomplete quantised expert tensors, e.g. {missing}")
