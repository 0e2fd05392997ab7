"""Quantised linear methods and their checkpoint formats.

Registered names (the reference registers the same schemes with a ``_gcu`` suffix and
auto-selects them for HF ``quant_method`` values, vllm_gcu/gcu.py:53-64,
vllm_gcu/kernels/quantization/*.py); both spellings are accepted here:

=============  ==========================================================================
``fp8``        e4m3 weights.  Per-tensor / per-channel ``weight_scale`` with dynamic
               per-token (or static ``input_scale``) activations -> row x column scaled
               tcgen05 fp8 GEMM; or ``weight_block_size: [128, 128]`` with
               ``weight_scale_inv`` and dynamic 1x128 activation scales -> block-scaled GEMM
               (vllm_gcu/kernels/quantization/fp8.py:22-212)
``w8a8``       int8 weights ``[N, K]``, per-channel ``out_scales`` (or ``weight_scale``),
               optional smooth-quant ``in_scales`` (static per-tensor activation scale),
               else dynamic per-token (w8a8.py:26-348, compressed-tensors int8)
``awq``        ``qweight int32 [K, N/8]``, ``qzeros int32 [K/g, N/8]``, ``scales [K/g, N]``,
               AWQ nibble order (awq.py:21-134, rearrange.py:61-133)
``gptq``       ``qweight int32 [K/8 | K/4, N]``, ``qzeros``, ``scales``, ``g_idx`` (contiguous
               groups only, gptq.py:141-143); 4 and 8 bit (gptq.py:31-296)
=============  ==========================================================================

Weights are re-packed once after loading into this library's own K-major device layouts;
the checkpoint files are read unchanged.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops
from ...ops import cuda as C
from ...ops import ref
from ..linear import LinearBase, LinearMethod, UnquantizedLinearMethod

FP8 = torch.float8_e4m3fn
AWQ_REVERSE_ORDER = [0, 4, 1, 5, 2, 6, 3, 7]


def _param(t: torch.Tensor) -> nn.Parameter:
    return nn.Parameter(t, requires_grad=False)


# =============================================================================
# fp8
# =============================================================================
class Fp8LinearMethod(LinearMethod):
    def __init__(self, block_size: Optional[list[int]], activation_static: bool):
        self.block = block_size
        self.static_act = activation_static

    def create_weights(self, layer: LinearBase) -> None:
        N, K = layer.out_per_rank, layer.in_per_rank
        layer.weight = _param(torch.empty(N, K, dtype=FP8, device=layer.device))
        if self.block:
            bn, bk = self.block
            layer.weight_scale_inv = _param(torch.ones(-(-N // bn), -(-K // bk),
                                                       dtype=torch.float32, device=layer.device))
        else:
            layer.weight_scale = _param(torch.ones(N, dtype=torch.float32, device=layer.device))
            if self.static_act:
                layer.input_scale = _param(torch.ones(1, dtype=torch.float32,
                                                      device=layer.device))

    def load_weight(self, layer: LinearBase, name: str, full: torch.Tensor, shard_id) -> bool:
        if name == "weight":
            if full.dtype != FP8:       # bf16 checkpoint quantised on the fly (per channel)
                w = torch.empty(layer.weight.shape, dtype=full.dtype, device=full.device)
                layer.copy_sharded(w, full, shard_id, 0, 1)
                if self.block:
                    raise ValueError("block-scaled fp8 needs a pre-quantised checkpoint")
                q, s = ref.dynamic_per_token_fp8_quant(w)
                layer.weight.data.copy_(q)
                layer.weight_scale.data.copy_(s.flatten())
                layer._online_quant = True
                return True
            layer.copy_sharded(layer.weight.data.view(torch.uint8), full.view(torch.uint8),
                               shard_id, 0, 1)
            return True
        if name == "weight_scale_inv":
            bn, bk = self.block
            layer.copy_sharded(layer.weight_scale_inv.data, full.float(), shard_id, 0, 1, bn, bk)
            return True
        if name == "weight_scale":
            if getattr(layer, "_online_quant", False):
                return True
            f = full.float().reshape(-1)
            if f.numel() == 1:          # per-tensor (per merged shard): broadcast over its rows
                segs, _ = layer.shard_spec(shard_id)
                if segs is None:
                    layer.weight_scale.data.fill_(float(f))
                else:
                    for so, n, do in segs:
                        layer.weight_scale.data[do:do + n] = float(f)
            else:
                layer.copy_sharded(layer.weight_scale.data, f, shard_id, 0, -1)
            return True
        if name == "input_scale":
            if self.static_act:
                layer.input_scale.data = torch.maximum(layer.input_scale.data,
                                                       full.float().reshape(-1)[:1].to(
                                                           layer.input_scale.device))
            return True
        return False

    def input_quant(self, layer: LinearBase):
        if self.block:
            return ("fp8_group128", None) if self.block[1] == 128 else None
        if self.static_act:
            return "fp8_static", layer.input_scale
        return "fp8_token", None

    def apply(self, layer: LinearBase, x: torch.Tensor, skip_bias=False, x_scale=None, **kw):
        """``x`` may already be fp8 with ``x_scale`` given (producer fused the quantisation,
        vllm_gcu/kernels/quantization/fp8.py:50-69)."""
        bias = None if skip_bias else layer.bias
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        N = layer.weight.shape[0]
        if ops.use_native(x2):
            if x2.dtype != FP8:
                if self.block:
                    x2, x_scale = C.activation(x2, "identity", mode="plain", quant="fp8_group128")
                elif self.static_act:
                    x2 = C.activation(x2, "identity", mode="plain", quant="fp8_static",
                                      scale=layer.input_scale)
                    x_scale = layer.input_scale.expand(x2.shape[0]).contiguous()
                else:
                    x2, x_scale = C.per_token_quant(x2, "fp8")
            if self.block:
                y = C.gemm_q8(x2, layer.weight, x_scale, layer.weight_scale_inv, bias, kind=1)
            else:
                y = C.gemm_q8(x2, layer.weight, x_scale.reshape(-1), layer.weight_scale, bias,
                              kind=0)
            return y.view(*shape[:-1], N)
        # reference path
        out_dtype = torch.bfloat16 if x.dtype == FP8 else x.dtype
        if x2.dtype != FP8:
            if self.block:
                x2, x_scale = ref.per_token_group_fp8_quant(x2, self.block[1])
            elif self.static_act:
                x_scale = layer.input_scale
                x2 = ref.static_scaled_fp8_quant(x2, x_scale)
            else:
                x2, x_scale = ref.dynamic_per_token_fp8_quant(x2)
        if self.block:
            bn, bk = self.block
            K = x2.shape[1]
            xs = x2.float().view(-1, K // bk, bk) * x_scale[..., None]
            ws = layer.weight_scale_inv.repeat_interleave(bn, 0)[:N].repeat_interleave(bk, 1)[:, :K]
            y = xs.view(-1, K) @ (layer.weight.float() * ws).t()
        else:
            y = (x2.float() * x_scale.reshape(-1, 1)) @ (layer.weight.float()
                                                       * layer.weight_scale[:, None]).t()
        if bias is not None:
            y = y + bias.float()
        return y.to(out_dtype).view(*shape[:-1], N)


# =============================================================================
# int8 w8a8
# =============================================================================
class Int8LinearMethod(LinearMethod):
    def __init__(self, static_act: bool):
        self.static_act = static_act

    def create_weights(self, layer: LinearBase) -> None:
        N, K = layer.out_per_rank, layer.in_per_rank
        layer.weight = _param(torch.zeros(N, K, dtype=torch.int8, device=layer.device))
        layer.out_scales = _param(torch.ones(N, dtype=torch.float32, device=layer.device))
        if self.static_act:
            layer.in_scale = _param(torch.ones(1, dtype=torch.float32, device=layer.device))

    def load_weight(self, layer, name, full, shard_id) -> bool:
        if name == "weight":
            layer.copy_sharded(layer.weight.data, full, shard_id, 0, 1)
            return True
        if name in ("out_scales", "weight_scale"):
            layer.copy_sharded(layer.out_scales.data, full.float().reshape(-1), shard_id, 0, -1)
            return True
        if name in ("in_scales", "input_scale"):
            if self.static_act:
                # smooth-quant stores a per-input-channel vector whose maximum is the
                # static activation scale of the quantised matmul
                layer.in_scale.data.fill_(float(full.float().max()))
            return True
        return False

    def input_quant(self, layer):
        return ("int8_static", layer.in_scale) if self.static_act else ("int8_token", None)

    def apply(self, layer, x, skip_bias=False, x_scale=None, **kw):
        bias = None if skip_bias else layer.bias
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        N = layer.weight.shape[0]
        if ops.use_native(x2) and x2.dtype == torch.int8:
            # the producing norm / activation kernel quantised the rows already
            y = C.gemm_q8(x2, layer.weight, x_scale.reshape(-1), layer.out_scales, bias, kind=2)
            return y.view(*shape[:-1], N)
        if ops.use_native(x2):
            if self.static_act:
                q = C.activation(x2, "identity", mode="plain", quant="int8_static",
                                 scale=layer.in_scale)
                s = layer.in_scale.expand(x2.shape[0]).contiguous()
            else:
                q, s = C.per_token_quant(x2, "int8")
            y = C.gemm_q8(q, layer.weight, s.reshape(-1), layer.out_scales, bias, kind=2)
            return y.view(*shape[:-1], N)
        if self.static_act:
            q = ref.static_scaled_int8_quant(x2, layer.in_scale)
            s = layer.in_scale.reshape(1, 1)
        else:
            q, s = ref.dynamic_scaled_int8_quant(x2)
        y = (q.float() @ layer.weight.float().t()) * s * layer.out_scales[None, :]
        if bias is not None:
            y = y + bias.float()
        return y.to(x.dtype).view(*shape[:-1], N)


# =============================================================================
# weight-only 4 / 8 bit (AWQ, GPTQ)
# =============================================================================
def unpack_awq(qweight: torch.Tensor, qzeros: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """int32 ``[K, N/8]`` / ``[K/g, N/8]`` -> uint8 ``[K, N]`` / ``[K/g, N]`` in natural order."""
    shifts = torch.arange(0, 32, 4, device=qweight.device)
    order = torch.tensor(AWQ_REVERSE_ORDER, device=qweight.device)

    def un(t):
        v = (t[:, :, None] >> shifts[None, None, :]) & 0xF        # [R, N/8, 8] nibble order
        return v[:, :, order].reshape(t.shape[0], -1).to(torch.uint8)

    return un(qweight), un(qzeros)


def unpack_gptq(qweight: torch.Tensor, qzeros: torch.Tensor, bits: int
                ) -> tuple[torch.Tensor, torch.Tensor]:
    """qweight int32 ``[K*bits/32, N]`` -> uint8 ``[K, N]``; qzeros int32
    ``[K/g, N*bits/32]`` -> ``[K/g, N]`` (stored value + 1 = zero point)."""
    per = 32 // bits
    mask = (1 << bits) - 1
    shifts = torch.arange(0, 32, bits, device=qweight.device)
    w = ((qweight[:, None, :] >> shifts[None, :, None]) & mask).reshape(-1, qweight.shape[1])
    z = ((qzeros[:, :, None] >> shifts[None, None, :]) & mask).reshape(qzeros.shape[0], -1)
    return w.to(torch.uint8), (z + 1).to(torch.int16)


class WNA16LinearMethod(LinearMethod):
    """AWQ / GPTQ weight-only quantisation.  Device layout after loading: ``qw`` uint8
    ``[N, K/2]`` (two nibbles per byte, low = even k) or ``[N, K]`` for 8 bit, ``scales``
    and ``zs = zero * scale`` as ``[N, K/g]``.  On the GPU, inputs of up to 256 rows go
    through the fused de-quantising GEMM (csrc/gemm_wna16.cu); larger ones de-quantise the
    layer into a shared bf16 scratch and run the bf16 tcgen05 GEMM on it."""

    _scratch: dict = {}

    def __init__(self, fmt: str, bits: int, group_size: int, sym: bool = False):
        self.fmt, self.bits, self.g, self.sym = fmt, bits, group_size, sym

    def create_weights(self, layer: LinearBase) -> None:
        N, K = layer.out_per_rank, layer.in_per_rank
        g = self.g if self.g > 0 else K
        dev = layer.device
        per = 32 // self.bits
        if self.fmt == "awq":
            layer.qweight = _param(torch.zeros(K, N // 8, dtype=torch.int32, device=dev))
            layer.qzeros = _param(torch.zeros(K // g, N // 8, dtype=torch.int32, device=dev))
        else:
            layer.qweight = _param(torch.zeros(K // per, N, dtype=torch.int32, device=dev))
            layer.qzeros = _param(torch.zeros(K // g, N // per, dtype=torch.int32, device=dev))
            layer.g_idx = _param(torch.zeros(K, dtype=torch.int32, device=dev))
        layer.scales = _param(torch.zeros(K // g, N, dtype=layer.dtype, device=dev))

    def load_weight(self, layer, name, full, shard_id) -> bool:
        per = 32 // self.bits
        g = self.g if self.g > 0 else layer.in_features
        if name == "qweight":
            if self.fmt == "awq":
                layer.copy_sharded(layer.qweight.data, full, shard_id, 1, 0, 8, 1)
            else:
                layer.copy_sharded(layer.qweight.data, full, shard_id, 1, 0, 1, per)
            return True
        if name == "qzeros":
            layer.copy_sharded(layer.qzeros.data, full, shard_id, 1, 0,
                               8 if self.fmt == "awq" else per, g)
            return True
        if name == "scales":
            layer.copy_sharded(layer.scales.data, full, shard_id, 1, 0, 1, g)
            return True
        if name == "g_idx":
            if self.fmt == "gptq":
                _, rng = layer.shard_spec(shard_id)
                gi = full if rng is None else full.narrow(0, rng[0], rng[1])
                expect = torch.arange(gi.numel(), device=gi.device) // g + (
                    0 if rng is None else rng[0] // g)
                if not torch.equal(gi.long().cpu(), expect.long().cpu()):
                    raise ValueError("GPTQ act-order (shuffled g_idx) is not supported")
            return True
        return False

    def process_weights_after_loading(self, layer: LinearBase) -> None:
        if hasattr(layer, "qw"):
            return
        if self.fmt == "awq":
            w, z = unpack_awq(layer.qweight.data, layer.qzeros.data)
            z = z.to(torch.int16)
        else:
            w, z = unpack_gptq(layer.qweight.data, layer.qzeros.data, self.bits)
            if self.sym and self.bits == 8:
                pass
        K, N = w.shape
        wt = w.t().contiguous()                                   # [N, K]
        if self.bits == 4:
            qw = (wt[:, 0::2] | (wt[:, 1::2] << 4)).contiguous()
        else:
            qw = wt
        sc = layer.scales.data.t().contiguous()                   # [N, K/g]
        zs = (z.t().float() * sc.float()).to(sc.dtype).contiguous()
        layer.qw, layer.sc, layer.zs = _param(qw), _param(sc), _param(zs)
        for n in ("qweight", "qzeros", "scales", "g_idx"):
            if hasattr(layer, n):
                delattr(layer, n)

    def dequantize(self, layer: LinearBase) -> torch.Tensor:
        g = self.g if self.g > 0 else layer.in_per_rank
        N = layer.qw.shape[0]
        K = layer.in_per_rank
        if ops.use_native(layer.qw) and layer.sc.dtype in (torch.bfloat16, torch.float16):
            key = (layer.qw.device, layer.sc.dtype)
            buf = WNA16LinearMethod._scratch.get(key)
            if buf is None or buf.numel() < N * K:
                buf = torch.empty(max(N * K, 1 << 20), dtype=layer.sc.dtype, device=layer.qw.device)
                WNA16LinearMethod._scratch[key] = buf
            w = buf[: N * K].view(N, K)
            C.weight_dequant(layer.qw, layer.sc, layer.zs, w, g, self.bits)
            return w
        if self.bits == 4:
            q = torch.stack([layer.qw & 0xF, layer.qw >> 4], dim=-1).reshape(N, K)
        else:
            q = layer.qw
        s = layer.sc.float().repeat_interleave(g, 1)
        z = layer.zs.float().repeat_interleave(g, 1)
        return (q.float() * s - z).to(layer.sc.dtype)

    def apply(self, layer, x, skip_bias=False, residual=None, **kw):
        if not hasattr(layer, "qw"):
            self.process_weights_after_loading(layer)
        bias = None if skip_bias else layer.bias
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if (ops.use_native(x2) and x2.dtype == torch.bfloat16
                and x2.shape[0] <= C.WNA16_FUSED_MAX_M):
            # decode-sized input: de-quantise inside the GEMM (reads the packed weights only)
            g = self.g if self.g > 0 else layer.in_per_rank
            y = C.gemm_wna16(x2, layer.qw, layer.sc, layer.zs, g, self.bits, bias)
            if y is not None:
                return y.view(*shape[:-1], y.shape[1])
        w = self.dequantize(layer)
        if ops.use_native(x2) and x2.dtype == torch.bfloat16:
            y = C.gemm_bf16(x2, w, bias=bias)
        else:
            y = F.linear(x2, w.to(x2.dtype), bias)
        return y.view(*shape[:-1], w.shape[0])


# =============================================================================
# configs
# =============================================================================
class QuantConfig:
    name = "none"

    def __init__(self, cfg: dict):
        self.cfg = cfg or {}
        ignore = self.cfg.get("ignored_layers") or self.cfg.get("modules_to_not_convert") or []
        self.ignored = list(ignore)

    def is_ignored(self, prefix: str) -> bool:
        if "lm_head" in prefix:
            return True
        return any(ig and ig in prefix for ig in self.ignored)

    def get_linear_method(self, prefix: str) -> Optional[LinearMethod]:
        if self.is_ignored(prefix):
            return None
        return self._method(prefix)

    def _method(self, prefix: str) -> Optional[LinearMethod]:
        raise NotImplementedError


class Fp8Config(QuantConfig):
    name = "fp8"

    def _method(self, prefix):
        return Fp8LinearMethod(self.cfg.get("weight_block_size"),
                               self.cfg.get("activation_scheme", "dynamic") == "static")


class W8A8Config(QuantConfig):
    name = "w8a8"

    def _method(self, prefix):
        return Int8LinearMethod(bool(self.cfg.get("static_activation",
                                                  self.cfg.get("smooth_quant", False))))


class AWQConfig(QuantConfig):
    name = "awq"

    def _method(self, prefix):
        bits = int(self.cfg.get("bits", self.cfg.get("w_bit", 4)))
        g = int(self.cfg.get("group_size", self.cfg.get("q_group_size", 128)))
        if bits != 4:
            raise ValueError("AWQ supports 4-bit weights only")
        return WNA16LinearMethod("awq", 4, g)


class GPTQConfig(QuantConfig):
    name = "gptq"

    def _method(self, prefix):
        bits = int(self.cfg.get("bits", 4))
        if bits not in (4, 8):
            raise ValueError("GPTQ supports 4- and 8-bit weights")
        if self.cfg.get("desc_act", False):
            raise ValueError("GPTQ act-order (desc_act) is not supported")
        return WNA16LinearMethod("gptq", bits, int(self.cfg.get("group_size", 128)),
                                 bool(self.cfg.get("sym", False)))


class MoeWNA16Config(QuantConfig):
    """``moe_wna16``: AWQ or GPTQ tensors for the experts (de-quantised at load, see
    ``layers.quant.moe``) and the matching weight-only method for the linear layers
    (vllm_gcu/kernels/quantization/moe_wna16.py:26-643)."""
    name = "moe_wna16"

    def __init__(self, cfg: dict):
        super().__init__(cfg)
        inner = (self.cfg.get("quant_method") or "awq").replace("_gcu", "")
        self.inner = (GPTQConfig if inner == "gptq" else AWQConfig)(cfg)

    def _method(self, prefix):
        return self.inner._method(prefix)


class W4A8Config(Fp8Config):
    """``w4a8``: int4 expert tensors (group scales), fp8 128x128 block-scaled dense layers
    (vllm_gcu/kernels/quantization/w4a8.py:134-235)."""
    name = "w4a8"


_CONFIGS = {"fp8": Fp8Config, "fp8_gcu": Fp8Config, "w8a8": W8A8Config, "w8a8_gcu": W8A8Config,
            "compressed-tensors": W8A8Config, "awq": AWQConfig, "awq_gcu": AWQConfig,
            "gptq": GPTQConfig, "gptq_gcu": GPTQConfig, "moe_wna16": MoeWNA16Config,
            "moe_wna16_gcu": MoeWNA16Config, "w4a8": W4A8Config, "w4a8_gcu": W4A8Config}

SUPPORTED_QUANTIZATION = sorted(_CONFIGS)


def register_quantization_config(name: str, cls) -> None:
    """Same role as ``register_gcu_quantization_config``
    (vllm_gcu/kernels/quantization/utils.py:10-13)."""
    _CONFIGS[name] = cls


def get_quant_config(model_cfg) -> QuantConfig:
    cached = getattr(model_cfg, "_quant_config_obj", None)
    if cached is not None:
        return cached
    name = model_cfg.quantization
    if name not in _CONFIGS:
        raise ValueError(f"unsupported quantization {name!r}; known: {sorted(_CONFIGS)}")
    obj = _CONFIGS[name](model_cfg.quant_config or {})
    object.__setattr__(model_cfg, "_quant_config_obj", obj)
    return obj
