"""8-bit linear layers of vLLM on this package's GEMMs.

vLLM picks the kernel of a quantised linear layer from per-platform priority lists
(``vllm.model_executor.kernels.linear``); ``register_linear_kernels`` puts the two classes
below at the head of the CUDA lists, so fp8 (``quantization="fp8"``, compressed-tensors fp8)
and int8 w8a8 layers quantise their activations with ``b200_per_token_quant`` /
``b200_activation`` and multiply with ``b200_gemm_q8`` (tcgen05, ``csrc/gemm_q8.cu``).  The
reference reaches its own quantised GEMMs from vLLM through its quantisation configs
(vllm_gcu/kernels/quantization/fp8.py:50-69,169-205, w8a8.py:174-342).

Covered: fp8 e4m3 weights with one scale per tensor or per output channel and activations
quantised per token (dynamic), per tensor (dynamic) or with a static scale; int8 weights with
symmetric activations (per token or static).  Everything else stays on vLLM's own kernels.
"""
from __future__ import annotations

import torch

_DONE = False


def _on_b200_platform() -> bool:
    from vllm.platforms import current_platform
    return type(current_platform).__name__ == "B200Platform"


def register_linear_kernels() -> bool:
    """Idempotent; returns False when this vLLM has no kernel lists to extend."""
    global _DONE
    if _DONE:
        return True
    try:
        import vllm.model_executor.kernels.linear as vk
        from vllm.model_executor.kernels.linear.scaled_mm.ScaledMMLinearKernel import (
            FP8ScaledMMLinearKernel, Int8ScaledMMLinearKernel)
        from vllm.platforms import PlatformEnum
    except Exception:  # noqa: BLE001
        return False
    from ..ops import cuda as C

    def _channel_scales(scale: torch.Tensor, n: int, widths) -> torch.Tensor:
        """fp32 ``[n]`` from a per-tensor scalar, one scalar per fused shard, or ``[n(, 1)]``."""
        s = scale.detach().float().reshape(-1)
        if s.numel() == n:
            return s.contiguous()
        if s.numel() == 1:
            return s.expand(n).contiguous()
        if widths is not None and s.numel() == len(widths) and sum(widths) == n:
            return torch.cat([s[i].expand(w) for i, w in enumerate(widths)]).contiguous()
        raise ValueError(f"cannot broadcast {tuple(scale.shape)} weight scales over {n} channels")

    class B200FP8ScaledMMLinearKernel(FP8ScaledMMLinearKernel):  # type: ignore[misc, valid-type]
        @classmethod
        def is_supported(cls, compute_capability=None):
            if not _on_b200_platform():
                return False, "needs the B200 platform plugin"
            return True, None

        @classmethod
        def can_implement(cls, c):
            if c.out_dtype not in (None, torch.bfloat16) or c.input_dtype != torch.bfloat16:
                return False, "b200_gemm_q8 writes bf16"
            a, w = c.activation_quant_key.scale, c.weight_quant_key.scale
            if a.group_shape.is_per_group() or w.group_shape.is_per_group():
                return False, "grouped scales go to the block-scaled kernels"
            n, k = c.weight_shape
            if n % 16 or k % 16:
                return False, "N and K must be multiples of 16"
            return True, None

        def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
            w_name, ws_name, _, _ = self.layer_param_names
            w = getattr(layer, w_name)             # [K, N]: the transpose of the stored [N, K]
            w_nk = w.t()
            layer._b200_w = w_nk if w_nk.is_contiguous() else w_nk.contiguous()
            layer._b200_ws = _channel_scales(getattr(layer, ws_name), layer._b200_w.shape[0],
                                             getattr(layer, "logical_widths", None))

        def _quantise(self, x2: torch.Tensor, x_s):
            a = self.config.activation_quant_key.scale
            M = x2.shape[0]
            if a.static:
                s = x_s.detach().float().reshape(-1)[:1]
                q = C.activation(x2, "identity", mode="plain", quant="fp8_static", scale=s)
                return q, s.expand(M).contiguous()
            if a.group_shape.is_per_token():
                q, s = C.per_token_quant(x2, "fp8")
                return q, s.reshape(-1)
            q, s = C.per_tensor_fp8_quant(x2)
            return q, s.expand(M).contiguous()

        def apply_weights(self, layer, x, bias=None):
            _, _, x_s, x_s_ub = self._get_layer_params(layer)
            x2 = x.reshape(-1, x.shape[-1])
            ok = (x2.is_cuda and x2.shape[0] > 0 and x_s_ub is None and hasattr(layer, "_b200_w")
                  and (x2.dtype == torch.bfloat16 or x2.dtype == self.fp8_dtype)
                  and (bias is None or bias.dtype == torch.bfloat16))
            if not ok:
                return self._fallback(layer, x, bias)
            if x2.dtype == self.fp8_dtype:
                q, s = x2, x_s.detach().float().reshape(-1)
                if s.numel() == 1:
                    s = s.expand(x2.shape[0]).contiguous()
            else:
                q, s = self._quantise(x2.contiguous() if x2.stride(-1) != 1 else x2, x_s)
            y = C.gemm_q8(q, layer._b200_w, s, layer._b200_ws, bias, kind=0)
            return y.view(*x.shape[:-1], layer._b200_w.shape[0])

        def _fallback(self, layer, x, bias):
            # de-quantised weights through the bf16 path (empty batches, unusual dtypes)
            w = layer._b200_w.to(torch.float32) * layer._b200_ws[:, None]
            y = torch.nn.functional.linear(x.float(), w, None if bias is None else bias.float())
            return y.to(x.dtype if x.dtype != self.fp8_dtype else torch.bfloat16)

        def apply_scaled_mm(self, *, A, B, out_dtype, As, Bs, bias, output_shape):
            n = B.shape[1]
            b_nk = B.t()
            b_nk = b_nk if b_nk.is_contiguous() else b_nk.contiguous()
            a_s = As.detach().float().reshape(-1)
            if a_s.numel() == 1:
                a_s = a_s.expand(A.shape[0]).contiguous()
            y = C.gemm_q8(A, b_nk, a_s, _channel_scales(Bs, n, None), bias, kind=0)
            return y.view(*output_shape)

    class B200Int8ScaledMMLinearKernel(Int8ScaledMMLinearKernel):  # type: ignore[misc, valid-type]
        @classmethod
        def is_supported(cls, compute_capability=None):
            if not _on_b200_platform():
                return False, "needs the B200 platform plugin"
            return True, None

        @classmethod
        def can_implement(cls, c):
            if not c.input_symmetric:
                return False, "asymmetric activations stay on the upstream kernel"
            return True, None

        def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
            w_name, ws_name, i_s_name, i_zp_name, azp_name = self.layer_param_names
            w = getattr(layer, w_name)             # [N, K] as stored
            layer._b200_w = w.data if w.is_contiguous() else w.data.contiguous()
            layer._b200_ws = _channel_scales(getattr(layer, ws_name), w.shape[0],
                                             getattr(layer, "logical_widths", None))
            if self.config.is_static_input_scheme:
                s = getattr(layer, i_s_name).detach().float().max().reshape(1)
                layer._b200_is = s.contiguous()
            setattr(layer, i_zp_name, None)
            setattr(layer, azp_name, None)

        def apply_weights(self, layer, x, bias=None):
            x2 = x.reshape(-1, x.shape[-1])
            if x2.stride(-1) != 1:
                x2 = x2.contiguous()
            M = x2.shape[0]
            if M == 0 or not x2.is_cuda or x2.dtype not in (torch.bfloat16, torch.float16) \
                    or (bias is not None and bias.dtype != torch.bfloat16):
                w = layer._b200_w.float() * layer._b200_ws[:, None]
                return torch.nn.functional.linear(x.float(), w, None if bias is None
                                                  else bias.float()).to(x.dtype)
            if self.config.is_static_input_scheme:
                q = C.activation(x2, "identity", mode="plain", quant="int8_static",
                                 scale=layer._b200_is)
                s = layer._b200_is.expand(M).contiguous()
            else:
                q, s = C.per_token_quant(x2, "int8")
                s = s.reshape(-1)
            y = C.gemm_q8(q, layer._b200_w, s, layer._b200_ws, bias, kind=2)
            return y.to(x.dtype).view(*x.shape[:-1], layer._b200_w.shape[0])

    for table, cls in ((vk._POSSIBLE_FP8_KERNELS, B200FP8ScaledMMLinearKernel),
                       (vk._POSSIBLE_INT8_KERNELS, B200Int8ScaledMMLinearKernel)):
        lst = table.setdefault(PlatformEnum.CUDA, [])
        if not any(k.__name__ == cls.__name__ for k in lst):
            lst.insert(0, cls)
    backend_map = getattr(vk, "_LINEAR_BACKEND_KERNEL_MAP", None)
    if isinstance(backend_map, dict):
        backend_map.setdefault("b200", set()).update({B200FP8ScaledMMLinearKernel,
                                                      B200Int8ScaledMMLinearKernel})
    globals()["B200FP8ScaledMMLinearKernel"] = B200FP8ScaledMMLinearKernel
    globals()["B200Int8ScaledMMLinearKernel"] = B200Int8ScaledMMLinearKernel
    _DONE = True
    return True
