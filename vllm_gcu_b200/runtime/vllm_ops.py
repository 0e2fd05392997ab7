"""This package's kernels behind vLLM's layer classes.

vLLM instantiates the class registered with ``CustomOp.register_oot`` in place of its own
whenever one exists under the same name, and a platform with the CUDA enum dispatches to
``forward_cuda``.  The subclasses below override ``forward_cuda`` with the sm_100a kernels
(RMSNorm with fused residual add, SiLU-and-mul) and fall back to the upstream method for what
they do not cover; the unquantised GEMM of every linear layer goes to the tcgen05 GEMM.  The
reference swaps its kernels into vLLM the same way (vllm_gcu/kernels/layernorm.py:10-41,
vllm_gcu/kernels/activation.py:20-32, vllm_gcu/kernels/linear.py).

These are eager (ctypes) launches: they are used when vLLM runs without ``torch.compile``
(``enforce_eager`` / compilation mode NONE, which ``B200Platform.check_and_update_config``
selects unless ``VLLM_B200_VLLM_NATIVE_OPS=0``).
"""
from __future__ import annotations

import torch

_DONE = False


def _ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and x.shape[-1] % 8 == 0 \
        and x.stride(-1) == 1


def register_ops() -> bool:
    """Idempotent; returns False when vLLM is not importable."""
    global _DONE
    if _DONE:
        return True
    try:
        from vllm.model_executor.layers.activation import SiluAndMul
        from vllm.model_executor.layers.layernorm import RMSNorm
        import vllm.model_executor.layers.utils as vutils
    except Exception:  # noqa: BLE001
        return False
    from ..ops import cuda as C

    @RMSNorm.register_oot
    class B200RMSNorm(RMSNorm):  # type: ignore[misc, valid-type]
        def forward_cuda(self, x, residual=None):
            if (not _ok(x) or getattr(self, "variance_size_override", None) is not None
                    or not getattr(self, "has_weight", True) or x.numel() == 0
                    or self.weight.dtype != x.dtype):
                return super().forward_cuda(x, residual)
            if residual is None:
                return C.norm(x, self.weight.data, self.variance_epsilon)
            out = C.norm(x, self.weight.data, self.variance_epsilon, residual=residual)
            return out, residual

    @SiluAndMul.register_oot
    class B200SiluAndMul(SiluAndMul):  # type: ignore[misc, valid-type]
        def forward_cuda(self, x):
            if not _ok(x) or (x.shape[-1] // 2) % 8 or x.numel() == 0:
                return super().forward_cuda(x)
            return C.activation(x, "silu", mode="act_mul")

    upstream_gemm = vutils.default_unquantized_gemm

    def b200_unquantized_gemm(layer, x, weight, bias=None):
        if (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                and weight.dim() == 2 and weight.stride(1) == 1 and x.shape[-1] % 8 == 0
                and weight.shape[0] % 8 == 0 and weight.stride(0) % 8 == 0 and x.numel() > 0
                and (bias is None or bias.dtype == torch.bfloat16)):
            x2 = x.reshape(-1, x.shape[-1])
            y = C.gemm_bf16(x2, weight, bias=bias)
            return y.view(*x.shape[:-1], weight.shape[0])
        return upstream_gemm(layer, x, weight, bias)

    vutils.default_unquantized_gemm = b200_unquantized_gemm
    _DONE = True
    return True
