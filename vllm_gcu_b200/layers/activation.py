"""Activation layers: gated ``act(x[:d]) * x[d:]`` family and element-wise variants,
dispatched to the sm_100a kernel on GPUs (vllm_gcu/kernels/activation.py:16-80)."""
from __future__ import annotations

import torch

from .. import ops
from ..ops import cuda as C
from ..ops import ref

_GATED = {"silu": "silu", "swiglu": "silu", "gelu": "gelu", "gelu_tanh": "gelu_tanh",
          "gelu_pytorch_tanh": "gelu_tanh", "fatrelu": "fatrelu"}
_PLAIN = {"gelu_new": "gelu_new", "gelu_fast": "gelu_fast", "quick_gelu": "gelu_quick",
          "gelu_quick": "gelu_quick", "silu": "silu", "gelu": "gelu"}


def act_and_mul(x: torch.Tensor, act: str = "silu", threshold: float = 0.0) -> torch.Tensor:
    name = _GATED[act]
    if ops.use_native(x) and x.dtype in (torch.bfloat16, torch.float16) \
            and (x.shape[-1] // 2) % 8 == 0:
        return C.activation(x, name, mode="act_mul", threshold=threshold)
    return ref.act_and_mul(x, name, threshold)


def mul_and_silu(x: torch.Tensor) -> torch.Tensor:
    if ops.use_native(x) and x.dtype in (torch.bfloat16, torch.float16) \
            and (x.shape[-1] // 2) % 8 == 0:
        return C.activation(x, "silu", mode="mul_act")
    return ref.mul_and_silu(x)


def activation(x: torch.Tensor, act: str) -> torch.Tensor:
    name = _PLAIN[act]
    if ops.use_native(x) and x.dtype in (torch.bfloat16, torch.float16) and x.shape[-1] % 8 == 0:
        return C.activation(x, name, mode="plain")
    return ref.activation(x, name)
