"""Op surface of the package.

``ref``   – PyTorch reference of every op (semantics, CPU execution path, test oracle)
``cuda``  – launchers of the hand-written sm_100a kernels (``_b200.so``)

Layers pick ``cuda`` for CUDA tensors and ``ref`` otherwise through
:func:`use_native`.
"""
from __future__ import annotations

import torch

from . import _native, cuda, ref  # noqa: F401


def use_native(t: torch.Tensor) -> bool:
    """True when ``t`` lives on a GPU (the native library must then be present)."""
    if not t.is_cuda:
        return False
    if _native.lib() is None:  # raises on a GPU machine without the build
        return False
    return True
