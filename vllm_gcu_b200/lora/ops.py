"""LoRA kernels behind the punica wrapper.

``bgmv_*`` take one adapter index per token; ``sgmv_*`` take one adapter index per sequence
plus sequence lengths and are evaluated as bgmv after expanding the indices per token, which
is how the reference implements them (vllm_gcu/lora/lora_ops.py:173-175,283,381).

* shrink:  ``y[t] (+)= scale * A[idx[t]] @ x[t]``           A ``[L, r, h_in]``
* expand:  ``y[t, off:off+n] += B[idx[t]] @ x[t]``           B ``[L, h_out, r]``
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..ops import ref
from ..ops._native import DTYPE_CODE, call, ptr, stream_ptr


def _w3(w: torch.Tensor) -> torch.Tensor:
    return w[:, 0] if w.dim() == 4 else w


def _bgmv(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, idx: torch.Tensor, scale: float,
          y_off: int, add: bool) -> torch.Tensor:
    w = _w3(w)
    h_out, h_in = w.shape[1], w.shape[2]
    if ops.use_native(x) and x.dtype in (torch.bfloat16, torch.float16) and x.stride(-1) == 1 \
            and (h_in <= 256 or h_in % 8 == 0) and y.dtype in (x.dtype, torch.float32):
        if not w.is_contiguous():
            w = w.contiguous()
        i32 = idx if idx.dtype == torch.int32 else idx.to(torch.int32)
        call("b200_bgmv", ptr(y), y.stride(0), ptr(x), x.stride(0), ptr(w), ptr(i32), x.shape[0],
             h_in, h_out, y_off, float(scale), int(add), DTYPE_CODE[x.dtype], DTYPE_CODE[y.dtype],
             stream_ptr())
        return y
    if not add:
        y[:, y_off:y_off + h_out] = 0
    return ref.bgmv(y, x, w, idx, scale, y_off, h_out)


def bgmv_shrink(x: torch.Tensor, lora_a: torch.Tensor, y: torch.Tensor, idx: torch.Tensor,
                scale: float = 1.0) -> torch.Tensor:
    """``y = scale * A[idx] @ x`` (overwrites y; rows with idx < 0 are left untouched)."""
    return _bgmv(y, x, lora_a, idx, scale, 0, add=False)


def bgmv_expand(x: torch.Tensor, lora_b: torch.Tensor, y: torch.Tensor, idx: torch.Tensor,
                add_inputs: bool = True) -> torch.Tensor:
    return _bgmv(y, x, lora_b, idx, 1.0, 0, add=add_inputs)


def bgmv_expand_slice(x: torch.Tensor, lora_b: torch.Tensor, y: torch.Tensor, idx: torch.Tensor,
                      slice_offset: int, slice_size: int, add_inputs: bool = True
                      ) -> torch.Tensor:
    assert _w3(lora_b).shape[1] == slice_size
    return _bgmv(y, x, lora_b, idx, 1.0, slice_offset, add=add_inputs)


def _expand_seq_indices(lora_indices: torch.Tensor, seq_lens: torch.Tensor) -> torch.Tensor:
    return torch.repeat_interleave(lora_indices, seq_lens.long())


def sgmv_shrink(x, lora_a, y, seq_lens: torch.Tensor, lora_indices: torch.Tensor,
                scale: float = 1.0) -> torch.Tensor:
    return bgmv_shrink(x, lora_a, y, _expand_seq_indices(lora_indices, seq_lens), scale)


def sgmv_expand(x, lora_b, y, seq_lens: torch.Tensor, lora_indices: torch.Tensor,
                add_inputs: bool = True, slice_offset: int = 0,
                slice_size: Optional[int] = None) -> torch.Tensor:
    idx = _expand_seq_indices(lora_indices, seq_lens)
    if slice_size is None:
        return bgmv_expand(x, lora_b, y, idx, add_inputs)
    return bgmv_expand_slice(x, lora_b, y, idx, slice_offset, slice_size, add_inputs)
