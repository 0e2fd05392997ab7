"""Sequence parallelism over the tensor-parallel group (DeepSeek family).

Between attention and the MLP / MoE the activations are sharded by token rows over the TP
ranks: the row-parallel ``o_proj`` output is reduce-scattered instead of all-reduced
(``tp_to_sp``), norms and the MoE input work on ``T / tp`` rows, and the rows are gathered
again (``sp_to_tp``) before the next attention block and before the logits.  The split is
uneven when ``T`` is not a multiple of ``tp``: part i gets ``(T + i) // tp - i // tp`` rows, so
later ranks receive the extra rows and no padding is needed
(vllm_gcu/distributed/sp.py:9-77).
"""
from __future__ import annotations

import torch

from .communicator import get_comm, scatter_sizes
from .state import tp_rank, tp_size


def scatter(n: int, p: int) -> list[int]:
    return scatter_sizes(n, p)


def tp_to_sp(x: torch.Tensor) -> torch.Tensor:
    """Partial sums ``[T, H]`` on every rank -> reduced rows of this rank ``[T_r, H]``."""
    p = tp_size()
    if p == 1:
        return x
    return get_comm("tp").reduce_scatter_v(x, scatter(x.shape[0], p))


def sp_to_tp(x: torch.Tensor, total_rows: int) -> torch.Tensor:
    """Rows of this rank ``[T_r, H]`` -> all rows ``[T, H]`` on every rank."""
    p = tp_size()
    if p == 1:
        return x
    return get_comm("tp").all_gather_v(x, scatter(total_rows, p))


def slice_tensor_sp(x: torch.Tensor) -> torch.Tensor:
    """The rows of a replicated tensor (e.g. the residual) that this rank owns."""
    p = tp_size()
    if p == 1:
        return x
    sizes = scatter(x.shape[0], p)
    r = tp_rank()
    start = sum(sizes[:r])
    return x[start:start + sizes[r]]


def sp_gather_linear(layer, x_local: torch.Tensor, sizes: list[int]) -> torch.Tensor:
    """``layer(all_gather(x_local))`` for a column-parallel layer whose input is sharded by
    rows.  On the GPU with bf16 unquantised weights the gather runs inside the GEMM
    (``FusedGather.all_gather_gemm``: gather warps pull the peers' rows while the tensor
    cores work on the rows that have arrived); otherwise all-gather-v then the layer."""
    comm = get_comm("tp")
    fg = getattr(comm, "fused_gather", None)
    w = getattr(layer, "weight", None)
    if (fg is not None and x_local.is_cuda and x_local.dtype == torch.bfloat16 and w is not None
            and w.dtype == torch.bfloat16 and getattr(layer, "bias", None) is None
            and not getattr(layer, "fuse_silu", False) and fg.sp_k == x_local.shape[-1]
            and type(layer.quant_method).__name__ == "UnquantizedLinearMethod"):
        y = fg.all_gather_gemm(x_local.contiguous(), w, list(sizes))
        if y is not None:
            return y
    return layer(sp_to_tp(x_local, sum(sizes)))


def reduce_scatter_rows(partial: torch.Tensor, sizes: list[int]) -> torch.Tensor:
    """Partial sums ``[T, H]`` -> this rank's reduced rows."""
    return get_comm("tp").reduce_scatter_v(partial, list(sizes))
