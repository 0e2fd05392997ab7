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
