"""Collectives used by the layers, per process group.

Two implementations sit behind the same methods:

* ``nccl`` – ``torch.distributed`` collectives (NCCL over NVLink 5 / NVSwitch on GPUs,
  gloo on CPU ranks).  This is the measured baseline and the fallback.
* ``fused`` – the symmetric-memory kernels of ``vllm_gcu_b200.parallel.symm`` (one-shot /
  two-shot P2P all-reduce, GEMM + all-reduce in one kernel, ...), selected per call when
  the message fits the symmetric buffers.

Role of ``GCUCommunicator`` in the reference (vllm_gcu/distributed/gcu_communicator.py:40-126):
all-reduce for TP, all-gather-v / reduce-scatter-v for sequence parallelism
(vllm_gcu/distributed/parallel_state.py:107-203) and the dispatch / combine of the
"ETP" mode (gcu_communicator.py:22-31,113-126).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .state import GroupCoordinator, get_state


def scatter_sizes(n: int, p: int) -> list[int]:
    """Uneven split of ``n`` rows over ``p`` ranks: part i gets ``(n+i)//p - i//p`` rows,
    so later ranks receive the extra rows (vllm_gcu/distributed/sp.py:9-12)."""
    return [(n + i) // p - i // p for i in range(p)]


class Communicator:
    def __init__(self, group: GroupCoordinator, mode: str = "nccl"):
        self.group = group
        self.mode = mode
        self.fused = None          # set by parallel.symm.attach() when available
        self.fused_gather = None   # gather-fused GEMMs (LM head, sequence-parallel input)

    @property
    def world_size(self) -> int:
        return self.group.world_size

    @property
    def rank(self) -> int:
        return self.group.rank_in_group

    # -- dense collectives ---------------------------------------------------
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world_size == 1:
            return x
        if self.fused is not None:
            y = self.fused.all_reduce(x)
            if y is not None:
                x.copy_(y)      # keep the in-place contract; the workspace is reused
                return x
        dist.all_reduce(x, group=self.group.device_group)
        return x

    def all_gather(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if self.world_size == 1:
            return x
        ws = self.world_size
        xc = x.contiguous()
        flat = torch.empty((ws * xc.shape[0],) + tuple(xc.shape[1:]), dtype=x.dtype,
                           device=x.device)
        dist.all_gather_into_tensor(flat, xc, group=self.group.device_group)
        out = flat.view((ws,) + tuple(xc.shape))
        dim = dim % x.dim()
        out = out.movedim(0, dim)
        return out.reshape(x.shape[:dim] + (ws * x.shape[dim],) + x.shape[dim + 1:])

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        """Sum over ranks, rank r keeps rows ``[r*n/p, (r+1)*n/p)`` (n divisible by p)."""
        if self.world_size == 1:
            return x
        out = torch.empty((x.shape[0] // self.world_size,) + tuple(x.shape[1:]), dtype=x.dtype,
                          device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group.device_group)
        return out

    # -- variable-size collectives ------------------------------------------
    def all_gather_v(self, x: torch.Tensor, sizes: Optional[Sequence[int]] = None
                     ) -> torch.Tensor:
        """Concatenates row blocks of different heights (``sizes[r]`` rows from rank r).
        Semantics of ``torch.ops.vllm.all_gather_v``
        (vllm_gcu/distributed/parallel_state.py:152-187)."""
        if self.world_size == 1:
            return x
        if sizes is None:
            t = torch.tensor([x.shape[0]], dtype=torch.int64)
            lst = [torch.zeros_like(t) for _ in range(self.world_size)]
            dist.all_gather(lst, t, group=self.group.cpu_group or self.group.device_group)
            sizes = [int(v) for v in lst]
        sizes = [int(v) for v in sizes]
        m = max(sizes)
        if m == 0:
            return x.new_zeros((0,) + tuple(x.shape[1:]))
        # pad every contribution to the largest one, gather, then drop the padding
        pad = torch.zeros((m,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        pad[: x.shape[0]] = x
        flat = torch.empty((self.world_size * m,) + tuple(x.shape[1:]), dtype=x.dtype,
                           device=x.device)
        dist.all_gather_into_tensor(flat, pad, group=self.group.device_group)
        parts = flat.view((self.world_size, m) + tuple(x.shape[1:]))
        return torch.cat([parts[r, : sizes[r]] for r in range(self.world_size)], dim=0)

    def reduce_scatter_v(self, x: torch.Tensor, sizes: Optional[Sequence[int]] = None
                         ) -> torch.Tensor:
        """Sum over ranks; rank r keeps its ``sizes[r]`` rows (default: uneven
        ``scatter_sizes`` split).  Semantics of ``torch.ops.vllm.reduce_scatter_v``
        (parallel_state.py:107-129)."""
        if self.world_size == 1:
            return x
        sizes = list(sizes) if sizes is not None else scatter_sizes(x.shape[0], self.world_size)
        start = sum(sizes[: self.rank])
        if dist.get_backend(self.group.device_group) == "gloo":
            # gloo has no reduce-scatter: reduce everything, keep the own rows
            y = x.contiguous().clone()
            dist.all_reduce(y, group=self.group.device_group)
            return y[start:start + sizes[self.rank]].contiguous()
        m = max(sizes)
        if m == 0:
            return x.new_zeros((0,) + tuple(x.shape[1:]))
        padded = torch.zeros((self.world_size, m) + tuple(x.shape[1:]), dtype=x.dtype,
                             device=x.device)
        off = 0
        for r, n in enumerate(sizes):
            padded[r, :n] = x[off:off + n]
            off += n
        out = torch.empty((m,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, padded.view((self.world_size * m,) + tuple(x.shape[1:])),
                                   group=self.group.device_group)
        return out[: sizes[self.rank]]

    def all_to_all_v(self, x: torch.Tensor, send_sizes: Sequence[int],
                     recv_sizes: Sequence[int]) -> torch.Tensor:
        """Row exchange with host-known split sizes (dynamic-shape EP path,
        vllm_gcu/kernels/prepare_finalize.py:400-573; reference semantics in
        parallel_state.py:73-104)."""
        if self.world_size == 1:
            return x
        out = torch.empty((int(sum(recv_sizes)),) + tuple(x.shape[1:]), dtype=x.dtype,
                          device=x.device)
        dist.all_to_all_single(out, x.contiguous(), list(recv_sizes), list(send_sizes),
                               group=self.group.device_group)
        return out

    def broadcast(self, x: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.world_size == 1:
            return x
        dist.broadcast(x, self.group.ranks[src], group=self.group.device_group)
        return x

    def send(self, x: torch.Tensor, dst: int) -> None:
        dist.send(x, self.group.ranks[dst], group=self.group.device_group)

    def recv(self, x: torch.Tensor, src: int) -> torch.Tensor:
        dist.recv(x, self.group.ranks[src], group=self.group.device_group)
        return x

    def barrier(self) -> None:
        if self.world_size > 1:
            dist.barrier(group=self.group.device_group)


_COMMS: dict[str, Communicator] = {}


def get_comm(name: str = "tp") -> Communicator:
    st = get_state()
    grp = getattr(st, name)
    c = _COMMS.get(name)
    if c is None or c.group is not grp:
        c = Communicator(grp)
        _COMMS[name] = c
    return c


def reset_comms() -> None:
    _COMMS.clear()
