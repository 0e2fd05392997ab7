"""Process-group state: one process per GPU, ``torch.distributed`` for the plumbing.

Rank layout (outermost to innermost): data parallel, pipeline parallel, tensor
parallel, i.e. ``rank = (dp * PP + pp) * TP + tp``.  Expert parallelism spans the
``DP x TP`` ranks of one pipeline stage (``ep_rank = dp * TP + tp``), as in the
reference where EP replaces TP for the experts while attention stays DP/TP
(vllm_gcu/worker/worker.py:222-266, vllm_gcu/kernels/prepare_finalize.py:126-128).
A gloo group mirrors every device group for host-side metadata exchange
(token counts of DP ranks, KV-block agreement), see worker.py:258-266.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class GroupCoordinator:
    name: str
    ranks: list[int]
    rank_in_group: int
    device_group: Optional[dist.ProcessGroup] = None
    cpu_group: Optional[dist.ProcessGroup] = None

    @property
    def world_size(self) -> int:
        return len(self.ranks)

    @property
    def first_rank(self) -> int:
        return self.ranks[0]

    @property
    def is_first(self) -> bool:
        return self.rank_in_group == 0

    @property
    def is_last(self) -> bool:
        return self.rank_in_group == len(self.ranks) - 1


_SINGLE = lambda name: GroupCoordinator(name, [0], 0)  # noqa: E731


class ParallelState:
    def __init__(self) -> None:
        self.initialized = False
        self.rank = 0
        self.world_size = 1
        self.local_rank = 0
        self.tp = _SINGLE("tp")
        self.pp = _SINGLE("pp")
        self.dp = _SINGLE("dp")
        self.ep = _SINGLE("ep")
        self.world = _SINGLE("world")
        self.backend = "none"
        # data-parallel attention: largest token count of any DP rank in the current step
        # (None outside a DP step); bounds the rows an expert-parallel rank can receive
        self.dp_max_tokens = None
        # rows of the current forward on every DP rank (ETP gather / scatter sizes); set by
        # the model for the duration of one forward
        self.dp_rows = None

    def reset(self) -> None:
        self.__init__()


_STATE = ParallelState()


def get_state() -> ParallelState:
    return _STATE


def _new_group(name: str, all_rank_lists: list[list[int]], my_rank: int, backend: str,
               with_cpu: bool) -> GroupCoordinator:
    mine: Optional[GroupCoordinator] = None
    for ranks in all_rank_lists:
        # every process must take part in every new_group call
        dg = dist.new_group(ranks, backend=backend) if len(ranks) > 1 else None
        cg = dist.new_group(ranks, backend="gloo") if (with_cpu and len(ranks) > 1) else None
        if my_rank in ranks:
            mine = GroupCoordinator(name, list(ranks), ranks.index(my_rank), dg, cg)
    assert mine is not None
    return mine


def init_distributed(tp: int = 1, pp: int = 1, dp: int = 1, backend: Optional[str] = None,
                     enable_ep: bool = False) -> ParallelState:
    """Initialises torch.distributed from the torchrun environment (RANK, WORLD_SIZE,
    LOCAL_RANK, MASTER_ADDR, MASTER_PORT) and builds the TP / PP / DP / EP groups."""
    st = _STATE
    world = tp * pp * dp
    if world == 1:
        st.initialized = True
        return st
    rank = int(os.environ.get("RANK", "0"))
    ws = int(os.environ.get("WORLD_SIZE", str(world)))
    if ws != world:
        raise ValueError(f"WORLD_SIZE={ws} does not match tp*pp*dp={world}")
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available()
    backend = backend or ("nccl" if use_cuda else "gloo")
    if use_cuda:
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29555")
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=ws, **kw)
    st.rank, st.world_size, st.local_rank, st.backend = rank, ws, local_rank, backend
    with_cpu = backend != "gloo"

    def rid(d: int, p: int, t: int) -> int:
        return (d * pp + p) * tp + t

    st.world = GroupCoordinator("world", list(range(ws)), rank, dist.group.WORLD, None)
    st.tp = _new_group("tp", [[rid(d, p, t) for t in range(tp)] for d in range(dp)
                              for p in range(pp)], rank, backend, with_cpu)
    st.pp = _new_group("pp", [[rid(d, p, t) for p in range(pp)] for d in range(dp)
                              for t in range(tp)], rank, backend, with_cpu)
    st.dp = _new_group("dp", [[rid(d, p, t) for d in range(dp)] for p in range(pp)
                              for t in range(tp)], rank, backend, True)
    if enable_ep:
        st.ep = _new_group("ep", [[rid(d, p, t) for d in range(dp) for t in range(tp)]
                                  for p in range(pp)], rank, backend, with_cpu)
    st.initialized = True
    return st


def exchange_dp_rows(n: int) -> list[int]:
    """Row count of every data-parallel rank for the forward that is about to run (host
    all-gather, the counterpart of ``cu_tokens_across_dp_cpu`` in
    vllm_gcu/patch/patch_0_9_2/forward_context.py:10-43)."""
    dpg = _STATE.dp
    if dpg.world_size == 1:
        return [int(n)]
    mine = torch.tensor([int(n)], dtype=torch.int64)
    parts = [torch.zeros_like(mine) for _ in range(dpg.world_size)]
    dist.all_gather(parts, mine, group=dpg.cpu_group or dpg.device_group)
    return [int(p[0]) for p in parts]


def destroy_distributed() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()
    _STATE.reset()


def tp_size() -> int:
    return _STATE.tp.world_size


def tp_rank() -> int:
    return _STATE.tp.rank_in_group


def ep_size() -> int:
    return _STATE.ep.world_size


def ep_rank() -> int:
    return _STATE.ep.rank_in_group
