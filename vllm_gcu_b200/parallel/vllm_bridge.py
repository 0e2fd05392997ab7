"""Builds the fused tensor-parallel workspace for a process group that vLLM created."""
from __future__ import annotations

import torch
import torch.distributed as dist

from .state import GroupCoordinator, get_state
from .symm import FusedTP

_CACHE: dict = {}


def fused_for_group(pg: dist.ProcessGroup, device: torch.device, max_tokens: int = 8192,
                    max_n: int = 8192) -> FusedTP:
    key = id(pg)
    if key in _CACHE:
        return _CACHE[key]
    ranks = dist.get_process_group_ranks(pg)
    st = get_state()
    st.tp = GroupCoordinator("tp", list(ranks), dist.get_rank(pg), pg, None)
    st.initialized = True
    fused = FusedTP(max_tokens, max_n, device)
    _CACHE[key] = fused
    return fused
