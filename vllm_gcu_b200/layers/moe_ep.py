"""Expert-parallel token dispatch / combine for data-parallel attention.

Every rank holds different tokens; a token must visit each rank that owns one of its top-k
experts.  The flow follows the reference's all-to-all prepare / finalize
(vllm_gcu/kernels/prepare_finalize.py:126-394):

1. route: per destination rank, the tokens with at least one expert there – a token is sent
   **once per destination rank**, not once per expert (``get_ep_indices``);
2. pack ``[hidden | topk_ids | topk_weights]`` rows in rank-major order and exchange them
   (all-to-all-v; a rank with no tokens still takes part, so idle data-parallel ranks do
   not stall the others);
3. the receiver runs its local experts on the received rows (ids mapped global -> local,
   experts living elsewhere contribute nothing), producing **one row per received row**,
   already weighted and summed over that token's local experts;
4. the reverse all-to-all returns those rows and the sender adds them onto the token
   (``index_add``), seeded with the shared-expert output.

``AllToAllDispatcher`` is the collective-library implementation (NCCL on GPUs, gloo on
CPU ranks) and the baseline for the fused symmetric-memory kernels in ``csrc/ep.cu``; both
share this contract, so the CPU multi-process tests pin the semantics of the GPU path.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..ops import cuda as C
from ..ops import ref
from ..parallel.communicator import get_comm
from ..parallel.state import get_state


def ep_route(topk_ids: torch.Tensor, experts_per_rank: int, ep: int):
    """(send counts list[int], token indices rank-major int64 tensor)."""
    if topk_ids.shape[0] == 0:
        return [0] * ep, torch.zeros(0, dtype=torch.long, device=topk_ids.device)
    if ops.use_native(topk_ids):
        cnt, idx, total = C.get_ep_indices(topk_ids, experts_per_rank, ep)
        cnt_l = cnt.tolist()              # dynamic-shape path: sizes are needed on the host
        return cnt_l, idx[: sum(cnt_l)].long()
    cnt, idx, total = ref.get_ep_indices(topk_ids, experts_per_rank, ep)
    return cnt.tolist(), idx.long()


class AllToAllDispatcher:
    def __init__(self, experts, cfg):
        self.experts = experts
        self.cfg = cfg
        st = get_state()
        self.ep = st.ep.world_size
        self.rank = st.ep.rank_in_group
        self.epr = experts.local_experts

    def __call__(self, x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor,
                 shared: Optional[torch.Tensor]) -> torch.Tensor:
        comm = get_comm("ep")
        T, H = x.shape
        k = topk_ids.shape[1]
        send_counts, tok_idx = ep_route(topk_ids, self.epr, self.ep)
        # exchange the split sizes (the static-shape device path keeps them on the GPU)
        sc = torch.tensor(send_counts, dtype=torch.int64)
        rc = torch.zeros_like(sc)
        grp = comm.group.cpu_group or comm.group.device_group
        if grp is comm.group.device_group and x.is_cuda:
            sc_d, rc_d = sc.to(x.device), rc.to(x.device)
            dist.all_to_all_single(rc_d, sc_d, group=grp)
            rc = rc_d.cpu()
        else:
            dist.all_to_all_single(rc, sc, group=grp)
        recv_counts = rc.tolist()
        # packed rows: hidden | ids (as float bits are avoided: separate exchanges keep dtypes)
        xs = x[tok_idx]
        ids_s = topk_ids[tok_idx]
        w_s = topk_w[tok_idx]
        xr = comm.all_to_all_v(xs, send_counts, recv_counts)
        ids_r = comm.all_to_all_v(ids_s, send_counts, recv_counts)
        w_r = comm.all_to_all_v(w_s, send_counts, recv_counts)
        # local experts: one output row per received row
        yr = self.experts(xr, w_r, ids_r)
        # combine
        ys = comm.all_to_all_v(yr, recv_counts, send_counts)
        out = shared.clone() if shared is not None else torch.zeros_like(x)
        if tok_idx.numel():
            out.index_add_(0, tok_idx, ys.to(out.dtype))
        return out
