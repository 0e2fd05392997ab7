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


def packed_width(hidden: int) -> int:
    """Width, in 16-bit elements, of a row that carries ``hidden`` fp8 values and one fp32
    scale per 128 of them."""
    return hidden // 2 + hidden // 64


def pack_fp8_rows(x: torch.Tensor) -> torch.Tensor:
    """``x [T, H]`` -> ``[T, H/2 + H/64]`` 16-bit words: the row quantised to fp8 e4m3 in groups
    of 128 with one fp32 scale per group, scales behind the values in the same row, so that the
    row moves through the dispatch as one piece (the reference sends quantised rows with their
    scales packed alongside, vllm_gcu/kernels/prepare_finalize.py:281-304,343).  About half the
    bytes of the bf16 row."""
    T, H = x.shape
    assert H % 128 == 0
    if ops.use_native(x) and x.dtype == torch.bfloat16:
        q, s = C.activation(x, "identity", "plain", quant="fp8_group128")
    else:
        q, s = ref.per_token_group_fp8_quant(x, 128)
    out = torch.empty((T, packed_width(H)), dtype=torch.int16, device=x.device)
    out[:, :H // 2] = q.contiguous().view(torch.int16).view(T, H // 2)
    out[:, H // 2:] = s.float().contiguous().view(torch.int16).view(T, H // 64)
    return out


def unpack_fp8_rows(packed: torch.Tensor, hidden: int, dtype: torch.dtype) -> torch.Tensor:
    """Inverse of :func:`pack_fp8_rows`: the de-quantised ``[T, hidden]`` rows.  Quantising
    them again in groups of 128 reproduces the same codes and scales, so experts that quantise
    their input see exactly what they would have seen without the detour."""
    T = packed.shape[0]
    packed = packed.contiguous()
    q = packed[:, :hidden // 2].contiguous().view(torch.float8_e4m3fn).view(T, hidden // 128, 128)
    s = packed[:, hidden // 2:].contiguous().view(torch.float32).view(T, hidden // 128, 1)
    return (q.float() * s).view(T, hidden).to(dtype)


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


def fp8_payload_wanted(experts, cfg) -> bool:
    """Rows travel as fp8 when the experts quantise their input to fp8 in groups of 128 anyway
    (block-scaled fp8 checkpoints) and ``VLLM_B200_EP_FP8_DISPATCH`` asks for it;
    ``extra["ep_fp8_dispatch"]`` overrides the flag for one model."""
    from .. import envs
    want = cfg.extra.get("ep_fp8_dispatch")
    if want is None:
        want = envs.EP_FP8_DISPATCH and bool(getattr(experts, "fp8_block", False))
    return bool(want) and cfg.hidden_size % 128 == 0


class AllToAllDispatcher:
    def __init__(self, experts, cfg):
        self.experts = experts
        self.cfg = cfg
        st = get_state()
        self.ep = st.ep.world_size
        self.rank = st.ep.rank_in_group
        self.epr = experts.local_experts
        self.fp8_payload = fp8_payload_wanted(experts, cfg)
        self.bytes_sent = 0                    # hidden-state bytes handed to the exchange

    def __call__(self, x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor,
                 shared: Optional[torch.Tensor],
                 max_tokens_per_rank: Optional[int] = None) -> torch.Tensor:
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
        if self.fp8_payload:
            xs = pack_fp8_rows(xs).view(torch.uint8)      # bytes: every backend moves them
        self.bytes_sent += xs.numel() * xs.element_size()
        xr = comm.all_to_all_v(xs, send_counts, recv_counts)
        if self.fp8_payload:
            xr = unpack_fp8_rows(xr.view(torch.int16), H, x.dtype)
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


class EPWorkspace:
    """Dispatch / combine with the peer-memory kernels of ``csrc/ep.cu`` (same contract as
    :class:`AllToAllDispatcher`).  Rows travel with plain peer stores into symmetric receive
    buffers; the only hop before data moves is the ep x ep count matrix; every row count stays
    on the device (``recv_total`` is handed to the expert kernels as their valid-row bound), so
    a layer is three launches around the expert GEMMs and can be captured in a CUDA graph.

    ``max_tokens`` bounds the tokens of one rank per call; the receive buffer holds
    ``ep * max_tokens`` rows (every token of every rank can land on one rank).  One
    workspace serves all MoE layers of a model (``EPWorkspace.get``)."""

    _cache: dict = {}

    @classmethod
    def get(cls, hidden: int, top_k: int, experts_per_rank: int, max_tokens: int,
            device: torch.device, group_name: str = "ep") -> "EPWorkspace":
        key = (hidden, top_k, experts_per_rank, max_tokens, str(device), group_name)
        if key not in cls._cache:
            cls._cache[key] = cls(hidden, top_k, experts_per_rank, max_tokens, device, group_name)
        return cls._cache[key]

    def __init__(self, hidden: int, top_k: int, experts_per_rank: int, max_tokens: int,
                 device: torch.device, group_name: str = "ep"):
        import ctypes

        from ..ops import _native
        from ..parallel.symm import SymmetricBuffer
        st = get_state()
        grp = getattr(st, group_name)
        self.ep = grp.world_size
        self.rank = grp.rank_in_group
        assert self.ep <= 8, "the fused dispatch supports up to 8 expert-parallel ranks"
        self.epr = experts_per_rank
        self.k = top_k
        self.H = hidden
        self.max_tokens = max_tokens
        self.device = device
        lib = _native.lib()
        P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        lib.b200_ep_meta_ints.restype = I
        lib.b200_ep_route.restype = I
        lib.b200_ep_route.argtypes = [P, I, I, I, I, I, P, P, P, P, P]
        lib.b200_ep_dispatch.restype = I
        lib.b200_ep_dispatch.argtypes = [P, L, P, P, P, I, I, I, I, I, I, P, P, P, P, P, P, P, P, P]
        lib.b200_ep_combine.restype = I
        lib.b200_ep_combine.argtypes = [P, L, I, P, P, L, P, L, F, I, I, I, I, P, P, P, P, P, P]
        ep, k, H = self.ep, self.k, self.H
        self.recv_cap = ep * max_tokens
        self.send_cap = max_tokens * min(k, ep)

        def al(n):
            return -(-n // 256) * 256
        self.off_cmat = 0
        self.off_flags = al(2 * ep * ep * 8)                # data_flag | ret_flag, 256 B each
        self.off_recv_x = self.off_flags + 512
        self.off_recv_ids = self.off_recv_x + al(self.recv_cap * H * 2)
        self.off_recv_w = self.off_recv_ids + al(self.recv_cap * k * 4)
        self.off_ret = self.off_recv_w + al(self.recv_cap * k * 4)
        total = self.off_ret + al(self.send_cap * H * 2)
        self.buf = SymmetricBuffer(total, grp.device_group, device)
        self.meta = torch.zeros(lib.b200_ep_meta_ints(), dtype=torch.int32, device=device)
        self.words = torch.zeros(8, dtype=torch.int32, device=device)   # epochs and counters
        self.tok_idx = torch.zeros(max(self.send_cap, 1), dtype=torch.int32, device=device)
        self.tok_pos = torch.zeros(max(max_tokens, 1) * ep, dtype=torch.int32, device=device)
        loc = self.buf.local
        self.recv_x = loc[self.off_recv_x:self.off_recv_x + self.recv_cap * H * 2] \
            .view(torch.bfloat16).view(self.recv_cap, H)
        self.recv_ids = loc[self.off_recv_ids:self.off_recv_ids + self.recv_cap * k * 4] \
            .view(torch.int32).view(self.recv_cap, k)
        self.recv_w = loc[self.off_recv_w:self.off_recv_w + self.recv_cap * k * 4] \
            .view(torch.float32).view(self.recv_cap, k)
        self.recv_total = self.meta[0:1]
        dist.barrier(group=grp.device_group)
        torch.cuda.synchronize()

    def _parr(self, off: int):
        from ..parallel.symm import _ptr_array
        return _ptr_array(self.buf.peer_ptrs(off))

    def dispatch(self, x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor,
                 max_tokens_per_rank: Optional[int] = None):
        """Returns (recv_x, recv_w, recv_ids, recv_total): static-size views of the receive
        buffers (``ep * max_tokens_per_rank`` rows) and the device scalar of valid rows."""
        from ..ops._native import call, ptr, stream_ptr
        T, H = x.shape
        # rows narrower than the workspace's hidden size (packed fp8 payloads) use the front of
        # the receive area with their own pitch
        assert T <= self.max_tokens and H <= self.H and H % 8 == 0 and x.dtype == torch.bfloat16
        assert topk_ids.dtype == torch.int32 and topk_w.dtype == torch.float32
        if T and x.stride(1) != 1:
            x = x.contiguous()
        topk_ids = topk_ids.contiguous()
        topk_w = topk_w.contiguous()
        w = self.words.data_ptr()
        call("b200_ep_route", ptr(topk_ids), T, self.k, self.epr, self.ep, self.rank,
             ptr(self.tok_idx), ptr(self.tok_pos), self._parr(self.off_cmat), w, stream_ptr())
        call("b200_ep_dispatch", ptr(x) if T else None, x.stride(0) if T else H, ptr(topk_ids),
             ptr(topk_w), ptr(self.tok_idx), T, H, self.k, self.ep, self.rank, self.recv_cap,
             self.buf.ptrs[self.rank] + self.off_cmat, self._parr(self.off_recv_x),
             self._parr(self.off_recv_ids), self._parr(self.off_recv_w),
             self._parr(self.off_flags), w, w + 4, ptr(self.meta), stream_ptr())
        rows = self.ep * min(self.max_tokens, max_tokens_per_rank or self.max_tokens)
        recv_x = self.recv_x[:rows] if H == self.H else \
            self.recv_x.view(-1)[:rows * H].view(rows, H)
        return recv_x, self.recv_w[:rows], self.recv_ids[:rows], self.recv_total

    def combine(self, y: torch.Tensor, T: int, add: Optional[torch.Tensor], alpha: float = 1.0
                ) -> torch.Tensor:
        from ..ops._native import call, ptr, stream_ptr
        out = torch.empty((T, self.H), dtype=torch.bfloat16, device=self.device)
        w = self.words.data_ptr()
        call("b200_ep_combine", ptr(y), y.stride(0), y.shape[0], ptr(self.tok_pos), ptr(add),
             add.stride(0) if add is not None else 0, ptr(out) if T else None, self.H,
             float(alpha), T, self.H, self.ep, self.rank, ptr(self.meta),
             self._parr(self.off_ret), self._parr(self.off_flags + 256), w + 8, w + 12,
             stream_ptr())
        return out



class FusedEPDispatcher:
    """Per-layer front end of :class:`EPWorkspace` (call contract of
    :class:`AllToAllDispatcher`)."""

    def __init__(self, experts, cfg, max_tokens: int, device: torch.device):
        self.experts = experts
        self.ws = EPWorkspace.get(cfg.hidden_size, cfg.num_experts_per_tok,
                                  experts.local_experts, max_tokens, device)
        self.fp8_payload = fp8_payload_wanted(experts, cfg)
        self.hidden = cfg.hidden_size

    def __call__(self, x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor,
                 shared: Optional[torch.Tensor],
                 max_tokens_per_rank: Optional[int] = None) -> torch.Tensor:
        T = x.shape[0]
        if self.fp8_payload:
            # quantised rows with their scales ride through the same dispatch kernel as narrower
            # 16-bit rows; the receive area is reinterpreted and de-quantised on arrival
            packed = pack_fp8_rows(x).view(torch.bfloat16)
            pr, w_r, ids_r, total = self.ws.dispatch(packed, topk_w.float(),
                                                     topk_ids.to(torch.int32),
                                                     max_tokens_per_rank)
            xr = unpack_fp8_rows(pr.view(torch.int16), self.hidden, x.dtype)
        else:
            xr, w_r, ids_r, total = self.ws.dispatch(x, topk_w.float(),
                                                     topk_ids.to(torch.int32),
                                                     max_tokens_per_rank)
        if any(getattr(self.experts, f, False) for f in ("_interleaved", "fp8_block", "q8_channel")):
            yr = self.experts(xr, w_r, ids_r, valid_tokens=total)
        else:           # layout without the grouped-GEMM path: run on the valid rows only
            n = int(total.item())
            yr = self.experts(xr[:n], w_r[:n], ids_r[:n]) if n else xr[:0]
        return self.ws.combine(yr, T, shared)
