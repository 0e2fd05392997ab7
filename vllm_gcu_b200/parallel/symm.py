"""Symmetric memory and the fused compute + collective paths built on it.

Plumbing: ``torch.distributed._symmetric_memory`` allocates one buffer per rank and
exchanges handles, so every rank holds peer-visible addresses of every other rank's
buffer (NVLink 5 through NVSwitch).  The kernels of this package then move data with
plain peer loads / stores issued from inside the kernel and synchronise with
release / acquire flags at system scope; no TMA load ever targets peer memory.

``FusedTP`` owns the workspace of one tensor-parallel group and offers

* ``gemm_all_reduce(x, w)`` – row-parallel GEMM whose epilogue performs a tile-granular
  two-shot all-reduce (``b200_gemm_bf16_allreduce``), replacing
  ``RowParallelLinear`` + ``GCUCommunicator.all_reduce`` of the reference
  (vllm_gcu/distributed/gcu_communicator.py:88-111);
* ``all_reduce(x)`` – stand-alone all-reduce for tensors produced elsewhere (embedding).

Every wait inside the kernels is bounded; a timeout is reported through the status word
(``ops._native.check_status``) and raises ``KernelTimeoutError`` on the host.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _native
from ..ops._native import call, ptr, stream_ptr
from .communicator import get_comm
from .state import get_state

_SIG_DONE = False


def _register_sigs() -> None:
    global _SIG_DONE
    if _SIG_DONE:
        return
    lib = _native.lib()
    P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    lib.b200_gemm_ar_tile_n.restype = I
    lib.b200_gemm_ar_tile_n.argtypes = [I, I]
    lib.b200_gemm_bf16_allreduce.restype = I
    lib.b200_gemm_bf16_allreduce.argtypes = [P, L, P, L, L, I, I, I, P, P, P, P, P, P, I, I, P, L,
                                             I, L, P]
    lib.b200_allreduce.restype = I
    lib.b200_allreduce.argtypes = [P, P, P, P, P, P, L, I, I, I, P]
    _SIG_DONE = True


def _ptr_array(ptrs: list[int]):
    arr = (ctypes.c_void_p * 8)()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


class SymmetricBuffer:
    """One symmetric allocation: local tensor + peer-visible base addresses."""

    def __init__(self, nbytes: int, group: dist.ProcessGroup, device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem
        nbytes = -(-nbytes // 256) * 256
        self.local = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.local.zero_()
        self.handle = symm_mem.rendezvous(self.local, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.rank = self.handle.rank
        self.world_size = self.handle.world_size
        self.nbytes = nbytes
        try:
            self.multicast_ptr = int(self.handle.multicast_ptr)
        except Exception:
            self.multicast_ptr = 0

    def peer_ptrs(self, offset: int) -> list[int]:
        return [p + offset for p in self.ptrs]


class FusedTP:
    BM = 128
    ONESHOT_MAX_TOKENS = 1024

    def __init__(self, max_tokens: int, max_n: int, device: torch.device, group_name: str = "tp"):
        _register_sigs()
        st = get_state()
        grp = getattr(st, group_name)
        self.group = grp
        self.p = grp.world_size
        self.rank = grp.rank_in_group
        self.device = device
        self.max_tokens = max_tokens
        self.max_n = max_n
        pg = grp.device_group
        rows = -(-max_tokens // self.BM) * self.BM
        # one-shot (push to every peer, reduce locally) for every size when p == 2, for
        # decode-sized batches otherwise; two-shot (owner reduces, broadcasts) above that
        self.oneshot_rows = rows if self.p == 2 else min(rows, self.ONESHOT_MAX_TOKENS)
        self.slot_elems = self.oneshot_rows * max_n
        self.part_bytes = max(rows * max_n * 2, 2 * self.p * self.slot_elems * 2)
        self.out_bytes = rows * max_n * 2
        max_tiles = (rows // self.BM) * (-(-max_n // 64))
        self.ready_bytes = max_tiles * self.p * 4
        self.done_bytes = max_tiles * 4
        self.max_tiles = max_tiles
        self.off_part = 0
        self.off_out = [self.part_bytes, self.part_bytes + self.out_bytes]   # double buffered
        self.off_ready = self.part_bytes + 2 * self.out_bytes
        self.off_done = self.off_ready + self.ready_bytes
        self.off_ar_flag = self.off_done + self.done_bytes                   # stand-alone all-reduce
        total = self.off_ar_flag + 4096
        self.buf = SymmetricBuffer(total, pg, device)
        self.local_words = torch.zeros(16, dtype=torch.int32, device=device)  # epoch, ctr, ...
        self.out_sel = 0
        dist.barrier(group=pg)
        torch.cuda.synchronize()

    # ------------------------------------------------------------------------------
    def gemm_all_reduce(self, x: torch.Tensor, w: torch.Tensor,
                        residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """``sum_ranks(x_r @ w_r^T)`` as a view of the symmetric output buffer, or None when
        the problem does not fit the workspace / dtype (caller falls back to NCCL)."""
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            return None
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        M, K = x2.shape
        N = w.shape[0]
        if M == 0:
            return x.new_empty(*shape[:-1], N)
        if M > self.max_tokens or N > self.max_n or K % 8 or N % 8:
            return None
        lib = _native.lib()
        bn = lib.b200_gemm_ar_tile_n(M, N)
        tiles = (-(-M // self.BM)) * (-(-N // bn))
        if tiles > self.max_tiles:
            return None
        self.out_sel ^= 1
        off_out = self.off_out[self.out_sel]
        out_local = self.buf.local[off_out:off_out + M * N * 2].view(torch.bfloat16).view(M, N)
        words = self.local_words.data_ptr()
        call("b200_gemm_bf16_allreduce", ptr(x2), x2.stride(0), ptr(w), w.stride(0), N, M, N, K,
             _ptr_array(self.buf.peer_ptrs(self.off_part)),
             _ptr_array(self.buf.peer_ptrs(off_out)),
             _ptr_array(self.buf.peer_ptrs(self.off_ready)),
             _ptr_array(self.buf.peer_ptrs(self.off_done)),
             words, words + 4, self.rank, self.p, ptr(residual),
             residual.stride(0) if residual is not None else 0,
             int(-(-M // self.BM) * self.BM <= self.oneshot_rows), self.slot_elems, stream_ptr())
        return out_local.view(*shape[:-1], N)

    def all_reduce(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        """Two-shot all-reduce of a bf16 tensor through the symmetric workspace (pull the
        owned slice from every peer, push the sum to every peer).  Returns None when the
        tensor does not fit."""
        if x.dtype != torch.bfloat16 or not x.is_contiguous():
            return None
        n = x.numel()
        if n == 0:
            return x
        if n * 2 > self.part_bytes or n % 8:
            return None
        self.out_sel ^= 1
        off_out = self.off_out[self.out_sel]
        src_local = self.buf.local[self.off_part:self.off_part + n * 2].view(torch.bfloat16)
        src_local.copy_(x.view(-1))
        words = self.local_words.data_ptr()
        call("b200_allreduce", _ptr_array(self.buf.peer_ptrs(self.off_part)),
             _ptr_array(self.buf.peer_ptrs(off_out)),
             _ptr_array(self.buf.peer_ptrs(self.off_ar_flag)), words + 8, words + 12, None,
             n, self.rank, self.p, 0, stream_ptr())
        out = self.buf.local[off_out:off_out + n * 2].view(torch.bfloat16).view(x.shape)
        return out


def attach(cfg) -> Optional[FusedTP]:
    """Creates the fused-TP workspace for the engine configuration and hooks it into the
    tensor-parallel communicator."""
    st = get_state()
    if st.tp.world_size <= 1 or not torch.cuda.is_available():
        return None
    mc = cfg.model
    max_tokens = max(cfg.scheduler.max_num_batched_tokens, cfg.scheduler.max_num_seqs)
    fused = FusedTP(max_tokens, mc.hidden_size, torch.device("cuda", torch.cuda.current_device()))
    get_comm("tp").fused = fused
    return fused
