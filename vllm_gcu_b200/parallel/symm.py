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
* ``all_reduce(x)`` – stand-alone all-reduce for tensors produced elsewhere (embedding);
* ``gemm_all_gather(x, w_shard)`` – column-parallel GEMM whose epilogue stores its column
  block into every peer's full-width output (``b200_gemm_bf16_allgather``): the
  vocabulary-parallel LM head + logits gather of the reference
  (vllm_gcu/distributed/gcu_communicator.py:112-160 ``gather`` / ``all_gather``);
* ``all_gather_gemm(x_shard, w)`` – all-gather of sequence-parallel activations fused into
  the following column-parallel GEMM (``b200_gemm_bf16_gather_a``; the reference runs
  ``all_gather`` then the matmul, vllm_gcu/patch/sp_model.py).

Every wait inside the kernels is bounded; a timeout is reported through the status word
(``ops._native.check_status``) and raises ``KernelTimeoutError`` on the host.
"""
from __future__ import annotations

import ctypes
import os
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
    lib.b200_gemm_bf16_allgather.restype = I
    lib.b200_gemm_bf16_allgather.argtypes = [P, L, P, L, L, L, I, I, I, P, P, P, P, P, I, I, P]
    lib.b200_gemm_bf16_gather_a.restype = I
    lib.b200_gemm_bf16_gather_a.argtypes = [P, L, P, P, L, P, L, P, L, I, I, I, P, P, P, P, P, P,
                                            I, I, P]
    F = ctypes.c_float
    lib.b200_gemm_bf16_ar_norm.restype = I
    lib.b200_gemm_bf16_ar_norm.argtypes = [P, L, P, L, L, I, I, I, P, P, P, P, P, P, P, P, I, I, P, L,
                                           P, F, I, I, P, P, P, P, L, P, P]
    lib.b200_argmax_allgather.restype = I
    lib.b200_argmax_allgather.argtypes = [P, L, I, I, I, P, I, P, P, I, I, P, P]
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
    ARGMAX_ROWS = 1024
    LL_MAX_ROWS = 1024

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
        # row-owner reduce + norm: new-residual buffers (double buffered) and one flag per row
        self.off_res = [self.off_ar_flag + 4096, self.off_ar_flag + 4096 + self.out_bytes]
        self.off_row_done = self.off_res[1] + self.out_bytes
        # greedy sampling: 2 (epoch parity) x p x ARGMAX_ROWS records of 16 bytes
        self.off_rn_cnt = -(-(self.off_row_done + rows * 4) // 256) * 256    # arrival counters
        self.off_argmax = -(-(self.off_rn_cnt + (rows // self.BM) * 4) // 256) * 256
        # sentinel-tagged transport of decode-sized gemm_ar_norm calls: three rotating buffers
        # for the rows pushed to their owners and three for the finished rows
        self.ll_cap = min(rows, self.LL_MAX_ROWS) * max_n               # elements per buffer
        self.off_ll_slots = -(-(self.off_argmax + 2 * self.p * self.ARGMAX_ROWS * 16) // 256) * 256
        self.off_ll_out = self.off_ll_slots + 3 * self.ll_cap * 2
        total = self.off_ll_out + 3 * self.ll_cap * 2 + 256
        self.buf = SymmetricBuffer(total, pg, device)
        self.local_words = torch.zeros(16, dtype=torch.int32, device=device)  # epoch, ctr, ...
        self.rn_base = torch.zeros(rows // self.BM + 1, dtype=torch.int32, device=device)
        self.ll_used = torch.zeros(6, dtype=torch.int64, device=device)
        ll = self.buf.local[self.off_ll_slots:self.off_ll_out + 3 * self.ll_cap * 2]
        ll.view(torch.int32).fill_(-2147450880)          # 0x80008000: "nothing has landed here"
        self.out_sel = 0
        self.res_sel = 0
        self.force_mode: Optional[str] = None     # benchmarks: "oneshot" | "twoshot"
        self.force_rn_mode: Optional[int] = None  # benchmarks / tests: transport of gemm_ar_norm
        self.row_owner: Optional[bool] = None     # benchmarks / tests: force the choice
        # thousands of rows with four or more ranks: owners pull their rows (through the
        # switch when the allocation has a multicast view); VLLM_B200_TP_LARGE_M=ar keeps
        # the tile-wise all-reduce + norm kernel
        self.large_m_row_owner = os.environ.get("VLLM_B200_TP_LARGE_M", "rn") != "ar"
        self.sm_count = int(_native.lib().b200_sm_count())
        from .. import envs
        # in-switch reduction and broadcast (NVLS multimem) when the allocation has a multicast
        # view; VLLM_B200_MULTIMEM=0 keeps the kernels on plain peer loads and stores
        self.use_multimem = bool(self.buf.multicast_ptr) and bool(getattr(envs, "MULTIMEM", True))
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
             int(self._oneshot(M)), self.slot_elems, stream_ptr())
        return out_local.view(*shape[:-1], N)

    def gemm_ar_norm(self, x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor],
                     norm_weight: Optional[torch.Tensor], eps: float = 1e-6,
                     bcast_residual: bool = True
                     ) -> Optional[tuple[torch.Tensor, Optional[torch.Tensor]]]:
        """Row-parallel GEMM + all-reduce + residual add + RMSNorm in one kernel
        (``b200_gemm_bf16_ar_norm``): returns ``(normed, new_residual)`` as views of the
        symmetric workspace, or None when the problem does not fit (the caller then runs the
        un-fused sequence).  ``new_residual`` holds valid rows on every rank only with
        ``bcast_residual``; otherwise each rank holds the rows it owns
        (``[128 r / p, 128 (r + 1) / p)`` of every 128-row tile), which is all the next call of
        this method reads.  Without ``norm_weight`` the result is the plain all-reduced sum
        (+ residual) and ``new_residual`` is None.  Replaces ``RowParallelLinear`` +
        ``all_reduce`` + ``fused_add_rms_norm`` of the reference
        (vllm_gcu/distributed/gcu_communicator.py:88-111, vllm_gcu/kernels/layernorm.py:10-41)."""
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            return None
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        M, K = x2.shape
        N = w.shape[0]
        if M == 0 or M > self.max_tokens or N > self.max_n or N > 8192 or K % 8 or N % 8:
            return None
        if residual is not None:
            residual = residual.reshape(-1, N)
            if residual.stride(-1) != 1 or residual.stride(0) % 8 or residual.dtype != x.dtype:
                return None
        lib = _native.lib()
        bn = lib.b200_gemm_ar_tile_n(M, N)
        if not self._row_owner_pays(M, N, bn):
            # GEMM + tile-wise all-reduce, then the norm kernel: every rank ends up with the
            # whole new residual
            from ..ops import cuda as C
            y = self.gemm_all_reduce(x2, w, None if norm_weight is not None else residual)
            if y is None:
                return None
            if norm_weight is None:
                return y.view(*x.shape[:-1], N), None
            if residual is None:
                return C.norm(y, norm_weight, eps).view(*x.shape[:-1], N), y
            if residual.data_ptr() == x2.data_ptr():
                residual = residual.clone()
            out = C.norm(y, norm_weight, eps, residual=residual)
            return out.view(*x.shape[:-1], N), residual
        if (-(-M // self.BM)) * (-(-N // bn)) > self.max_tiles:
            return None
        self.out_sel ^= 1
        off_out = self.off_out[self.out_sel]
        off_res = 0
        if norm_weight is not None:
            self.res_sel ^= 1
            off_res = self.off_res[self.res_sel]
        mode = self._rn_mode(M, N, bn, bool(bcast_residual) and norm_weight is not None)
        mc = self.buf.multicast_ptr if (self.use_multimem and mode == 0) else 0
        off_part = self.off_ll_slots if mode == 3 else self.off_part
        off_dst = self.off_ll_out if mode == 3 else off_out
        words = self.local_words.data_ptr()
        call("b200_gemm_bf16_ar_norm", ptr(x2), x2.stride(0), ptr(w), w.stride(0), N, M, N, K,
             _ptr_array(self.buf.peer_ptrs(off_part)),
             _ptr_array(self.buf.peer_ptrs(off_dst)),
             _ptr_array(self.buf.peer_ptrs(off_res)) if norm_weight is not None else None,
             _ptr_array(self.buf.peer_ptrs(self.off_rn_cnt)),
             _ptr_array(self.buf.peer_ptrs(self.off_row_done)), ptr(self.rn_base),
             words + 40, words + 44, self.rank, self.p, ptr(residual),
             residual.stride(0) if residual is not None else 0, ptr(norm_weight), float(eps),
             int(bool(bcast_residual) and norm_weight is not None), mode,
             mc + self.off_part if mc else None, mc + off_out if mc else None,
             mc + off_res if (mc and norm_weight is not None) else None,
             self.buf.ptrs[self.rank] + off_out, self.ll_cap, ptr(self.ll_used), stream_ptr())
        out = self.buf.local[off_out:off_out + M * N * 2].view(torch.bfloat16).view(M, N)
        res = None
        if norm_weight is not None:
            res = self.buf.local[off_res:off_res + M * N * 2].view(torch.bfloat16).view(M, N)
        return out.view(*x.shape[:-1], N), res

    def greedy_argmax(self, local_logits: torch.Tensor, valid: int, vocab_offset: int
                      ) -> Optional[torch.Tensor]:
        """Token ids ``[B]`` (int64) of the maximum over the vocabulary-parallel logits: every
        rank passes its ``[B, V/p]`` block, ``valid`` = number of real (un-padded) columns in
        it and ``vocab_offset`` = id of its first column.  16 bytes per row and rank cross
        NVLink instead of the logits (``b200_argmax_allgather``); the reference exchanges
        sampled ids, not logits, in the same spirit (vllm_gcu/kernels/sampler.py:13-71)."""
        if local_logits.dtype != torch.bfloat16 or local_logits.dim() != 2 \
                or local_logits.stride(1) != 1 or local_logits.stride(0) % 8:
            return None
        B = local_logits.shape[0]
        if B == 0 or B > self.ARGMAX_ROWS:
            return None
        out = torch.empty(B, dtype=torch.int64, device=local_logits.device)
        words = self.local_words.data_ptr()
        call("b200_argmax_allgather", ptr(local_logits), local_logits.stride(0), B, int(valid),
             int(vocab_offset), _ptr_array(self.buf.peer_ptrs(self.off_argmax)), self.ARGMAX_ROWS,
             words + 32, words + 36, self.rank, self.p, ptr(out), stream_ptr())
        return out

    def _few_rows(self, M: int, N: int, bn: int) -> bool:
        tiles_m = -(-M // self.BM)
        grid = min(tiles_m * -(-N // bn), self.sm_count)
        return min(tiles_m * max(1, self.BM // self.p), M) <= 2 * grid

    def _row_owner_pays(self, M: int, N: int, bn: int) -> bool:
        """Whether ``gemm_ar_norm`` runs as the one row-owner kernel or as GEMM + tile-wise
        all-reduce followed by the norm kernel.  Measured with two ranks the latter is as fast
        for decode-sized problems (one hop against two) and faster for thousands of rows (the
        four reducer warps of a CTA cannot keep enough rows in flight when a rank owns half of
        them); with four or more ranks pushing every partial to every rank costs (p - 1) times
        the traffic and the row owners win."""
        if self.row_owner is not None:
            return bool(self.row_owner)
        if self.force_rn_mode is not None:
            return True
        if self.p < 4:
            return False
        if self._few_rows(M, N, bn):
            return True
        return self.large_m_row_owner

    def _rn_mode(self, M: int, N: int, bn: int, bcast_residual: bool = False) -> int:
        """Transport of ``gemm_ar_norm`` for this problem.  Decode-sized problems (few rows per
        rank): 3 = rows pushed to their owners through sentinel-tagged buffers, no flags and no
        fences (needs the residual to stay with its owner); otherwise 1 = rows pushed to their
        owners with arrival counters.  Many rows: 0 = owners pull whole rows (the
        multimem-capable transport).  2 (every rank reduces everything) only on request."""
        tiles_m = -(-M // self.BM)
        if self.force_rn_mode is not None:
            mode = self.force_rn_mode
        else:
            mode = 3 if self._few_rows(M, N, bn) else 0
        if mode and self.BM % self.p:
            mode = 0
        if mode == 3 and (bcast_residual or tiles_m * self.BM * N > self.ll_cap):
            mode = 1
        if mode == 2 and 2 * self.p * tiles_m * self.BM * N * 2 > self.part_bytes:
            mode = 1
        if mode == 1 and 2 * tiles_m * self.BM * N * 2 > self.part_bytes:
            mode = 0
        return mode

    def _oneshot(self, M: int) -> bool:
        fits = -(-M // self.BM) * self.BM <= self.oneshot_rows
        if self.force_mode == "twoshot":
            return False
        return fits

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


class FusedGather:
    """Workspaces of the two gather-fused GEMMs of one tensor-parallel group."""
    BM = 128

    def __init__(self, device: torch.device, out_rows: int = 0, out_cols: int = 0,
                 sp_tokens: int = 0, sp_k: int = 0, group_name: str = "tp"):
        _register_sigs()
        st = get_state()
        grp = getattr(st, group_name)
        self.p = grp.world_size
        self.rank = grp.rank_in_group
        self.device = device
        pg = grp.device_group
        self.out_rows, self.out_cols = out_rows, out_cols
        self.sp_tokens, self.sp_k = sp_tokens, sp_k
        rows = -(-max(out_rows, 1) // self.BM) * self.BM
        self.out_bytes = rows * out_cols * 2
        self.max_tiles = (rows // self.BM) * (-(-max(out_cols, 64) // self.p // 64) + 1)
        self.ready_bytes = self.max_tiles * self.p * 4
        self.m_loc_max = -(-max(sp_tokens, 1) // self.p) + 1
        self.shard_bytes = self.m_loc_max * sp_k * 2
        self.off_out = 0
        self.off_ready = -(-self.out_bytes // 256) * 256
        self.off_shard = self.off_ready + -(-self.ready_bytes // 256) * 256
        # flag words: in_ready | rd_done | started, 256 bytes each
        self.off_flags = self.off_shard + -(-self.shard_bytes // 256) * 256
        self.buf = SymmetricBuffer(self.off_flags + 768, pg, device)
        self.a_full = torch.empty((max(sp_tokens, 1), max(sp_k, 8)), dtype=torch.bfloat16,
                                  device=device)
        self.chunk_ready = torch.zeros(-(-max(sp_tokens, 1) // self.BM) + 1, dtype=torch.int32,
                                       device=device)
        self.local_words = torch.zeros(16, dtype=torch.int32, device=device)
        dist.barrier(group=pg)
        torch.cuda.synchronize()

    def gemm_all_gather(self, x: torch.Tensor, w: torch.Tensor) -> Optional[torch.Tensor]:
        """``concat_r(x @ w_r^T)`` on every rank ([M, p * N_local] view of the symmetric
        output buffer), or None when the problem does not fit."""
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2:
            return None
        if x.stride(-1) != 1:
            x = x.contiguous()
        M, K = x.shape
        N = w.shape[0]
        ldc = N * self.p
        if M == 0:
            return x.new_empty(0, ldc)
        if M > self.out_rows or ldc > self.out_cols or K % 8 or N % 8:
            return None
        lib = _native.lib()
        bn = lib.b200_gemm_ar_tile_n(M, N)
        if (-(-M // self.BM)) * (-(-N // bn)) > self.max_tiles:
            return None
        off_out = self.off_out
        words = self.local_words.data_ptr()
        call("b200_gemm_bf16_allgather", ptr(x), x.stride(0), ptr(w), w.stride(0), ldc,
             self.rank * N, M, N, K, _ptr_array(self.buf.peer_ptrs(off_out)),
             _ptr_array(self.buf.peer_ptrs(self.off_ready)),
             _ptr_array(self.buf.peer_ptrs(self.off_flags + 512)), words, words + 4, self.rank,
             self.p, stream_ptr())
        return self.buf.local[off_out:off_out + M * ldc * 2].view(torch.bfloat16).view(M, ldc)

    def all_gather_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, sizes: list[int]
                        ) -> Optional[torch.Tensor]:
        """``gather_r(x_r) @ w^T`` where rank r passes its ``[sizes[r], K]`` rows (the uneven
        sequence-parallel split of ``parallel.sp.scatter`` is allowed)."""
        if x_shard.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x_shard.dim() != 2:
            return None
        m_loc, K = x_shard.shape
        N = w.shape[0]
        M = sum(sizes)
        assert len(sizes) == self.p and sizes[self.rank] == m_loc
        if (M <= 0 or M > self.sp_tokens or K != self.sp_k or max(sizes) > self.m_loc_max
                or K % 8 or N % 8):
            return None
        row_off = (ctypes.c_int * (self.p + 1))()
        for i, n in enumerate(sizes):
            row_off[i + 1] = row_off[i] + n
        shard = self.buf.local[self.off_shard:self.off_shard + m_loc * K * 2] \
            .view(torch.bfloat16).view(m_loc, K)
        shard.copy_(x_shard)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x_shard.device)
        words = self.local_words.data_ptr()
        call("b200_gemm_bf16_gather_a", _ptr_array(self.buf.peer_ptrs(self.off_shard)), K, row_off,
             ptr(self.a_full), self.a_full.stride(0), ptr(w), w.stride(0), ptr(out), N, M, N, K,
             _ptr_array(self.buf.peer_ptrs(self.off_flags)),
             _ptr_array(self.buf.peer_ptrs(self.off_flags + 256)), ptr(self.chunk_ready),
             words + 12, words + 8, words + 16, self.rank, self.p, stream_ptr())
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
    comm = get_comm("tp")
    comm.fused = fused
    # LM head: logits are needed for the sampled rows only (one per sequence, plus the
    # speculative positions)
    tp = st.tp.world_size
    rows = cfg.scheduler.max_num_seqs * (1 + getattr(cfg.speculative, "num_speculative_tokens", 0))
    padded_vocab = -(-mc.vocab_size // (tp * 64)) * (tp * 64)
    sp_on = bool(mc.extra.get("sequence_parallel"))
    comm.fused_gather = FusedGather(fused.device, out_rows=max(rows, 128), out_cols=padded_vocab,
                                    sp_tokens=max_tokens if sp_on else 0,
                                    sp_k=mc.hidden_size if sp_on else 0)
    return fused
