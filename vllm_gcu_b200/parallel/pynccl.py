"""ctypes binding of the NCCL C API and a small communicator on top of it.

Used where a collective or a send / receive must run outside ``torch.distributed`` process
groups: the point-to-point KV connector creates two-rank communicators per peer on demand, and
tests compare the symmetric-memory kernels against plain NCCL.  The reference has the same
layer for its vendor library (``ECCLLibrary`` / ``PyEcclCommunicator``,
vllm_gcu/distributed/pyeccl_wrapper.py:31-278, pyeccl.py:30-140): unique-id bootstrap through
an existing CPU group, dtype / op enums, every non-zero result turned into ``RuntimeError``.

The library is loaded from ``VLLM_NCCL_SO_PATH``, else from the ``nvidia-nccl`` wheel next to
torch, else by soname.  A different object with the same function table can be injected
(``NCCLLibrary(lib=fake)``), which is how the error paths are tested without a GPU.
"""
from __future__ import annotations

import ctypes
import glob
import os
from typing import Any, Optional

import torch
import torch.distributed as dist

ncclResult_t = ctypes.c_int
ncclComm_t = ctypes.c_void_p


class ncclUniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


class ncclDataType:
    INT8, UINT8, INT32, UINT32, INT64, UINT64, FLOAT16, FLOAT32, FLOAT64, BFLOAT16 = range(10)
    FP8_E4M3, FP8_E5M2 = 10, 11
    _MAP = {torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6,
            torch.float32: 7, torch.float64: 8, torch.bfloat16: 9, torch.float8_e4m3fn: 10,
            torch.float8_e5m2: 11}

    @classmethod
    def from_torch(cls, dt: torch.dtype) -> int:
        try:
            return cls._MAP[dt]
        except KeyError:
            raise ValueError(f"dtype {dt} has no NCCL equivalent")


class ncclRedOp:
    SUM, PROD, MAX, MIN, AVG = range(5)
    _MAP = {dist.ReduceOp.SUM: 0, dist.ReduceOp.PRODUCT: 1, dist.ReduceOp.MAX: 2,
            dist.ReduceOp.MIN: 3, dist.ReduceOp.AVG: 4}

    @classmethod
    def from_torch(cls, op) -> int:
        try:
            return cls._MAP[op]
        except KeyError:
            raise ValueError(f"reduce op {op} has no NCCL equivalent")


def find_nccl_library() -> str:
    p = os.environ.get("VLLM_NCCL_SO_PATH")
    if p:
        return p
    base = os.path.dirname(os.path.dirname(torch.__file__))
    hits = sorted(glob.glob(os.path.join(base, "nvidia", "nccl", "lib", "libnccl.so*")))
    return hits[0] if hits else "libnccl.so.2"


class NCCLLibrary:
    """Function table of libnccl with checked calls."""

    _FUNCS = {
        "ncclGetErrorString": (ctypes.c_char_p, [ncclResult_t]),
        "ncclGetVersion": (ncclResult_t, [ctypes.POINTER(ctypes.c_int)]),
        "ncclGetUniqueId": (ncclResult_t, [ctypes.POINTER(ncclUniqueId)]),
        "ncclCommInitRank": (ncclResult_t, [ctypes.POINTER(ncclComm_t), ctypes.c_int,
                                            ncclUniqueId, ctypes.c_int]),
        "ncclAllReduce": (ncclResult_t, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                         ctypes.c_int, ctypes.c_int, ncclComm_t, ctypes.c_void_p]),
        "ncclAllGather": (ncclResult_t, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                         ctypes.c_int, ncclComm_t, ctypes.c_void_p]),
        "ncclReduceScatter": (ncclResult_t, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                             ctypes.c_int, ctypes.c_int, ncclComm_t,
                                             ctypes.c_void_p]),
        "ncclBroadcast": (ncclResult_t, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t,
                                         ctypes.c_int, ctypes.c_int, ncclComm_t, ctypes.c_void_p]),
        "ncclSend": (ncclResult_t, [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                    ncclComm_t, ctypes.c_void_p]),
        "ncclRecv": (ncclResult_t, [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                    ncclComm_t, ctypes.c_void_p]),
        "ncclGroupStart": (ncclResult_t, []),
        "ncclGroupEnd": (ncclResult_t, []),
        "ncclCommDestroy": (ncclResult_t, [ncclComm_t]),
    }

    def __init__(self, so_file: Optional[str] = None, lib: Any = None):
        if lib is None:
            lib = ctypes.CDLL(so_file or find_nccl_library())
            for name, (res, args) in self._FUNCS.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
        self.lib = lib

    def check(self, result: int) -> None:
        if result != 0:
            msg = self.lib.ncclGetErrorString(result)
            if isinstance(msg, bytes):
                msg = msg.decode()
            raise RuntimeError(f"NCCL error {result}: {msg}")

    def version(self) -> int:
        v = ctypes.c_int()
        self.check(self.lib.ncclGetVersion(ctypes.byref(v)))
        return v.value

    def get_unique_id(self) -> ncclUniqueId:
        uid = ncclUniqueId()
        self.check(self.lib.ncclGetUniqueId(ctypes.byref(uid)))
        return uid

    def comm_init_rank(self, world_size: int, uid: ncclUniqueId, rank: int) -> ncclComm_t:
        comm = ncclComm_t()
        self.check(self.lib.ncclCommInitRank(ctypes.byref(comm), world_size, uid, rank))
        return comm

    def __getattr__(self, name: str):
        # checked pass-through: lib.ncclAllReduce(...) -> self.all ... raise on error
        if name.startswith("nccl"):
            fn = getattr(self.lib, name)

            def call(*args):
                self.check(fn(*args))
            return call
        raise AttributeError(name)


class PyNcclCommunicator:
    """Communicator over an explicit rank set.  ``group`` is a torch CPU (gloo) process
    group used only to hand the unique id from rank 0 to the others; with ``unique_id`` given
    (point-to-point connector: the id travels over the connector's own control channel) no
    group is needed."""

    def __init__(self, rank: int, world_size: int, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None,
                 unique_id: Optional[bytes] = None, library: Optional[NCCLLibrary] = None):
        self.rank, self.world_size = rank, world_size
        self.device = torch.device(device)
        self.nccl = library or NCCLLibrary()
        self.available = world_size > 1
        self.comm: Optional[ncclComm_t] = None
        if not self.available:
            return
        if unique_id is not None:
            uid = ncclUniqueId()
            ctypes.memmove(ctypes.byref(uid), unique_id, 128)
        else:
            uid = self.nccl.get_unique_id() if rank == 0 else ncclUniqueId()
            assert group is not None, "a CPU group or a unique id is needed"
            t = torch.tensor(list(bytes(uid)), dtype=torch.uint8)
            dist.broadcast(t, src=dist.get_global_rank(group, 0), group=group)
            ctypes.memmove(ctypes.byref(uid), bytes(t.tolist()), 128)
        if self.device.type == "cuda":
            with torch.cuda.device(self.device):
                self.comm = self.nccl.comm_init_rank(world_size, uid, rank)
                warm = torch.zeros(1, device=self.device)      # first collective sets up rings
                self.all_reduce(warm)
                torch.cuda.current_stream().synchronize()
        else:
            self.comm = self.nccl.comm_init_rank(world_size, uid, rank)

    @staticmethod
    def new_unique_id(library: Optional[NCCLLibrary] = None) -> bytes:
        return bytes((library or NCCLLibrary()).get_unique_id())

    def _stream(self, stream) -> ctypes.c_void_p:
        if stream is None and self.device.type == "cuda":
            stream = torch.cuda.current_stream(self.device)
        return ctypes.c_void_p(stream.cuda_stream if stream is not None else 0)

    def all_reduce(self, t: torch.Tensor, op=dist.ReduceOp.SUM, out: Optional[torch.Tensor] = None,
                   stream=None) -> torch.Tensor:
        out = t if out is None else out
        self.nccl.ncclAllReduce(ctypes.c_void_p(t.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                t.numel(), ncclDataType.from_torch(t.dtype),
                                ncclRedOp.from_torch(op), self.comm, self._stream(stream))
        return out

    def all_gather(self, out: torch.Tensor, t: torch.Tensor, stream=None) -> torch.Tensor:
        self.nccl.ncclAllGather(ctypes.c_void_p(t.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                t.numel(), ncclDataType.from_torch(t.dtype), self.comm,
                                self._stream(stream))
        return out

    def reduce_scatter(self, out: torch.Tensor, t: torch.Tensor, op=dist.ReduceOp.SUM,
                       stream=None) -> torch.Tensor:
        self.nccl.ncclReduceScatter(ctypes.c_void_p(t.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                                    out.numel(), ncclDataType.from_torch(t.dtype),
                                    ncclRedOp.from_torch(op), self.comm, self._stream(stream))
        return out

    def broadcast(self, t: torch.Tensor, src: int, stream=None) -> torch.Tensor:
        self.nccl.ncclBroadcast(ctypes.c_void_p(t.data_ptr()), ctypes.c_void_p(t.data_ptr()),
                                t.numel(), ncclDataType.from_torch(t.dtype), src, self.comm,
                                self._stream(stream))
        return t

    def send(self, t: torch.Tensor, dst: int, stream=None) -> None:
        self.nccl.ncclSend(ctypes.c_void_p(t.data_ptr()), t.numel(),
                           ncclDataType.from_torch(t.dtype), dst, self.comm, self._stream(stream))

    def recv(self, t: torch.Tensor, src: int, stream=None) -> None:
        self.nccl.ncclRecv(ctypes.c_void_p(t.data_ptr()), t.numel(),
                           ncclDataType.from_torch(t.dtype), src, self.comm, self._stream(stream))

    def destroy(self) -> None:
        if self.comm is not None:
            self.nccl.ncclCommDestroy(self.comm)
            self.comm = None
