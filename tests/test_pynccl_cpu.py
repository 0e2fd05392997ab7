"""NCCL binding: enum mapping, library loading and error reporting against a fake function
table (failures are injected on the host; no GPU is involved)."""
import ctypes

import pytest
import torch
import torch.distributed as dist

from vllm_gcu_b200.parallel.pynccl import (NCCLLibrary, PyNcclCommunicator, ncclDataType,
                                           ncclRedOp)


class FakeNccl:
    """Stands in for libnccl: records calls, returns a chosen result code."""

    def __init__(self):
        self.calls = []
        self.fail = {}

    def ncclGetErrorString(self, code):
        return b"unhandled system error" if code == 2 else b"other"

    def _call(self, name, *args):
        self.calls.append((name, args))
        return self.fail.get(name, 0)

    def __getattr__(self, name):
        if name.startswith("nccl"):
            return lambda *a: self._call(name, *a)
        raise AttributeError(name)


def test_enums_and_real_library_loads():
    assert ncclDataType.from_torch(torch.bfloat16) == 9
    assert ncclDataType.from_torch(torch.float32) == 7
    assert ncclRedOp.from_torch(dist.ReduceOp.MAX) == 2
    with pytest.raises(ValueError):
        ncclDataType.from_torch(torch.complex64)
    lib = NCCLLibrary()                  # the NCCL that ships with torch; no device needed
    assert lib.version() >= 22000


def test_errors_become_runtime_errors_and_calls_carry_the_arguments():
    fake = FakeNccl()
    lib = NCCLLibrary(lib=fake)
    comm = PyNcclCommunicator(0, 2, torch.device("cpu"), unique_id=bytes(128), library=lib)
    assert fake.calls[0][0] == "ncclCommInitRank"
    t = torch.arange(6, dtype=torch.float32)
    comm.all_reduce(t)
    name, args = fake.calls[-1]
    assert name == "ncclAllReduce" and args[2] == 6 and args[3] == 7 and args[4] == 0
    comm.send(t, 1)
    assert fake.calls[-1][0] == "ncclSend" and fake.calls[-1][1][3] == 1
    fake.fail["ncclAllReduce"] = 2
    with pytest.raises(RuntimeError, match="NCCL error 2: unhandled system error"):
        comm.all_reduce(t)
    fake.fail["ncclCommInitRank"] = 2
    with pytest.raises(RuntimeError):
        PyNcclCommunicator(1, 2, torch.device("cpu"), unique_id=bytes(128), library=lib)
    comm.destroy()
    assert fake.calls[-1][0] == "ncclCommDestroy"
