"""Environment flags, evaluated lazily on attribute access.

Every flag is read as ``VLLM_B200_<NAME>``; the reference's ``VLLM_GCU_<NAME>`` spelling is
accepted as an alias so existing launch scripts keep working (vllm_gcu/envs.py:4-41).
"""
from __future__ import annotations

import os
from typing import Any, Callable


def _get(name: str, default: str | None = None) -> str | None:
    for prefix in ("VLLM_B200_", "VLLM_GCU_"):
        v = os.environ.get(prefix + name)
        if v is not None:
            return v
    return default


def _flag(name: str, default: str = "0") -> Callable[[], bool]:
    return lambda: bool(int(_get(name, default)))


def _path(name: str) -> Callable[[], str | None]:
    return lambda: (None if _get(name) is None else os.path.expanduser(_get(name)))


environment_variables: dict[str, Callable[[], Any]] = {
    # Megatron-style sequence parallelism over the TP group (DeepSeek family)
    "ENABLE_SEQUENCE_PARALLEL": _flag("ENABLE_SEQUENCE_PARALLEL"),
    # run the sampler with the torch reference on the host (debugging)
    "SAMPLER_ON_CPU": lambda: int(_get("SAMPLER_ON_CPU", "0")),
    # dump the allocator history every n engine steps and on exceptions (0 = off)
    "DUMP_SNAPSHOT_EVERY_N_STEP": lambda: int(
        os.environ.get("VLLM_DUMP_SNAPSHOT_EVERY_N_STEP", _get("DUMP_SNAPSHOT_EVERY_N_STEP", "0"))),
    # directory for per-rank stdout/stderr logs (worker_<rank>.log)
    "RANK_LOG_PATH": _path("RANK_LOG_PATH"),
    # overlap the shared-expert MLP with the expert dispatch on a side stream
    "ENABLE_PARALLEL_COMPUTE": _flag("ENABLE_PARALLEL_COMPUTE"),
    # fused MLA path (RMSNorm + RoPE + cache write in one kernel); on by default here
    "DEEPSEEK_FUSION": _flag("DEEPSEEK_FUSION", "1"),
    # cross-check the rejection-sampler kernels against the torch oracle at run time
    "REJECT_SAMPLER_CHECK": _flag("REJECT_SAMPLER_CHECK"),
    # synthetic round-robin routing (benchmarking expert-parallel balance)
    "FORCE_EP_BALANCE": _flag("FORCE_EP_BALANCE"),
    # routed-expert MLP processes at most this many token rows at a time (bounds the
    # permuted / intermediate buffers of very long prefill batches; the reference chunks by
    # VLLM_FUSED_MOE_CHUNK_SIZE, vllm_gcu/kernels/modular_kernel.py:167-286)
    "FUSED_MOE_CHUNK_SIZE": lambda: int(
        os.environ.get("VLLM_FUSED_MOE_CHUNK_SIZE", _get("FUSED_MOE_CHUNK_SIZE", "32768"))),
    # comma-separated list of enabled forward hooks (entry-point group vllm_gcu_b200.hooks)
    "HOOKS": lambda: None if _get("HOOKS") is None else _get("HOOKS").split(","),
    # JSON file mapping GPUs to NICs for multi-node KV transfer
    "NET_CONFIG": _path("NET_CONFIG"),
    # run selected ops through the torch reference and compare ("all" or op1,op2,...)
    "ORACLE": lambda: None if _get("ORACLE") is None else _get("ORACLE").split(","),
    # communication backend of the tensor-parallel collectives: fused | nccl
    "COMM": lambda: _get("COMM", "fused"),
    # in-switch reduction / broadcast (NVLS multimem instructions) inside the fused
    # tensor-parallel kernels when the symmetric allocation has a multicast view; 0 keeps them
    # on plain peer loads and stores
    "MULTIMEM": _flag("MULTIMEM", "1"),
    # NVTX range around every engine step, named by its kind (the reference opens a vendor
    # profiler range per step, vllm_gcu/worker/worker_v1.py:322-335)
    "NVTX": _flag("NVTX"),
    # pin every worker process to its own slice of the CPU cores (the reference's optional
    # worker affinity, vllm_gcu/worker/worker_v1.py:259-260)
    "CPU_AFFINITY": _flag("CPU_AFFINITY"),
    # disaggregated prefill (vllm_gcu/envs.py:30-36, used by patch_0_9_2/nixl_connector.py):
    # the decode instance takes the KV of a partly filled last block too (0: whole blocks
    # only, the rest is recomputed) ...
    # 8-bit linear layers take their input already quantised from the norm / activation kernel
    # in front of them (0: separate quantisation kernels, for comparison)
    "FUSE_ACT_QUANT": _flag("FUSE_ACT_QUANT", "1"),
    # the executor's commands reach the workers through a shared-memory broadcast ring
    # (0: one pipe-backed queue per worker)
    "SHM_BROADCAST": _flag("SHM_BROADCAST", "1"),
    # expert parallelism with tensor-parallel attention inside a replica: every tensor-parallel
    # rank dispatches its own slice of the replica's rows (0: every rank dispatches all rows)
    "EP_TP_SLICE": _flag("EP_TP_SLICE", "1"),
    # expert-parallel dispatch of block-scaled fp8 models sends rows as fp8 with their group
    # scales (half the bytes of bf16 rows) and de-quantises them on arrival
    "EP_FP8_DISPATCH": _flag("EP_FP8_DISPATCH", "0"),
    # under vLLM: the worker reads the native status word (one device-to-host copy) every this
    # many steps and raises when a kernel reported a wait that ran out (0 = never)
    "CHECK_STATUS_EVERY": lambda: int(_get("CHECK_STATUS_EVERY", "0")),
    # log the median wall time of an engine step per batch size every this many steps
    # (0 = off; the reference logs median forward time per batch size periodically)
    "LOG_FORWARD_TIME_EVERY": lambda: int(_get("LOG_FORWARD_TIME_EVERY", "0")),
    "NIXL_ENABLE_FULL_KV_TRANSFER": _flag("NIXL_ENABLE_FULL_KV_TRANSFER", "1"),
    # ... and starts at the first output token the prefill instance already produced
    "NIXL_ENABLE_FIRST_TOKEN_REUSE": _flag("NIXL_ENABLE_FIRST_TOKEN_REUSE"),
}


def __getattr__(name: str):
    if name in environment_variables:
        return environment_variables[name]()
    raise AttributeError(name)


def __dir__():
    return list(environment_variables.keys())
