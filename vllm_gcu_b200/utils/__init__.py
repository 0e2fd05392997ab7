"""Small shared utilities: logger, memory-snapshot decorator, hook discovery, thresholds."""
from __future__ import annotations

import functools
import logging
import os
import sys
from typing import Callable, Optional

import torch

from .. import envs

_FORMAT = "(Module: VLLM_B200) %(levelname)s %(asctime)s [%(filename)s:%(lineno)d] %(message)s"


def init_logger(name: str = "vllm_gcu_b200") -> logging.Logger:
    """Package logger with the module prefix (vllm_gcu/__init__.py:35-71)."""
    logger = logging.getLogger(name)
    if not logger.handlers:
        # stderr: tools of this package print their results (JSON lines) on stdout
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter(_FORMAT, datefmt="%m-%d %H:%M:%S"))
        logger.addHandler(h)
        logger.setLevel(os.environ.get("VLLM_LOGGING_LEVEL", "INFO"))
        logger.propagate = False
    return logger


logger = init_logger()

STR_DTYPE_TO_TORCH_DTYPE = {
    "half": torch.float16, "float16": torch.float16, "bfloat16": torch.bfloat16,
    "float": torch.float32, "float32": torch.float32, "fp8": torch.float8_e4m3fn,
    "fp8_e4m3": torch.float8_e4m3fn, "fp8_e5m2": torch.float8_e5m2, "int8": torch.int8,
    "uint8": torch.uint8,
}


def dump_memory_snapshot(func: Callable) -> Callable:
    """Wraps a step function: with ``DUMP_SNAPSHOT_EVERY_N_STEP = n`` the CUDA allocator
    history is recorded and written to ``/tmp/vllm_snapshot_rank{r}_{name}{step}.pkl`` every
    n calls and whenever the call raises (vllm_gcu/utils.py:51-82)."""
    state = {"step": 0, "recording": False}

    @functools.wraps(func)
    def wrapper(*args, **kwargs):
        n = envs.DUMP_SNAPSHOT_EVERY_N_STEP
        if n <= 0 or not torch.cuda.is_available():
            return func(*args, **kwargs)
        if not state["recording"]:
            torch.cuda.memory._record_memory_history(max_entries=100000)
            state["recording"] = True
        rank = int(os.environ.get("RANK", "0"))
        state["step"] += 1

        def dump(tag: str) -> None:
            path = f"/tmp/vllm_snapshot_rank{rank}_{func.__name__}{tag}.pkl"
            try:
                torch.cuda.memory._dump_snapshot(path)
            except Exception as e:  # pragma: no cover
                logger.warning("memory snapshot failed: %s", e)

        try:
            out = func(*args, **kwargs)
        except Exception:
            dump(f"{state['step']}_error")
            raise
        if state["step"] % n == 0:
            dump(str(state["step"]))
        return out

    return wrapper


def ep_alltoall_threshold(max_num_seqs: int, max_capture_size: int, dp_size: int, tp_size: int = 1,
                          sequence_parallel: bool = False) -> int:
    """Largest total token count (over all data-parallel ranks) served by the static-shape
    dispatch path: ``max(max_num_seqs, max_capture_size)`` (rounded up to the TP size under
    sequence parallelism) times the DP size (vllm_gcu/utils.py:95-112)."""
    n = max(max_num_seqs, max_capture_size)
    if sequence_parallel and tp_size > 1:
        n = -(-n // tp_size) * tp_size
    return n * dp_size


def discover_hooks() -> list[Callable]:
    """Forward hooks from the entry-point group ``vllm_gcu_b200.hooks``, filtered by the
    ``HOOKS`` flag (vllm_gcu/utils.py:115-123)."""
    allowed = envs.HOOKS
    out = []
    try:
        from importlib.metadata import entry_points
        eps = entry_points(group="vllm_gcu_b200.hooks")
    except Exception:  # pragma: no cover
        return out
    for ep in eps:
        if allowed is not None and ep.name not in allowed:
            continue
        try:
            out.append(ep.load())
        except Exception as e:  # pragma: no cover
            logger.warning("hook %s failed to load: %s", ep.name, e)
    return out


def redirect_rank_output(rank: int) -> Optional[str]:
    """Duplicates stdout / stderr of this process into ``RANK_LOG_PATH/worker_<rank>.log``
    (vllm_gcu/worker/worker.py:51-60).  Returns the log path or None."""
    d = envs.RANK_LOG_PATH
    if d is None:
        return None
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, f"worker_{rank}.log")
    fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_APPEND, 0o644)
    os.dup2(fd, sys.stdout.fileno())
    os.dup2(fd, sys.stderr.fileno())
    return path


def bind_cpu_affinity(rank: int, world: int) -> Optional[list[int]]:
    """Pins the calling process to the ``rank``-th of ``world`` equal slices of the cores it
    may run on.  Returns the cores, or None when the platform has no affinity call."""
    if not hasattr(os, "sched_getaffinity"):
        return None
    cores = sorted(os.sched_getaffinity(0))
    per = max(1, len(cores) // max(world, 1))
    mine = cores[rank * per:(rank + 1) * per] or cores[-per:]
    os.sched_setaffinity(0, mine)
    return mine
