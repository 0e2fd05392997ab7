"""Worker class that vLLM's executors start on every GPU when the platform plugin is active
(``parallel_config.worker_cls``, set by ``B200Platform.check_and_update_config``; the
reference points it at its own worker, vllm_gcu/gcu.py:192-209 and
vllm_gcu/worker/worker_v1.py:236).  It is vLLM's GPU worker plus the duties of this package:

* start-up: the native library must load (a missing ``_b200.so`` on a GPU box is an error, not
  a silent fallback), the layer kernels are registered before the model is built, the
  process's output goes to its per-rank log and the process is pinned to its share of the
  cores when the environment asks for it (vllm_gcu/worker/worker_v1.py:247-260);
* every step: an NVTX range named ``step`` when ``VLLM_B200_NVTX`` is set (the reference opens
  a vendor profiler range per step, :322-335), the allocator-history dump of
  ``DUMP_SNAPSHOT_EVERY_N_STEP`` (:320), and a look at the native status word every
  ``VLLM_B200_CHECK_STATUS_EVERY`` steps, so that a kernel wait that ran out surfaces as an
  exception in the worker instead of as wrong tokens.
"""
from __future__ import annotations

from vllm.v1.worker.gpu_worker import Worker


class B200Worker(Worker):
    _steps = 0

    def init_device(self):
        from .. import envs
        from ..ops import _native
        from ..utils import bind_cpu_affinity, redirect_rank_output
        from . import vllm_ops
        if _native.lib() is None:
            raise RuntimeError("vllm_gcu_b200: the native library is not built")
        rank = int(getattr(self, "rank", 0) or 0)
        redirect_rank_output(rank)                       # no-op without RANK_LOG_PATH
        if envs.CPU_AFFINITY:
            world = int(getattr(getattr(self, "parallel_config", None), "world_size", 1) or 1)
            bind_cpu_affinity(int(getattr(self, "local_rank", rank) or 0), world)
        vllm_ops.register_ops()
        return super().init_device()

    def execute_model(self, *args, **kwargs):
        return self._step(super().execute_model, *args, **kwargs)

    def _step(self, inner, *args, **kwargs):
        """One engine step through ``inner`` with this package's per-step hooks."""
        import torch
        from .. import envs
        from ..utils import dump_memory_snapshot
        nvtx = bool(envs.NVTX) and torch.cuda.is_available()
        if envs.DUMP_SNAPSHOT_EVERY_N_STEP > 0:
            if getattr(self, "_snapshot_step", None) is None:
                def execute_model(f, *a, **k):
                    return f(*a, **k)
                self._snapshot_step = dump_memory_snapshot(execute_model)
            call = lambda: self._snapshot_step(inner, *args, **kwargs)   # noqa: E731
        else:
            call = lambda: inner(*args, **kwargs)                        # noqa: E731
        if nvtx:
            torch.cuda.nvtx.range_push("step")
        try:
            out = call()
        finally:
            if nvtx:
                torch.cuda.nvtx.range_pop()
        self._steps += 1
        every = envs.CHECK_STATUS_EVERY
        if every > 0 and self._steps % every == 0:
            from ..ops import _native
            _native.check_status()
        return out

    def native_launch_count(self) -> int:
        """Kernels of this package launched by this worker process so far."""
        from ..ops import _native
        return int(_native.launch_count)
