"""Sleep mode is not offered.

The reference replaces vLLM's ``CuMemAllocator`` with a stub whose every method raises
(vllm_gcu/gcumem.py:4-26, patched in at vllm_gcu/worker/worker_v1.py:233-234) and lists sleep
mode as "no plan" in its feature matrix.  The same stub here keeps the call sites of an
engine that asks for ``enable_sleep_mode`` failing loudly instead of silently ignoring it.
"""
from __future__ import annotations

from contextlib import contextmanager


class CuMemAllocator:
    _instance = None

    @classmethod
    def get_instance(cls) -> "CuMemAllocator":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def _no(self, what: str):
        raise NotImplementedError(f"sleep mode is not supported ({what})")

    def sleep(self, offload_tags=None) -> None:
        self._no("sleep")

    def wake_up(self, tags=None) -> None:
        self._no("wake_up")

    @contextmanager
    def use_memory_pool(self, tag=None):
        self._no("use_memory_pool")
        yield

    def get_current_usage(self) -> int:
        return 0
