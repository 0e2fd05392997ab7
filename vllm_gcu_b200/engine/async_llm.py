"""Asynchronous front end over one in-process engine: a background thread runs the step loop,
callers await per-request output streams (single-GPU serving; multi-GPU serving uses
``AsyncMultiprocExecutor`` with the same ``generate_stream`` contract)."""
from __future__ import annotations

import asyncio
import itertools
import threading
import time
from typing import AsyncIterator, Optional, Sequence

from ..config import EngineConfig
from .llm import LLMEngine
from .request import RequestOutput, SamplingParams


class AsyncLLM:
    def __init__(self, cfg: EngineConfig):
        self.engine = LLMEngine(cfg)
        self._lock = threading.Lock()
        self._streams: dict[str, tuple[asyncio.AbstractEventLoop, asyncio.Queue]] = {}
        self._ids = itertools.count()
        self._stop = threading.Event()
        self._wake = threading.Event()
        self.error: Optional[BaseException] = None
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self) -> None:
        try:
            while not self._stop.is_set():
                with self._lock:
                    busy = self.engine.has_unfinished()
                    outs = self.engine.step() if busy else []
                for o in outs:
                    ent = self._streams.get(o.request_id)
                    if ent is not None:
                        loop, q = ent
                        loop.call_soon_threadsafe(q.put_nowait, o)
                if not busy:
                    self._wake.wait(0.01)
                    self._wake.clear()
        except BaseException as e:  # noqa: BLE001
            self.error = e
            for loop, q in list(self._streams.values()):
                loop.call_soon_threadsafe(q.put_nowait, e)

    async def generate_stream(self, prompt_token_ids: Sequence[int],
                              sampling_params: Optional[SamplingParams] = None,
                              request_id: Optional[str] = None, priority: int = 0,
                              lora_id: int = -1, kv_transfer_params: Optional[dict] = None
                              ) -> AsyncIterator[RequestOutput]:
        if self.error is not None:
            raise RuntimeError(f"engine failed: {self.error!r}")
        rid = request_id or f"areq-{next(self._ids)}"
        q: asyncio.Queue = asyncio.Queue()
        self._streams[rid] = (asyncio.get_running_loop(), q)
        with self._lock:
            self.engine.add_request(prompt_token_ids, sampling_params, rid, priority,
                                    lora_id=lora_id, kv_transfer_params=kv_transfer_params)
        self._wake.set()
        try:
            while True:
                item = await q.get()
                if isinstance(item, BaseException):
                    raise RuntimeError(f"engine failed: {item!r}")
                yield item
                if item.finished:
                    break
        except asyncio.CancelledError:
            with self._lock:
                self.engine.abort_request(rid)
            raise
        finally:
            self._streams.pop(rid, None)

    def stats(self) -> dict:
        with self._lock:
            s = dict(self.engine.scheduler.stats())
            s.update(self.engine.stats)
            if self.engine.spec_metrics is not None:
                s["spec_acceptance_rate"] = self.engine.spec_metrics.acceptance_rate
        return s

    def shutdown(self) -> None:
        self._stop.set()
        self._wake.set()
        self._thread.join(5.0)
