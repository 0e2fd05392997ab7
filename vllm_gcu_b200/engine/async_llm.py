"""Asynchronous front end over one in-process engine: a background thread runs the step loop,
callers await per-request output streams (single-GPU serving; multi-GPU serving uses
``AsyncMultiprocExecutor`` with the same ``generate_stream`` contract)."""
from __future__ import annotations

import asyncio
import itertools
import queue
import threading
import time
from typing import AsyncIterator, Optional, Sequence

from ..config import EngineConfig
from .llm import LLMEngine
from .request import RequestOutput, SamplingParams


class AsyncLLM:
    def __init__(self, cfg: EngineConfig):
        self.engine = LLMEngine(cfg)
        self._lock = threading.Lock()          # guards engine state against stats()
        self._inbox: queue.SimpleQueue = queue.SimpleQueue()   # ("add", kwargs) / ("abort", rid)
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
                    self._drain_inbox()
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

    def _drain_inbox(self) -> None:
        """Applies the submissions and aborts that arrived since the last step (engine thread)."""
        while True:
            try:
                kind, arg = self._inbox.get_nowait()
            except queue.Empty:
                return
            if kind == "abort":
                self.engine.abort_request(arg)
                continue
            if kind == "lora":
                req, tensors, config, done = arg
                try:
                    self.engine.add_lora(req, tensors, config)
                    done.set_result(None) if not done.done() else None
                except Exception as e:  # noqa: BLE001  (reported to the caller of add_lora)
                    done.set_exception(e) if not done.done() else None
                continue
            try:
                self.engine.add_request(**arg)
            except Exception as e:  # noqa: BLE001  (reported to the one caller, not fatal)
                ent = self._streams.get(arg["request_id"])
                if ent is not None:
                    ent[0].call_soon_threadsafe(ent[1].put_nowait, e)

    def validate_prompt(self, prompt_token_ids: Sequence[int], multimodal: bool = False) -> None:
        """Raises ValueError for a prompt the scheduler would refuse (empty, or longer than
        the model length); callable from any thread."""
        n = len(prompt_token_ids)
        if n == 0:
            raise ValueError("the prompt is empty")
        limit = self.engine.cfg.scheduler.max_model_len
        if n >= limit:
            raise ValueError(f"prompt of {n} tokens exceeds max_model_len {limit}")
        from .llm import check_token_ids
        check_token_ids(prompt_token_ids, self.engine.cfg.model.vocab_size,
                        allow_placeholders=multimodal)

    async def generate_stream(self, prompt_token_ids: Sequence[int],
                              sampling_params: Optional[SamplingParams] = None,
                              request_id: Optional[str] = None, priority: int = 0,
                              lora_id: int = -1, kv_transfer_params: Optional[dict] = None,
                              multi_modal_data: Optional[dict] = None
                              ) -> AsyncIterator[RequestOutput]:
        if self.error is not None:
            raise RuntimeError(f"engine failed: {self.error!r}")
        self.validate_prompt(prompt_token_ids)
        rid = request_id or f"areq-{next(self._ids)}"
        q: asyncio.Queue = asyncio.Queue()
        self._streams[rid] = (asyncio.get_running_loop(), q)
        # the engine thread holds its lock for a whole step: hand the request over through the
        # inbox instead of blocking the event loop on that lock
        self._inbox.put(("add", dict(prompt_token_ids=prompt_token_ids,
                                     sampling_params=sampling_params, request_id=rid,
                                     priority=priority, lora_id=lora_id,
                                     kv_transfer_params=kv_transfer_params,
                                     multi_modal_data=multi_modal_data)))
        self._wake.set()
        try:
            while True:
                item = await q.get()
                if isinstance(item, ValueError):
                    raise item
                if isinstance(item, BaseException):
                    raise RuntimeError(f"engine failed: {item!r}")
                yield item
                if item.finished:
                    break
        except asyncio.CancelledError:
            self._inbox.put(("abort", rid))
            self._wake.set()
            raise
        finally:
            self._streams.pop(rid, None)

    def add_lora(self, lora_request, tensors=None, config=None, timeout: float = 600.0) -> None:
        """Loads a LoRA adapter between two engine steps (the engine thread applies it);
        blocks until it is in place and re-raises a loading error."""
        import concurrent.futures
        done: concurrent.futures.Future = concurrent.futures.Future()
        self._inbox.put(("lora", (lora_request, tensors, config, done)))
        self._wake.set()
        done.result(timeout)

    def stats(self) -> dict:
        # read-only snapshot of counters: taken without the step lock so that a metrics
        # request never waits for a running step
        s = dict(self.engine.scheduler.stats())
        s.update(self.engine.stats)
        if self.engine.spec_metrics is not None:
            s["spec_acceptance_rate"] = self.engine.spec_metrics.acceptance_rate
        return s

    def shutdown(self) -> None:
        self._stop.set()
        self._wake.set()
        self._thread.join(5.0)
