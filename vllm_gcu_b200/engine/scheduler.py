"""Continuous-batching scheduler with chunked prefill, prefix caching, priority
preemption, speculative tokens and asynchronous (one-step-ahead) scheduling.

One class covers the reference's three schedulers:

* the unified token-budget policy of the v1 scheduler it forks
  (vllm_gcu/v1/core/sched/async_scheduler.py:51-476);
* ``async_scheduling``: step N+1 is scheduled before the token ids of step N
  exist, tracked by ``Request.num_output_placeholders``
  (async_scheduler.py:478-555);
* ``policy="priority"``: requests are served in (priority, arrival) order, a
  higher-priority arrival preempts the lowest-priority running request when the
  cache is full, and with ``separate_prefill_decode`` a step never mixes prefill
  and decode work and a running higher-priority decode is not displaced by a
  lower-priority prefill (vllm_gcu/scheduler.py:13-140).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Iterable, Optional, Sequence

from ..config import CacheConfig, SchedulerConfig
from .block_manager import KVCacheManager
from .request import (CompletionOutput, Request, RequestOutput, RequestStatus, check_stop)


@dataclass(eq=False)
class ScheduledRequest:
    req: Request
    start: int                 # first position computed in this step
    num_tokens: int            # positions computed in this step
    new_block_ids: list[int]
    is_new: bool               # first step since admission / resumption
    spec_token_ids: list[int] = field(default_factory=list)
    will_sample: bool = False  # this step produces the next token(s) of the request
    epoch: int = 0             # the request's preemption count when this step was planned
    sample_index: int = 0      # index of the first output token this step produces


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledRequest] = field(default_factory=list)
    total_tokens: int = 0
    finished_req_ids: set[str] = field(default_factory=set)
    preempted_req_ids: list[str] = field(default_factory=list)
    # swap preemption: (device block, host block) pairs to copy out / (host, device) to copy in,
    # executed by the runner before the forward pass of this step (copy-in first)
    swap_out: list[tuple[int, int]] = field(default_factory=list)
    swap_in: list[tuple[int, int]] = field(default_factory=list)
    step_id: int = 0

    @property
    def is_empty(self) -> bool:
        return not self.scheduled


class Scheduler:
    def __init__(self, sched_cfg: SchedulerConfig, cache_cfg: CacheConfig, num_blocks: int,
                 separate_prefill_decode: bool = False, num_lookahead_tokens: int = 0):
        self.cfg = sched_cfg
        self.block_size = cache_cfg.block_size
        self.kv = KVCacheManager(num_blocks, cache_cfg.block_size,
                                 cache_cfg.enable_prefix_caching)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.requests: dict[str, Request] = {}
        self.finished_since_last: set[str] = set()
        self.async_mode = sched_cfg.async_scheduling
        self.on_free = None              # optional callback(req), blocks still allocated
        self.priority = sched_cfg.policy == "priority"
        self.separate_prefill_decode = separate_prefill_decode
        self.num_lookahead_tokens = num_lookahead_tokens
        self.step_id = 0
        self.num_preemptions = 0
        self.num_running_last = 0          # requests in the most recent scheduler output
        # host blocks of the swap space (CacheConfig.num_cpu_blocks > 0 turns preemption by
        # recomputation into preemption by swapping where the victim's state allows it)
        self.cpu_free: list[int] = list(range(int(getattr(cache_cfg, "num_cpu_blocks", 0) or 0)))
        self.num_swaps = 0
        #: emit a RequestOutput for every sampled token (streaming); False: finished only
        self.emit_partial = True

    # -- request lifecycle ---------------------------------------------------
    def add_request(self, req: Request) -> None:
        if req.num_prompt_tokens == 0:
            # an empty prompt has nothing to prefill: at the head of the queue it would ask for
            # zero tokens forever and starve every request behind it
            raise ValueError("the prompt is empty")
        if req.num_prompt_tokens >= self.cfg.max_model_len:
            raise ValueError(f"prompt of {req.num_prompt_tokens} tokens exceeds max_model_len "
                             f"{self.cfg.max_model_len}")
        self.requests[req.request_id] = req
        req.status = RequestStatus.WAITING
        if self.priority:
            self._insert_by_priority(req)
        else:
            self.waiting.append(req)

    def _insert_by_priority(self, req: Request) -> None:
        key = (req.priority, req.arrival_time)
        items = list(self.waiting)
        pos = len(items)
        for i, r in enumerate(items):
            if (r.priority, r.arrival_time) > key:
                pos = i
                break
        items.insert(pos, req)
        self.waiting = deque(items)

    def stop_request(self, request_id: str) -> Optional[RequestOutput]:
        """Ends a running request as stopped (a stop string appeared in its text) and returns
        its final output; None when the request is unknown or already over."""
        req = self.requests.get(request_id)
        if req is None or req.finished:
            return None
        req.status = RequestStatus.FINISHED_STOPPED
        import time as _t
        req.finish_time = _t.monotonic()
        self._free(req)
        return self._make_output(req, 0)

    def abort_request(self, request_id: str) -> None:
        req = self.requests.get(request_id)
        if req is None or req.finished:
            return
        req.status = RequestStatus.FINISHED_ABORTED
        self._free(req)

    def _free(self, req: Request) -> None:
        if req in self.running:
            self.running.remove(req)
        else:
            try:
                self.waiting.remove(req)
            except ValueError:
                pass
        if self.on_free is not None:
            self.on_free(req)           # e.g. ship the KV to a decode instance
        if getattr(req, "cpu_block_ids", None):
            self.cpu_free.extend(req.cpu_block_ids)
            req.cpu_block_ids = []
        self.kv.free(req)
        self.finished_since_last.add(req.request_id)
        self.requests.pop(req.request_id, None)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    @property
    def num_unfinished(self) -> int:
        return len(self.waiting) + len(self.running)

    # -- scheduling ------------------------------------------------------------
    def _preempt(self, victim: Request, out: SchedulerOutput) -> None:
        self.running.remove(victim)
        bs = self.kv.block_size
        nb = -(-victim.num_computed_tokens // bs)
        if (0 < nb <= len(self.cpu_free) and victim.num_output_placeholders == 0
                and not victim.spec_token_ids and victim.mm_embeds is None
                and nb <= len(victim.block_ids)):
            # swap: the blocks that hold computed tokens go to host memory and the request
            # resumes where it stopped (the reference's legacy engine swaps the same way,
            # vllm_gcu/attention/ops/paged_attn.py:214-234 `swap_blocks`)
            cpu = [self.cpu_free.pop() for _ in range(nb)]
            out.swap_out.extend(zip(victim.block_ids[:nb], cpu))
            victim.cpu_block_ids = cpu
            self.kv.free(victim)
            victim.status = RequestStatus.SWAPPED
            victim.num_preemptions += 1
            self.num_preemptions += 1
            self.num_swaps += 1
            out.preempted_req_ids.append(victim.request_id)
            if self.priority:
                self._insert_by_priority(victim)
            else:
                self.waiting.appendleft(victim)
            return
        self.kv.free(victim)
        victim.status = RequestStatus.PREEMPTED
        victim.preempt_epoch = getattr(victim, "preempt_epoch", 0) + 1
        victim.num_computed_tokens = 0
        victim.num_output_placeholders = 0
        victim.spec_token_ids = []
        victim.num_preemptions += 1
        self.num_preemptions += 1
        out.preempted_req_ids.append(victim.request_id)
        if self.priority:
            self._insert_by_priority(victim)
        else:
            self.waiting.appendleft(victim)

    def _tokens_wanted(self, req: Request) -> int:
        return (req.num_tokens_with_placeholders + len(req.spec_token_ids)
                - req.num_computed_tokens)

    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput(step_id=self.step_id)
        self.step_id += 1
        out.finished_req_ids, self.finished_since_last = self.finished_since_last, set()
        budget = self.cfg.max_num_batched_tokens
        threshold = self.cfg.long_prefill_token_threshold

        if self.priority:
            self.running.sort(key=lambda r: (r.priority, r.arrival_time))

        # Under the priority policy with separated phases, decide the phase first:
        # prefill work is admitted only if no running decode outranks it.
        allow_waiting = True
        running_decodes = [r for r in self.running if r.num_computed_tokens >= r.num_prompt_tokens]
        if self.separate_prefill_decode and self.waiting and running_decodes:
            head = self.waiting[0]
            best_running = min((r.priority, r.arrival_time) for r in running_decodes)
            if (head.priority, head.arrival_time) > best_running:
                allow_waiting = False       # the low-priority prefill stays in `waiting`

        # Priority policy: a waiting request that outranks running ones takes their blocks
        # when the cache cannot hold its first chunk.
        if self.priority and self.waiting and allow_waiting:
            head = self.waiting[0]
            first = min(head.num_tokens - head.num_computed_tokens, budget)
            need = self.kv.pool.blocks_needed(first + self.num_lookahead_tokens, 0)
            while self.running and self.kv.pool.num_free_blocks < need:
                victim = max(self.running, key=lambda r: (r.priority, r.arrival_time))
                if (victim.priority, victim.arrival_time) <= (head.priority, head.arrival_time):
                    break
                self._preempt(victim, out)
        priority_preempted = len(out.preempted_req_ids)

        # 1) requests that are already running
        scheduled_ids: set[str] = set()
        i = 0
        while i < len(self.running) and budget > 0:
            req = self.running[i]
            want = self._tokens_wanted(req)
            if self.async_mode:
                sp = req.sampling_params
                if len(req.output_token_ids) + req.num_output_placeholders >= sp.max_tokens:
                    want = 0                # the last token is already in flight
                elif req.num_output_placeholders > 0 and sp.needs_host_history:
                    want = 0                # its mask / penalties need the token in flight
            if self.separate_prefill_decode and allow_waiting and self.waiting \
                    and req.num_computed_tokens >= req.num_prompt_tokens:
                want = 0                    # prefill phase: decodes sit this step out
            if want <= 0:
                i += 1
                continue
            n = min(want, budget)
            if threshold > 0:
                n = min(n, threshold)
            if not self.cfg.enable_chunked_prefill and n < want:
                i += 1
                continue
            new_blocks = None
            while True:
                new_blocks = self.kv.allocate_slots(
                    req, n, num_lookahead_tokens=self.num_lookahead_tokens)
                if new_blocks is not None:
                    break
                # out of blocks: preempt the lowest-priority running request
                victim = self.running[-1]
                if victim.request_id in scheduled_ids:
                    # never preempt a request already placed in this step
                    cands = [r for r in self.running if r.request_id not in scheduled_ids]
                    if not cands:
                        break
                    victim = cands[-1]
                self._preempt(victim, out)
                if victim is req:
                    break
            if new_blocks is None:
                if req in self.running:
                    i += 1
                continue
            spec = list(req.spec_token_ids)
            out.scheduled.append(ScheduledRequest(req, req.num_computed_tokens, n, new_blocks,
                                                  False, spec))
            scheduled_ids.add(req.request_id)
            budget -= n
            i += 1

        # 2) admit waiting requests (only if nothing was preempted in this step)
        if allow_waiting and len(out.preempted_req_ids) == priority_preempted:
            while self.waiting and budget > 0 and len(self.running) < self.cfg.max_num_seqs:
                req = self.waiting[0]
                computed_blocks: list[int] = []
                num_cached = 0
                if req.num_computed_tokens == 0 and req.sampling_params.prompt_logprobs is None:
                    # (prompt log-probabilities need every prompt position computed)
                    computed_blocks, num_cached = self.kv.get_computed_blocks(req)
                want = req.num_tokens - num_cached - req.num_computed_tokens
                n = min(want, budget)
                if threshold > 0:
                    n = min(n, threshold)
                if want <= 0:
                    # nothing left to compute (cannot be scheduled): drop it instead of
                    # blocking the queue
                    self.waiting.popleft()
                    req.status = RequestStatus.FINISHED_ABORTED
                    self._free(req)
                    continue
                if n <= 0 or (not self.cfg.enable_chunked_prefill and n < want):
                    break
                new_blocks = self.kv.allocate_slots(
                    req, n, computed_blocks, num_lookahead_tokens=self.num_lookahead_tokens)
                if new_blocks is None:
                    if self.priority and self._preempt_for(req, out, scheduled_ids):
                        continue
                    break
                self.waiting.popleft()
                if req.status == RequestStatus.SWAPPED:
                    cpu = req.cpu_block_ids
                    out.swap_in.extend(zip(cpu, req.block_ids[:len(cpu)]))
                    self.cpu_free.extend(cpu)
                    req.cpu_block_ids = []
                if num_cached:
                    req.num_computed_tokens = num_cached
                    if req.num_preemptions == 0:
                        req.num_cached_tokens = num_cached
                req.status = RequestStatus.RUNNING
                self.running.append(req)
                out.scheduled.append(ScheduledRequest(req, req.num_computed_tokens, n,
                                                      list(req.block_ids), True, []))
                scheduled_ids.add(req.request_id)
                budget -= n

        out.total_tokens = sum(s.num_tokens for s in out.scheduled)
        self._update_after_schedule(out)
        return out

    def _preempt_for(self, newcomer: Request, out: SchedulerOutput, placed: set[str]) -> bool:
        """Priority policy: evict the lowest-priority running request if the waiting
        head outranks it.  Returns True when something was evicted."""
        cands = [r for r in self.running if r.request_id not in placed]
        if not cands:
            return False
        victim = max(cands, key=lambda r: (r.priority, r.arrival_time))
        if (victim.priority, victim.arrival_time) <= (newcomer.priority, newcomer.arrival_time):
            return False
        self._preempt(victim, out)
        return True

    def _update_after_schedule(self, out: SchedulerOutput) -> None:
        """Advances ``num_computed_tokens`` right away so the next step can be planned
        before this one returns (async_scheduler.py:478-515)."""
        self.num_running_last = len(out.scheduled)
        for s in out.scheduled:
            req = s.req
            s.epoch = getattr(req, "preempt_epoch", 0)
            req.num_computed_tokens += s.num_tokens
            will_sample = req.num_computed_tokens >= (req.num_tokens_with_placeholders
                                                      + len(s.spec_token_ids))
            s.will_sample = will_sample
            # tokens already produced or in flight: the same number whether earlier steps have
            # been retired yet or not, so a seeded draw does not depend on the scheduling mode
            s.sample_index = len(req.output_token_ids) + req.num_output_placeholders
            if self.async_mode and will_sample:
                req.num_output_placeholders += 1 + len(s.spec_token_ids)
            if s.spec_token_ids:
                req.spec_token_ids = []

    # -- results -----------------------------------------------------------------
    def update_from_output(self, out: SchedulerOutput,
                           sampled: dict[str, Sequence[int]],
                           draft: Optional[dict[str, Sequence[int]]] = None,
                           logprobs: Optional[dict[str, dict]] = None,
                           ) -> list[RequestOutput]:
        """``sampled[req_id]`` holds the token ids emitted by the step (one, or up to
        ``1 + len(spec)`` accepted tokens under speculative decoding; empty for a
        partial prefill chunk)."""
        results: list[RequestOutput] = []
        for s in out.scheduled:
            req = s.req
            if req.finished or req.request_id not in self.requests:
                continue                    # aborted / finished while the step was in flight
            if req.status != RequestStatus.RUNNING:
                continue
            if getattr(req, "preempt_epoch", 0) != s.epoch:
                continue                    # preempted and re-admitted since this step was planned
            toks = list(sampled.get(req.request_id, ()))
            if not s.will_sample:
                # partial prefill: nothing to emit, tokens are all known -> cacheable
                self.kv.cache_blocks(req, req.num_computed_tokens)
                continue
            n_spec = len(s.spec_token_ids)
            if n_spec:
                rejected = n_spec + 1 - len(toks)
                if rejected > 0:
                    req.num_computed_tokens -= rejected
            if self.async_mode:
                req.num_output_placeholders -= 1 + n_spec
                assert req.num_output_placeholders >= 0
            stopped = False
            emitted = 0
            for t in toks:
                req.output_token_ids.append(int(t))
                emitted += 1
                if logprobs is not None and req.request_id in logprobs:
                    req.logprobs.append(logprobs[req.request_id])
                if req.first_token_time is None:
                    import time as _t
                    req.first_token_time = _t.monotonic()
                if check_stop(req, self.cfg.max_model_len):
                    stopped = True
                    break
            if draft is not None and not stopped:
                req.spec_token_ids = list(draft.get(req.request_id, ()))
            self.kv.cache_blocks(req, req.num_computed_tokens - req.num_output_placeholders)
            if stopped:
                import time as _t
                req.finish_time = _t.monotonic()
                self._free(req)
            if stopped or self.emit_partial:
                results.append(self._make_output(req, emitted))
        return results

    @staticmethod
    def _make_output(req: Request, num_new: int) -> RequestOutput:
        reason = None
        if req.status == RequestStatus.FINISHED_STOPPED:
            reason = "stop"
        elif req.status == RequestStatus.FINISHED_LENGTH:
            reason = "length"
        elif req.status == RequestStatus.FINISHED_ABORTED:
            reason = "abort"
        # token_ids is the request's live list (no per-step copy); treat it as read-only
        cum = None
        if req.logprobs:
            cum = sum(d.get(t, 0.0) for d, t in zip(req.logprobs, req.output_token_ids))
        comp = CompletionOutput(0, req.output_token_ids, reason,
                                req.logprobs if req.logprobs else None, cum)
        return RequestOutput(req.request_id, req.prompt_token_ids, [comp], req.finished,
                             req.num_cached_tokens, req.prompt_logprobs,
                             kv_transfer_params=req.kv_transfer_params_out)

    # -- stats -------------------------------------------------------------------
    def stats(self) -> dict[str, float]:
        return {"num_running": len(self.running), "num_waiting": len(self.waiting),
                "kv_cache_usage": self.kv.usage,
                "prefix_cache_queries": self.kv.pool.queries,
                "prefix_cache_hits": self.kv.pool.hits,
                "num_preemptions": self.num_preemptions, "num_swaps": self.num_swaps}
