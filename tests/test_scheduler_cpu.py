"""Scheduler unit tests with scripted token ids (no model, no device)."""
import itertools

import pytest

from vllm_gcu_b200.config import CacheConfig, SchedulerConfig
from vllm_gcu_b200.engine.request import Request, RequestStatus, SamplingParams
from vllm_gcu_b200.engine.scheduler import Scheduler


def make(num_blocks=64, policy="fcfs", async_mode=False, budget=64, max_seqs=8, separate=False,
         prefix=True, max_len=512):
    sc = SchedulerConfig(max_num_seqs=max_seqs, max_num_batched_tokens=budget,
                         max_model_len=max_len, policy=policy, async_scheduling=async_mode)
    cc = CacheConfig(block_size=16, enable_prefix_caching=prefix)
    return Scheduler(sc, cc, num_blocks, separate_prefill_decode=separate)


_ids = itertools.count()


def req(n_prompt, max_tokens=8, priority=0, arrival=None, prompt=None, eos=None, **kw):
    i = next(_ids)
    # distinct contents per request so that prefix caching does not link unrelated prompts
    r = Request(f"r{i}", prompt or [1000 * (i + 1) + t for t in range(n_prompt)],
                SamplingParams(max_tokens=max_tokens, ignore_eos=eos is None, **kw),
                eos_token_id=eos, priority=priority)
    if arrival is not None:
        r.arrival_time = arrival
    return r


def run_sync(s, script=None, max_steps=1000):
    """Drives the scheduler to completion; every sampling request gets ``script(req)``."""
    done = {}
    for _ in range(max_steps):
        if not s.has_unfinished():
            break
        so = s.schedule()
        toks = {x.req.request_id: [script(x.req) if script else 7] for x in so.scheduled
                if x.will_sample}
        for o in s.update_from_output(so, toks):
            if o.finished:
                done[o.request_id] = o
    return done


def test_chunked_prefill_respects_budget_and_finishes():
    s = make(budget=32)
    a, b = req(50, max_tokens=3), req(20, max_tokens=3)
    s.add_request(a)
    s.add_request(b)
    so = s.schedule()
    assert so.total_tokens <= 32 and so.scheduled[0].req is a and so.scheduled[0].num_tokens == 32
    assert not so.scheduled[0].will_sample
    s.update_from_output(so, {})
    so = s.schedule()                       # rest of a (18) + first chunk of b (14)
    assert [x.num_tokens for x in so.scheduled] == [18, 14]
    assert so.scheduled[0].will_sample and not so.scheduled[1].will_sample
    s.update_from_output(so, {a.request_id: [5]})
    done = run_sync(s)
    assert len(done) == 2 and all(len(o.outputs[0].token_ids) == 3 for o in done.values())
    assert s.kv.pool.num_free_blocks == s.kv.pool.num_blocks


def test_prefix_cache_hit_skips_computed_blocks():
    s = make()
    p = list(range(100, 148))               # 3 full blocks
    a = req(0, prompt=p + [1, 2], max_tokens=2)
    s.add_request(a)
    run_sync(s)
    b = req(0, prompt=p + [9, 9, 9], max_tokens=2)
    s.add_request(b)
    so = s.schedule()
    assert so.scheduled[0].start == 48 and so.scheduled[0].num_tokens == 3
    assert b.num_cached_tokens == 48
    run_sync(s)


def test_preemption_by_recompute_when_cache_is_full():
    s = make(num_blocks=8, budget=128)
    a, b = req(60, max_tokens=40), req(60, max_tokens=40)
    s.add_request(a)
    s.add_request(b)
    done = run_sync(s)
    assert len(done) == 2
    assert s.num_preemptions > 0
    assert all(len(o.outputs[0].token_ids) == 40 for o in done.values())


def test_priority_keeps_high_priority_decode_running():
    """A large low-priority prefill must not displace a running high-priority decode
    (the reference's only scheduler test, tests/core/test_scheduler.py:13-42)."""
    s = make(policy="priority", separate=True, budget=64)
    hi = req(8, max_tokens=6, priority=0, arrival=0.0)
    s.add_request(hi)
    so = s.schedule()
    s.update_from_output(so, {hi.request_id: [3]})
    lo = req(60, max_tokens=2, priority=5, arrival=1.0)
    s.add_request(lo)
    for _ in range(3):
        so = s.schedule()
        assert [x.req for x in so.scheduled] == [hi]        # decode continues, prefill waits
        s.update_from_output(so, {hi.request_id: [3]})
    assert lo.status == RequestStatus.WAITING
    done = run_sync(s)
    assert set(done) == {hi.request_id, lo.request_id}


def test_priority_preempts_lower_priority_when_out_of_blocks():
    s = make(policy="priority", num_blocks=8, budget=128)
    lo = req(70, max_tokens=30, priority=9, arrival=0.0)
    s.add_request(lo)
    so = s.schedule()
    s.update_from_output(so, {lo.request_id: [1]})
    hi = req(60, max_tokens=4, priority=0, arrival=1.0)
    s.add_request(hi)
    so = s.schedule()
    assert lo.request_id in so.preempted_req_ids
    assert any(x.req is hi for x in so.scheduled)
    s.update_from_output(so, {hi.request_id: [1]} if so.scheduled[0].will_sample else {})
    done = run_sync(s)
    assert len(done) == 2


def test_async_placeholders_match_sync_stream():
    def script(r):
        return 100 + len(r.output_token_ids)

    def drive(async_mode):
        s = make(async_mode=async_mode, budget=24)
        rs = [req(30, max_tokens=6), req(10, max_tokens=4), req(5, max_tokens=9)]
        for r in rs:
            s.add_request(r)
        out = {}
        pending = []
        for _ in range(200):
            if not s.has_unfinished() and not pending:
                break
            so = s.schedule() if s.has_unfinished() else None
            if so is not None and not so.is_empty:
                pending.append(so)
            if pending and (len(pending) >= (2 if async_mode else 1) or so is None or so.is_empty):
                so0 = pending.pop(0)
                toks = {x.req.request_id: [script(x.req)] for x in so0.scheduled
                        if x.will_sample and not x.req.finished}
                for o in s.update_from_output(so0, toks):
                    if o.finished:
                        out[o.request_id] = o.outputs[0].token_ids
        assert s.kv.pool.num_free_blocks == s.kv.pool.num_blocks
        return [out[r.request_id] for r in rs]

    assert drive(True) == drive(False)


def test_async_stop_token_and_abort_in_flight():
    s = make(async_mode=True)
    a = req(6, max_tokens=50, eos=42)
    b = req(6, max_tokens=50)
    s.add_request(a)
    s.add_request(b)
    so1 = s.schedule()
    so2 = s.schedule()                       # scheduled before so1's ids are known
    assert a.num_output_placeholders == 2
    outs = s.update_from_output(so1, {a.request_id: [42], b.request_id: [7]})   # a hits EOS
    assert any(o.finished and o.request_id == a.request_id for o in outs)
    s.abort_request(b.request_id)            # b aborted while so2 is in flight
    assert s.update_from_output(so2, {a.request_id: [1], b.request_id: [1]}) == []
    assert not s.has_unfinished()
    assert s.kv.pool.num_free_blocks == s.kv.pool.num_blocks


def test_spec_tokens_rollback_on_rejection():
    s = make()
    r = req(10, max_tokens=20)
    s.add_request(r)
    so = s.schedule()
    s.update_from_output(so, {r.request_id: [5]}, draft={r.request_id: [6, 7, 8]})
    so = s.schedule()
    assert so.scheduled[0].num_tokens == 4 and so.scheduled[0].spec_token_ids == [6, 7, 8]
    before = r.num_computed_tokens
    s.update_from_output(so, {r.request_id: [6, 9]})     # first draft accepted, second rejected
    assert r.output_token_ids == [5, 6, 9]
    assert r.num_computed_tokens == before - 2
    assert r.num_computed_tokens == r.num_tokens - 1


def test_preemption_by_swap_keeps_computed_tokens_and_returns_host_blocks():
    """With swap space a victim keeps its computed tokens: its blocks are copied out
    (swap_out pairs), it waits as SWAPPED, and comes back with swap_in pairs onto fresh blocks
    instead of recomputing the prompt."""
    sc = SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=128, max_model_len=512)
    cc = CacheConfig(block_size=16, enable_prefix_caching=False, num_cpu_blocks=16)
    s = Scheduler(sc, cc, 8)
    a, b = req(60, max_tokens=40), req(60, max_tokens=40)
    s.add_request(a)
    s.add_request(b)
    outs, ins, computed_after_prefill = [], [], 0
    done = {}
    for _ in range(500):
        if not s.has_unfinished():
            break
        so = s.schedule()
        outs += so.swap_out
        ins += so.swap_in
        for x in so.scheduled:
            # a request that was swapped out never re-runs its prompt
            if x.req.num_preemptions > 0 and x.req.status == RequestStatus.RUNNING:
                assert x.num_tokens == 1
        toks = {x.req.request_id: [7] for x in so.scheduled if x.will_sample}
        for o in s.update_from_output(so, toks):
            if o.finished:
                done[o.request_id] = o
    assert len(done) == 2 and all(len(o.outputs[0].token_ids) == 40 for o in done.values())
    assert s.num_swaps > 0 and s.stats()["num_swaps"] == s.num_swaps
    assert len(outs) == len(ins) > 0
    assert sorted(c for _, c in outs) == sorted(c for c, _ in ins)     # every host block returns
    assert sorted(s.cpu_free) == list(range(16))
    # an aborted swapped request gives its host blocks back
    s2 = Scheduler(sc, cc, 8)
    a, b = req(60, max_tokens=40), req(60, max_tokens=40)
    s2.add_request(a)
    s2.add_request(b)
    for _ in range(200):
        so = s2.schedule()
        s2.update_from_output(so, {x.req.request_id: [7] for x in so.scheduled if x.will_sample})
        victim = next((r for r in (a, b) if r.status == RequestStatus.SWAPPED), None)
        if victim is not None:
            break
    assert victim is not None and len(s2.cpu_free) < 16
    s2.abort_request(victim.request_id)
    assert sorted(s2.cpu_free) == list(range(16))
