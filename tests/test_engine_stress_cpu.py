"""Randomised engine runs on the CPU path: staggered arrivals, random priorities, aborts, small
KV pools that force pre-emption (by recomputation or by swapping), prefix caching, chunked
prefill, asynchronous and multi-step scheduling in random combinations.  Every request that
was not aborted must produce exactly the tokens of an engine with ample cache that runs all
prompts at once, and every KV block must be free again at the end."""
import random

import pytest
import torch

from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams

def reference(prompts, sps):
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=16, max_num_batched_tokens=256, max_model_len=256,
              num_gpu_blocks=512, dtype="float32", enable_prefix_caching=False)
    return [o.outputs[0].token_ids for o in llm.generate(prompts, sps)]

def trial(seed):
    rng = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    n = rng.randint(4, 10)
    shared = torch.randint(0, 32000, (rng.randint(16, 48),), generator=g).tolist()
    prompts = []
    for i in range(n):
        body = torch.randint(0, 32000, (rng.randint(3, 60),), generator=g).tolist()
        prompts.append((shared + body) if rng.random() < 0.4 else body)
    sps = [SamplingParams(max_tokens=rng.randint(1, 24), temperature=0.0, ignore_eos=True) for _ in prompts]
    want = reference(prompts, sps)
    kw = dict(max_num_seqs=rng.choice([2, 4, 8]), max_num_batched_tokens=rng.choice([16, 32, 64]),
              num_gpu_blocks=rng.choice([10, 14, 24, 64]), num_cpu_blocks=rng.choice([0, 0, 16]),
              enable_prefix_caching=rng.random() < 0.6, async_scheduling=rng.random() < 0.5,
              scheduling_policy=rng.choice(["fcfs", "priority"]), num_scheduler_steps=rng.choice([1, 1, 3]))
    if kw["async_scheduling"] and kw["num_scheduler_steps"] > 1:
        kw["num_scheduler_steps"] = 1
    llm = LLM("tiny-llama", device="cpu", max_model_len=256, dtype="float32", **kw)
    eng = llm.engine
    free0 = eng.scheduler.kv.pool.num_free_blocks
    # staggered arrivals, random priorities, a few aborts
    pending = list(range(n)); rng.shuffle(pending)
    ids = {}; aborted = set(); got = {}
    steps = 0
    while pending or eng.has_unfinished():
        for _ in range(rng.randint(0, 2)):
            if pending:
                i = pending.pop()
                ids[eng.add_request(prompts[i], sps[i], priority=rng.randint(0, 3))] = i
        if ids and rng.random() < 0.05:
            rid = rng.choice(list(ids))
            if ids[rid] not in got and ids[rid] not in aborted:
                eng.abort_request(rid); aborted.add(ids[rid])
        for o in eng.step():
            if o.finished:
                got[ids[o.request_id]] = o.outputs[0].token_ids
        steps += 1
        if steps > 5000:
            raise AssertionError(f"no progress after {steps} steps: {kw}")
    # drain async leftovers
    for _ in range(4):
        eng.step()
    for i in range(n):
        if i not in aborted:
            assert got.get(i) == want[i], (i, kw)
    assert eng.scheduler.kv.pool.num_free_blocks == free0, kw
    if kw["num_cpu_blocks"]:
        assert sorted(eng.scheduler.cpu_free) == list(range(kw["num_cpu_blocks"])), kw


@pytest.mark.timeout(600)
@pytest.mark.parametrize("seed", [0, 3, 4, 8, 11, 17, 23, 42])
def test_random_engine_schedules_reproduce_the_reference_tokens(seed):
    trial(seed)
