"""Randomised engine runs with per-request sampling features on the CPU path: penalties,
allowed-token masks, guided choices, log-probabilities and seeded sampling, mixed in one batch,
with n-gram draft tokens, asynchronous scheduling, small KV pools and staggered arrivals in
random combinations.  Tokens and log-probabilities must equal those of a plain synchronous
engine that runs all prompts at once."""
import random

import pytest
import torch

from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams

def mk_sp(rng, allow_seeded):
    kind = rng.choice(["plain", "plain", "penalty", "allowed", "logprobs", "choice", "seeded" if allow_seeded else "plain", "minp"])
    mt = rng.randint(1, 16)
    if kind == "penalty":
        return SamplingParams(max_tokens=mt, temperature=0.0, ignore_eos=True, repetition_penalty=1.0 + rng.random(), presence_penalty=rng.random(), frequency_penalty=rng.random() * 0.5)
    if kind == "allowed":
        return SamplingParams(max_tokens=mt, temperature=0.0, ignore_eos=True, allowed_token_ids=tuple(rng.sample(range(32000), 5)))
    if kind == "logprobs":
        return SamplingParams(max_tokens=mt, temperature=0.0, ignore_eos=True, logprobs=rng.randint(0, 3))
    if kind == "choice":
        c = tuple(tuple(rng.sample(range(100, 200), rng.randint(2, 4))) for _ in range(3))
        return SamplingParams(max_tokens=8, temperature=0.0, guided_choice=c)
    if kind == "seeded":
        return SamplingParams(max_tokens=mt, temperature=0.8, top_k=rng.choice([0, 20]), top_p=rng.choice([1.0, 0.9]), seed=rng.randint(0, 99), ignore_eos=True)
    return SamplingParams(max_tokens=mt, temperature=0.0, ignore_eos=True)

def run(prompts, sps, rng, **kw):
    llm = LLM("tiny-llama", device="cpu", max_model_len=256, dtype="float32", **kw)
    eng = llm.engine
    if rng is None:
        return [(o.outputs[0].token_ids, o.outputs[0].logprobs) for o in llm.generate(prompts, sps)]
    pending = list(range(len(prompts))); rng.shuffle(pending)
    ids, got, steps = {}, {}, 0
    while pending or eng.has_unfinished():
        for _ in range(rng.randint(0, 2)):
            if pending:
                i = pending.pop(); ids[eng.add_request(prompts[i], sps[i])] = i
        for o in eng.step():
            if o.finished: got[ids[o.request_id]] = (o.outputs[0].token_ids, o.outputs[0].logprobs)
        steps += 1
        assert steps < 5000
    return [got[i] for i in range(len(prompts))]

def trial(seed):
    rng = random.Random(seed)
    g = torch.Generator().manual_seed(seed)
    n = rng.randint(3, 8)
    spec = rng.random() < 0.5
    prompts = []
    for i in range(n):
        if rng.random() < 0.4:
            pat = torch.randint(0, 32000, (rng.randint(2, 5),), generator=g).tolist()
            prompts.append(pat * rng.randint(3, 8))
        else:
            prompts.append(torch.randint(0, 32000, (rng.randint(3, 50),), generator=g).tolist())
    sps = [mk_sp(rng, not spec) for _ in prompts]
    want = run(prompts, sps, None, max_num_seqs=16, max_num_batched_tokens=256, num_gpu_blocks=512)
    kw = dict(max_num_seqs=rng.choice([2, 4, 8]), max_num_batched_tokens=rng.choice([16, 32, 64]),
              num_gpu_blocks=rng.choice([16, 24, 64]), async_scheduling=rng.random() < 0.5)
    if spec:
        kw.update(speculative_method="ngram", num_speculative_tokens=rng.randint(1, 3))
    got = run(prompts, sps, rng, **kw)
    for i, (a, b) in enumerate(zip(got, want)):
        assert a[0] == b[0], (i, sps[i], kw)
        assert (a[1] is None) == (b[1] is None), (i, kw)
        for da, db, t in zip(a[1] or [], b[1] or [], a[0]):
            assert abs(da[t] - db[t]) < 1e-3, (i, kw)


@pytest.mark.timeout(600)
@pytest.mark.parametrize("seed", [0, 2, 4, 5, 9, 13, 21, 34])
def test_random_feature_mixes_reproduce_the_reference(seed):
    trial(seed)
