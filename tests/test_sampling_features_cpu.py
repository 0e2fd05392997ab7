"""Sampling extras of the engine on the CPU path: log-probabilities, prompt log-probabilities,
penalties, n / best_of and beam search (ReadMe-EN.md:283-292 and
docs/source/user_guide/support_matrix/supported_features.md:11-64 list them as supported)."""
import math

import torch

from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams


def _llm(**kw):
    return LLM("tiny-llama", device="cpu", max_num_seqs=8, max_num_batched_tokens=64,
               max_model_len=128, num_gpu_blocks=128, dtype="float32", **kw)


def _prompt(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 32000, (n,), generator=g).tolist()


def test_logprobs_and_prompt_logprobs_are_consistent():
    llm = _llm()
    p = _prompt(21, 1)
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True, logprobs=3,
                        prompt_logprobs=2)
    out = llm.generate([p], sp)[0]
    comp = out.outputs[0]
    assert len(comp.logprobs) == 5
    for tok, d in zip(comp.token_ids, comp.logprobs):
        assert tok in d and len(d) >= 3
        assert d[tok] == max(d.values())            # greedy: the sampled token is the arg-max
        assert all(v <= 1e-6 for v in d.values())
    assert math.isclose(comp.cumulative_logprob,
                        sum(d[t] for t, d in zip(comp.token_ids, comp.logprobs)), rel_tol=1e-6)
    assert out.prompt_logprobs[0] is None and len(out.prompt_logprobs) == len(p)
    for tok, d in zip(p[1:], out.prompt_logprobs[1:]):
        assert tok in d and d[tok] <= 1e-6
    # chunked prefill (budget 64 > 21 here; force chunks of 8) gives the same prompt logprobs
    llm2 = LLM("tiny-llama", device="cpu", max_num_seqs=8, max_num_batched_tokens=8,
               max_model_len=128, num_gpu_blocks=128, dtype="float32")
    out2 = llm2.generate([p], sp)[0]
    for a, b, tok in zip(out.prompt_logprobs[1:], out2.prompt_logprobs[1:], p[1:]):
        assert abs(a[tok] - b[tok]) < 1e-4
    assert out2.outputs[0].token_ids == comp.token_ids


def test_repetition_penalty_changes_greedy_choice_and_presence_blocks_repeats():
    llm = _llm()
    p = _prompt(12, 2)
    base = llm.generate([p], SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))[0]
    pen = llm.generate([p], SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True,
                                           presence_penalty=1e4))[0]
    toks = pen.outputs[0].token_ids
    assert len(set(toks)) == len(toks), "a huge presence penalty forbids repeating a token"
    assert len(base.outputs[0].token_ids) == 12


def test_n_best_of_and_beam_search():
    llm = _llm()
    p = _prompt(9, 3)
    outs = llm.generate([p], SamplingParams(max_tokens=4, temperature=1.0, n=2, best_of=4,
                                            ignore_eos=True, seed=5))[0]
    assert len(outs.outputs) == 2
    assert outs.outputs[0].cumulative_logprob >= outs.outputs[1].cumulative_logprob
    beam = llm.beam_search(p, beam_width=3, max_tokens=4, num_return=2)
    greedy = llm.generate([p], SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True,
                                              logprobs=0))[0]
    assert len(beam.outputs) == 2 and len(beam.outputs[0].token_ids) == 4
    # the best beam is at least as likely as the greedy continuation
    assert beam.outputs[0].cumulative_logprob >= greedy.outputs[0].cumulative_logprob - 1e-5


def test_allowed_tokens_and_guided_choice():
    llm = _llm()
    p = _prompt(10, 4)
    out = llm.generate([p], SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True,
                                           allowed_token_ids=(11, 22, 33)))[0]
    assert set(out.outputs[0].token_ids) <= {11, 22, 33}
    choices = ((5, 6, 7), (5, 9), (100, 101, 102, 103))
    out = llm.generate([p], SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True,
                                           guided_choice=choices))[0]
    toks = tuple(out.outputs[0].token_ids)
    assert toks in choices and out.outputs[0].finish_reason == "stop"


def test_text_prompts_and_chat_with_a_tokenizer():
    """``LLM(tokenizer=...)``: text prompts are encoded, completions carry ``text``, ``chat``
    renders conversations with the tokenizer's template."""
    class Tok:
        def encode(self, text):
            return [3 + b for b in text.encode()]

        def decode(self, ids):
            return bytes((i - 3) % 256 for i in ids).decode("latin-1")

        def apply_chat_template(self, conv, tokenize=True, add_generation_prompt=True):
            return self.encode("".join(f"<{m['role']}>{m['content']}" for m in conv) + "<assistant>")

    llm = _llm(tokenizer=Tok())
    sp = SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True)
    a = llm.generate("hello world", sp)[0]
    b = llm.generate([Tok().encode("hello world")], sp)[0]
    assert a.outputs[0].token_ids == b.outputs[0].token_ids
    assert a.outputs[0].text == Tok().decode(a.outputs[0].token_ids)
    c = llm.chat([{"role": "user", "content": "hi"}], sp)[0]
    assert c.prompt_token_ids == Tok().encode("<user>hi<assistant>") and len(c.outputs[0].text) == 4
    import pytest
    with pytest.raises(ValueError):
        _llm().generate("text without a tokenizer", sp)


def test_constraints_hold_with_ngram_drafts_in_the_same_batch():
    """A constrained request gets no draft tokens, and its mask is applied even when another
    request of the batch is verifying drafts in the same step."""
    llm = _llm(speculative_method="ngram", num_speculative_tokens=3)
    base = _prompt(8, 5)
    rep = base * 3                      # repetitive: the proposer finds drafts for it
    sps = [SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True),
           SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True,
                          allowed_token_ids=(5, 6, 7)),
           SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True,
                          guided_choice=((11, 12, 13, 14), (11, 15)))]
    outs = llm.generate([rep, rep, rep], sps)
    assert set(outs[1].outputs[0].token_ids) <= {5, 6, 7}
    assert tuple(outs[2].outputs[0].token_ids) in ((11, 12, 13, 14), (11, 15))
    assert llm.engine.spec_metrics.num_drafts > 0


def test_guided_request_added_while_async_steps_are_in_flight():
    """The engine retires the steps in flight before a request whose mask depends on its own
    history starts, and goes back to asynchronous scheduling when that request is gone."""
    llm = _llm(async_scheduling=True)
    eng = llm.engine
    bg = eng.add_request(_prompt(12, 6), SamplingParams(max_tokens=40, temperature=0.0,
                                                         ignore_eos=True))
    for _ in range(4):
        eng.step()
    assert eng._pending, "a step should be in flight"
    gid = eng.add_request(_prompt(9, 7), SamplingParams(
        max_tokens=8, temperature=0.0, ignore_eos=True, guided_choice=((11, 12, 13, 14),)))
    done = {}
    while eng.has_unfinished():
        for o in eng.step():
            if o.finished:
                done[o.request_id] = o
    assert list(done[gid].outputs[0].token_ids) == [11, 12, 13, 14]
    assert len(done[bg].outputs[0].token_ids) == 40
    assert eng.cfg.scheduler.async_scheduling and eng.scheduler.async_mode


def test_empty_prompt_is_rejected_and_does_not_block_the_queue():
    import pytest
    llm = _llm()
    eng = llm.engine
    with pytest.raises(ValueError):
        eng.add_request([], SamplingParams(max_tokens=4))
    out = llm.generate([_prompt(6, 8)], SamplingParams(max_tokens=4, temperature=0.0,
                                                       ignore_eos=True))[0]
    assert len(out.outputs[0].token_ids) == 4


def test_seeded_sampling_depends_on_the_request_only():
    """A request with a seed draws the same tokens whatever shares its steps and whether the
    engine schedules ahead of its results or not: the draw of its i-th token is a function of
    (seed, i) alone."""
    sp = SamplingParams(max_tokens=10, temperature=0.9, top_p=0.95, top_k=50, seed=11,
                        ignore_eos=True)
    other = SamplingParams(max_tokens=7, temperature=1.2, seed=3, ignore_eos=True)
    p, q, r = _prompt(17, 2), _prompt(40, 3), _prompt(5, 4)
    llm = _llm()
    alone = llm.generate([p], sp)[0].outputs[0].token_ids
    mixed = llm.generate([q, p, r], [other, sp, other])[1].outputs[0].token_ids
    assert alone == mixed and len(alone) == 10
    ahead = _llm(async_scheduling=True).generate([q, p, r], [other, sp, other])
    assert ahead[1].outputs[0].token_ids == alone
    different = llm.generate([p], SamplingParams(max_tokens=10, temperature=0.9, top_p=0.95,
                                                 top_k=50, seed=12, ignore_eos=True))
    assert different[0].outputs[0].token_ids != alone


def test_token_ids_outside_the_vocabulary_are_refused():
    import pytest
    llm = _llm()
    sp = SamplingParams(max_tokens=2, temperature=0.0, ignore_eos=True)
    for bad in ([1, 2, 32000], [5, -1]):
        with pytest.raises(ValueError, match="vocabulary"):
            llm.engine.add_request(bad, sp)
    with pytest.raises(ValueError, match="max_tokens"):
        llm.engine.add_request([1, 2], SamplingParams(max_tokens=0))
    out = llm.generate([[1, 2, 31999]], sp)[0]            # the engine is unharmed
    assert len(out.outputs[0].token_ids) == 2


def test_mask_ids_and_adapters_are_checked_at_admission():
    import pytest
    llm = _llm()
    for sp in (SamplingParams(max_tokens=2, allowed_token_ids=(5, 40000)),
               SamplingParams(max_tokens=2, guided_choice=((1, 2), (3, -7)))):
        with pytest.raises(ValueError, match="token ids"):
            llm.engine.add_request([1, 2, 3], sp)
    with pytest.raises(ValueError, match="LoRA"):
        llm.engine.add_request([1, 2, 3], SamplingParams(max_tokens=2), lora_id=3)
    assert not llm.engine.has_unfinished()


def test_out_of_range_sampling_values_are_normalised():
    llm = _llm()
    p = _prompt(9, 1)
    ref_ = llm.generate([p], SamplingParams(max_tokens=4, temperature=0.8, seed=1,
                                            ignore_eos=True))[0].outputs[0].token_ids
    wild = llm.generate([p], SamplingParams(max_tokens=4, temperature=0.8, seed=1, top_k=10 ** 9,
                                            top_p=7.0, ignore_eos=True))[0].outputs[0].token_ids
    off = llm.generate([p], SamplingParams(max_tokens=4, temperature=0.8, seed=1, top_k=-1,
                                           top_p=1.0, ignore_eos=True))[0].outputs[0].token_ids
    assert ref_ == wild == off
    cold = llm.generate([p], SamplingParams(max_tokens=4, temperature=float("nan"),
                                            ignore_eos=True))[0].outputs[0].token_ids
    greedy = llm.generate([p], SamplingParams(max_tokens=4, temperature=0.0,
                                              ignore_eos=True))[0].outputs[0].token_ids
    assert cold == greedy
    tiny = llm.generate([p], SamplingParams(max_tokens=4, temperature=0.8, seed=1, top_p=0.0,
                                            ignore_eos=True))[0].outputs[0].token_ids
    assert len(tiny) == 4
