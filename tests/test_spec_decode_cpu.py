"""Speculative decoding on CPU: greedy outputs must be identical with and without drafts."""
import torch

from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams
from vllm_gcu_b200.ops import ref
from vllm_gcu_b200.spec import NgramProposer, RejectionSampler


def _run(model, n_out=24, **kw):
    torch.manual_seed(0)
    llm = LLM(model, device="cpu", block_size=16, max_num_seqs=8, max_num_batched_tokens=64,
              max_model_len=256, num_gpu_blocks=96, **kw)
    g = torch.Generator().manual_seed(2)
    V = llm.engine.cfg.model.vocab_size
    # repetitive prompts so that prompt lookup finds matches
    base = torch.randint(0, V, (12,), generator=g).tolist()
    prompts = [base * 3 + base[:5], base[::-1] * 2 + base[:3], base * 2]
    outs = llm.generate(prompts, SamplingParams(max_tokens=n_out, temperature=0.0, ignore_eos=True))
    return llm, [o.outputs[0].token_ids for o in outs]


def test_ngram_spec_decode_is_lossless_under_greedy():
    _, base = _run("tiny-llama")
    llm, spec = _run("tiny-llama", speculative_method="ngram", num_speculative_tokens=3)
    assert base == spec
    m = llm.engine.spec_metrics
    assert m.num_drafts > 0 and m.num_draft_tokens > 0
    assert 0.0 <= m.acceptance_rate <= 1.0


def test_mtp_spec_decode_is_lossless_under_greedy():
    _, base = _run("tiny-deepseek", n_out=12)
    llm, spec = _run("tiny-deepseek", n_out=12, speculative_method="mtp",
                     num_speculative_tokens=1)
    assert base == spec
    assert llm.engine.spec_metrics.num_drafts > 0


def test_rejection_sampler_oracles():
    rs = RejectionSampler()
    draft = torch.tensor([[5, 6, 7], [1, 2, 3], [9, 9, 9]], dtype=torch.int32)
    tgt = torch.tensor([[5, 6, 7, 8], [1, 4, 3, 2], [9, 9, 1, 0]])
    nd = torch.tensor([3, 3, 2], dtype=torch.int32)
    out = rs.greedy(draft, tgt, nd)
    assert out.tolist() == [[5, 6, 7, 8], [1, 4, -1, -1], [9, 9, 1, -1]]
    # random: target puts all mass on the draft token -> always accepted; zero mass -> rejected
    V = 11
    tp = torch.zeros(2, 2, V)
    tp[0, 0, 3] = 1.0
    tp[0, 1, 4] = 1.0
    tp[1, 0, 0] = 1.0           # draft token 7 has zero target probability
    tp[1, 1, 2] = 1.0
    d = torch.tensor([[3, 4], [7, 2]], dtype=torch.int32)
    out = rs.random(d, None, tp, torch.tensor([10, 10]), torch.tensor([2, 2], dtype=torch.int32))
    assert out[0].tolist() == [3, 4, 10]
    assert out[1].tolist() == [0, -1, -1]


def test_ngram_proposer():
    p = NgramProposer(3, 3, 1)
    assert p.propose([1, 2, 3, 9, 1, 2, 3]) == [9, 1, 2]
    assert p.propose([1, 2, 3]) == []


def test_medusa_and_mlp_speculator_heads_are_lossless_under_greedy():
    """Draft heads propose from the target's hidden state; whatever they propose, greedy
    verification keeps the output identical to plain decoding."""
    _, base = _run("tiny-llama", n_out=12)
    for method in ("medusa", "mlp_speculator"):
        llm, spec = _run("tiny-llama", n_out=12, speculative_method=method,
                         num_speculative_tokens=2)
        assert spec == base, method
        m = llm.engine.spec_metrics
        assert m.num_drafts > 0 and m.num_draft_tokens == 2 * m.num_drafts


def test_draft_heads_propose_shapes():
    from vllm_gcu_b200.spec import MedusaProposer, MLPSpeculatorProposer
    h = torch.randn(5, 64)
    last = torch.randint(0, 100, (5,))
    for cls in (MedusaProposer, MLPSpeculatorProposer):
        p = cls(64, 100, 3, dtype=torch.float32)
        p.init_random(1)
        out = p.propose(h, last)
        assert out.shape == (5, 3) and out.dtype == torch.int64
        sd = {k: v.clone() for k, v in p.state_dict().items()}
        q = cls(64, 100, 3, dtype=torch.float32)
        assert len(q.load_weights(sd.items())) == len(sd)
        assert torch.equal(q.propose(h, last), out)
