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


def test_eagle_spec_decode_is_lossless_and_loads_its_checkpoint(tmp_path):
    """EAGLE draft head (fc + one decoder layer without input norm, target's embedding and LM
    head): greedy outputs are those of the target alone; a head whose weights make it repeat
    the target's own next-token computation is loaded from a checkpoint in the EAGLE layout."""
    from vllm_gcu_b200.spec import EagleDrafter
    from vllm_gcu_b200.utils.weights import write_safetensors
    _, base = _run("tiny-llama", n_out=12)
    llm, spec = _run("tiny-llama", n_out=12, speculative_method="eagle",
                     num_speculative_tokens=1)
    assert base == spec
    m = llm.engine.spec_metrics
    assert m.num_drafts > 0
    d = llm.engine.runner.drafter
    assert isinstance(d, EagleDrafter) and len(llm.engine.runner.drafter_caches) == 1
    # checkpoint round trip in the EAGLE layout (q / k / v and gate / up as separate tensors)
    cfg = llm.engine.cfg.model
    D, Hq, Hkv, I = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, \
        cfg.intermediate_size
    sd = {}
    for name, p in d.state_dict().items():
        if ".qkv_proj.weight" in name:
            q, k, v = p.split([Hq * D, Hkv * D, Hkv * D], 0)
            for n, t in (("q_proj", q), ("k_proj", k), ("v_proj", v)):
                sd[name.replace("qkv_proj", n)] = t.clone() + 0.01
        elif ".gate_up_proj.weight" in name:
            g, u = p.split([I, I], 0)
            sd[name.replace("gate_up_proj", "gate_proj")] = g.clone() + 0.01
            sd[name.replace("gate_up_proj", "up_proj")] = u.clone() + 0.01
        elif "input_layernorm" not in name:
            sd[name] = p.clone() + 0.01
    sd["embed_tokens.weight"] = torch.zeros(4, 4)            # ignored: the target's is shared
    write_safetensors(str(tmp_path / "model.safetensors"), sd)
    before = {k: v.clone() for k, v in d.state_dict().items()}
    llm2, spec2 = _run("tiny-llama", n_out=12, speculative_method="eagle",
                       num_speculative_tokens=1, speculative_model=str(tmp_path))
    assert spec2 == base
    after = llm2.engine.runner.drafter.state_dict()
    for k, v in before.items():
        if "input_layernorm" in k:
            continue
        assert torch.allclose(after[k], v + 0.01, atol=1e-6), k
