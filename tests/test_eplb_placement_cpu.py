"""Redundant experts with a static placement file (``expert_map_path`` of the reference,
vllm_gcu/models/deepseek_v3/deepseek_v3.py:880-913): checkpoint tensors of a logical expert
reach every physical replica, and the model computes what the model without replicas does."""
import torch

from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams


def _llm(**extra):
    return LLM("tiny-qwen3-moe", device="cpu", dtype="float32", max_num_seqs=4,
               max_num_batched_tokens=64, max_model_len=128, num_gpu_blocks=32,
               extra=extra or {})


def test_static_placement_loads_replicas_and_matches_the_plain_model(tmp_path):
    plain = _llm()
    cfg = plain.engine.cfg.model
    E, L = cfg.num_experts, cfg.num_hidden_layers
    n_moe = sum(cfg.is_moe_layer(i) for i in range(L))
    g = torch.Generator().manual_seed(0)
    # every layer its own placement: a permutation of the logical experts plus two replicas
    table = torch.stack([torch.cat([torch.randperm(E, generator=g),
                                    torch.randint(0, E, (2,), generator=g)]) for _ in range(n_moe)])
    path = tmp_path / "expert_map.pt"
    torch.save((table.view(n_moe, 1, E + 2), torch.zeros(1)), path)
    red = _llm(num_redundant_experts=2, expert_map_path=str(path))
    src, dst = plain.engine.model, red.engine.model
    sd = src.state_dict()
    dst.load_state_dict({k: v for k, v in sd.items() if ".experts." not in k}, strict=False)
    I = cfg.moe_intermediate_size
    for name, layer in src.layers.items():
        if not hasattr(layer.mlp, "experts"):
            continue
        a, b = layer.mlp.experts, dst.layers[name].mlp.experts
        assert b.w13.shape[0] == E + 2
        for e in range(E):
            assert b.load_expert_weight(e, "gate", a.w13.data[e, :I])
            b.load_expert_weight(e, "up", a.w13.data[e, I:])
            b.load_expert_weight(e, "down", a.w2.data[e])
        li = int(name) - int(cfg.first_k_dense_replace or 0)
        for p, l in enumerate(table[li].tolist()):          # every replica holds its expert
            assert torch.equal(b.w13.data[p], a.w13.data[l])
            assert torch.equal(b.w2.data[p], a.w2.data[l])
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (19, 7, 30)]
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    plain.engine.runner.keep_logits = red.engine.runner.keep_logits = True
    want = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    got = [o.outputs[0].token_ids for o in red.generate(prompts, sp)]
    assert got == want
    assert torch.allclose(red.engine.runner.last_logits, plain.engine.runner.last_logits, atol=1e-4)


def test_moe_chunking_gives_the_same_result(monkeypatch):
    """``VLLM_FUSED_MOE_CHUNK_SIZE``: the routed-expert MLP over chunks of token rows equals the
    unchunked computation (vllm_gcu/kernels/modular_kernel.py:167-286)."""
    llm = _llm()
    moe = next(l.mlp.experts for l in llm.engine.model.layers.values() if hasattr(l.mlp, "experts"))
    cfg = llm.engine.cfg.model
    g = torch.Generator().manual_seed(3)
    T = 37
    x = torch.randn(T, cfg.hidden_size, generator=g)
    tw, ti = torch.topk(torch.softmax(torch.randn(T, cfg.num_experts, generator=g), -1),
                        cfg.num_experts_per_tok, dim=-1)
    add = torch.randn(T, cfg.hidden_size, generator=g)
    want = moe(x, tw, ti.to(torch.int32), add=add)
    monkeypatch.setenv("VLLM_FUSED_MOE_CHUNK_SIZE", "8")
    got = moe(x, tw, ti.to(torch.int32), add=add)
    assert torch.allclose(got, want, atol=1e-5)
