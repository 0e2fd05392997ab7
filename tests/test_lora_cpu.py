"""Multi-LoRA on CPU: a batch mixing two adapters and no adapter must equal running each
request alone with merged weights."""
import torch

from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams
from vllm_gcu_b200.lora import LoRARequest, bgmv_expand_slice, bgmv_shrink
from vllm_gcu_b200.ops import ref


def _adapter(cfg, seed, r=4):
    g = torch.Generator().manual_seed(seed)
    H, I = cfg.hidden_size, cfg.intermediate_size
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    shapes = {"self_attn.q_proj": (Hq * D, H), "self_attn.k_proj": (Hkv * D, H),
              "self_attn.v_proj": (Hkv * D, H), "self_attn.o_proj": (H, Hq * D),
              "mlp.gate_proj": (I, H), "mlp.up_proj": (I, H), "mlp.down_proj": (H, I)}
    t = {}
    for l in range(cfg.num_hidden_layers):
        for name, (o, i) in shapes.items():
            base = f"base_model.model.model.layers.{l}.{name}"
            t[base + ".lora_A.weight"] = torch.randn(r, i, generator=g) * 0.05
            t[base + ".lora_B.weight"] = torch.randn(o, r, generator=g) * 0.05
    return t, {"r": r, "lora_alpha": 2 * r}


def _merged_llm(tensors, conf):
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, max_num_batched_tokens=64,
              max_model_len=128, num_gpu_blocks=32)
    scale = conf["lora_alpha"] / conf["r"]
    model = llm.engine.model
    cfg = model.cfg
    D, Hq, Hkv, I = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, \
        cfg.intermediate_size
    for l in range(cfg.num_hidden_layers):
        layer = model.layers[str(l)]
        pre = f"base_model.model.model.layers.{l}."

        def delta(n):
            return scale * tensors[pre + n + ".lora_B.weight"] @ tensors[pre + n + ".lora_A.weight"]
        w = layer.self_attn.qkv_proj.weight.data
        w[:Hq * D] += delta("self_attn.q_proj")
        w[Hq * D:Hq * D + Hkv * D] += delta("self_attn.k_proj")
        w[Hq * D + Hkv * D:] += delta("self_attn.v_proj")
        layer.self_attn.o_proj.weight.data += delta("self_attn.o_proj")
        layer.mlp.gate_up_proj.weight.data[:I] += delta("mlp.gate_proj")
        layer.mlp.gate_up_proj.weight.data[I:] += delta("mlp.up_proj")
        layer.mlp.down_proj.weight.data += delta("mlp.down_proj")
    return llm


def test_multi_lora_batch_matches_merged_weights():
    torch.manual_seed(0)
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, max_num_batched_tokens=64,
              max_model_len=128, num_gpu_blocks=32, enable_lora=True, max_loras=2,
              max_lora_rank=8)
    cfg = llm.engine.cfg.model
    a1, c1 = _adapter(cfg, 1)
    a2, c2 = _adapter(cfg, 2, r=8)
    llm.engine.add_lora(LoRARequest("a1", 1, ""), a1, c1)
    llm.engine.add_lora(LoRARequest("a2", 2, ""), a2, c2)
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, 32000, (20,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    ids = [llm.engine.add_request(p, sp, lora_id=l) for p, l in zip(prompts, (1, -1, 2))]
    final = {}
    while llm.engine.has_unfinished():
        for o in llm.engine.step():
            if o.finished:
                final[o.request_id] = o.outputs[0].token_ids
    base = LLM("tiny-llama", device="cpu", max_num_seqs=4, max_num_batched_tokens=64,
               max_model_len=128, num_gpu_blocks=32)
    want_plain = base.generate([prompts[1]], sp)[0].outputs[0].token_ids
    want1 = _merged_llm(a1, c1).generate([prompts[0]], sp)[0].outputs[0].token_ids
    want2 = _merged_llm(a2, c2).generate([prompts[2]], sp)[0].outputs[0].token_ids
    assert final[ids[1]] == want_plain
    assert final[ids[0]] == want1
    assert final[ids[2]] == want2


def test_bgmv_ops_reference():
    torch.manual_seed(1)
    T, hin, r, hout, Lw = 6, 32, 4, 24, 3
    x = torch.randn(T, hin)
    A = torch.randn(Lw, r, hin)
    Bm = torch.randn(Lw, hout, r)
    idx = torch.tensor([0, 2, -1, 1, 1, 0], dtype=torch.int32)
    buf = torch.zeros(T, r)
    bgmv_shrink(x, A, buf, idx, 0.5)
    y = torch.ones(T, 40)
    bgmv_expand_slice(buf, Bm, y, idx, 8, hout)
    for t in range(T):
        want = torch.ones(40)
        if idx[t] >= 0:
            want[8:8 + hout] += Bm[idx[t]] @ (0.5 * A[idx[t]] @ x[t])
        assert torch.allclose(y[t], want, atol=1e-5)
