"""The CPU configuration of the baseline list: a tiny Llama (2 layers, hidden 256, 4 query /
2 KV heads of 64, FFN 688, vocabulary 32000, fp32, seed 0) through the engine with a paged KV
cache of block size 16; four prompts of 32 uniform-random token ids, 16 greedy tokens each.
Reports the largest absolute difference between the engine's logits (paged cache, prefill
then decode steps) and a dense forward without a cache over the same tokens, whether every
generated token is the dense arg-max, and tokens per second (informational: torch on CPU).

Usage: python benchmarks/tiny_llama_cpu.py
"""
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from vllm_gcu_b200.engine.llm import LLM  # noqa: E402
from vllm_gcu_b200.engine.request import SamplingParams  # noqa: E402
from vllm_gcu_b200.ops import ref  # noqa: E402


def dense_logits(model, ids: torch.Tensor) -> torch.Tensor:
    """No-cache forward of the same weights: logits ``[S, V]``."""
    cfg = model.cfg
    S = ids.shape[0]
    x = model.embed_tokens.weight[ids]
    pos = torch.arange(S)
    residual = None
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    for i in range(cfg.num_hidden_layers):
        layer = model.layers[str(i)]
        if residual is None:
            residual, h = x, ref.rms_norm(x, layer.input_layernorm.weight, cfg.rms_norm_eps)
        else:
            h, residual = ref.fused_add_rms_norm(x, residual, layer.input_layernorm.weight,
                                                 cfg.rms_norm_eps)
        att = layer.self_attn
        q, k, v = (h @ att.qkv_proj.weight.t()).split([Hq * D, Hkv * D, Hkv * D], -1)
        q, k = ref.rotary_embedding(pos, q, k, D, att.attn.rotary.cos_sin_cache, True)
        o = ref.dense_causal_attention(q.view(S, Hq, D), k.view(S, Hkv, D), v.view(S, Hkv, D),
                                       D ** -0.5).reshape(S, Hq * D)
        h, residual = ref.fused_add_rms_norm(o @ att.o_proj.weight.t(), residual,
                                             layer.post_attention_layernorm.weight,
                                             cfg.rms_norm_eps)
        x = ref.silu_and_mul(h @ layer.mlp.gate_up_proj.weight.t()) @ layer.mlp.down_proj.weight.t()
    x, _ = ref.fused_add_rms_norm(x, residual, model.norm.weight, cfg.rms_norm_eps)
    return x @ model.lm_head.weight[: cfg.vocab_size].t()


def main():
    torch.manual_seed(0)
    llm = LLM("tiny-llama", device="cpu", block_size=16, max_num_seqs=8,
              max_num_batched_tokens=128, max_model_len=256, num_gpu_blocks=64, seed=0)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 32000, (32,), generator=g).tolist() for _ in range(4)]
    llm.engine.runner.keep_logits = True
    sp = SamplingParams(max_tokens=16, temperature=0.0, ignore_eos=True)
    t0 = time.perf_counter()
    outs = llm.generate(prompts, sp)
    dt = time.perf_counter() - t0
    model = llm.engine.model
    all_argmax = True
    worst = 0.0
    for p, o in zip(prompts, outs):
        toks = o.outputs[0].token_ids
        dense = dense_logits(model, torch.tensor(p + toks)[:-1])
        all_argmax &= dense[len(p) - 1:].argmax(-1).tolist() == toks
    # logits of the engine's last step (one decode row per request, in request order) against
    # the dense rows
    last = llm.engine.runner.last_logits
    for i in range(last.shape[0]):
        r = i
        full = torch.tensor(prompts[i] + outs[i].outputs[0].token_ids)
        dense = dense_logits(model, full[:-1])[-1]
        worst = max(worst, float((last[r].float() - dense).abs().max()))
    print(json.dumps({"config": "tiny llama, CPU, fp32, block 16, 4 x 32 in / 16 out",
                      "max_abs_logit_error": worst, "all_tokens_are_dense_argmax": all_argmax,
                      "output_tokens_per_s": 64 / dt}))


if __name__ == "__main__":
    main()
