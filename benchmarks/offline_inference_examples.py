"""Feature smoke scripts (the reference ships offline_inference_with_prefix /
_chunked_prefill / _speculative_decoding and multilora_inference under benchmarks/):

  python benchmarks/offline_inference_examples.py prefix|chunked|spec|lora [--device cpu]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from vllm_gcu_b200.engine.llm import LLM  # noqa: E402
from vllm_gcu_b200.engine.request import SamplingParams  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["prefix", "chunked", "spec", "lora"])
    ap.add_argument("--model", default="tiny-llama")
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args()
    kw = dict(device=a.device, max_num_seqs=8, max_model_len=256, num_gpu_blocks=256,
              dtype="float32" if a.device == "cpu" else None)
    g = torch.Generator().manual_seed(0)
    sp = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
    if a.what == "prefix":
        llm = LLM(a.model, enable_prefix_caching=True, **kw)
        V = llm.engine.cfg.model.vocab_size
        shared = torch.randint(0, V, (64,), generator=g).tolist()
        first = llm.generate([shared + [1, 2, 3]], sp)       # computes and caches the prefix
        second = llm.generate([shared + [4, 5, 6]], sp)      # reuses its blocks
        print("cached tokens per request:",
              [first[0].num_cached_tokens, second[0].num_cached_tokens])
    elif a.what == "chunked":
        llm = LLM(a.model, max_num_batched_tokens=16, **kw)
        V = llm.engine.cfg.model.vocab_size
        outs = llm.generate([torch.randint(0, V, (100,), generator=g).tolist()], sp)
        print("engine steps:", llm.engine.stats["steps"], "tokens:", outs[0].outputs[0].token_ids)
    elif a.what == "spec":
        llm = LLM(a.model, speculative_method="ngram", num_speculative_tokens=3, **kw)
        outs = llm.generate([[7, 8, 9, 7, 8, 9, 7, 8, 9, 7, 8]], sp)
        m = llm.engine.spec_metrics
        print("tokens:", outs[0].outputs[0].token_ids, "acceptance rate:",
              round(m.acceptance_rate, 3), "mean accepted length:",
              round(m.mean_acceptance_length, 2))
    else:
        from vllm_gcu_b200.lora import LoRARequest
        llm = LLM(a.model, enable_lora=True, max_loras=2, max_lora_rank=8, **kw)
        mc = llm.engine.cfg.model
        r = 4
        tensors = {}
        for i in range(mc.num_hidden_layers):
            base = f"base_model.model.model.layers.{i}.self_attn.q_proj"
            tensors[base + ".lora_A.weight"] = torch.randn(r, mc.hidden_size, generator=g) * 0.5
            tensors[base + ".lora_B.weight"] = torch.randn(
                mc.num_attention_heads * mc.head_dim, r, generator=g) * 0.5
        llm.engine.add_lora(LoRARequest("demo", 1, ""), tensors,
                            {"r": r, "lora_alpha": 8, "target_modules": ["q_proj"]})
        lid = 1                                  # requests name the adapter by lora_int_id
        plain = llm.generate([[1, 2, 3, 4]], sp)[0].outputs[0].token_ids
        rid = llm.engine.add_request([1, 2, 3, 4], sp, lora_id=lid)
        tuned = None
        while llm.engine.has_unfinished():
            for o in llm.engine.step():
                if o.finished and o.request_id == rid:
                    tuned = o.outputs[0].token_ids
        print("base:", plain, "with adapter:", tuned)


if __name__ == "__main__":
    main()
