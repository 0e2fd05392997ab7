"""Prefix-cache benchmark: the same long shared prefix with different suffixes, timed with the
prefix cache on and off (the reference ships benchmarks/benchmark_prefix_caching.py).

  python benchmarks/benchmark_prefix_caching.py --model tiny-llama --device cpu \
      --prefix-len 96 --suffix-len 8 --num-prompts 16 --output-len 4
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from vllm_gcu_b200.engine.llm import LLM  # noqa: E402
from vllm_gcu_b200.engine.request import SamplingParams  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--prefix-len", type=int, default=2048)
    ap.add_argument("--suffix-len", type=int, default=64)
    ap.add_argument("--num-prompts", type=int, default=64)
    ap.add_argument("--output-len", type=int, default=16)
    ap.add_argument("--dtype", default=None)
    a = ap.parse_args()
    res = {}
    for on in (False, True):
        llm = LLM(a.model, device=a.device, enable_prefix_caching=on, dtype=a.dtype,
                  max_model_len=a.prefix_len + a.suffix_len + a.output_len + 16)
        V = llm.engine.cfg.model.vocab_size
        g = torch.Generator().manual_seed(0)
        prefix = torch.randint(0, V, (a.prefix_len,), generator=g).tolist()
        prompts = [prefix + torch.randint(0, V, (a.suffix_len,), generator=g).tolist()
                   for _ in range(a.num_prompts)]
        sp = SamplingParams(max_tokens=a.output_len, temperature=0.0, ignore_eos=True)
        llm.generate(prompts[:1], sp)               # fills the cache with the shared prefix
        t0 = time.perf_counter()
        outs = llm.generate(prompts[1:], sp)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        st = llm.engine.scheduler.stats()
        res["cache_on" if on else "cache_off"] = {
            "seconds": dt, "cached_tokens": sum(o.num_cached_tokens for o in outs),
            "hits": st["prefix_cache_hits"], "queries": st["prefix_cache_queries"]}
    res["speedup"] = res["cache_off"]["seconds"] / max(res["cache_on"]["seconds"], 1e-9)
    print(json.dumps(res, indent=1))


if __name__ == "__main__":
    main()
