"""Fixed-batch latency: one batch of identical-length requests, repeated; reports mean and
percentiles of the end-to-end batch latency (benchmarks/benchmark_latency.py:21-159).

Example: python benchmarks/benchmark_latency.py --model llama-3-8b --batch-size 8 \
             --input-len 32 --output-len 128 --num-iters 10
"""
import argparse
import json
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from vllm_gcu_b200.engine.llm import LLM  # noqa: E402
from vllm_gcu_b200.engine.request import SamplingParams  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--input-len", type=int, default=32)
    ap.add_argument("--output-len", type=int, default=128)
    ap.add_argument("--num-iters-warmup", type=int, default=3)
    ap.add_argument("--num-iters", type=int, default=10)
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--num-hidden-layers", type=int, default=0)
    a = ap.parse_args()
    kw = {"num_hidden_layers": a.num_hidden_layers} if a.num_hidden_layers else {}
    llm = LLM(a.model, tensor_parallel_size=a.tensor_parallel_size,
              max_num_seqs=max(a.batch_size, 8),
              max_num_batched_tokens=max(a.batch_size * a.input_len, 2048),
              max_model_len=a.input_len + a.output_len + 16, device=a.device,
              enable_prefix_caching=False, **kw)
    V = llm.engine.cfg.model.vocab_size
    sp = SamplingParams(max_tokens=a.output_len, temperature=0.0, ignore_eos=True)
    lat = []
    for it in range(a.num_iters_warmup + a.num_iters):
        g = torch.Generator().manual_seed(it)
        prompts = torch.randint(0, V, (a.batch_size, a.input_len), generator=g).tolist()
        t0 = time.perf_counter()
        llm.generate(prompts, sp)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if it >= a.num_iters_warmup:
            lat.append(time.perf_counter() - t0)
    lat = np.array(lat)
    res = {"avg_latency_s": float(lat.mean()),
           "percentiles_s": {str(p): float(np.percentile(lat, p)) for p in (10, 25, 50, 75, 90, 99)},
           "tpot_ms": float(lat.mean() / a.output_len * 1e3)}
    print(json.dumps(res, indent=1))


if __name__ == "__main__":
    main()
