"""Offline data-parallel generation: one engine replica per DP rank, requests spread over
the replicas, all replicas stepping together (idle ones run a zero-token forward so that
expert-parallel collectives line up).  The reference's ``dpllm`` does this with one Ray actor
per rank and a fake one-token request for idle ranks (benchmarks/dpllm.py:57-94); here the
multi-process executor has it built in.

  python benchmarks/dpllm.py --model tiny-qwen3-moe --dp 2 --device cpu --num-prompts 8
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from vllm_gcu_b200.config import (CacheConfig, EngineConfig, ParallelConfig,  # noqa: E402
                                  SchedulerConfig, preset)
from vllm_gcu_b200.engine.executor import MultiprocExecutor  # noqa: E402
from vllm_gcu_b200.engine.request import SamplingParams  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-qwen3-moe")
    ap.add_argument("--dp", type=int, default=2)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--num-prompts", type=int, default=16)
    ap.add_argument("--input-len", type=int, default=32)
    ap.add_argument("--output-len", type=int, default=16)
    ap.add_argument("--expert-parallel", action="store_true")
    a = ap.parse_args()
    mc = preset(a.model)
    if a.expert_parallel:
        mc.extra["dp_attention"] = True
    cfg = EngineConfig(model=mc, cache=CacheConfig(block_size=16),
                       scheduler=SchedulerConfig(max_num_seqs=64, max_num_batched_tokens=2048,
                                                 max_model_len=a.input_len + a.output_len + 16),
                       parallel=ParallelConfig(tensor_parallel_size=a.tp,
                                               data_parallel_size=a.dp,
                                               enable_expert_parallel=a.expert_parallel,
                                               comm_backend="nccl"),
                       device=a.device if a.device != "auto" else
                       ("cuda" if torch.cuda.is_available() else "cpu"))
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, mc.vocab_size, (a.num_prompts, a.input_len), generator=g).tolist()
    sp = SamplingParams(max_tokens=a.output_len, temperature=0.0, ignore_eos=True)
    ex = MultiprocExecutor(cfg)
    try:
        t0 = time.perf_counter()
        outs = ex.generate(prompts, sp)
        dt = time.perf_counter() - t0
    finally:
        ex.shutdown()
    n = sum(len(o.outputs[0].token_ids) for o in outs)
    print(json.dumps({"requests": len(outs), "output_tokens": n, "seconds": dt,
                      "output_tokens_per_s": n / dt, "dp": a.dp, "tp": a.tp}))


if __name__ == "__main__":
    main()
