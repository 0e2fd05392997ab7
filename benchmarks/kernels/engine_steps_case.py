"""A short engine run for per-kernel launch lists of whole decode / prefill steps.

  VLLM_B200_NVTX=1 python benchmarks/kernels/engine_steps_case.py --batch 256 --input-len 1024 \
      --output-len 6

With the NVTX flag every engine step is wrapped in a range named decode_step, prefill_step or
mixed_step, so Nsight Compute can list the kernels of one kind of step with their device time
(one metric, one pass, nothing saved or restored):

  ncu --metrics gpu__time_duration.sum --clock-control none --nvtx \
      --nvtx-include "decode_step/" -c 700 --csv --log-file <output dir>/decode_launches.csv \
      python benchmarks/kernels/engine_steps_case.py --batch 256 --input-len 1024 --output-len 4
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from vllm_gcu_b200.engine.llm import LLM  # noqa: E402
from vllm_gcu_b200.engine.request import SamplingParams  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=6)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = model's)")
    ap.add_argument("--eager", action="store_true")
    a = ap.parse_args()
    kw = {"num_hidden_layers": a.layers} if a.layers else {}
    llm = LLM(a.model, max_num_seqs=a.batch, max_num_batched_tokens=8192,
              max_model_len=a.input_len + a.output_len + 16, async_scheduling=True,
              enforce_eager=a.eager, load_format="dummy", cuda_graph_sizes=[a.batch],
              num_gpu_blocks=(a.batch * (a.input_len + a.output_len + 32)) // 16 + 64, **kw)
    g = torch.Generator().manual_seed(0)
    vocab = llm.engine.cfg.model.vocab_size
    prompts = [torch.randint(0, vocab, (a.input_len,), generator=g).tolist()
               for _ in range(a.batch)]
    sp = SamplingParams(max_tokens=a.output_len, temperature=0.0, ignore_eos=True)
    t0 = time.time()
    outs = llm.generate(prompts, sp)
    torch.cuda.synchronize()
    print(f"ok {len(outs)} requests, {time.time() - t0:.2f} s")


if __name__ == "__main__":
    main()
