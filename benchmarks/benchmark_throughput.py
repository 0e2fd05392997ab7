"""Offline throughput: all requests submitted up front, ``ignore_eos``, fixed lengths.
Reports requests/s, total tokens/s and output tokens/s (the reference's
benchmarks/benchmark_throughput.py:448-450 protocol on the built-in engine).

Example: python benchmarks/benchmark_throughput.py --model llama-3-8b --num-prompts 512 \
             --input-len 1024 --output-len 256

Several GPUs (one process per GPU; tensor-parallel attention, experts spread over the ranks):
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/benchmark_throughput.py --model qwen3-30b-a3b --tensor-parallel-size 8 \
        --enable-expert-parallel --num-prompts 256 --input-len 2048 --output-len 512
Every rank runs the same requests; the elapsed time is the maximum over ranks and rank 0 prints.
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
    ap.add_argument("--num-prompts", type=int, default=512)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--enable-expert-parallel", action="store_true")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--num-hidden-layers", type=int, default=0)
    ap.add_argument("--output-json", default=None)
    ap.add_argument("--quantization", default=None, choices=[None, "fp8", "fp8_block", "w8a8"],
                    help="random-init quantised weights: fp8 per-channel, fp8 with 128 x 128 "
                         "blocks (DeepSeek-V3 layout), or int8 w8a8")
    a = ap.parse_args()
    kw = {"num_hidden_layers": a.num_hidden_layers} if a.num_hidden_layers else {}
    if a.quantization == "fp8_block":
        kw.update(quantization="fp8", quant_config={"quant_method": "fp8",
                                                    "weight_block_size": [128, 128]})
    elif a.quantization:
        kw.update(quantization=a.quantization, quant_config={"quant_method": a.quantization})
    llm = LLM(a.model, tensor_parallel_size=a.tensor_parallel_size, max_num_seqs=a.max_num_seqs,
              max_num_batched_tokens=a.max_num_batched_tokens,
              max_model_len=a.input_len + a.output_len + 16, async_scheduling=True,
              enable_expert_parallel=a.enable_expert_parallel, device=a.device, **kw)
    V = llm.engine.cfg.model.vocab_size
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, V, (a.num_prompts, a.input_len), generator=g).tolist()
    sp = SamplingParams(max_tokens=a.output_len, temperature=a.temperature, ignore_eos=True)
    llm.generate(prompts[: min(8, len(prompts))], SamplingParams(max_tokens=4, ignore_eos=True))
    t0 = time.perf_counter()
    outs = llm.generate(prompts, sp)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    rank = 0
    if a.tensor_parallel_size > 1:
        import torch.distributed as dist
        rank = dist.get_rank()
        t = torch.tensor([dt], dtype=torch.float64,
                         device="cuda" if torch.cuda.is_available() else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t[0])
    n_out = sum(len(o.outputs[0].token_ids) for o in outs)
    n_in = a.num_prompts * a.input_len
    res = {"elapsed_s": dt, "requests_per_s": a.num_prompts / dt,
           "total_tokens_per_s": (n_in + n_out) / dt, "output_tokens_per_s": n_out / dt}
    res["config"] = {"model": a.model, "num_prompts": a.num_prompts, "input_len": a.input_len,
                     "output_len": a.output_len, "tensor_parallel_size": a.tensor_parallel_size,
                     "expert_parallel": a.enable_expert_parallel, "quantization": a.quantization}
    if rank != 0:
        return
    print(json.dumps(res, indent=1))
    if a.output_json:
        with open(a.output_json, "w") as f:
            json.dump(res, f)


if __name__ == "__main__":
    main()
