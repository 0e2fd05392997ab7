"""Stand-in baseline: stock vLLM (the copy installed in the image, CUDA platform, its own
kernels and NCCL) on the workload of ``bench.py``.

The reference plugin needs the Enflame SDK and has no CUDA path, so it cannot run on a B200;
stock vLLM on the CUDA platform is the closest thing to "the reference with NCCL and library
kernels" and is measured with the same protocol as the reference's
``benchmarks/benchmark_throughput.py:448-450``: all requests submitted up front, fixed
lengths, EOS ignored, output tokens / elapsed.

Workload: Llama-3-8B architecture (random "dummy" weights, bf16), ``--num-prompts`` requests
of ``--input-len`` uniform-random token ids, ``--output-len`` output tokens each,
``max_num_seqs`` 256, block size 16, tensor parallel over ``--gpus`` GPUs.

    python benchmarks/baseline_vllm_stock.py --gpus 1 --steps 1 --warmup 1
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29700 benchmarks/baseline_vllm_stock.py --gpus N

With N > 1 every rank runs this script with the same prompts (vLLM's ``external_launcher``
executor).  vLLM exposes no per-step device timing, so ``value`` and ``e2e`` are both the wall
clock around ``LLM.generate`` between ``torch.cuda.synchronize()`` calls (maximum over ranks).
No plugin of this repository is loaded (``VLLM_PLUGINS`` is set to an empty list).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time

LLAMA3_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 4096,
    "intermediate_size": 14336, "num_hidden_layers": 32, "num_attention_heads": 32,
    "num_key_value_heads": 8, "vocab_size": 128256, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0, "max_position_embeddings": 8192, "torch_dtype": "bfloat16",
    "tie_word_embeddings": False, "hidden_act": "silu", "attention_bias": False,
    "mlp_bias": False, "bos_token_id": 128000, "eos_token_id": 128001,
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--num-prompts", type=int, default=512)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--attention-backend", default=None,
                    help="vLLM attention backend name (default: vLLM's own choice)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model")
    ap.add_argument("--prefill-only-pass", action="store_true",
                    help="also time one pass with a single output token per request (attributes "
                         "the total to prefill and decode)")
    args = ap.parse_args()

    os.environ["VLLM_PLUGINS"] = ""                   # stock code path only
    os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1:
        os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")

    import torch
    from vllm import LLM, SamplingParams

    cfg = dict(LLAMA3_8B)
    if args.layers > 0:
        cfg["num_hidden_layers"] = args.layers
    d = tempfile.mkdtemp(prefix="llama3_8b_cfg_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)

    kw = dict(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16",
              tensor_parallel_size=max(1, world), max_num_seqs=args.max_num_seqs,
              max_num_batched_tokens=args.max_num_batched_tokens, block_size=16,
              max_model_len=args.input_len + args.output_len + 16, enable_prefix_caching=True,
              gpu_memory_utilization=0.9, seed=0)
    if world > 1:
        kw["distributed_executor_backend"] = "external_launcher"
    if args.attention_backend:
        kw["attention_config"] = {"backend": args.attention_backend}
    llm = LLM(**kw)
    sp = SamplingParams(max_tokens=args.output_len, temperature=0.0, ignore_eos=True,
                        detokenize=False)

    def prompts(seed: int):
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(0, cfg["vocab_size"], (args.num_prompts, args.input_len), generator=g)
        return [{"prompt_token_ids": row} for row in ids.tolist()]

    def one_pass(seed: int, params=None):
        ps = prompts(seed)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(ps, params or sp, use_tqdm=False)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        return sum(len(o.outputs[0].token_ids) for o in outs), dt

    for w in range(args.warmup):
        one_pass(1000 + w)
    tot_out, tot_s = 0, 0.0
    for k in range(args.steps):
        n, dt = one_pass(2000 + k)
        tot_out += n
        tot_s += dt
    prefill_s = None
    if args.prefill_only_pass:
        sp1 = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True, detokenize=False)
        one_pass(3000, sp1)
        _, prefill_s = one_pass(3001, sp1)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([tot_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        tot_s = float(t[0])
    if rank == 0:
        import vllm
        value = tot_out / tot_s
        print(json.dumps({
            "impl": "vllm-stock", "vllm_version": vllm.__version__,
            "metric": (f"output tok/s per box (offline throughput, {args.num_prompts} req x "
                       f"{args.input_len} in / {args.output_len} out)"),
            "value": round(value, 2), "unit": "tok/s", "n_gpus": max(1, world),
            "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(tot_s * 1e3 / max(1, args.steps), 3),
            "higher_is_better": True, "scaling": "strong", "dtype": "bf16",
            "data": "synthetic (uniform-random token ids, dummy weights)",
            "timing": "wall clock around LLM.generate, max over ranks",
            "config": {"model": "llama-3-8b", "global_batch": args.num_prompts,
                       "input_len": args.input_len, "output_len": args.output_len,
                       "max_num_seqs": args.max_num_seqs, "block_size": 16,
                       "parallelism": f"tp{max(1, world)}",
                       "attention_backend": args.attention_backend or "default",
                       "layers_override": args.layers or None},
            "e2e": {"value": round(value, 2), "unit": "tok/s"},
            "prefill_only_pass_ms": None if prefill_s is None else round(prefill_s * 1e3, 1),
        }), flush=True)
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
