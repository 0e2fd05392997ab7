"""Offline-throughput benchmark: output tokens per second of the whole job.

Workload (the reference's ``benchmark_throughput`` protocol, benchmarks/benchmark_throughput.py:
448-450, on the Llama-3-8B configuration): ``--num-prompts`` requests (default 512) of
``--input-len`` (1024) uniform-random token ids each, exactly ``--output-len`` (256) output
tokens (EOS ignored), all submitted up front, ``max_num_seqs`` 256, paged KV block 16, bf16,
random-init weights, tensor parallel over ``--gpus`` GPUs.

One *step* is one complete pass of that workload through ``LLM.generate``.  After
``--warmup`` untimed passes, ``--steps`` passes are timed between barriers +
``torch.cuda.synchronize()``.  Reported:

* ``value``  – output tok/s from device time: the sum over engine steps of the CUDA-event
  interval that brackets each step's host-to-device copies and kernels (max over ranks);
* ``e2e``    – output tok/s from the wall clock around ``LLM.generate`` (scheduling, host
  preparation, per-step pinned-memory H2D copies of the inputs and the D2H read of the
  sampled ids all included);
* ``gpu_launches`` – kernels of this repository launched in the timed region (graph replays
  counted by their captured launches).

Launch: ``python bench.py`` (1 GPU) or
``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``.
``--impl reference`` reports why the reference cannot run on this hardware;
``--impl vllm-stock`` runs the same workload through stock vLLM on the CUDA platform (the
stand-in baseline, benchmarks/baseline_vllm_stock.py).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

BASELINE_PUBLISHED = None   # the reference publishes no number for this configuration

CLOCK_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
               "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
               "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self) -> None:
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={CLOCK_QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.gpu_index)], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        busy = [c for c in sm if c > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def run_reference(args) -> None:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "vllm-gcu cannot be installed here: setup.py imports tops_extension and the "
                       "package needs torch_gcu/topsaten/libeccl (Enflame GCU SDK); it has no CUDA "
                       "code path, so there is nothing to run on a B200"}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "vllm-stock"])
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--num-prompts", type=int, default=512)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--no-async", action="store_true")
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.impl == "vllm-stock":
        # stand-in baseline (stock vLLM on the CUDA platform, none of this repository's code):
        # the same workload through benchmarks/baseline_vllm_stock.py, in this process slot
        script = os.path.join(os.path.dirname(os.path.abspath(__file__)), "benchmarks",
                              "baseline_vllm_stock.py")
        argv = [sys.executable, script, "--gpus", str(args.gpus), "--steps", str(args.steps),
                "--warmup", str(args.warmup), "--num-prompts", str(args.num_prompts),
                "--input-len", str(args.input_len), "--output-len", str(args.output_len),
                "--max-num-seqs", str(args.max_num_seqs),
                "--max-num-batched-tokens", str(args.max_num_batched_tokens)]
        if args.layers > 0:
            argv += ["--layers", str(args.layers)]
        os.execv(sys.executable, argv)

    import torch
    import torch.distributed as dist
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    from vllm_gcu_b200.ops import _native
    from vllm_gcu_b200.parallel.state import get_state, init_distributed

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run "
                             "(--nproc-per-node N)")
        args.gpus = world
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local_rank)
    if args.gpus > 1:
        init_distributed(tp=args.gpus)

    overrides = {}
    if args.layers > 0:
        overrides["num_hidden_layers"] = args.layers
    llm = LLM(args.model, tensor_parallel_size=args.gpus, max_num_seqs=args.max_num_seqs,
              max_num_batched_tokens=args.max_num_batched_tokens,
              max_model_len=args.input_len + args.output_len + 16, block_size=16,
              async_scheduling=not args.no_async, enforce_eager=args.eager,
              enable_prefix_caching=True, comm_backend=args.comm, **overrides)
    eng = llm.engine
    vocab = eng.cfg.model.vocab_size
    sp = SamplingParams(max_tokens=args.output_len, temperature=0.0, ignore_eos=True)

    def make_prompts(seed: int):
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(0, vocab, (args.num_prompts, args.input_len), generator=g)
        return ids.tolist()

    def barrier():
        if args.gpus > 1:
            dist.barrier()
        torch.cuda.synchronize()

    breakdown: dict = {}

    def one_pass(seed: int, timed: bool):
        prompts = make_prompts(seed)       # fresh ids: no prefix-cache reuse across passes
        eng.runner.timing_events = [] if timed else None
        eng.runner.timing_meta = []
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        n_out = sum(len(o.outputs[0].token_ids) for o in outs)
        dev_ms = 0.0
        if timed:
            times = [a.elapsed_time(b) for a, b in eng.runner.timing_events]
            dev_ms = sum(times)
            for t, (nd, npf, ntok) in zip(times, eng.runner.timing_meta):
                kind = "decode" if npf == 0 else ("prefill" if nd == 0 else "mixed")
                acc = breakdown.setdefault(kind, [0, 0.0, 0])
                acc[0] += 1
                acc[1] += t
                acc[2] += ntok
            eng.runner.timing_events = None
        return n_out, wall, dev_ms

    for w in range(args.warmup):
        one_pass(1000 + w, False)

    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _native.launch_count + eng.runner.graph_launches
    h2d0, d2h0, steps0 = eng.runner.h2d_bytes, eng.runner.d2h_bytes, eng.stats["steps"]
    tot_out, tot_wall, tot_dev = 0, 0.0, 0.0
    for k in range(args.steps):
        n_out, wall, dev_ms = one_pass(2000 + k, True)
        tot_out += n_out
        tot_wall += wall
        tot_dev += dev_ms
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    launches = _native.launch_count + eng.runner.graph_launches - launches0
    engine_steps = eng.stats["steps"] - steps0
    _native.check_status()

    t = torch.tensor([tot_dev, tot_wall * 1e3], dtype=torch.float64, device="cuda")
    if args.gpus > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms = float(t[0]), float(t[1])
    if rank == 0:
        value = tot_out / (dev_ms / 1e3)
        e2e = tot_out / (wall_ms / 1e3)
        line = {
            "metric": (f"output tok/s per box (offline throughput, {args.num_prompts} req x "
                       f"{args.input_len} in / {args.output_len} out)"),
            "value": round(value, 2), "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dev_ms / args.steps, 3), "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": (value / BASELINE_PUBLISHED) if BASELINE_PUBLISHED else None,
            "dtype": "bf16", "data": "synthetic (uniform-random token ids, random-init weights)",
            "impl": "ours",
            "config": {"model": args.model, "global_batch": args.num_prompts,
                       "seq_len": args.input_len + args.output_len,
                       "input_len": args.input_len, "output_len": args.output_len,
                       "max_num_seqs": args.max_num_seqs, "block_size": 16,
                       "parallelism": f"tp{args.gpus}", "comm": args.comm,
                       "async_scheduling": not args.no_async,
                       "cuda_graphs": not args.eager,
                       "l2_policy": "inputs larger than L2 (weights 16 GB + KV cache are "
                                    "streamed every step)",
                       "engine_steps_per_step": engine_steps // max(1, args.steps),
                       "layers_override": args.layers or None},
            "e2e": {"value": round(e2e, 2), "unit": "tok/s",
                    "h2d_bytes_per_step": (eng.runner.h2d_bytes - h2d0) // max(1, args.steps),
                    "d2h_bytes_per_step": (eng.runner.d2h_bytes - d2h0) // max(1, args.steps),
                    "wall_ms_per_step": round(wall_ms / args.steps, 3)},
            "gpu_launches": int(launches),
            "step_breakdown": {k: {"engine_steps": v[0], "device_ms": round(v[1], 1),
                                   "tokens": v[2]} for k, v in breakdown.items()},
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if args.gpus > 1:
        # Leave without tearing down NCCL communicators that captured CUDA graphs still
        # reference: that teardown can block forever after the result has been printed.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
