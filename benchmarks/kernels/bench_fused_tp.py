"""Latency of the fused GEMM + all-reduce kernel against GEMM followed by an NCCL all-reduce.

Launch with one rank per GPU:
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
      --master-port 29650 benchmarks/kernels/bench_fused_tp.py

Shapes are the two row-parallel layers of Llama-3-8B at tensor-parallel degree N (o_proj and
down_proj) for a decode batch (M = 256) and a prefill chunk (M = 8192).  Times are CUDA-event
times on the launching stream after warm-up, maximum over ranks, per call inside a chain of
16 calls that use 16 different weights (together larger than L2).
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from vllm_gcu_b200.ops import _native  # noqa: E402
from vllm_gcu_b200.ops import cuda as C  # noqa: E402
from vllm_gcu_b200.parallel import symm  # noqa: E402
from vllm_gcu_b200.parallel.state import init_distributed  # noqa: E402


CHAIN = 16


def timed(fn, iters, graph=False):
    """Average time of one call inside a chain of CHAIN back-to-back calls (each on its own
    weight, together larger than L2), so that launch skew between the ranks is amortised.
    With ``graph`` the chain is captured into a CUDA graph first (no host launch cost, as in
    the engine's decode steps)."""
    def chain():
        for i in range(CHAIN):
            fn(i)
    for _ in range(2):
        chain()
    torch.cuda.synchronize()
    run = chain
    if graph:
        g = torch.cuda.CUDAGraph()
        s_ = torch.cuda.Stream()
        s_.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s_):
            chain()
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=s_):
                chain()
        torch.cuda.current_stream().wait_stream(s_)
        torch.cuda.synchronize()
        run = g.replay
        run()
        torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        tot += e0.elapsed_time(e1)
    t = torch.tensor([tot / iters / CHAIN], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return round(float(t.item()) * 1e3, 2)     # microseconds


def main():
    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    st = init_distributed(tp=world)
    dev = torch.device("cuda", st.local_rank)
    fused = symm.FusedTP(max_tokens=8192, max_n=4096, device=dev)
    rows = []
    for M in (256, 8192):
        for name, K in (("o_proj", 4096 // world), ("down_proj", 14336 // world)):
            N = 4096
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            ws = [(torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
                  for _ in range(CHAIN)]

            def nccl(i):
                y = C.gemm_bf16(x, ws[i])
                dist.all_reduce(y)
                return y
            gr = M <= 1024          # decode-sized: time graph replays, as the engine runs them
            res = {"M": M, "layer": name, "K": K, "graph": gr, "nccl_us": timed(nccl, 5, gr),
                   "gemm_only_us": timed(lambda i: C.gemm_bf16(x, ws[i]), 5, gr)}
            for mode in ("oneshot", "twoshot"):
                if mode == "oneshot" and not fused._oneshot(M):
                    continue            # does not fit the one-shot slots at this size
                fused.force_mode = mode
                res[mode + "_us"] = timed(lambda i: fused.gemm_all_reduce(x, ws[i]), 5, gr)
                _native.check_status()
                fused.force_mode = None
            rows.append(res)
    if rank == 0:
        print(json.dumps({"world": world, "results": rows}))
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
