"""Latency of the fused row-parallel kernels against GEMM followed by an NCCL all-reduce.

Three fused forms are timed: GEMM + tile-wise all-reduce (one-shot / two-shot), and
GEMM + all-reduce + residual add + RMSNorm with row owners (``gemm_ar_norm``), the latter
over plain peer loads / stores and over multimem (in-switch reduction), against the un-fused
sequence GEMM, NCCL all-reduce, fused-add RMSNorm kernel.  ``roofline_us`` is the slowest of
FLOPs / measured bf16 peak, operand bytes / measured HBM bandwidth and the bytes that must
cross NVLink per direction and GPU / 770 GB/s; ``*_frac`` = roofline / measured.

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
    peaks = {"bf16_tflops": 1632.2, "hbm_gbs": 6552.3}
    try:
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        peaks.update(json.load(open(os.path.join(root, "MEASURED_PEAKS.json"))))
    except Exception:
        pass
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
            # GEMM + all-reduce + residual + RMSNorm: one kernel against three
            resid = torch.randn(M, N, device=dev).to(torch.bfloat16)
            nw = torch.ones(N, device=dev, dtype=torch.bfloat16)

            def unfused(i):
                y = C.gemm_bf16(x, ws[i])
                dist.all_reduce(y)
                return C.norm(y, nw, 1e-5, residual=resid)
            res["nccl_norm_us"] = timed(unfused, 5, gr)
            variants = [("ar_norm_pull_us", False, 0), ("ar_norm_push_us", False, 1),
                        ("ar_norm_pushall_us", False, 2), ("ar_norm_ll_us", False, 3),
                        ("ar_norm_us", False, None)]
            if fused.buf.multicast_ptr:
                variants.append(("ar_norm_mc_us", True, 0))
            for key, mc, mode in variants:
                if mode in (1, 2, 3) and M > 1024:
                    continue            # the push transports are for decode-sized problems
                fused.use_multimem = mc
                fused.force_rn_mode = mode
                fused.row_owner = True if mode is None else None
                res[key] = timed(lambda i: fused.gemm_ar_norm(x, ws[i], resid, nw, 1e-5,
                                                              bcast_residual=False), 5, gr)
                _native.check_status()
            fused.force_rn_mode = None
            fused.row_owner = None
            fused.use_multimem = bool(fused.buf.multicast_ptr)
            res["ar_norm_default_us"] = timed(lambda i: fused.gemm_ar_norm(
                x, ws[i], resid, nw, 1e-5, bcast_residual=False), 5, gr)
            flop_us = 2.0 * M * N * K / (peaks["bf16_tflops"] * 1e12) * 1e6
            hbm_us = (N * K + M * K + 2 * M * N) * 2 / (peaks["hbm_gbs"] * 1e9) * 1e6
            # per GPU and direction: (p-1)/p of the partial matrix in, (p-1)/p of the result in
            nvl_us = 2.0 * (world - 1) / world * M * N * 2 / 770e9 * 1e6
            # multimem: the switch adds the partials, 1/p of the matrix comes in reduced
            nvl_mc_us = ((world - 1) / world + 1.0 / world) * M * N * 2 / 770e9 * 1e6
            res["roofline_us"] = round(max(flop_us, hbm_us, nvl_us), 2)
            res["roofline_mc_us"] = round(max(flop_us, hbm_us, nvl_mc_us), 2)
            res["ar_norm_frac"] = round(res["roofline_us"] / res["ar_norm_us"], 3)
            if "ar_norm_mc_us" in res:
                res["ar_norm_mc_frac"] = round(res["roofline_mc_us"] / res["ar_norm_mc_us"], 3)
            rows.append(res)
    if rank == 0:
        print(json.dumps({"world": world, "results": rows}))
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
