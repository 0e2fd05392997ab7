"""Decode-sized bf16 GEMMs of Llama-3-8B timed the way the engine runs them: 20 launches
captured in a CUDA graph and replayed (a single launch from Python costs more host time than
these kernels take on the device), weights cycling through copies that exceed L2.

Per shape: the kernel the dispatcher picks (persistent tiles, weight-streaming kernel, two-kernel
K split for up to 128 rows), the same with the K split switched off, the CTA-pair kernel
(one 256 x 256 tile per cluster of two, no K split) and torch.matmul (cuBLAS).

Usage: python benchmarks/kernels/bench_decode_gemm.py [--rows 256 128 64 16 1]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from vllm_gcu_b200.ops import _native  # noqa: E402
from vllm_gcu_b200.ops import cuda as C  # noqa: E402

SHAPES = ((6144, 4096, "qkv"), (4096, 4096, "o_proj"), (28672, 4096, "gate_up"),
          (4096, 14336, "down"), (128256, 4096, "lm_head"))


def replay_time(fn, iters=20):
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(iters):
                fn(i)
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(True), torch.cuda.Event(True)
    s.record()
    graph.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, nargs="+", default=[256, 128, 64, 16, 1])
    a = ap.parse_args()
    keep = C.SKINNY_SPLIT2_MAX_M
    print(f"{'rows':>5} {'layer':>8} {'N x K':>14} {'ours us':>8} {'no split us':>12} "
          f"{'pair us':>8} {'cuBLAS us':>10}")
    for M in a.rows:
        for Nn, K, name in SHAPES:
            copies = max(2, (200 << 20) // (Nn * K * 2) + 1)
            ws = [torch.randn(Nn, K, device="cuda", dtype=torch.bfloat16) * 0.02
                  for _ in range(copies)]
            x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            out = torch.empty(M, Nn, device="cuda", dtype=torch.bfloat16)
            C.SKINNY_SPLIT2_MAX_M = keep
            t_ours = replay_time(lambda i: C.gemm_bf16(x, ws[i % copies], out=out))
            C.SKINNY_SPLIT2_MAX_M = 0
            t_nosplit = replay_time(lambda i: C.gemm_bf16(x, ws[i % copies], out=out))
            C.SKINNY_SPLIT2_MAX_M = keep

            def pair(i):
                w = ws[i % copies]
                rc = _native.lib().b200_gemm_pair(x.data_ptr(), x.stride(0), w.data_ptr(),
                                                  w.stride(0), out.data_ptr(), out.stride(0), M,
                                                  Nn, K, None, 0, _native.stream_ptr())
                assert rc == 0, rc
            t_pair = replay_time(pair) if Nn % 256 == 0 else float("nan")
            t_ref = replay_time(lambda i: torch.matmul(x, ws[i % copies].t(), out=out))
            print(f"{M:>5} {name:>8} {Nn:>7} x {K:<5} {t_ours:8.1f} {t_nosplit:12.1f} "
                  f"{t_pair:8.1f} {t_ref:10.1f}", flush=True)
            del ws


if __name__ == "__main__":
    main()
