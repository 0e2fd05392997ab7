"""Large-M bf16 GEMMs of Llama-3-8B (8192 rows): the CTA-pair kernel (`csrc/gemm_pair.cu`,
256 x 256 tile per cluster of two, and its 512 x 256 variant), the single-CTA 256 x 256 kernel
and torch.matmul (cuBLAS).  CUDA events around 20 launches after 3 warm-up launches; every
operand set is larger than L2.

Usage: python benchmarks/kernels/bench_gemm_pair.py [--rows 8192]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from vllm_gcu_b200.ops import _native  # noqa: E402
from vllm_gcu_b200.ops import cuda as C  # noqa: E402

SHAPES = ((6144, 4096, 0, "qkv"), (4096, 4096, 0, "o_proj"), (28672, 4096, 2, "gate_up+silu"),
          (4096, 14336, 0, "down"))


def timed(fn, iters=20):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=8192)
    a = ap.parse_args()
    M = a.rows
    print(f"{'layer':>13} {'N x K':>14} | pair 256x256 | pair 512x256 | single CTA | cuBLAS   "
          "(us, TFLOP/s)")
    for N, K, epi, name in SHAPES:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
        flops = 2.0 * M * N * K
        cols = []
        for pair, mt in ((True, "1"), (True, "2"), (False, "1")):
            C.USE_PAIR_GEMM = pair
            os.environ["VLLM_B200_PAIR_MT"] = mt
            t = timed(lambda: C.gemm_bf16(x, w, epilogue=epi))
            cols.append(f"{t:7.1f} {flops / t / 1e6:5.0f}")
        C.USE_PAIR_GEMM = True
        os.environ["VLLM_B200_PAIR_MT"] = "1"
        t = timed(lambda: torch.matmul(x, w.t()))
        cols.append(f"{t:7.1f} {flops / t / 1e6:5.0f}")
        print(f"{name:>13} {N:>7} x {K:<5} | " + " | ".join(cols), flush=True)
    _native.check_status()


if __name__ == "__main__":
    main()
