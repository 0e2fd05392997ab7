"""Times the tcgen05 bf16 GEMM against torch.matmul (cuBLAS) on Llama-shaped problems.

Usage: python benchmarks/kernels/bench_gemm.py [--iters 20]
Prints one line per shape: device time (CUDA events, L2 flushed between
iterations), TFLOP/s, effective weight bandwidth and the ratio to cuBLAS.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from vllm_gcu_b200.ops import cuda as C  # noqa: E402

SHAPES = [  # (M, N, K, label)
    (8192, 6144, 4096, "8B qkv prefill"),
    (8192, 4096, 4096, "8B o_proj prefill"),
    (8192, 28672, 4096, "8B gate_up prefill"),
    (8192, 4096, 14336, "8B down prefill"),
    (256, 6144, 4096, "8B qkv decode"),
    (256, 4096, 4096, "8B o_proj decode"),
    (256, 28672, 4096, "8B gate_up decode"),
    (256, 4096, 14336, "8B down decode"),
    (256, 128256, 4096, "8B lm_head decode"),
    (64, 6144, 4096, "8B qkv decode b64"),
    (64, 28672, 4096, "8B gate_up decode b64"),
    (64, 4096, 14336, "8B down decode b64"),
    (256, 2048, 2048, "o_proj tp2 decode"),
    (256, 4096, 7168, "down tp2 decode"),
    (8192, 8192, 8192, "square 8k"),
]


def timeit(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(True), torch.cuda.Event(True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        tot += s.elapsed_time(e)
    return tot / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for M, N, K, label in SHAPES:
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t_ours = timeit(lambda: C.gemm_bf16(x, w, out=out), a.iters, flush)
        t_ref = timeit(lambda: torch.matmul(x, w.t(), out=out), a.iters, flush)
        fl = 2.0 * M * N * K
        if M >= C.WIDE2_MIN_M and N % 256 == 0:     # large M: also time the 128 x 256 tile kernel
            C.USE_WIDE2_GEMM = False
            t_tile = timeit(lambda: C.gemm_bf16(x, w, out=out), a.iters, flush)
            C.USE_WIDE2_GEMM = True
            label = f"{label} [128x256 tiles {t_tile*1e3:.1f} us]"
        if M <= C.SKINNY_MAX_M:          # decode-sized: also time the persistent-tile kernel
            C.USE_SKINNY_GEMM = False
            t_tile = timeit(lambda: C.gemm_bf16(x, w, out=out), a.iters, flush)
            C.USE_SKINNY_GEMM = True
            ref = x.float() @ w.float().t()
            err = (C.gemm_bf16(x, w).float() - ref).abs().max().item() / ref.abs().max().item()
            label = f"{label} [tile kernel {t_tile*1e3:.1f} us, rel err {err:.1e}]"
        print(f"{label:22s} M={M:5d} N={N:6d} K={K:5d}  ours {t_ours*1e3:8.1f} us "
              f"{fl/t_ours/1e9:7.1f} TFLOP/s  w-bw {N*K*2/t_ours/1e6:6.0f} GB/s | cublas "
              f"{t_ref*1e3:8.1f} us {fl/t_ref/1e9:7.1f} TFLOP/s | ratio {t_ref/t_ours:.2f}",
              flush=True)


if __name__ == "__main__":
    main()
