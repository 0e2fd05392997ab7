"""Times the tcgen05 multi-head latent attention kernel (csrc/attention_mla.cu) against the
gather + batched-GEMM formulation it replaces (models/deepseek.py ``mla_decode_batched``).
CUDA events, latent cache larger than L2 by default.

Usage: python benchmarks/kernels/bench_mla.py [--batch 256] [--ctx 1152] [--heads 128]
       python benchmarks/kernels/bench_mla.py --prefill 2048 --batch 4 --heads 16
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from vllm_gcu_b200.models.deepseek import mla_decode_batched  # noqa: E402
from vllm_gcu_b200.ops import cuda as C  # noqa: E402


def timeit(fn, iters=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(True), torch.cuda.Event(True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=1152)
    ap.add_argument("--heads", type=int, default=128)
    ap.add_argument("--bs", type=int, default=16)
    ap.add_argument("--prefill", type=int, default=0, help="query tokens per request (0: decode)")
    ap.add_argument("--splits", type=int, default=0)
    a = ap.parse_args()
    B, ctx, Nh, bs = a.batch, a.ctx, a.heads, a.bs
    dev = torch.device("cuda")
    mb = (ctx + bs - 1) // bs
    cache = (torch.randn(B * mb, bs, 576, device=dev) * 0.3).to(torch.bfloat16)
    bt = torch.randperm(B * mb, device=dev).view(B, mb).to(torch.int32)
    sl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
    ql = a.prefill or 1
    T = B * ql
    q = (torch.randn(T, Nh, 576, device=dev) * 0.3).to(torch.bfloat16)
    cu = None if not a.prefill else torch.arange(0, T + 1, ql, dtype=torch.int32, device=dev)
    tq = 128 // Nh
    tiles = B * (-(-ql // tq))
    scale = 576 ** -0.5
    out = torch.empty(T, Nh, 512, dtype=torch.bfloat16, device=dev)
    splits = a.splits or None
    t = timeit(lambda: C.mla_attention(q, cache, bt, sl, cu, tiles, ctx, scale, out=out,
                                       splits=splits))
    keys = ctx if not a.prefill else ctx - (ql - 1) / 2          # mean visible keys per token
    flops = 2.0 * T * Nh * keys * (576 + 512)
    cache_bytes = B * ctx * 576 * 2
    print(f"mla_attention  B={B} ctx={ctx} heads={Nh} q_len={ql}: {t * 1e3:8.1f} us  "
          f"{flops / t / 1e9:7.1f} TFLOP/s  cache {cache_bytes / t / 1e6:7.1f} GB/s")
    if not a.prefill:
        t2 = timeit(lambda: mla_decode_batched(q, cache, bt, sl, ctx, scale, 512))
        print(f"gather + bmm   {t2 * 1e3:8.1f} us  ({t2 / t:.2f}x the kernel's time)")


if __name__ == "__main__":
    main()
