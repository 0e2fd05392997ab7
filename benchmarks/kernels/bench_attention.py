"""Times the paged decode and varlen prefill attention kernels (CUDA events, inputs larger
than L2) and reports achieved KV-cache bandwidth / FLOP rate.

Usage: python benchmarks/kernels/bench_attention.py [--batch 256] [--ctx 1152]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
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
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--hd", type=int, default=128)
    ap.add_argument("--bs", type=int, default=16)
    a = ap.parse_args()
    B, ctx, Hq, Hkv, D, bs = a.batch, a.ctx, a.hq, a.hkv, a.hd, a.bs
    mb = (ctx + bs - 1) // bs
    nb = B * mb
    kc = torch.randn(nb, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(nb, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    bt = torch.randperm(nb, device="cuda").to(torch.int32).view(B, mb)
    sl = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    scale = D ** -0.5
    kv_bytes = 2 * B * ctx * Hkv * D * 2
    for tma in (True, False):
        C.USE_TMA_DECODE = tma
        for splits in (1, 2, 4):
            ms = timeit(lambda: C.paged_decode(q, kc, vc, bt, sl, scale, out=out,
                                               num_splits=splits))
            print(f"decode {'tma     ' if tma else 'cp.async'} B={B} ctx={ctx} splits={splits}: "
                  f"{ms*1e3:8.1f} us  {kv_bytes/ms/1e6:7.0f} GB/s "
                  f"(KV bytes {kv_bytes/1e6:.0f} MB)", flush=True)
    C.USE_TMA_DECODE = True
    # prefill: 8 sequences of 1024 new tokens
    nseq, ql = 8, 1024
    T = nseq * ql
    qp = torch.randn(T, Hq, D, device="cuda", dtype=torch.bfloat16)
    cu = torch.arange(0, T + 1, ql, device="cuda", dtype=torch.int32)
    slp = torch.full((nseq,), ql, device="cuda", dtype=torch.int32)
    btp = bt[:nseq, : (ql + bs - 1) // bs].contiguous()
    outp = torch.empty_like(qp)
    tiles = nseq * (ql // 64)
    fl = 4.0 * nseq * Hq * D * ql * ql / 2
    for name, flag in (("tcgen05", True), ("mma.sync", False)):
        C.USE_FMHA_PREFILL = flag
        ms = timeit(lambda: C.varlen_prefill(qp, kc, vc, btp, cu, slp, scale, tiles, out=outp,
                                             num_q_tiles_128=nseq * (ql // 128)))
        print(f"prefill {name:8s} {nseq}x{ql}: {ms*1e3:8.1f} us  {fl/ms/1e9:7.1f} TFLOP/s (causal)",
              flush=True)
    C.USE_FMHA_PREFILL = True


if __name__ == "__main__":
    main()
