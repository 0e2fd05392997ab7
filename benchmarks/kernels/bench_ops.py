"""Micro-benchmarks of the memory-bound ops against the measured copy bandwidth: RMSNorm
(plain, fused add, fp8 epilogue), SiLU-mul, RoPE + cache write, per-token quantisation, MoE
routing / align / permute, sampling (the reference keeps one script per op under
benchmarks/kernels/).  CUDA events, L2 flushed between iterations.

  python benchmarks/kernels/bench_ops.py [--tokens 8192] [--hidden 4096]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from vllm_gcu_b200.ops import cuda as C  # noqa: E402


def timeit(fn, flush, iters=10):
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
    return tot / iters * 1e3          # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    a = ap.parse_args()
    T, H = a.tokens, a.hidden
    dev = "cuda"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    res = torch.randn_like(x)
    w = torch.ones(H, device=dev, dtype=torch.bfloat16)
    rows = []

    def add(name, fn, nbytes):
        us = timeit(fn, flush)
        rows.append((name, us, nbytes / us / 1e3))

    add("rms_norm", lambda: C.norm(x, w, 1e-6), 2 * T * H * 2)
    add("fused_add_rms_norm", lambda: C.norm(x, w, 1e-6, residual=res), 4 * T * H * 2)
    add("rms_norm + fp8 per-token", lambda: C.norm(x, w, 1e-6, quant="fp8_token"), T * H * 3)
    gu = torch.randn(T, 2 * H, device=dev, dtype=torch.bfloat16)
    add("silu_and_mul", lambda: C.activation(gu, "silu"), 3 * T * H * 2)
    add("per_token_quant fp8", lambda: C.per_token_quant(x, "fp8"), T * H * 3)
    Hq, Hkv, D, bs = 32, 8, 128, 16
    q = torch.randn(T, Hq * D, device=dev, dtype=torch.bfloat16)
    k = torch.randn(T, Hkv * D, device=dev, dtype=torch.bfloat16)
    v = torch.randn_like(k)
    nb = T // bs + 1
    kc = torch.zeros(nb, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    pos = torch.arange(T, device=dev)
    from vllm_gcu_b200.ops import ref
    cs = ref.make_cos_sin_cache(D, T + 1).to(dev)
    add("rope + cache write", lambda: C.rope_cache_flash(q, k, v, pos, cs, True, D, pos, kc, vc),
        (2 * T * Hq * D + 4 * T * Hkv * D) * 2)
    E, topk = 128, 8
    gate = torch.randn(T, E, device=dev, dtype=torch.float32)
    add("moe_topk (128 experts, top-8)", lambda: C.moe_topk(gate, topk, True), T * E * 4)
    _, ids = C.moe_topk(gate, topk, True)
    add("moe_align", lambda: C.moe_align(ids, E), T * topk * 8)
    V = 128256
    logits = torch.randn(256, V, device=dev, dtype=torch.bfloat16)
    add("greedy sample 256 x 128256", lambda: C.sample(logits), 256 * V * 2)
    temp = torch.full((256,), 0.8, device=dev)
    tk = torch.full((256,), 50, device=dev, dtype=torch.int32)
    tp = torch.full((256,), 0.9, device=dev)
    seeds = torch.arange(256, device=dev)
    add("top-k/top-p sample 256 x 128256", lambda: C.sample(logits, temp, tk, tp, seeds=seeds),
        256 * V * 2)
    print(f"{'op':36s} {'us':>9s} {'GB/s':>9s}")
    for name, us, gbs in rows:
        print(f"{name:36s} {us:9.1f} {gbs:9.0f}")


if __name__ == "__main__":
    main()
