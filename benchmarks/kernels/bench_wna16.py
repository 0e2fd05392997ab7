"""Times the fused de-quantising GEMM (csrc/gemm_wna16.cu) against de-quantise + bf16 GEMM on
the decode shapes of Llama-3-8B (CUDA events; each shape cycles through enough weight copies
to exceed L2).

Usage: python benchmarks/kernels/bench_wna16.py [--m 256] [--bits 4] [--group 128]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from vllm_gcu_b200.ops import cuda as C  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=256)
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--group", type=int, default=128)
    a = ap.parse_args()
    dev, M, g, bits = "cuda", a.m, a.group, a.bits
    print(f"M={M} bits={bits} group={g}")
    print(f"{'N x K':>16} {'fused us':>9} {'GB/s':>7} {'dequant+gemm us':>16} {'speedup':>8}")
    for Nn, K in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)):
        wbytes = Nn * K * bits // 8
        copies = max(2, (160 << 20) // wbytes + 1)
        qws = [torch.randint(0, 256, (Nn, K * bits // 8), dtype=torch.uint8, device=dev)
               for _ in range(copies)]
        sc = (torch.rand(Nn, K // g, device=dev) * 0.02).to(torch.bfloat16)
        zs = (torch.rand(Nn, K // g, device=dev) * 0.1).to(torch.bfloat16)
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.empty(Nn, K, dtype=torch.bfloat16, device=dev)

        def fused(i):
            C.gemm_wna16(x, qws[i % copies], sc, zs, g, bits)

        def unfused(i):
            C.weight_dequant(qws[i % copies], sc, zs, w, g, bits)
            C.gemm_bf16(x, w)

        # The kernels take 10-100 us and the Python call path about 25 us per launch, so each
        # variant is captured into a CUDA graph (as the engine's decode step is) and replayed.
        res = []
        iters = 20
        for fn in (fused, unfused):
            for i in range(3):
                fn(i)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
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
            res.append(s.elapsed_time(e) / iters * 1e3)
        print(f"{Nn:>8} x {K:<6} {res[0]:9.1f} {wbytes / res[0] / 1e3:7.0f} {res[1]:16.1f} "
              f"{res[1] / res[0]:8.2f}")


if __name__ == "__main__":
    main()
