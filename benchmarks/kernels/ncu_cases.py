"""Small, self-terminating workloads for Nsight Compute captures of single kernels.

Each case allocates well under 2 GB, uses inputs larger than L2 where DRAM figures matter and
launches the kernel of interest a handful of times:

  python benchmarks/kernels/ncu_cases.py --case gemm_prefill   # 8192 x 4096 x 4096 bf16
  python benchmarks/kernels/ncu_cases.py --case gemm_decode    # 256 x 4096 x 14336 bf16
  python benchmarks/kernels/ncu_cases.py --case decode_attn    # B=256, ctx=1152, GQA 32/8
  python benchmarks/kernels/ncu_cases.py --case prefill_attn   # 8 x 1024 tokens, causal
  python benchmarks/kernels/ncu_cases.py --case gemm_fp8       # 4096 x 4096 x 4096 fp8
  python benchmarks/kernels/ncu_cases.py --case gemm_ar_single # fused all-reduce epilogue, p = 1
  python benchmarks/kernels/ncu_cases.py --case gemm_ar_norm_single      # + residual + RMSNorm,
                                                                        # 8192 rows, owners pull
  python benchmarks/kernels/ncu_cases.py --case gemm_ar_norm_single_ll   # 256 rows, tagged push
  python benchmarks/kernels/ncu_cases.py --case mla_decode     # latent attention, 128 heads
  python benchmarks/kernels/ncu_cases.py --case mla_decode_small  # latent attention, 16 heads
  python benchmarks/kernels/ncu_cases.py --case wna16_decode   # fused 4-bit de-quantising GEMM

Capture (one GPU):
  ncu --set full --clock-control none -k regex:<kernel> -s 2 -c 2 -o <output dir>/<name> \
      python benchmarks/kernels/ncu_cases.py --case <case>
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from vllm_gcu_b200.ops import _native  # noqa: E402
from vllm_gcu_b200.ops import cuda as C  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    dev = "cuda"
    torch.manual_seed(0)
    if a.case in ("gemm_prefill", "gemm_decode"):
        M, N, K = (8192, 4096, 4096) if a.case == "gemm_prefill" else (256, 4096, 14336)
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        fn = lambda: C.gemm_bf16(x, w, out=out)  # noqa: E731
    elif a.case == "gemm_fp8":
        M = N = K = 4096
        x = torch.randn(M, K, device=dev).to(torch.float8_e4m3fn)
        w = torch.randn(N, K, device=dev).to(torch.float8_e4m3fn)
        sa = torch.ones(M, device=dev)
        sb = torch.ones(N, device=dev)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        fn = lambda: C.gemm_q8(x, w, sa, sb, None, kind=0, out=out)  # noqa: E731
    elif a.case == "decode_attn":
        B, ctx, Hq, Hkv, D, bs = 256, 1152, 32, 8, 128, 16
        mb = ctx // bs
        nb = B * mb
        kc = torch.randn(nb, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
        vc = torch.randn(nb, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
        bt = torch.randperm(nb, device=dev).to(torch.int32).view(B, mb)
        sl = torch.full((B,), ctx, device=dev, dtype=torch.int32)
        q = torch.randn(B, Hq, D, device=dev, dtype=torch.bfloat16)
        out = torch.empty_like(q)
        fn = lambda: C.paged_decode(q, kc, vc, bt, sl, D ** -0.5, out=out, num_splits=1)  # noqa
    elif a.case == "prefill_attn":
        nseq, ql, Hq, Hkv, D, bs = 8, 1024, 32, 8, 128, 16
        nb = nseq * ql // bs
        kc = torch.randn(nb, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
        vc = torch.randn(nb, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
        bt = torch.randperm(nb, device=dev).to(torch.int32).view(nseq, ql // bs)
        q = torch.randn(nseq * ql, Hq, D, device=dev, dtype=torch.bfloat16)
        cu = torch.arange(0, nseq * ql + 1, ql, device=dev, dtype=torch.int32)
        sl = torch.full((nseq,), ql, device=dev, dtype=torch.int32)
        out = torch.empty_like(q)
        fn = lambda: C.varlen_prefill(q, kc, vc, bt, cu, sl, D ** -0.5, nseq * ql // 64,  # noqa
                                      out=out)
    elif a.case == "gemm_ar_single":
        # the fused row-parallel GEMM + all-reduce kernel with a one-rank "group": same code
        # path (partial tile -> flags -> reduce -> output) without a second process
        import ctypes
        M, N, K = 8192, 4096, 2048
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        part = torch.zeros(2 * M * N, device=dev, dtype=torch.bfloat16)
        out = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
        flags = torch.zeros(1 << 16, device=dev, dtype=torch.int32)
        words = torch.zeros(16, device=dev, dtype=torch.int32)
        lib = _native.lib()
        P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.b200_gemm_bf16_allreduce.argtypes = [P, L, P, L, L, I, I, I, P, P, P, P, P, P, I, I,
                                                 P, L, I, L, P]

        def arr(p):
            v = (ctypes.c_void_p * 8)()
            v[0] = p
            return v

        def fn():
            rc = lib.b200_gemm_bf16_allreduce(
                x.data_ptr(), K, w.data_ptr(), K, N, M, N, K, arr(part.data_ptr()),
                arr(out.data_ptr()), arr(flags.data_ptr()), arr(flags.data_ptr() + (1 << 17)),
                words.data_ptr(), words.data_ptr() + 16, 0, 1, None, 0, 1, M * N,
                torch.cuda.current_stream().cuda_stream)
            assert rc == 0, rc
    elif a.case in ("gemm_ar_norm_single", "gemm_ar_norm_single_ll"):
        # row-parallel GEMM + all-reduce + residual + RMSNorm in one kernel, one-rank group
        # (down_proj shard of Llama-3-8B at 8 ranks: K = 1792): park the partial rows, raise
        # the flags (or tag the rows), the row owners reduce, add the residual, normalise
        import ctypes
        from vllm_gcu_b200.parallel import symm
        symm._register_sigs()
        ll = a.case.endswith("_ll")
        M, N, K = (256, 4096, 1792) if ll else (8192, 4096, 1792)
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        res = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
        nw = torch.ones(N, device=dev, dtype=torch.bfloat16)
        partial = torch.zeros(2 * M, N, dtype=torch.bfloat16, device=dev)
        out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        res_out = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        ready = torch.zeros(M // 128 * (N // 64) + 64, dtype=torch.int32, device=dev)
        done = torch.zeros(M, dtype=torch.int32, device=dev)
        words = torch.zeros(16, dtype=torch.int32, device=dev)
        base = torch.zeros(M // 128 + 1, dtype=torch.int32, device=dev)
        cap = M * N
        tag = -2147450880                      # 0x80008000: two bf16 "row not written" marks
        ll_slots = torch.full((3 * cap // 2,), tag, dtype=torch.int32, device=dev)
        ll_out = torch.full((3 * cap // 2,), tag, dtype=torch.int32, device=dev)
        ll_used = torch.zeros(6, dtype=torch.int64, device=dev)

        def arr(t):
            v = (ctypes.c_void_p * 8)()
            v[0] = t.data_ptr()
            return v

        def fn():
            wp = words.data_ptr()
            _native.call("b200_gemm_bf16_ar_norm", x.data_ptr(), K, w.data_ptr(), K, N, M, N, K,
                         arr(ll_slots if ll else partial), arr(ll_out if ll else out),
                         arr(res_out), arr(ready), arr(done), base.data_ptr(), wp, wp + 16, 0, 1,
                         res.data_ptr(), N, nw.data_ptr(), 1e-5, 0, 3 if ll else 0, None, None,
                         None, out.data_ptr(), cap, ll_used.data_ptr(), _native.stream_ptr())
    elif a.case in ("mla_decode", "mla_decode_small"):
        # latent attention, B = 256, ctx = 1152: 340 MB of latent cache (larger than L2);
        # 128 heads (data-parallel attention) or 16 heads (tensor parallel 8)
        B, ctx, bs = 256, 1152, 16
        Nh = 128 if a.case == "mla_decode" else 16
        mb = ctx // bs
        cache = (torch.randn(B * mb, bs, 576, device=dev) * 0.3).to(torch.bfloat16)
        bt = torch.randperm(B * mb, device=dev).to(torch.int32).view(B, mb)
        sl = torch.full((B,), ctx, device=dev, dtype=torch.int32)
        q = (torch.randn(B, Nh, 576, device=dev) * 0.3).to(torch.bfloat16)
        out = torch.empty(B, Nh, 512, device=dev, dtype=torch.bfloat16)
        fn = lambda: C.mla_attention(q, cache, bt, sl, None, B, ctx, 576 ** -0.5, out=out,  # noqa
                                     splits=1)
    elif a.case == "wna16_decode":
        # fused de-quantising GEMM, 4-bit weights, M = 64, N = 28672, K = 4096 (59 MB packed;
        # three weight copies so that consecutive launches miss L2)
        M, Nn, K, g = 64, 28672, 4096, 128
        qws = [torch.randint(0, 256, (Nn, K // 2), dtype=torch.uint8, device=dev)
               for _ in range(3)]
        sc = (torch.rand(Nn, K // g, device=dev) * 0.02).to(torch.bfloat16)
        zs = (torch.rand(Nn, K // g, device=dev) * 0.1).to(torch.bfloat16)
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        state = {"i": 0}

        def fn():
            state["i"] += 1
            C.gemm_wna16(x, qws[state["i"] % 3], sc, zs, g, 4)
    else:
        raise SystemExit(f"unknown case {a.case}")
    for _ in range(a.iters):
        fn()
    torch.cuda.synchronize()
    _native.check_status()
    print("ok", a.case)


if __name__ == "__main__":
    main()
