"""Quantised linear layers under tensor parallelism (two CPU ranks, gloo): every checkpoint
format is loaded from full tensors, each rank keeps its shard (packed words, group scales and
zero points, per-channel scales, 128 x 128 block scales) and the sharded result equals the
product with the de-quantised full weight: merged column-parallel layers with the outputs
gathered, row-parallel layers through their all-reduce."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

def _check(rank, world):
    from vllm_gcu_b200.layers import quant as Q
    from vllm_gcu_b200.layers.linear import MergedColumnParallelLinear, RowParallelLinear, QKVParallelLinear
    from vllm_gcu_b200.ops import ref
    from vllm_gcu_b200.parallel.communicator import get_comm
    from test_quant_cpu import _awq_pack, _to_i32
    comm = get_comm("tp")
    torch.manual_seed(0)
    K, N1, N2, g = 512, 256, 256, 64
    N = N1 + N2
    x = torch.randn(5, K)
    xr = torch.randn(5, N)
    def report(name, got, want, tol):
        err = (got - want).abs().max().item()
        assert got.shape == want.shape and err < tol, f"{name}: error {err:.3e} (limit {tol})"
    def gather_cols(y, sizes):
        # merged column layer output on each rank: [n1/tp | n2/tp]; rebuild [n1 | n2]
        parts = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(parts, y.contiguous())
        outs, off = [], 0
        for s in sizes:
            loc = s // world
            outs.append(torch.cat([p[:, off:off + loc] for p in parts], 1))
            off += loc
        return torch.cat(outs, 1)
    # ---- AWQ
    q = torch.randint(0, 16, (K, N), dtype=torch.uint8)
    z = torch.randint(0, 16, (K // g, N), dtype=torch.uint8)
    s = torch.rand(K // g, N) * 0.02 + 0.01
    w = ((q.float() - z.float().repeat_interleave(g, 0)) * s.repeat_interleave(g, 0)).t()
    col = MergedColumnParallelLinear(K, [N1, N2], dtype=torch.float32, device="cpu",
          quant_method=Q.WNA16LinearMethod("awq", 4, g))
    for i, (lo, hi) in enumerate(((0, N1), (N1, N))):
        col.load_weight("qweight", _awq_pack(q[:, lo:hi]), i)
        col.load_weight("qzeros", _awq_pack(z[:, lo:hi]), i)
        col.load_weight("scales", s[:, lo:hi], i)
    col.finalize()
    report("awq col", gather_cols(col(x), [N1, N2]), x @ w.t(), 1e-3)
    # row: in = N (use w2 [K_out=K? ] ) : build row layer in_features=N, out=K
    q2 = torch.randint(0, 16, (N, K), dtype=torch.uint8)
    z2 = torch.randint(0, 16, (N // g, K), dtype=torch.uint8)
    s2 = torch.rand(N // g, K) * 0.02 + 0.01
    w2 = ((q2.float() - z2.float().repeat_interleave(g, 0)) * s2.repeat_interleave(g, 0)).t()   # [K, N]
    row = RowParallelLinear(N, K, dtype=torch.float32, device="cpu",
          quant_method=Q.WNA16LinearMethod("awq", 4, g))
    row.load_weight("qweight", _awq_pack(q2))
    row.load_weight("qzeros", _awq_pack(z2))
    row.load_weight("scales", s2)
    row.finalize()
    loc = N // world
    report("awq row", row(xr[:, rank * loc:(rank + 1) * loc].contiguous()), xr @ w2.t(), 1e-3)
    # ---- GPTQ 4/8
    for bits in (4, 8):
        per = 32 // bits
        qq = torch.randint(0, 2 ** bits, (N, K), dtype=torch.int64)
        zp = torch.randint(1, 2 ** bits, (N // g, K), dtype=torch.int64)
        ss = torch.rand(N // g, K) * 0.02 + 0.01
        wg = ((qq.float() - zp.float().repeat_interleave(g, 0)) * ss.repeat_interleave(g, 0)).t()
        qw = torch.zeros(N // per, K, dtype=torch.int64)
        for i in range(per):
            qw |= qq[i::per] << (bits * i)
        qz = torch.zeros(N // g, K // per, dtype=torch.int64)
        for i in range(per):
            qz |= (zp[:, i::per] - 1) << (bits * i)
        row = RowParallelLinear(N, K, dtype=torch.float32, device="cpu",
              quant_method=Q.WNA16LinearMethod("gptq", bits, g))
        row.load_weight("qweight", _to_i32(qw))
        row.load_weight("qzeros", _to_i32(qz))
        row.load_weight("scales", ss)
        row.load_weight("g_idx", torch.arange(N, dtype=torch.int32) // g)
        row.finalize()
        report(f"gptq{bits} row", row(xr[:, rank * loc:(rank + 1) * loc].contiguous()), xr @ wg.t(), 1e-3)
        # column (merged) gptq
        qc = torch.randint(0, 2 ** bits, (K, N), dtype=torch.int64)
        zc = torch.randint(1, 2 ** bits, (K // g, N), dtype=torch.int64)
        sc = torch.rand(K // g, N) * 0.02 + 0.01
        wc = ((qc.float() - zc.float().repeat_interleave(g, 0)) * sc.repeat_interleave(g, 0)).t()
        col = MergedColumnParallelLinear(K, [N1, N2], dtype=torch.float32, device="cpu",
              quant_method=Q.WNA16LinearMethod("gptq", bits, g))
        for i, (lo, hi) in enumerate(((0, N1), (N1, N))):
            qwc = torch.zeros(K // per, hi - lo, dtype=torch.int64)
            for j in range(per):
                qwc |= qc[j::per, lo:hi] << (bits * j)
            qzc = torch.zeros(K // g, (hi - lo) // per, dtype=torch.int64)
            for j in range(per):
                qzc |= (zc[:, lo:hi][:, j::per] - 1) << (bits * j)
            col.load_weight("qweight", _to_i32(qwc), i)
            col.load_weight("qzeros", _to_i32(qzc), i)
            col.load_weight("scales", sc[:, lo:hi], i)
            col.load_weight("g_idx", torch.arange(K, dtype=torch.int32) // g, i)
        col.finalize()
        report(f"gptq{bits} col", gather_cols(col(x), [N1, N2]), x @ wc.t(), 1e-3)
    # ---- fp8 per channel and block
    w = torch.randn(N, K) * 0.05
    qw, sw = ref.dynamic_per_token_fp8_quant(w)
    col = MergedColumnParallelLinear(K, [N1, N2], dtype=torch.float32, device="cpu",
          quant_method=Q.Fp8LinearMethod(None, False))
    col.load_weight("weight", qw[:N1], 0)
    col.load_weight("weight", qw[N1:], 1)
    col.load_weight("weight_scale", sw.flatten()[:N1], 0)
    col.load_weight("weight_scale", sw.flatten()[N1:], 1)
    report("fp8 ch col", gather_cols(col(x), [N1, N2]), x @ w.t(), 0.25)
    wr = torch.randn(K, N) * 0.05
    qwr, swr = ref.dynamic_per_token_fp8_quant(wr)
    row = RowParallelLinear(N, K, dtype=torch.float32, device="cpu",
          quant_method=Q.Fp8LinearMethod(None, False))
    row.load_weight("weight", qwr)
    row.load_weight("weight_scale", swr.flatten())
    report("fp8 ch row", row(xr[:, rank * loc:(rank + 1) * loc].contiguous()), xr @ wr.t(), 0.25)
    wb = w.view(N // 128, 128, K // 128, 128)
    sb = wb.abs().amax(dim=(1, 3)) / 448.0
    qb = (wb / sb[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(N, K)
    col = MergedColumnParallelLinear(K, [N1, N2], dtype=torch.float32, device="cpu",
          quant_method=Q.Fp8LinearMethod([128, 128], False))
    col.load_weight("weight", qb[:N1], 0)
    col.load_weight("weight", qb[N1:], 1)
    col.load_weight("weight_scale_inv", sb[:N1 // 128], 0)
    col.load_weight("weight_scale_inv", sb[N1 // 128:], 1)
    report("fp8 blk col", gather_cols(col(x), [N1, N2]), x @ w.t(), 0.25)
    wb = wr.view(K // 128, 128, N // 128, 128)
    sb = wb.abs().amax(dim=(1, 3)) / 448.0
    qb = (wb / sb[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(K, N)
    row = RowParallelLinear(N, K, dtype=torch.float32, device="cpu",
          quant_method=Q.Fp8LinearMethod([128, 128], False))
    row.load_weight("weight", qb)
    row.load_weight("weight_scale_inv", sb)
    report("fp8 blk row", row(xr[:, rank * loc:(rank + 1) * loc].contiguous()), xr @ wr.t(), 0.25)
    # ---- int8
    ws = w.abs().amax(1) / 127
    qi = torch.round(w / ws[:, None]).clamp(-128, 127).to(torch.int8)
    col = MergedColumnParallelLinear(K, [N1, N2], dtype=torch.float32, device="cpu",
          quant_method=Q.Int8LinearMethod(False))
    col.load_weight("weight", qi[:N1], 0)
    col.load_weight("weight", qi[N1:], 1)
    col.load_weight("out_scales", ws[:N1], 0)
    col.load_weight("out_scales", ws[N1:], 1)
    report("int8 col", gather_cols(col(x), [N1, N2]), x @ w.t(), 0.1)
    wsr = wr.abs().amax(1) / 127
    qir = torch.round(wr / wsr[:, None]).clamp(-128, 127).to(torch.int8)
    row = RowParallelLinear(N, K, bias=True, dtype=torch.float32, device="cpu",
          quant_method=Q.Int8LinearMethod(False))
    row.load_weight("weight", qir)
    row.load_weight("out_scales", wsr)
    row.load_weight("bias", torch.ones(K))
    report("int8 row", row(xr[:, rank * loc:(rank + 1) * loc].contiguous()), xr @ wr.t() + 1, 0.15)

def _worker(rank, world, port):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    from vllm_gcu_b200.parallel.state import init_distributed
    init_distributed(tp=world, backend="gloo")
    _check(rank, world)
    dist.barrier()
    dist.destroy_process_group()
@pytest.mark.timeout(300)
def test_quantised_linear_layers_shard_correctly_over_two_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port), nprocs=2, join=True)
