"""Quantised linear methods on the CPU reference path: checkpoint formats, load-time
re-packing and numerics against the de-quantised weights."""
import torch

from vllm_gcu_b200.layers import quant as Q
from vllm_gcu_b200.layers.linear import (ColumnParallelLinear, MergedColumnParallelLinear,
                                         RowParallelLinear)
from vllm_gcu_b200.ops import ref


def _to_i32(x: torch.Tensor) -> torch.Tensor:
    x = x & 0xFFFFFFFF
    return torch.where(x >= 2 ** 31, x - 2 ** 32, x).to(torch.int32)


def test_awq_linear_matches_dequantised():
    torch.manual_seed(0)
    K, N, g = 256, 128, 64
    q = torch.randint(0, 16, (K, N), dtype=torch.uint8)
    z = torch.randint(0, 16, (K // g, N), dtype=torch.uint8)
    s = (torch.rand(K // g, N) * 0.02 + 0.01)
    w = ((q.float() - z.float().repeat_interleave(g, 0)) * s.repeat_interleave(g, 0)).t()  # [N,K]
    order = Q.AWQ_REVERSE_ORDER

    def pack(t):
        R, C = t.shape
        v = t.view(R, C // 8, 8).to(torch.int64)
        out = torch.zeros(R, C // 8, dtype=torch.int64)
        for c in range(8):
            out |= v[:, :, c] << (4 * order[c])
        return _to_i32(out)

    layer = ColumnParallelLinear(K, N, dtype=torch.float32, device="cpu",
                                 quant_method=Q.WNA16LinearMethod("awq", 4, g))
    layer.load_weight("qweight", pack(q))
    layer.load_weight("qzeros", pack(z))
    layer.load_weight("scales", s)
    layer.finalize()
    x = torch.randn(5, K)
    assert torch.allclose(layer(x), x @ w.t(), atol=1e-4, rtol=1e-4)


def test_gptq_linear_4_and_8_bit():
    torch.manual_seed(1)
    for bits in (4, 8):
        K, N, g = 128, 64, 32
        per = 32 // bits
        q = torch.randint(0, 2 ** bits, (K, N), dtype=torch.int64)
        zp = torch.randint(1, 2 ** bits, (K // g, N), dtype=torch.int64)
        s = torch.rand(K // g, N) * 0.02 + 0.01
        w = ((q.float() - zp.float().repeat_interleave(g, 0)) * s.repeat_interleave(g, 0)).t()
        qw = torch.zeros(K // per, N, dtype=torch.int64)
        for i in range(per):
            qw |= q[i::per] << (bits * i)
        qz = torch.zeros(K // g, N // per, dtype=torch.int64)
        for i in range(per):
            qz |= (zp[:, i::per] - 1) << (bits * i)
        layer = RowParallelLinear(K, N, dtype=torch.float32, device="cpu",
                                  quant_method=Q.WNA16LinearMethod("gptq", bits, g))
        layer.load_weight("qweight", _to_i32(qw))
        layer.load_weight("qzeros", _to_i32(qz))
        layer.load_weight("scales", s)
        layer.load_weight("g_idx", torch.arange(K, dtype=torch.int32) // g)
        layer.finalize()
        x = torch.randn(3, K)
        assert torch.allclose(layer(x), x @ w.t(), atol=1e-4, rtol=1e-4)


def test_fp8_per_channel_and_block():
    torch.manual_seed(2)
    K, N = 256, 384
    w = torch.randn(N, K) * 0.05
    x = torch.randn(7, K)
    # per channel, dynamic per-token activations
    qw, sw = ref.dynamic_per_token_fp8_quant(w)
    layer = ColumnParallelLinear(K, N, dtype=torch.float32, device="cpu",
                                 quant_method=Q.Fp8LinearMethod(None, False))
    layer.load_weight("weight", qw)
    layer.load_weight("weight_scale", sw.flatten())
    y = layer(x)
    assert (y - x @ w.t()).abs().max() < 0.15
    # 128x128 block scales + 1x128 activation scales
    wb = w.view(N // 128, 128, K // 128, 128)
    sb = wb.abs().amax(dim=(1, 3)) / 448.0
    qb = (wb / sb[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(N, K)
    layer2 = MergedColumnParallelLinear(K, [256, 128], dtype=torch.float32, device="cpu",
                                        quant_method=Q.Fp8LinearMethod([128, 128], False))
    layer2.load_weight("weight", qb[:256], 0)
    layer2.load_weight("weight", qb[256:], 1)
    layer2.load_weight("weight_scale_inv", sb[:2], 0)
    layer2.load_weight("weight_scale_inv", sb[2:], 1)
    y2 = layer2(x)
    assert (y2 - x @ w.t()).abs().max() < 0.15


def test_int8_w8a8():
    torch.manual_seed(3)
    K, N = 128, 96
    w = torch.randn(N, K) * 0.05
    ws = w.abs().amax(1) / 127
    qw = torch.round(w / ws[:, None]).clamp(-128, 127).to(torch.int8)
    x = torch.randn(4, K)
    layer = ColumnParallelLinear(K, N, bias=True, dtype=torch.float32, device="cpu",
                                 quant_method=Q.Int8LinearMethod(False))
    layer.load_weight("weight", qw)
    layer.load_weight("out_scales", ws)
    layer.load_weight("bias", torch.ones(N))
    assert (layer(x) - (x @ w.t() + 1)).abs().max() < 0.05
