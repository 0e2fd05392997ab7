"""GPU numerics of the 8-bit GEMMs, quantisation kernels and quantised linear methods."""
import pytest
import torch

from vllm_gcu_b200.layers import quant as Q
from vllm_gcu_b200.layers.linear import ColumnParallelLinear
from vllm_gcu_b200.ops import _native, ref

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def C():
    from vllm_gcu_b200.ops import cuda
    return cuda


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    if torch.cuda.is_available():
        _native.check_status()


def _close(a, b, rtol, atol):
    err = (a.float() - b.float()).abs()
    assert bool((err <= atol + rtol * b.float().abs()).all()), err.max().item()


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 1024, 4096), (8, 3584, 8192),
                                   (1000, 136, 272)])
def test_gemm_fp8_rowcol(C, M, N, K):
    torch.manual_seed(0)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    xq, xs = C.per_token_quant(x, "fp8")
    xr, xsr = ref.dynamic_per_token_fp8_quant(x)
    _close(xs, xsr, 1e-3, 1e-8)
    wq, ws = ref.dynamic_per_token_fp8_quant(w)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    got = C.gemm_q8(xq, wq, xs.flatten(), ws.flatten(), bias, kind=0)
    want = (xq.float() * xs) @ (wq.float() * ws).t() + bias.float()
    _close(got, want, 1e-2, 2e-2)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (257, 512, 7168), (16, 2048, 512)])
def test_gemm_fp8_block(C, M, N, K):
    torch.manual_seed(1)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda") * 0.05
    xq, xs = C.activation(x, "identity", mode="plain", quant="fp8_group128")
    xr, xsr = ref.per_token_group_fp8_quant(x, 128)
    _close(xs, xsr, 1e-3, 1e-8)
    nb, kb = (N + 127) // 128, K // 128
    wp = torch.zeros(nb * 128, K, device="cuda")
    wp[:N] = w
    wb = wp.view(nb, 128, kb, 128)
    sb = (wb.abs().amax(dim=(1, 3)) / 448.0).clamp_min(1e-12)
    wq = (wb / sb[:, None, :, None]).clamp(-448, 448).to(FP8).view(nb * 128, K)[:N].contiguous()
    got = C.gemm_q8(xq, wq, xs, sb, None, kind=1)
    wdq = (wq.float().view(-1) if False else
           (torch.cat([wq.float(), torch.zeros(nb * 128 - N, K, device="cuda")]).view(nb, 128, kb, 128)
            * sb[:, None, :, None]).view(nb * 128, K)[:N])
    xdq = (xq.float().view(M, kb, 128) * xs[..., None]).view(M, K)
    _close(got, xdq @ wdq.t(), 1e-2, 2e-2)


def test_gemm_int8(C):
    torch.manual_seed(2)
    M, N, K = 200, 768, 1024
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda") * 0.05
    xq, xs = C.per_token_quant(x, "int8")
    xr, xsr = ref.dynamic_scaled_int8_quant(x)
    assert ((xq.int() - xr.int()).abs() <= 1).all()
    ws = w.abs().amax(1) / 127
    wq = torch.round(w / ws[:, None]).clamp(-128, 127).to(torch.int8)
    got = C.gemm_q8(xq, wq, xs.flatten(), ws, None, kind=2)
    want = (xq.float() @ wq.float().t()) * xs * ws[None, :]
    _close(got, want, 1e-2, 2e-2)


def test_weight_dequant_and_quant_linear(C):
    torch.manual_seed(3)
    K, N, g = 512, 256, 128
    # AWQ layer on the GPU vs the same layer on the CPU reference path
    q = torch.randint(0, 16, (K, N), dtype=torch.uint8)
    z = torch.randint(0, 16, (K // g, N), dtype=torch.uint8)
    s = (torch.rand(K // g, N) * 0.02 + 0.01).to(torch.bfloat16)
    order = Q.AWQ_REVERSE_ORDER

    def pack(t):
        R, Cc = t.shape
        v = t.view(R, Cc // 8, 8).to(torch.int64)
        out = torch.zeros(R, Cc // 8, dtype=torch.int64)
        for c in range(8):
            out |= v[:, :, c] << (4 * order[c])
        out = out & 0xFFFFFFFF
        return torch.where(out >= 2 ** 31, out - 2 ** 32, out).to(torch.int32)

    outs = {}
    x = torch.randn(9, K, dtype=torch.bfloat16)
    for dev in ("cpu", "cuda"):
        layer = ColumnParallelLinear(K, N, dtype=torch.bfloat16, device=dev,
                                     quant_method=Q.WNA16LinearMethod("awq", 4, g))
        layer.load_weight("qweight", pack(q).to(dev))
        layer.load_weight("qzeros", pack(z).to(dev))
        layer.load_weight("scales", s.to(dev))
        layer.finalize()
        outs[dev] = layer(x.to(dev)).float().cpu()
    _close(outs["cuda"], outs["cpu"], 2e-2, 2e-2)
    # fp8 per-channel layer with on-the-fly weight quantisation from a bf16 checkpoint
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    res = {}
    for dev in ("cpu", "cuda"):
        layer = ColumnParallelLinear(K, N, dtype=torch.bfloat16, device=dev,
                                     quant_method=Q.Fp8LinearMethod(None, False))
        layer.load_weight("weight", w.to(dev))
        res[dev] = layer(x.to(dev)).float().cpu()
    # both sides quantise activations to fp8 independently: one e4m3 step (6 %) apart at most
    _close(res["cuda"], res["cpu"], 0.1, 0.1)
    _close(res["cuda"], (x.float() @ w.float().t()), 0.15, 0.15)
    qd, sd = C.per_tensor_fp8_quant(x.cuda())
    qr, sr = ref.dynamic_per_tensor_fp8_quant(x)
    _close(sd.cpu(), sr, 1e-3, 0)
    i8 = torch.randint(-128, 127, (1000,), dtype=torch.int8, device="cuda")
    sc = torch.tensor([0.03], device="cuda")
    zp = torch.tensor([5], dtype=torch.int32, device="cuda")
    _close(C.int8_dequant(i8, sc, zp, torch.float32),
           ref.static_scaled_int8_dequant(i8, sc, zp), 1e-5, 1e-6)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M,N,K,g", [(1, 256, 512, 128), (37, 200, 1024, 64), (128, 4096, 4096, 128),
                                     (256, 1024, 2048, 32), (200, 96, 256, 256)])
def test_fused_wna16_gemm_matches_dequant_reference(C, bits, M, N, K, g):
    """De-quantising GEMM (gemm_wna16.cu) against fp32 matmul on the de-quantised weights;
    the weights the kernel builds in shared memory are the ones the stand-alone kernel writes."""
    torch.manual_seed(bits * 100 + M)
    dev = "cuda"
    qmax = 16 if bits == 4 else 256
    q = torch.randint(0, qmax, (N, K), dtype=torch.uint8, device=dev)
    qw = (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous() if bits == 4 else q.contiguous()
    sc = (torch.rand(N, K // g, device=dev) * 0.02 + 0.005).to(torch.bfloat16)
    zero = torch.randint(0, qmax, (N, K // g), device=dev).float()
    zs = (zero * sc.float()).to(torch.bfloat16)
    x = (torch.randn(M, K, device=dev) * 0.5).to(torch.bfloat16)
    bias = torch.randn(N, device=dev).to(torch.bfloat16) if M % 2 else None
    got = C.gemm_wna16(x, qw, sc, zs, g, bits, bias)
    assert got is not None
    torch.cuda.synchronize()
    from vllm_gcu_b200.ops import _native
    _native.check_status()
    w = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
    C.weight_dequant(qw, sc, zs, w, g, bits)
    w_ref = (q.float() * sc.float().repeat_interleave(g, 1)
             - zs.float().repeat_interleave(g, 1)).to(torch.bfloat16)
    assert torch.equal(w, w_ref)
    want = x.float() @ w.float().t()
    if bias is not None:
        want = want + bias.float()
    err = (got.float() - want).abs().max().item()
    assert err < 1e-2 * want.abs().max().item() + 1e-2, err
    # shapes outside the kernel's range are declined, not mis-computed
    assert C.gemm_wna16(torch.zeros(300, K, dtype=torch.bfloat16, device=dev), qw, sc, zs, g,
                        bits) is None
