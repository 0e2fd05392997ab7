"""One-GPU checks of the fused tensor-parallel kernels with a group of one rank (the same
code path as with peers: park the partial rows, raise the flags, row owners reduce, add the
residual, normalise and store), plus a bounded wait that is made to run out."""
import ctypes

import pytest
import torch

from vllm_gcu_b200.ops import _native

pytestmark = pytest.mark.gpu


def _arr(*tensors):
    a = (ctypes.c_void_p * 8)()
    for i, t in enumerate(tensors):
        a[i] = t.data_ptr()
    return a


class _Ws:
    """Plain device tensors standing in for the symmetric buffers of a one-rank group."""

    def __init__(self, rows, n, dev):
        self.partial = torch.zeros(2 * rows, n, dtype=torch.bfloat16, device=dev)   # two parities
        self.out = torch.zeros(rows, n, dtype=torch.bfloat16, device=dev)
        self.res = torch.zeros(rows, n, dtype=torch.bfloat16, device=dev)
        self.ready = torch.zeros(rows // 128 * (n // 64) + 64, dtype=torch.int32, device=dev)
        self.done = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.words = torch.zeros(16, dtype=torch.int32, device=dev)
        self.base = torch.zeros(rows // 128 + 1, dtype=torch.int32, device=dev)
        # sentinel-tagged transport (mode 3): three rotating buffers each way
        self.cap = rows * n
        self.ll_slots = torch.full((3 * self.cap // 2,), -2147450880, dtype=torch.int32, device=dev)
        self.ll_out = torch.full((3 * self.cap // 2,), -2147450880, dtype=torch.int32, device=dev)
        self.ll_used = torch.zeros(6, dtype=torch.int64, device=dev)


def _run(ws, x, w, residual, norm_w, eps, bcast, mode=0):
    from vllm_gcu_b200.parallel import symm
    symm._register_sigs()
    M, K = x.shape
    N = w.shape[0]
    wp = ws.words.data_ptr()
    ll = mode == 3
    _native.call("b200_gemm_bf16_ar_norm", x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0),
                 N, M, N, K, _arr(ws.ll_slots if ll else ws.partial),
                 _arr(ws.ll_out if ll else ws.out),
                 _arr(ws.res) if norm_w is not None else None, _arr(ws.ready), _arr(ws.done),
                 ws.base.data_ptr(), wp, wp + 16, 0, 1, None if residual is None else residual.data_ptr(),
                 0 if residual is None else residual.stride(0),
                 None if norm_w is None else norm_w.data_ptr(), float(eps), int(bcast), mode,
                 None, None, None, ws.out.data_ptr(), ws.cap, ws.ll_used.data_ptr(),
                 _native.stream_ptr())


@pytest.mark.parametrize("M,N,K", [(8, 4096, 512), (256, 4096, 1792), (300, 2048, 1024),
                                   (1100, 4096, 512), (64, 8192, 256)])
@pytest.mark.parametrize("mode", ["norm", "norm_nores", "plain", "plain_res"])
def test_gemm_reduce_norm_one_rank(M, N, K, mode):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(M + N + K)
    x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    res = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16)
    nw = (1.0 + 0.1 * torch.randn(N, device=dev, generator=g)).to(torch.bfloat16)
    rows = -(-M // 128) * 128
    ws = _Ws(rows, N, dev)
    use_res = mode in ("norm", "plain_res")
    use_norm = mode.startswith("norm")
    for it in range(8):                       # later calls run on advanced epochs / rotated buffers
        # transports: owners pull / rows pushed to the owner / rows pushed to everyone /
        # sentinel-tagged push (needs the residual to stay with the owner)
        mode = (M + it) % 4
        _run(ws, x, w, res if use_res else None, nw if use_norm else None, 1e-5,
             0 if mode == 3 else it % 2, mode=mode)
        torch.cuda.synchronize()
        _native.check_status()
        z = x.float() @ w.float().t()
        z = z.to(torch.bfloat16).float()      # the partial product is parked as bf16
        if use_res:
            z = z + res.float()
        zb = z.to(torch.bfloat16)
        if use_norm:
            zf = zb.float()
            want = zf * torch.rsqrt(zf.pow(2).mean(-1, keepdim=True) + 1e-5) * nw.float()
            got_res = ws.res[:M].float()
            assert (got_res - zf).abs().max().item() <= 0.02 * max(1.0, zf.abs().max().item())
        else:
            want = zb.float()
        got = ws.out[:M].float()
        err = (got - want).abs().max().item()
        assert err <= 0.03 * max(1.0, want.abs().max().item()), (mode, it, err)
        ws.out.zero_()


def test_flag_wait_runs_out_and_the_context_stays_usable():
    """A two-rank all-reduce whose second rank never starts: the wait on its flag gives up
    after the (shortened) budget, the kernel returns, the status word names the timeout, and
    the next launch on the same context works."""
    from vllm_gcu_b200.parallel import symm
    symm._register_sigs()
    lib = _native.lib()
    lib.b200_set_flag_wait_limit.argtypes = [ctypes.c_uint]
    lib.b200_set_flag_wait_limit.restype = ctypes.c_int
    dev = torch.device("cuda")
    n = 4096
    src = [torch.ones(n, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    out = [torch.zeros(n, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(2)]
    words = torch.zeros(16, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    assert lib.b200_set_flag_wait_limit(2000) == 0
    try:
        _native.call("b200_allreduce", _arr(*src), _arr(*out), _arr(*flags), words.data_ptr(),
                     words.data_ptr() + 16, None, n, 0, 2, 0, _native.stream_ptr())
        torch.cuda.synchronize()              # returns: the wait was bounded
        with pytest.raises(_native.KernelTimeoutError):
            _native.check_status()
    finally:
        assert lib.b200_set_flag_wait_limit(0) == 0
    # same context, next launch: a one-rank all-reduce completes and is correct
    words.zero_()
    flags[0].zero_()
    _native.call("b200_allreduce", _arr(src[0]), _arr(out[0]), _arr(flags[0]), words.data_ptr(),
                 words.data_ptr() + 16, None, n, 0, 1, 0, _native.stream_ptr())
    torch.cuda.synchronize()
    _native.check_status()
    assert torch.equal(out[0], src[0])
