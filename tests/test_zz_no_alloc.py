"""The allocation-free decode entry point, called through its exported C symbol.

Some hosts of this library cannot give it a workspace: code running after a memory pool
has claimed the whole GPU, callbacks that may not call cudaMalloc/cudaFree because those
synchronise the device, or an embedding through the plain C ABI with no allocator at hand.
``b200_paged_decode_noalloc`` serves them from a fixed workspace inside the library.  This
test checks it against the regular entry point (which gets a torch-allocated workspace) on
two consecutive calls with different inputs, so leftovers of the first call in the shared
workspace would show up in the second, and checks the size limit.

The file name sorts last on purpose: a run that stops at the first failure has then
already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _lib():
    from vllm_gcu_b200.ops import _native
    lib = ctypes.CDLL(str(_native.lib_path()))
    lib.b200_paged_decode_noalloc.restype = I
    lib.b200_paged_decode_noalloc.argtypes = [P, L, P, L, P, P, L, L, L, P, I, I, P, I, I, I, I, I,
                                              F, I, P]
    lib.b200_paged_decode.restype = I
    lib.b200_paged_decode.argtypes = [P, L, P, L, P, P, L, L, L, P, I, I, P, P, P, I, I, I, I, I,
                                      F, I, P]
    lib.b200_noalloc_last_error.restype = ctypes.c_char_p
    lib.b200_noalloc_last_error.argtypes = []
    return lib


def _case(seed, B, lens, Hq=32, Hkv=8, D=128, bs=16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mb = (max(lens) + bs - 1) // bs + 1
    nb = B * mb + 2
    kc = torch.randn(nb, bs, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    vc = torch.randn(nb, bs, Hkv, D, device="cuda", dtype=torch.bfloat16, generator=g)
    bt = torch.randperm(nb, device="cuda", generator=g)[: B * mb].to(torch.int32).view(B, mb)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16, generator=g)
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    return q, kc, vc, bt.contiguous(), sl


def _run(lib, use_noalloc, q, kc, vc, bt, sl, splits):
    B, Hq, D = q.shape
    nb, bs, Hkv, _ = kc.shape
    out = torch.empty_like(q)
    stream = torch.cuda.current_stream().cuda_stream
    common_a = (q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kc.data_ptr(),
                vc.data_ptr(), kc.stride(1), kc.stride(2), nb * bs, bt.data_ptr(), bt.stride(0), bs,
                sl.data_ptr())
    common_b = (splits, B, Hq, Hkv, D, float(D ** -0.5), 0, stream)
    if use_noalloc:
        rc = lib.b200_paged_decode_noalloc(*common_a, *common_b)
    else:
        tmp_out = torch.empty(B * Hq * splits * D, device="cuda", dtype=torch.float32)
        tmp_lse = torch.empty(B * Hq * splits, device="cuda", dtype=torch.float32)
        rc = lib.b200_paged_decode(*common_a, tmp_out.data_ptr(), tmp_lse.data_ptr(), *common_b)
    torch.cuda.synchronize()
    return rc, out


def test_noalloc_decode_matches_regular_entry_point_twice():
    lib = _lib()
    cases = [(11, 5, [700, 33, 1200, 64, 257], 4), (12, 3, [90, 2000, 511], 6)]
    for seed, B, lens, splits in cases:          # two calls in a row share the workspace
        args = _case(seed, B, lens)
        rc_a, want = _run(lib, False, *args, splits)
        rc_b, got = _run(lib, True, *args, splits)
        assert rc_a == 0 and rc_b == 0, lib.b200_noalloc_last_error()
        err = (got.float() - want.float()).abs()
        tol = 2e-2 + 2e-2 * want.float().abs()
        assert bool((err <= tol).all()), err.max().item()


def test_noalloc_rejects_oversized_problem():
    lib = _lib()
    args = _case(13, 64, [64] * 64)
    rc, _ = _run(lib, True, *args, 32)     # 64 * 32 * 32 * 128 floats > the built-in workspace
    assert rc == -12
    assert b"workspace" in lib.b200_noalloc_last_error()
