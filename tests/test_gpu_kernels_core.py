"""GPU numerics of the core kernels against the fp32 PyTorch reference."""
import math

import pytest
import torch

from vllm_gcu_b200.ops import _native, ref

pytestmark = pytest.mark.gpu


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
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = (err > tol).float().mean().item()
    assert bad == 0.0, f"{bad:.2%} out of tolerance, max err {err.max().item():.4g}"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 4096), (1, 4096, 4096),
                                   (77, 6144, 4096), (333, 256, 200), (1024, 28672, 4096),
                                   (8192, 4096, 4096), (130, 136, 72)])
def test_gemm_bf16(C, M, N, K):
    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    out = C.gemm_bf16(a, b)
    want = ref.gemm(a, b, out_dtype=torch.float32)
    _close(out, want, 2e-2, 2e-2 * math.sqrt(K) * 0.05)


@pytest.mark.parametrize("M,N,K", [(256, 6144, 4096), (256, 4096, 14336), (200, 4096, 4096),
                                   (129, 28672, 4096), (64, 2048, 2048), (7, 136, 72),
                                   (256, 128256, 1024), (128, 64, 8192), (256, 1024, 256)])
def test_gemm_skinny_decode_shapes(C, M, N, K, monkeypatch):
    """Weight-streaming kernel for M <= 256 (column tile x K slice per CTA, split-K reduce):
    same result as the fp32 reference, also on repeated launches (the counters must come back
    to zero) and identical to the persistent-tile kernel within bf16 rounding."""
    assert C.USE_SKINNY_GEMM and M <= C.SKINNY_MAX_M
    monkeypatch.setattr(C, "USE_PAIR_GEMM", False)          # (wide shapes would go to CTA pairs)
    monkeypatch.setattr(C, "SKINNY_ALLOW_SPLIT", True)      # exercise the split-K path too
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") / math.sqrt(K)).to(torch.bfloat16)
    want = ref.gemm(a, b, out_dtype=torch.float32)
    first = None
    for _ in range(3):
        out = C.gemm_bf16(a, b)
        _close(out, want, 2e-2, 2e-2)
        if first is None:
            first = out.clone()
        assert torch.equal(out, first), "split-K reduction must be reproducible"
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    _close(C.gemm_bf16(a, b, bias=bias), want + bias.float(), 2e-2, 3e-2)
    if N % 256 == 0:
        got = C.gemm_bf16(a, b, epilogue=C.EPI_SILU_MUL)
        w4 = want.view(M, N // 64, 2, 32)
        _close(got, (torch.nn.functional.silu(w4[:, :, 0]) * w4[:, :, 1]).reshape(M, N // 2),
               3e-2, 3e-2)


@pytest.mark.parametrize("M,N,K", [(1100, 512, 320), (2048, 1024, 4096), (1024, 256, 64)])
def test_gemm_wide2_large_m(C, M, N, K, monkeypatch):
    """Persistent 256 x 256 tile kernel (large M, N a multiple of 256): plain, bias and
    SiLU-mul epilogues, ragged last row tile."""
    monkeypatch.setattr(C, "USE_PAIR_GEMM", False)
    assert C.USE_WIDE2_GEMM and M >= C.WIDE2_MIN_M
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") / math.sqrt(K)).to(torch.bfloat16)
    want = ref.gemm(a, b, out_dtype=torch.float32)
    _close(C.gemm_bf16(a, b), want, 2e-2, 2e-2)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    _close(C.gemm_bf16(a, b, bias=bias), want + bias.float(), 2e-2, 3e-2)
    got = C.gemm_bf16(a, b, epilogue=C.EPI_SILU_MUL)
    w4 = want.view(M, N // 64, 2, 32)
    _close(got, (torch.nn.functional.silu(w4[:, :, 0]) * w4[:, :, 1]).reshape(M, N // 2),
           3e-2, 3e-2)


@pytest.mark.parametrize("mt", ["1", "2"])
@pytest.mark.parametrize("M,N,K", [(1100, 512, 320 + 64), (2048, 1024, 4096), (1024, 256, 64),
                                   (4096, 3584, 4096), (8192, 768, 512), (256, 28672, 512),
                                   (200, 16384, 256), (600, 8192, 128)])
def test_gemm_cta_pair_large_m(C, M, N, K, mt, monkeypatch):
    """One output tile per pair of CTAs (`tcgen05.mma.cta_group::2`, a cluster of two): plain,
    bias and SiLU-mul epilogues, ragged last row tile, both tile shapes (256 x 256 with two
    accumulator sets, 512 x 256 with one), repeated launches."""
    monkeypatch.setenv("VLLM_B200_PAIR_MT", mt)
    assert C.USE_PAIR_GEMM and (M >= C.WIDE2_MIN_M or
                                -(-M // 256) * (N // 256) >= C.PAIR_MIN_TILES)
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") / math.sqrt(K)).to(torch.bfloat16)
    want = ref.gemm(a, b, out_dtype=torch.float32)
    direct = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    rc = _native.lib().b200_gemm_pair(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0),
                                      direct.data_ptr(), N, M, N, K, None, 0,
                                      _native.stream_ptr())
    assert rc == 0, rc                         # the pair kernel takes this shape on this device
    _close(direct, want, 2e-2, 2e-2)
    first = C.gemm_bf16(a, b)
    _close(first, want, 2e-2, 2e-2)
    assert torch.equal(C.gemm_bf16(a, b), first)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    _close(C.gemm_bf16(a, b, bias=bias), want + bias.float(), 2e-2, 3e-2)
    got = C.gemm_bf16(a, b, epilogue=C.EPI_SILU_MUL)
    w4 = want.view(M, N // 64, 2, 32)
    _close(got, (torch.nn.functional.silu(w4[:, :, 0]) * w4[:, :, 1]).reshape(M, N // 2),
           3e-2, 3e-2)
    torch.cuda.synchronize()
    _native.check_status()


@pytest.mark.parametrize("M,N,K,epi", [(256, 4096, 4096, 0), (256, 6144, 1024, 0),
                                       (200, 1024, 2048, 1), (512, 4096, 4096, 0),
                                       (130, 2048, 1024, 2)])
def test_gemm_cta_pair_k_split(C, M, N, K, epi, monkeypatch):
    """K split of the CTA-pair kernel (one tile and K slice per pair, fp32 partial sums meet at
    a counter, every CTA reduces a row slice): off by default (measured slower than the
    weight-streaming kernel), kept correct: same result as the reference, bitwise equal on
    repeated launches (the counters return to zero)."""
    monkeypatch.setattr(C, "USE_PAIR_SPLIT", True)
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") / math.sqrt(K)).to(torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16) if epi == 1 else None
    wsp = C._pair_split_workspace(a.device)
    assert wsp is not None
    want = ref.gemm(a, b, out_dtype=torch.float32)
    if epi == 1:
        want = want + bias.float()
    if epi == 2:
        w4 = want.view(M, N // 64, 2, 32)
        want = (torch.nn.functional.silu(w4[:, :, 0]) * w4[:, :, 1]).reshape(M, N // 2)
    first = C.gemm_bf16(a, b, bias=bias, epilogue=epi)
    _close(first, want, 3e-2, 3e-2)
    assert torch.equal(C.gemm_bf16(a, b, bias=bias, epilogue=epi), first)
    torch.cuda.synchronize()
    assert int(wsp[1].abs().sum()) == 0
    _native.check_status()


def test_gemm_bf16_epilogues(C):
    torch.manual_seed(1)
    M, N, K = 200, 1024, 512
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    atol = 2e-2 * math.sqrt(K) * 0.05
    _close(C.gemm_bf16(a, b, bias=bias), ref.gemm(a, b, bias=bias, out_dtype=torch.float32),
           2e-2, atol)
    _close(C.gemm_bf16(a, b, residual=res),
           ref.gemm(a, b, residual=res, out_dtype=torch.float32), 2e-2, atol)
    out32 = C.gemm_bf16(a, b, epilogue=C.EPI_FP32)
    assert out32.dtype == torch.float32
    _close(out32, ref.gemm(a, b, out_dtype=torch.float32), 1e-3, 1e-3)
    wg, wu = b[: N // 2].contiguous(), b[N // 2:].contiguous()
    wi = ref.interleave_gate_up(wg, wu)
    got = C.gemm_bf16(a, wi, epilogue=C.EPI_SILU_MUL)
    want = ref.silu_and_mul(torch.cat([ref.gemm(a, wg, out_dtype=torch.float32),
                                       ref.gemm(a, wu, out_dtype=torch.float32)], -1))
    _close(got, want, 3e-2, 3e-2)


def test_gemm_bf16_strided_views(C):
    torch.manual_seed(2)
    big = torch.randn(300, 1024, device="cuda", dtype=torch.bfloat16)
    a = big[:, 256:768]
    b = (torch.randn(384, 512, device="cuda") * 0.05).to(torch.bfloat16)
    outbuf = torch.zeros(300, 1024, device="cuda", dtype=torch.bfloat16)
    C.gemm_bf16(a, b, out=outbuf[:, 128:512])
    _close(outbuf[:, 128:512], ref.gemm(a, b, out_dtype=torch.float32), 2e-2, 3e-2)
    assert outbuf[:, :128].abs().sum().item() == 0 and outbuf[:, 512:].abs().sum().item() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,H", [(1, 256), (7, 4096), (33, 7168), (5, 8192 + 128)])
def test_rms_norm_family(C, dtype, T, H):
    torch.manual_seed(3)
    x = torch.randn(T, H, device="cuda", dtype=dtype)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(dtype)
    r = torch.randn(T, H, device="cuda", dtype=dtype)
    _close(C.norm(x, w, 1e-6), ref.rms_norm(x, w, 1e-6), 1e-2, 1e-2)
    r2 = r.clone()
    got = C.norm(x, w, 1e-6, residual=r2)
    want, want_r = ref.fused_add_rms_norm(x, r, w, 1e-6)
    _close(got, want, 1e-2, 1e-2)
    _close(r2, want_r, 1e-2, 1e-2)
    # dynamic group quant
    q, s = C.norm(x, w, 1e-6, quant="fp8_group128")
    qr, sr, _ = ref.rms_norm_quant(x, w, 1e-6, "fp8_group128")
    _close(s, sr, 2e-2, 1e-6)
    deq = q.float().view(T, H // 128, 128) * s[..., None]
    deqr = qr.float().view(T, H // 128, 128) * sr[..., None]
    _close(deq, deqr, 0.13, 0.02)
    q, s = C.norm(x, w, 1e-6, quant="fp8_token")
    qr, sr, _ = ref.rms_norm_quant(x, w, 1e-6, "fp8_token")
    _close(s, sr, 2e-2, 1e-6)
    _close(q.float() * s, qr.float() * sr, 0.13, 0.05)
    sc = torch.tensor([0.05], device="cuda")
    q = C.norm(x, w, 1e-6, quant="int8_static", scale=sc)
    qr, _, _ = ref.rms_norm_quant(x, w, 1e-6, "int8_static", scale=sc)
    assert ((q.int() - qr.int()).abs() <= 1).all()


@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_tanh", "fatrelu"])
def test_act_and_mul(C, act):
    torch.manual_seed(4)
    x = torch.randn(19, 2 * 1408, device="cuda", dtype=torch.bfloat16)
    _close(C.activation(x, act, threshold=0.1), ref.act_and_mul(x, act, 0.1), 2e-2, 2e-2)
    if act == "silu":
        q, s = C.activation(x, act, quant="fp8_group128")
        qr, sr = ref.per_token_group_fp8_quant(ref.silu_and_mul(x), 128)
        _close(s, sr, 2e-2, 1e-6)
        n = torch.tensor([5], device="cuda", dtype=torch.int32)
        out = torch.zeros(19, 1408, device="cuda", dtype=torch.bfloat16)
        C.activation(x, act, out=out, valid_rows=n)
        assert out[5:].abs().sum().item() == 0
        _close(out[:5], ref.silu_and_mul(x[:5]), 2e-2, 2e-2)
        _close(C.activation(x, "silu", mode="mul_act"), ref.mul_and_silu(x), 2e-2, 2e-2)
    for name in ("gelu_new", "gelu_fast", "gelu_quick"):
        _close(C.activation(x, name, mode="plain"), ref.activation(x, name), 2e-2, 2e-2)


@pytest.mark.parametrize("is_neox", [True, False])
def test_rope_and_cache_flash(C, is_neox):
    torch.manual_seed(5)
    T, Hq, Hkv, D, bs, nb = 37, 8, 2, 128, 16, 12
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    pos = torch.randint(0, 500, (T,), device="cuda")
    cs = ref.make_cos_sin_cache(D, 512, 10000.0).cuda().to(torch.bfloat16)
    slots = torch.randperm(nb * bs, device="cuda")[:T]
    slots[3] = -1
    kc = torch.zeros(nb, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q_ref, k_ref = ref.rotary_embedding(pos, q, k, D, cs, is_neox)
    kc_r, vc_r = kc.clone(), vc.clone()
    ref.reshape_and_cache_flash(k_ref, v, kc_r, vc_r, slots)
    C.rope_cache_flash(q, k, v, pos, cs, is_neox, D, slots, kc, vc)
    _close(q, q_ref, 2e-2, 2e-2)
    _close(k, k_ref, 2e-2, 2e-2)
    _close(kc, kc_r, 2e-2, 2e-2)
    assert torch.equal(vc, vc_r)


def _make_paged(B, lens, Hkv, D, bs, dtype=torch.bfloat16):
    max_blocks = (max(lens) + bs - 1) // bs + 1
    nb = B * max_blocks + 3
    kc = torch.randn(nb, bs, Hkv, D, device="cuda", dtype=dtype)
    vc = torch.randn(nb, bs, Hkv, D, device="cuda", dtype=dtype)
    perm = torch.randperm(nb, device="cuda")[: B * max_blocks].to(torch.int32)
    bt = perm.view(B, max_blocks).contiguous()
    return kc, vc, bt


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (4, 2, 64), (8, 1, 128), (16, 16, 128)])
@pytest.mark.parametrize("splits", [1, 3])
def test_paged_decode(C, Hq, Hkv, D, splits):
    torch.manual_seed(6)
    lens = [1, 17, 64, 65, 300, 1000, 33]
    B = len(lens)
    kc, vc, bt = _make_paged(B, lens, Hkv, D, 16)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    scale = D ** -0.5
    got = C.paged_decode(q, kc, vc, bt, sl, scale, num_splits=splits)
    want = ref.paged_attention_decode(q, kc, vc, bt, sl, scale)
    _close(got, want, 2e-2, 2e-2)


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 128), (4, 2, 64)])
def test_varlen_prefill(C, Hq, Hkv, D):
    torch.manual_seed(7)
    q_lens = [5, 64, 130, 1, 77]
    ctx = [0, 16, 50, 200, 3]
    lens = [a + b for a, b in zip(q_lens, ctx)]
    B = len(lens)
    kc, vc, bt = _make_paged(B, lens, Hkv, D, 16)
    T = sum(q_lens)
    q = torch.randn(T, Hq, D, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device="cuda",
                      dtype=torch.int32)
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    tiles = sum((x + 63) // 64 for x in q_lens)
    scale = D ** -0.5
    got, lse = C.varlen_prefill(q, kc, vc, bt, cu, sl, scale, tiles, return_lse=True)
    want, lse_r = ref.varlen_prefill_attention(q, kc, vc, bt, cu, sl, scale, return_lse=True)
    _close(got, want, 2e-2, 2e-2)
    _close(lse, lse_r, 1e-2, 1e-2)


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 8, 128), (12, 4, 64)])
def test_alibi_decode_and_prefill(C, Hq, Hkv, D):
    """ALiBi slopes in the decode kernel (with and without KV splits) and in the prefill kernel
    (cached prefixes, causal): slope * (key position - query position) added to the scores."""
    from vllm_gcu_b200.layers.attention import alibi_slopes
    torch.manual_seed(23)
    slopes = alibi_slopes(Hq).cuda()
    assert slopes.shape == (Hq,) and float(slopes[0]) == pytest.approx(2.0 ** (-8.0 / 8), rel=1e-6)
    lens = [1, 17, 64, 65, 300, 1000, 33]
    B = len(lens)
    kc, vc, bt = _make_paged(B, lens, Hkv, D, 16)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    scale = D ** -0.5
    want = ref.paged_attention_decode(q, kc, vc, bt, sl, scale, alibi_slopes=slopes)
    plain = ref.paged_attention_decode(q, kc, vc, bt, sl, scale)
    assert (want.float() - plain.float()).abs().max() > 0.05     # the bias matters here
    for splits in (1, 4):
        got = C.paged_decode(q, kc, vc, bt, sl, scale, num_splits=splits, alibi_slopes=slopes)
        _close(got, want, 2e-2, 2e-2)
    q_lens = [5, 64, 130, 1, 77]
    ctx = [0, 16, 50, 200, 3]
    lens = [a + b for a, b in zip(q_lens, ctx)]
    kc, vc, bt = _make_paged(len(lens), lens, Hkv, D, 16)
    T = sum(q_lens)
    q = torch.randn(T, Hq, D, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device="cuda",
                      dtype=torch.int32)
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    tiles = sum((x + 63) // 64 for x in q_lens)
    got, lse = C.varlen_prefill(q, kc, vc, bt, cu, sl, scale, tiles, return_lse=True,
                                alibi_slopes=slopes)
    want, lse_r = ref.varlen_prefill_attention(q, kc, vc, bt, cu, sl, scale, return_lse=True,
                                               alibi_slopes=slopes)
    _close(got, want, 2e-2, 2e-2)
    _close(lse, lse_r, 1e-2, 1e-2)


@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (4, 4), (8, 1)])
@pytest.mark.parametrize("window", [0, 100])
def test_fmha_prefill_tcgen05(C, Hq, Hkv, window):
    """tcgen05 prefill attention (128-row query tiles, scores and output in tensor memory):
    long and short sequences, cached prefixes, tiles that end inside a page, sliding window;
    also equal to the mma.sync kernel within bf16 rounding."""
    torch.manual_seed(17)
    D = 128
    q_lens = [5, 64, 130, 1, 77, 300, 1024, 128]
    ctx = [0, 16, 50, 200, 3, 500, 0, 128]
    lens = [a + b for a, b in zip(q_lens, ctx)]
    B = len(lens)
    kc, vc, bt = _make_paged(B, lens, Hkv, D, 16)
    T = sum(q_lens)
    q = torch.randn(T, Hq, D, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device="cuda",
                      dtype=torch.int32)
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    tiles = sum((x + 63) // 64 for x in q_lens)
    scale = D ** -0.5
    assert C.USE_FMHA_PREFILL
    got, lse = C.varlen_prefill(q, kc, vc, bt, cu, sl, scale, tiles, window=window,
                                return_lse=True)
    C.USE_FMHA_PREFILL = False
    try:
        old, lse_old = C.varlen_prefill(q, kc, vc, bt, cu, sl, scale, tiles, window=window,
                                        return_lse=True)
    finally:
        C.USE_FMHA_PREFILL = True
    _close(got, old, 2e-2, 2e-2)
    _close(lse, lse_old, 1e-2, 1e-2)
    if window == 0:
        want, lse_r = ref.varlen_prefill_attention(q, kc, vc, bt, cu, sl, scale, return_lse=True)
        _close(got, want, 2e-2, 2e-2)
        _close(lse, lse_r, 1e-2, 1e-2)


@pytest.mark.parametrize("kind", ["fp8", "int8"])
def test_attention_over_8bit_kv_cache(C, kind):
    """Decode and prefill attention reading an fp8 / int8 KV cache (dequantised inside the
    kernel) against the reference on the dequantised cache; the cache is filled by the fused
    RoPE + cache-write kernel so the write path is covered too."""
    torch.manual_seed(23)
    Hq, Hkv, D, bs = 8, 2, 128, 16
    lens = [40, 300, 17, 129]
    B = len(lens)
    max_blocks = max(lens) // bs + 2
    nb = B * max_blocks + 1
    qdt = torch.float8_e4m3fn if kind == "fp8" else torch.int8
    scale_k, scale_v = (0.5, 0.25) if kind == "fp8" else (1 / 24.0, 1 / 20.0)
    kc = torch.zeros(nb, bs, Hkv, D, device="cuda", dtype=qdt)
    vc = torch.zeros_like(kc)
    bt = torch.randperm(nb - 1, device="cuda")[: B * max_blocks].add_(1).to(torch.int32).view(
        B, max_blocks)
    kc_ref = torch.zeros(nb, bs, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc_ref = torch.zeros_like(kc_ref)
    sc = torch.tensor([scale_k, scale_v], device="cuda")
    for b, n in enumerate(lens):
        k = torch.randn(n, Hkv * D, device="cuda", dtype=torch.bfloat16)
        v = torch.randn(n, Hkv * D, device="cuda", dtype=torch.bfloat16)
        pos = torch.arange(n, device="cuda")
        slots = (bt[b, pos // bs].long() * bs + pos % bs)
        C.rope_cache_flash(None, k, v, None, None, True, D, slots, kc, vc, sc[0:1], sc[1:2])
        if kind == "fp8":
            kd = (k.float() / scale_k).to(qdt).float() * scale_k
            vd = (v.float() / scale_v).to(qdt).float() * scale_v
        else:
            kd = (k.float() / scale_k).round().clamp(-128, 127) * scale_k
            vd = (v.float() / scale_v).round().clamp(-128, 127) * scale_v
        kc_ref.view(-1, Hkv * D)[slots] = kd.to(torch.bfloat16)
        vc_ref.view(-1, Hkv * D)[slots] = vd.to(torch.bfloat16)
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    att = D ** -0.5
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    got = C.paged_decode(q, kc, vc, bt, sl, att, num_splits=2,
                         kv_quant=(scale_k, scale_v, 0.0, 0.0))
    want = ref.paged_attention_decode(q, kc_ref, vc_ref, bt, sl, att)
    _close(got, want, 3e-2, 3e-2)
    q_lens = [8, 100, 17, 64]
    T = sum(q_lens)
    qp = torch.randn(T, Hq, D, device="cuda", dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device="cuda",
                      dtype=torch.int32)
    tiles = sum((x + 63) // 64 for x in q_lens)
    gotp = C.varlen_prefill(qp, kc, vc, bt, cu, sl, att, tiles,
                            kv_quant=(scale_k, scale_v, 0.0, 0.0))
    wantp = ref.varlen_prefill_attention(qp, kc_ref, vc_ref, bt, cu, sl, att)
    _close(gotp, wantp, 3e-2, 3e-2)


def test_sampler(C):
    torch.manual_seed(8)
    B, V = 9, 32000
    logits = torch.randn(B, V, device="cuda", dtype=torch.float32) * 3
    ids = C.sample(logits)
    assert torch.equal(ids, logits.argmax(-1))
    ids16 = C.sample(logits.to(torch.bfloat16))
    assert torch.equal(ids16, logits.to(torch.bfloat16).float().argmax(-1))
    temp = torch.full((B,), 0.8, device="cuda")
    temp[0] = 0.0
    k = torch.tensor([0, 1, 5, 50, 0, 0, 20, 1000, 3], device="cuda", dtype=torch.int32)
    p = torch.tensor([1.0, 1.0, 1.0, 1.0, 0.5, 0.9, 0.7, 0.95, 1.0], device="cuda")
    noise = torch.empty(B, V, device="cuda").exponential_()
    got = C.sample(logits, temp, k, p, noise=noise)
    want = ref.sample(logits, temp, k, p, noise=noise)
    # ties at the nucleus boundary may differ by one token; the pick must be in the kept set
    masked = ref.apply_top_k_top_p(logits / torch.where(temp > 0, temp, torch.ones_like(temp))[:, None],
                                   k, p)
    for b in range(B):
        assert torch.isfinite(masked[b, got[b]]) or got[b] == want[b]
    assert (got == want).float().mean().item() >= 0.8
    # built-in generator: valid ids, different draws for different steps
    seeds = torch.arange(B, device="cuda", dtype=torch.int64)
    a = C.sample(logits, temp, k, p, seeds=seeds, step=1)
    b2 = C.sample(logits, temp, k, p, seeds=seeds, step=1)
    assert torch.equal(a, b2)
    assert ((a >= 0) & (a < V)).all()
    lg = logits.clone()
    C.top_k_top_p_(lg, k, p)
    kept = torch.isfinite(lg).sum(-1)
    kept_ref = torch.isfinite(ref.apply_top_k_top_p(logits, k, p)).sum(-1)
    assert ((kept - kept_ref).abs() <= 2).all(), (kept, kept_ref)


def test_advance_step(C):
    torch.manual_seed(9)
    n, pad, bs, mb = 50, 64, 16, 40
    toks = torch.zeros(pad, device="cuda", dtype=torch.int64)
    sampled = torch.randint(0, 1000, (n,), device="cuda")
    pos = torch.zeros(pad, device="cuda", dtype=torch.int64)
    sl = torch.randint(1, bs * mb - 1, (pad,), device="cuda", dtype=torch.int32)
    slots = torch.zeros(pad, device="cuda", dtype=torch.int64)
    bt = torch.randint(0, 5000, (pad, mb), device="cuda", dtype=torch.int32)
    r = [t.clone() for t in (toks, pos, sl, slots)]
    ref.advance_step(pad, n, bs, r[0], sampled, r[1], r[2], r[3], bt)
    C.advance_step(pad, n, bs, toks, sampled, pos, sl, slots, bt)
    for a, b in zip((toks, pos, sl, slots), r):
        assert torch.equal(a, b)


@pytest.mark.parametrize("M,N,K", [(64, 4096, 14336), (1, 4096, 4096), (100, 1024, 8192)])
def test_skinny_gemm_two_kernel_k_split_matches_reference(M, N, K):
    """Rows <= 128: wide column tiles with a K split whose fp32 partial sums are added by a
    second kernel (gemm_skinny.cu, ``make_plan2``), with and without a bias."""
    import ctypes
    from vllm_gcu_b200.ops import _native
    from vllm_gcu_b200.ops import cuda as C
    torch.manual_seed(M + N)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ref = x.float() @ w.float().t()
    for b in (None, bias):
        got = C.gemm_bf16(x, w, bias=b)
        want = ref if b is None else ref + b.float()
        err = (got.float() - want).abs().max().item()
        assert err < 1e-2 * want.abs().max().item() + 1e-2, err
    torch.cuda.synchronize()
    _native.check_status()
    # twice the same: the summation order is fixed
    assert torch.equal(C.gemm_bf16(x, w), C.gemm_bf16(x, w))
