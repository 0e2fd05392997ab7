"""GPU numerics of the smaller kernels (LoRA, speculative decoding, cache maintenance,
attention-state merge, token feed) against the fp32 / integer references of ``ops.ref``."""
import pytest
import torch

from vllm_gcu_b200.ops import _native, ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def C():
    from vllm_gcu_b200.ops import cuda
    return cuda


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    if torch.cuda.is_available():
        _native.check_status()


def _close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float(), b.float()
    bad = ((a - b).abs() > atol + rtol * b.abs()).float().mean().item()
    assert bad == 0.0, f"{bad:.2%} out of tolerance, max err {(a - b).abs().max().item():.4g}"


# -- multi-LoRA -------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_bgmv_shrink_expand_slice(dtype):
    from vllm_gcu_b200.lora import ops as L
    g = torch.Generator(device=DEV).manual_seed(0)
    T, h, r, n_lora = 37, 1024, 16, 4
    x = torch.randn(T, h, device=DEV, generator=g).to(dtype)
    A = (torch.randn(n_lora, r, h, device=DEV, generator=g) * 0.05).to(dtype)
    B = (torch.randn(n_lora, 3 * 256, r, device=DEV, generator=g) * 0.05).to(dtype)
    idx = torch.randint(-1, n_lora, (T,), device=DEV, generator=g)
    idx[0], idx[1] = -1, n_lora - 1                        # rows without an adapter stay as they are
    # shrink: y = scale * A[idx] x, rows with idx < 0 untouched
    y = torch.full((T, r), 7.0, device=DEV, dtype=torch.float32)
    want = y.clone()
    want[idx >= 0] = 0
    ref.bgmv(want, x, A, idx, 0.5)
    L.bgmv_shrink(x, A, y, idx, 0.5)
    _close(y, want)
    # expand with accumulation into a slice of a wider output
    h_mid = y.to(dtype)
    out = torch.randn(T, 1024, device=DEV, generator=g).to(dtype)
    want = out.clone().float()
    ref.bgmv(want, h_mid, B[:, 256:512], idx, 1.0, y_offset=300, y_slice=256)
    L.bgmv_expand_slice(h_mid, B[:, 256:512].contiguous(), out, idx, 300, 256, add_inputs=True)
    _close(out, want, 3e-2, 3e-2)
    # expand without accumulation
    out2 = torch.randn(T, 768, device=DEV, generator=g).to(dtype)
    want2 = out2.clone().float()
    want2[idx >= 0] = 0      # rows with an adapter are overwritten ...
    ref.bgmv(want2, h_mid, B, idx, 1.0)
    L.bgmv_expand(h_mid, B, out2, idx, add_inputs=False)
    _close(out2[idx >= 0], want2[idx >= 0], 3e-2, 3e-2)


# -- speculative decoding ----------------------------------------------------------------------
def test_rejection_kernels_match_the_oracles():
    from vllm_gcu_b200.spec import RejectionSampler
    g = torch.Generator(device=DEV).manual_seed(1)
    B, S, V = 33, 4, 1000
    draft = torch.randint(0, V, (B, S), device=DEV, generator=g, dtype=torch.int32)
    tgt = torch.randint(0, V, (B, S + 1), device=DEV, generator=g)
    tgt[:, :S] = torch.where(torch.rand(B, S, device=DEV, generator=g) < 0.7, draft.long(), tgt[:, :S])
    nd = torch.randint(0, S + 1, (B,), device=DEV, generator=g, dtype=torch.int32)
    rs = RejectionSampler()
    got = rs.greedy(draft, tgt, nd)
    assert torch.equal(got.cpu(), rs._greedy_ref(draft.cpu(), tgt.cpu(), nd.cpu()))
    # random verification: kernel pair (recovered tokens + accept / reject) against the oracles
    probs = torch.rand(B, S, V, device=DEV, generator=g).softmax(-1)
    dprobs = torch.rand(B, S, V, device=DEV, generator=g).softmax(-1)
    bonus = torch.randint(0, V, (B,), device=DEV, generator=g)
    for dp in (None, dprobs):
        uniform = torch.rand(B, S, device=DEV, generator=g)
        noise = torch.empty(B, S, V, device=DEV).exponential_(generator=g)
        rec = torch.empty(B, S, dtype=torch.int32, device=DEV)
        _native.call("b200_sample_recovered_tokens", rec.data_ptr(), draft.data_ptr(),
                     None if dp is None else dp.data_ptr(), probs.data_ptr(), noise.data_ptr(),
                     B, S, V, _native.stream_ptr())
        want_rec = ref.sample_recovered_tokens(draft, dp, probs, noise)
        assert torch.equal(rec, want_rec)
        out = torch.empty(B, S + 1, dtype=torch.int32, device=DEV)
        _native.call("b200_rejection_random", out.data_ptr(), draft.data_ptr(),
                     None if dp is None else dp.data_ptr(), probs.data_ptr(), bonus.data_ptr(),
                     rec.data_ptr(), uniform.data_ptr(), nd.data_ptr(), B, S, V,
                     _native.stream_ptr())
        want = ref.rejection_random_sample(draft.cpu(), None if dp is None else dp.cpu(),
                                           probs.cpu(), bonus.cpu(), rec.cpu(), uniform.cpu(),
                                           nd.cpu())
        assert torch.equal(out.cpu(), want)
    # the sampler class end to end (same seed, same result on a second call)
    gen = torch.Generator(device=DEV).manual_seed(5)
    a = rs.random(draft, None, probs, bonus, nd, generator=gen)
    gen.manual_seed(5)
    b = rs.random(draft, None, probs, bonus, nd, generator=gen)
    assert torch.equal(a, b)


def test_expand_batch_to_tokens():
    x = torch.tensor([5, -1, 9, 0], dtype=torch.int64, device=DEV)
    cu = torch.tensor([3, 3, 10, 12], dtype=torch.int32, device=DEV)
    out = torch.empty(12, dtype=torch.int64, device=DEV)
    _native.call("b200_expand_batch_to_tokens", out.data_ptr(), x.data_ptr(), cu.data_ptr(), 4,
                 -1, 77, _native.stream_ptr())
    want = ref.expand_batch_to_tokens(x, cu.long(), -1, 77)
    assert torch.equal(out, want)


# -- attention state merge ---------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_merge_attn_states(C, dtype):
    g = torch.Generator(device=DEV).manual_seed(2)
    T, H, D = 19, 8, 128
    p_out = torch.randn(T, H, D, device=DEV, generator=g).to(dtype)
    s_out = torch.randn(T, H, D, device=DEV, generator=g).to(dtype)
    p_lse = torch.randn(H, T, device=DEV, generator=g) * 3      # log-sum-exp values: [H, T]
    s_lse = torch.randn(H, T, device=DEV, generator=g) * 3
    s_lse[:, 0] = float("-inf")             # an empty suffix contributes nothing
    out, lse = C.merge_attn_states(p_out, p_lse, s_out, s_lse)
    want, want_lse = ref.merge_attn_states(p_out, p_lse, s_out, s_lse)
    _close(out, want)
    _close(lse, want_lse, 1e-3, 1e-3)


# -- cache maintenance -------------------------------------------------------------------------
def test_gather_cache_and_copy_blocks(C):
    g = torch.Generator(device=DEV).manual_seed(3)
    nb, bs, W = 40, 16, 576
    cache = torch.randn(nb, bs, W, device=DEV, generator=g).to(torch.bfloat16)
    lens = [5, 33, 16, 1]
    starts = torch.tensor([0, 7, 16, 3], dtype=torch.int32, device=DEV)
    bt = torch.randperm(nb, device=DEV, generator=g)[:4 * 4].view(4, 4).to(torch.int32)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    for st in (None, starts):
        got = C.gather_cache(cache, bt, cu, sum(lens), seq_starts=st)
        want = ref.gather_cache(cache, bt, cu, st)
        assert torch.equal(got, want)
    # copy_blocks over several layers at once
    caches = [torch.randn(nb, bs, 2, 64, device=DEV, generator=g).to(torch.bfloat16)
              for _ in range(3)]
    want = [c.clone() for c in caches]
    mapping = torch.tensor([[1, 30], [2, 31], [1, 32], [17, 0]], dtype=torch.int64, device=DEV)
    ref.copy_blocks(want, mapping)
    C.copy_blocks(caches, mapping)
    for a, b in zip(caches, want):
        assert torch.equal(a, b)


@pytest.mark.parametrize("cache_dtype", [torch.bfloat16, torch.int8])
def test_reshape_and_cache_x_packed_layout(C, cache_dtype):
    g = torch.Generator(device=DEV).manual_seed(4)
    T, H, D, bs, nb, x = 21, 4, 128, 16, 6, 8
    key = torch.randn(T, H, D, device=DEV, generator=g).to(torch.bfloat16)
    val = torch.randn(T, H, D, device=DEV, generator=g).to(torch.bfloat16)
    slots = torch.randperm(nb * bs, device=DEV, generator=g)[:T]
    slots[3] = -1
    kc = torch.zeros(nb, H, D // x, bs, x, device=DEV, dtype=cache_dtype)
    vc = torch.zeros(nb, H, D, bs, device=DEV, dtype=cache_dtype)
    kr, vr = kc.clone(), vc.clone()
    kw = dict(k_scale=0.05, v_scale=0.04, k_zp=2.0, v_zp=-1.0) if cache_dtype == torch.int8 else {}
    C.reshape_and_cache(key, val, kc, vc, slots, **kw)
    ref.reshape_and_cache(key, val, kr, vr, slots, **kw)
    if cache_dtype == torch.int8:
        assert (kc.int() - kr.int()).abs().max().item() <= 1      # rounding at .5
        assert (vc.int() - vr.int()).abs().max().item() <= 1
    else:
        assert torch.equal(kc, kr) and torch.equal(vc, vr)


@pytest.mark.parametrize("is_neox", [False, True])
def test_mla_rope_cache_and_concat_mode(C, is_neox):
    g = torch.Generator(device=DEV).manual_seed(5)
    T, H, L, R, bs, nb = 29, 16, 512, 64, 16, 8
    q_pe = torch.randn(T, H, R, device=DEV, generator=g).to(torch.bfloat16)
    kv = torch.randn(T, L + R, device=DEV, generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(L, device=DEV, generator=g)).to(torch.bfloat16)
    pos = torch.randint(0, 500, (T,), device=DEV, generator=g)
    cs = ref.make_cos_sin_cache(R, 512, 10000.0).to(DEV).float()
    slots = torch.randperm(nb * bs, device=DEV, generator=g)[:T]
    slots[5] = -1
    cache = torch.zeros(nb, bs, L + R, device=DEV, dtype=torch.bfloat16)
    cache_ref = cache.clone()
    q_want, k_want, c_want = ref.mla_rope_cache(q_pe.clone(), kv, pos, cs, w, 1e-6, cache_ref,
                                                slots, L, is_neox)
    q_got = q_pe.clone()
    k_got, c_got = C.mla_rope_cache(q_got, kv, pos, cs, w, 1e-6, cache, slots, L, is_neox,
                                    want_k_pe=True, want_kv_c=True)
    _close(q_got, q_want)
    _close(k_got, k_want)
    _close(c_got, c_want)
    _close(cache, cache_ref)
    # concat mode: cache[slot] = [kv_c | k_pe] without norm / rotation
    cache2 = torch.zeros_like(cache)
    cache2_ref = torch.zeros_like(cache)
    C.concat_and_cache_mla(kv[:, :L], kv[:, L:], cache2, slots)
    ref.concat_and_cache_mla(kv[:, :L], kv[:, L:], cache2_ref, slots)
    assert torch.equal(cache2, cache2_ref)


def test_feed_tokens(C):
    ids = torch.arange(40, dtype=torch.int64, device=DEV)
    prev = torch.arange(100, 110, dtype=torch.int64, device=DEV)
    dst = torch.tensor([3, 0, 39, 7], dtype=torch.int32, device=DEV)
    src = torch.tensor([9, 1, 0, 4], dtype=torch.int32, device=DEV)
    want = ids.clone()
    want[dst[:3].long()] = prev[src[:3].long()]
    C.feed_tokens(ids, prev, dst, src, 3)                 # only the first n pairs are live
    assert torch.equal(ids, want)


@pytest.mark.parametrize("D", [128, 64])
def test_cascade_attention_matches_the_full_pass(C, D):
    """Shared-prefix attention (one non-causal pass over the common blocks + causal passes over
    the suffixes, merged by log-sum-exp) against one ordinary pass over everything."""
    from vllm_gcu_b200.layers.attention import cascade_attention
    g = torch.Generator(device=DEV).manual_seed(6)
    nb, bs, Hq, Hkv = 64, 16, 8, 2
    kc = torch.randn(nb, bs, Hkv, D, device=DEV, generator=g).to(torch.bfloat16)
    vc = torch.randn(nb, bs, Hkv, D, device=DEV, generator=g).to(torch.bfloat16)
    prefix = list(range(20, 36))                            # 256 shared tokens
    rows = [prefix + [1, 2, 3, 0], prefix + [4, 0, 0, 0], prefix + [5, 6, 0, 0], prefix + [7, 8, 9, 10]]
    bt = torch.tensor(rows, dtype=torch.int32, device=DEV)
    q_lens = [33, 1, 1, 64]
    seq_lens = torch.tensor([256 + 40, 256 + 3, 256 + 17, 256 + 64], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, 33, 34, 35, 99], dtype=torch.int32, device=DEV)
    q = torch.randn(99, Hq, D, device=DEV, generator=g).to(torch.bfloat16)
    want = ref.varlen_prefill_attention(q, kc, vc, bt, cu, seq_lens, D ** -0.5)
    got = cascade_attention(q, kc, vc, bt, cu, seq_lens, D ** -0.5, 256, q_lens, native=True)
    _close(got, want, 3e-2, 3e-2)
