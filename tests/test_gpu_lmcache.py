"""LMCache offload kernels on the GPU against the host reference implementations."""
import pytest
import torch

from vllm_gcu_b200.ops import _native, ref
from vllm_gcu_b200.parallel.kv_transfer import lmcache_ops as O

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    if torch.cuda.is_available():
        _native.check_status()


def test_multi_layer_transfer_matches_host():
    torch.manual_seed(0)
    L, slots, W, T = 4, 256, 1024, 70
    layers = [torch.randn(2, slots, W, device="cuda", dtype=torch.bfloat16) for _ in range(L)]
    ptrs = torch.tensor([t.data_ptr() for t in layers], dtype=torch.int64, device="cuda")
    sm = torch.randperm(slots, device="cuda")[:T]
    sm[5] = -1
    buf = torch.zeros(2, L, T, W, device="cuda", dtype=torch.bfloat16)
    O.multi_layer_kv_transfer(buf, ptrs, sm, "cuda", slots, True, False)
    ok = sm >= 0
    for l in range(L):
        assert torch.equal(buf[0, l][ok], layers[l][0, sm[ok]])
        assert torch.equal(buf[1, l][ok], layers[l][1, sm[ok]])
    fresh = [torch.zeros_like(t) for t in layers]
    ptrs2 = torch.tensor([t.data_ptr() for t in fresh], dtype=torch.int64, device="cuda")
    O.multi_layer_kv_transfer(buf, ptrs2, sm, "cuda", slots, False, False)
    for l in range(L):
        assert torch.equal(fresh[l][:, sm[ok]], layers[l][:, sm[ok]])


def test_rerotation_matches_fresh_rotation():
    torch.manual_seed(1)
    T, H, D = 33, 8, 128
    cs = ref.make_cos_sin_cache(D, 512).cuda()
    k = torch.randn(T, H * D, device="cuda", dtype=torch.bfloat16)
    old = torch.randint(0, 200, (T,), device="cuda")
    new = old + torch.randint(0, 200, (T,), device="cuda")
    _, k_old = ref.rotary_embedding(old, k.clone(), k.clone(), D, cs, True)
    _, k_new = ref.rotary_embedding(new, k.clone(), k.clone(), D, cs, True)
    moved = k_old.clone()
    O.rotary_embedding_k_fused(old, new, moved, D, cs, True)
    assert (moved.float() - k_new.float()).abs().max().item() < 0.05


def test_cachegen_cdf_and_codec_match_host_bit_for_bit():
    torch.manual_seed(2)
    L, T, C, bins = 3, 40, 96, 32
    probs = torch.softmax(torch.randn(bins) * 2, 0)
    sym = torch.multinomial(probs, L * T * C, replacement=True).view(L, T, C).to(torch.int8)
    cdf_h = O.calculate_cdf(sym, bins)
    cdf_d = O.calculate_cdf(sym.cuda(), bins)
    assert torch.equal(cdf_d.cpu(), cdf_h)
    mb = 2 * C + 16
    out_h = torch.zeros(L, T, mb, dtype=torch.uint8)
    len_h = torch.zeros(L, T, dtype=torch.int32)
    O.encode_fast_new(cdf_h, sym, out_h, len_h)
    out_d = torch.zeros(L, T, mb, dtype=torch.uint8, device="cuda")
    len_d = torch.zeros(L, T, dtype=torch.int32, device="cuda")
    O.encode_fast_new(cdf_d, sym.cuda(), out_d, len_d)
    assert torch.equal(len_d.cpu(), len_h)
    assert torch.equal(out_d.cpu(), out_h)
    dec = torch.zeros(L, T, C, dtype=torch.int8, device="cuda")
    O.decode_fast_new(cdf_d, out_d, len_d, dec)
    assert torch.equal(dec.cpu(), sym)
    # packed streams
    lens = len_d.flatten().long()
    offs = torch.zeros(L * T + 1, dtype=torch.int64, device="cuda")
    offs[1:] = lens.cumsum(0)
    packed = torch.cat([out_d.view(L * T, mb)[i, :int(lens[i])] for i in range(L * T)])
    dec2 = torch.zeros_like(dec)
    O.decode_fast_prefsum(cdf_d, packed, offs, dec2)
    assert torch.equal(dec2.cpu(), sym)
    assert int(lens.sum()) < L * T * C * 5 // 8 + L * T * 8      # better than 5 raw bits / symbol
