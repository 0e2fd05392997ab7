"""tcgen05 multi-head latent attention kernel (csrc/attention_mla.cu) against the fp32 torch
reference of the same op (models/deepseek.py ``mla_attention_ref``): decode, multi-token
requests with a cached prefix, split contexts, padded (empty) requests."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(N, q_lens, seq_lens, bs=16, seed=0):
    from vllm_gcu_b200.ops import cuda as C
    dev = torch.device("cuda")
    g = torch.Generator(device="cuda").manual_seed(seed)
    B = len(q_lens)
    max_blocks = max((max(seq_lens) + bs - 1) // bs, 1) + 1
    nb = B * max_blocks + 3
    cache = (torch.randn(nb, bs, 576, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(nb - 1, device=dev, generator=g)[:B * max_blocks] + 1
    bt = perm.view(B, max_blocks).to(torch.int32).contiguous()
    T = sum(q_lens)
    q = (torch.randn(T, N, 576, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=dev)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev)
    return C, q, cache, bt, sl, cu


def _check(N, q_lens, seq_lens, decode=False, splits=None, seed=0):
    from vllm_gcu_b200.models.deepseek import mla_attention_ref
    from vllm_gcu_b200.ops import _native
    C, q, cache, bt, sl, cu = _setup(N, q_lens, seq_lens, seed=seed)
    scale = 576 ** -0.5
    tq = 128 // N
    tiles = sum(-(-x // tq) for x in q_lens)
    got = C.mla_attention(q, cache, bt, sl, None if decode else cu, tiles, max(seq_lens), scale,
                          splits=splits)
    torch.cuda.synchronize()
    _native.check_status()
    want = mla_attention_ref(q.float(), cache.float(), bt, q_lens, seq_lens, scale, 512)
    err = (got.float() - want).abs().max().item()
    ref = want.abs().max().item()
    assert err < 0.02 * ref + 0.01, (N, q_lens, seq_lens, splits, err, ref)
    return got


@pytest.mark.parametrize("N", [16, 128])
def test_mla_decode_matches_reference(N):
    _check(N, [1] * 5, [1, 17, 64, 65, 300], decode=True, splits=1)


def test_mla_decode_with_empty_request_and_splits():
    got = _check(16, [1] * 4, [130, 0, 1000, 77], decode=True, splits=4, seed=1)
    assert got[1].abs().max().item() == 0.0          # nothing to attend to: zeros
    _check(32, [1] * 3, [513, 64, 2], decode=True, splits=None, seed=2)


@pytest.mark.parametrize("N", [16, 64, 128])
def test_mla_multi_token_requests_with_prefix(N):
    _check(N, [40, 7, 130, 1], [40, 100, 130, 9], splits=1, seed=3)
    _check(N, [40, 7, 130, 1], [40, 100, 130, 9], splits=3, seed=4)
