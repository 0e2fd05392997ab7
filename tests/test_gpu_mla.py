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


def test_deepseek_engine_with_mla_kernel_tracks_torch_path(monkeypatch):
    """DeepSeek-V3-shaped model (512 + 64 latent, 16 heads) through the engine: the tcgen05
    latent attention (prefill chunks, decode under CUDA graphs) against the same engine with
    the torch formulation; logits of a prefill step agree."""
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    from vllm_gcu_b200.models import deepseek
    from vllm_gcu_b200.ops import _native
    kw = dict(hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
              num_attention_heads=16, num_key_value_heads=16, q_lora_rank=128, kv_lora_rank=512,
              qk_nope_head_dim=64, qk_rope_head_dim=64, v_head_dim=64, head_dim=128,
              moe_intermediate_size=128, num_nextn_predict_layers=0, dtype="bfloat16",
              max_num_seqs=8, max_num_batched_tokens=128, max_model_len=512, num_gpu_blocks=256)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (150, 33, 64, 7)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    calls = {"n": 0}
    from vllm_gcu_b200.ops import cuda as C
    real = C.mla_attention

    def counted(*a, **k):
        calls["n"] += 1
        return real(*a, **k)
    monkeypatch.setattr(C, "mla_attention", counted)
    res = {}
    for use in (True, False):
        monkeypatch.setattr(deepseek, "USE_MLA_KERNEL", use)
        llm = LLM("tiny-deepseek", device="cuda", cuda_graph_sizes=[4, 8], seed=0, **kw)
        n0 = calls["n"]
        outs = llm.generate(prompts, sp)
        torch.cuda.synchronize()
        _native.check_status()
        assert (calls["n"] > n0) == use
        llm.engine.runner.keep_logits = True
        llm.engine.runner.graphs = {}
        llm.generate(prompts[:3], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
        res[use] = ([o.outputs[0].token_ids for o in outs],
                    llm.engine.runner.last_logits.float().cpu())
        del llm
    assert all(len(t) == 6 for t in res[True][0])
    assert [t[0] for t in res[True][0]] == [t[0] for t in res[False][0]]
    lk, lt = res[True][1], res[False][1]
    err = (lk - lt).abs().max().item()
    assert err < 0.05 * lt.std().item() + 0.03, (err, lt.std().item())
