"""CPU checks of the MoE and MLA model paths (torch reference ops, fp32)."""
import torch

from vllm_gcu_b200.config import preset
from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams
from vllm_gcu_b200.layers.moe import SparseMoeBlock, select_experts
from vllm_gcu_b200.ops import ref


def _gen(model, max_tokens_per_step, async_sched=False, n=4, plen=40, out=10, **kw):
    torch.manual_seed(0)
    llm = LLM(model, device="cpu", block_size=16, max_num_seqs=8,
              max_num_batched_tokens=max_tokens_per_step, max_model_len=256,
              async_scheduling=async_sched, num_gpu_blocks=64, **kw)
    g = torch.Generator().manual_seed(1)
    V = llm.engine.cfg.model.vocab_size
    prompts = [torch.randint(0, V, (plen + 3 * i,), generator=g).tolist() for i in range(n)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=out, temperature=0.0, ignore_eos=True))
    return llm, prompts, [o.outputs[0].token_ids for o in outs]


def test_qwen3_moe_chunked_and_async_agree():
    _, _, a = _gen("tiny-qwen3-moe", 256)
    _, _, b = _gen("tiny-qwen3-moe", 24)
    _, _, c = _gen("tiny-qwen3-moe", 24, async_sched=True)
    assert a == b == c


def test_sparse_moe_block_matches_naive_loop():
    torch.manual_seed(0)
    cfg = preset("tiny-qwen3-moe")
    blk = SparseMoeBlock(cfg, "cpu", "m")
    for p in blk.parameters():
        p.data.normal_(0, 0.05)
    x = torch.randn(9, cfg.hidden_size)
    got = blk(x)
    logits = x @ blk.gate.weight.t()
    w, ids = ref.topk_softmax(logits, cfg.num_experts_per_tok, True)
    want = torch.zeros_like(x)
    I = cfg.moe_intermediate_size
    for t in range(x.shape[0]):
        for s in range(ids.shape[1]):
            e = int(ids[t, s])
            h = blk.experts.w13[e] @ x[t]
            a = torch.nn.functional.silu(h[:I]) * h[I:]
            want[t] += w[t, s] * (blk.experts.w2[e] @ a)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-4)


def test_grouped_topk_semantics():
    torch.manual_seed(0)
    T, E, k, ng, tg = 6, 16, 4, 4, 2
    g = torch.randn(T, E)
    bias = torch.randn(E) * 0.1
    w, ids = ref.grouped_topk(g, k, True, ng, tg, bias, "sigmoid", 2.5)
    s = torch.sigmoid(g)
    for t in range(T):
        sel = s[t] + bias
        gs = sel.view(ng, E // ng).topk(2, -1).values.sum(-1)
        groups = set(gs.topk(tg).indices.tolist())
        chosen = ids[t].tolist()
        assert all(c // (E // ng) in groups for c in chosen)
        ww = s[t, ids[t].long()]
        assert torch.allclose(w[t], ww / ww.sum() * 2.5, atol=1e-6)


def test_deepseek_mla_matches_plain_attention():
    """The absorbed latent-space attention equals textbook MLA (decompress k/v per head)."""
    llm, prompts, toks = _gen("tiny-deepseek", 256, n=2, plen=20, out=4)
    model = llm.engine.model
    cfg = model.cfg
    att = model.layers["0"].self_attn
    torch.manual_seed(3)
    S = 12
    x = torch.randn(S, cfg.hidden_size)
    pos = torch.arange(S)
    N, L, R, nope, vd = att.N, att.L, att.R, att.nope, att.vdim
    qkv_a = x @ att.qkv_a_proj.weight.t()
    q_c, kv = qkv_a.split([cfg.q_lora_rank, L + R], -1)
    q = (ref.rms_norm(q_c, att.q_a_layernorm.weight, cfg.rms_norm_eps)
         @ att.q_b_proj.weight.t()).view(S, N, nope + R)
    kv_c = ref.rms_norm(kv[:, :L].contiguous(), att.kv_a_layernorm.weight, cfg.rms_norm_eps)
    q_pe, k_pe = ref.rotary_embedding(pos, q[..., nope:].reshape(S, N * R),
                                      kv[:, L:].contiguous(), R, att.cos_sin_cache, False)
    kvb = (kv_c @ att.kv_b_proj.weight.t()).view(S, N, nope + vd)
    k = torch.cat([kvb[..., :nope], k_pe[:, None, :].expand(S, N, R)], -1)
    qq = torch.cat([q[..., :nope], q_pe.view(S, N, R)], -1)
    s = torch.einsum("qhd,nhd->hqn", qq, k) * att.scale
    s = s.masked_fill(~torch.tril(torch.ones(S, S, dtype=torch.bool))[None], float("-inf"))
    o = torch.einsum("hqn,nhd->qhd", s.softmax(-1), kvb[..., nope:]).reshape(S, N * vd)
    want = o @ att.o_proj.weight.t()
    # the engine path on a fresh paged cache
    from vllm_gcu_b200.layers.attention import AttentionMetadata
    cache = torch.zeros(4, 16, L + R)
    md = AttentionMetadata(num_tokens=S, num_decodes=0, num_prefills=1, num_decode_tokens=0,
                           positions=pos, slot_mapping=torch.arange(S),
                           block_tables=torch.tensor([[0, 1, 2, 3]], dtype=torch.int32),
                           seq_lens=torch.tensor([S], dtype=torch.int32), q_lens_cpu=[S],
                           seq_lens_cpu=[S])
    got = att(x, cache, md)
    assert torch.allclose(got, want, atol=2e-5, rtol=1e-4), (got - want).abs().max()


def test_deepseek_chunked_and_async_agree():
    _, _, a = _gen("tiny-deepseek", 256, n=3, plen=30, out=8)
    _, _, b = _gen("tiny-deepseek", 20, n=3, plen=30, out=8)
    _, _, c = _gen("tiny-deepseek", 20, async_sched=True, n=3, plen=30, out=8)
    assert a == b == c
