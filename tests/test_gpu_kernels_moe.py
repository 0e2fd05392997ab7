"""GPU numerics of the MoE kernels against the torch reference."""
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


@pytest.mark.parametrize("E,k,ng,tg,sigmoid,use_bias", [(128, 8, 1, 1, False, False),
                                                        (256, 8, 8, 4, True, True),
                                                        (16, 4, 4, 2, False, False),
                                                        (8, 2, 1, 1, False, False)])
def test_moe_topk(C, E, k, ng, tg, sigmoid, use_bias):
    torch.manual_seed(0)
    T = 37
    g = torch.randn(T, E, device="cuda", dtype=torch.float32)
    bias = (torch.randn(E, device="cuda") * 0.1) if use_bias else None
    w, ids = C.moe_topk(g, k, True, ng, tg, bias, sigmoid, 2.5 if ng > 1 else 1.0)
    if ng > 1 or sigmoid:
        wr, ir = ref.grouped_topk(g, k, True, ng, tg, bias, "sigmoid" if sigmoid else "softmax",
                                  2.5 if ng > 1 else 1.0)
    else:
        wr, ir = ref.topk_softmax(g, k, True)
    # compare as sets per row (order of equal-rank experts is not part of the contract)
    so, sr = ids.long().sort(-1), ir.long().sort(-1)
    assert torch.equal(so.values, sr.values)
    assert torch.allclose(w.gather(1, so.indices), wr.gather(1, sr.indices), atol=1e-5, rtol=1e-4)


def test_moe_align_and_ep_indices(C):
    torch.manual_seed(1)
    T, k, E = 50, 4, 16
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).to(torch.int32).cuda()
    sorted_ids, expert_ids, npp, pos_of = C.moe_align(ids, E)
    n = int(npp.item())
    assert n % 128 == 0
    flat = ids.reshape(-1).cpu()
    s = sorted_ids.cpu()
    for b in range(n // 128):
        e = int(expert_ids[b])
        rows = s[b * 128:(b + 1) * 128]
        real = rows[rows < T * k]
        assert (flat[real.long()] == e).all()
    placed = s[:n][s[:n] < T * k]
    assert sorted(placed.tolist()) == list(range(T * k))
    assert (s[pos_of.cpu().long()] == torch.arange(T * k)).all()
    # expert map: only experts 4..7 are local
    emap = torch.full((E,), -1, dtype=torch.int32)
    emap[4:8] = torch.arange(4, dtype=torch.int32)
    s2, e2, n2, p2 = C.moe_align(ids, 4, expert_map=emap.cuda())
    keep = ((flat >= 4) & (flat < 8)).nonzero().flatten()
    got = s2.cpu()[: int(n2)]
    assert sorted(got[got < T * k].tolist()) == keep.tolist()
    assert ((p2.cpu() >= 0) == ((flat >= 4) & (flat < 8))).all()
    cnt, idx, tot = C.get_ep_indices(ids, 4, 4)
    cr, ir, tr = ref.get_ep_indices(ids.cpu(), 4, 4)
    assert torch.equal(cnt.cpu(), cr) and int(tot) == tr
    off = 0
    for r in range(4):
        c = int(cr[r])
        assert sorted(idx.cpu()[off:off + c].tolist()) == sorted(ir[off:off + c].tolist())
        off += c


@pytest.mark.parametrize("T,E,k,H,I", [(33, 8, 2, 256, 128), (300, 16, 4, 512, 256),
                                       (1, 128, 8, 2048, 768)])
def test_fused_experts(C, T, E, k, H, I):
    torch.manual_seed(2)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w13 = (torch.randn(E, 2 * I, H, device="cuda") * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, device="cuda") * 0.05).to(torch.bfloat16)
    g = torch.randn(T, E, device="cuda")
    tw, ti = C.moe_topk(g, k, True)
    want = ref.fused_experts(x, w13, w2, tw, ti)
    w13i = torch.stack([ref.interleave_gate_up(w13[e, :I], w13[e, I:]) for e in range(E)])
    add = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    got = C.fused_experts(x, w13i.contiguous(), w2, tw, ti, add=add)
    err = (got.float() - (want.float() + add.float())).abs()
    tol = 3e-2 + 3e-2 * want.float().abs()
    assert bool((err <= tol).all()), err.max().item()
    # expert-parallel slice: only half of the experts are local
    emap = torch.full((E,), -1, dtype=torch.int32, device="cuda")
    emap[E // 2:] = torch.arange(E - E // 2, dtype=torch.int32, device="cuda")
    got2 = C.fused_experts(x, w13i[E // 2:].contiguous(), w2[E // 2:].contiguous(), tw, ti,
                           expert_map=emap)
    want2 = ref.fused_experts(x, w13[E // 2:], w2[E // 2:], tw, ti, expert_map=emap)
    err2 = (got2.float() - want2.float()).abs()
    assert bool((err2 <= 3e-2 + 3e-2 * want2.float().abs()).all()), err2.max().item()


def test_qwen3_moe_engine_gpu_vs_cpu():
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    kw = dict(num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
              head_dim=64, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
              vocab_size=1024, dtype="bfloat16", max_num_seqs=8, max_num_batched_tokens=128,
              max_model_len=256, num_gpu_blocks=64)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (33, 70, 9)]
    one = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
    gpu = LLM("tiny-qwen3-moe", device="cuda", enforce_eager=True, **kw)
    cpu = LLM("tiny-qwen3-moe", device="cpu", load_format="none", **kw)
    sd = {k: v.detach().cpu() for k, v in gpu.engine.model.state_dict().items()}
    for name, mod in gpu.engine.model.named_modules():
        if getattr(mod, "_interleaved", False) and hasattr(mod, "w13"):
            w = sd[name + ".w13"]
            E, I2, H = w.shape
            I = I2 // 2
            w4 = w.view(E, I // ref.GATE_UP_BLOCK, 2, ref.GATE_UP_BLOCK, H)
            sd[name + ".w13"] = torch.cat([w4[:, :, 0].reshape(E, I, H),
                                           w4[:, :, 1].reshape(E, I, H)], 1)
    cpu.engine.model.load_state_dict(sd, strict=False)
    gpu.engine.runner.keep_logits = True
    cpu.engine.runner.keep_logits = True
    gpu.generate(prompts, one)
    cpu.generate(prompts, one)
    lg, lc = gpu.engine.runner.last_logits, cpu.engine.runner.last_logits
    err = (lg - lc).abs().max().item()
    assert err < 0.08 * lc.std().item() + 0.03, (err, lc.std().item())


def _block_quant_fp8(w):
    """[..., N, K] float -> (fp8 codes, scales [..., N/128, K/128]) with one scale per block."""
    *lead, N, K = w.shape
    b = w.float().reshape(*lead, N // 128, 128, K // 128, 128)
    amax = b.abs().amax(dim=(-3, -1), keepdim=True).clamp_min(1e-8)
    s = amax / 448.0
    q = (b / s).to(torch.float8_e4m3fn)
    return q.reshape(*lead, N, K), s.reshape(*lead, N // 128, K // 128)


@pytest.mark.parametrize("T,E,k", [(7, 4, 2), (300, 8, 2), (64, 16, 4)])
def test_fused_experts_fp8_block_matches_dequantised_reference(T, E, k):
    """Grouped fp8 GEMMs with 128 x 128 weight scales and 1 x 128 activation scales against
    the fp32 reference on the de-quantised weights (activation quantisation is the only
    difference: a few percent of the output scale)."""
    from vllm_gcu_b200.ops import _native, ref
    from vllm_gcu_b200.ops import cuda as C
    torch.manual_seed(T)
    dev = "cuda"
    H, I = 256, 384
    w13 = torch.randn(E, 2 * I, H, device=dev) * 0.05
    w2 = torch.randn(E, H, I, device=dev) * 0.05
    q13, s13 = _block_quant_fp8(w13)
    q2, s2 = _block_quant_fp8(w2)
    x = (torch.randn(T, H, device=dev) * 0.5).to(torch.bfloat16)
    logits = torch.randn(T, E, device=dev)
    tw, ti = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    ti = ti.to(torch.int32)
    add = (torch.randn(T, H, device=dev) * 0.1).to(torch.bfloat16)
    got = C.fused_experts_fp8(x, q13.contiguous(), s13.contiguous(), q2.contiguous(),
                              s2.contiguous(), tw.float(), ti, add=add)
    torch.cuda.synchronize()
    _native.check_status()
    d13 = (q13.float().reshape(E, 2 * I // 128, 128, H // 128, 128)
           * s13[:, :, None, :, None]).reshape(E, 2 * I, H)
    d2 = (q2.float().reshape(E, H // 128, 128, I // 128, 128)
          * s2[:, :, None, :, None]).reshape(E, H, I)
    want = ref.fused_experts(x.float(), d13, d2, tw.float(), ti).float() + add.float()
    err = (got.float() - want).abs().max().item()
    scale = (want - add.float()).abs().max().item()
    assert err < 0.06 * scale + 0.02, (err, scale)
    # expert map (expert parallel rank owning the upper half): other experts contribute nothing
    emap = torch.full((E,), -1, dtype=torch.int32, device=dev)
    emap[E // 2:] = torch.arange(E - E // 2, dtype=torch.int32, device=dev)
    got_h = C.fused_experts_fp8(x, q13[E // 2:].contiguous(), s13[E // 2:].contiguous(),
                                q2[E // 2:].contiguous(), s2[E // 2:].contiguous(), tw.float(),
                                ti, expert_map=emap)
    want_h = ref.fused_experts(x.float(), d13[E // 2:], d2[E // 2:], tw.float(), ti, emap).float()
    torch.cuda.synchronize()
    _native.check_status()
    err = (got_h.float() - want_h).abs().max().item()
    assert err < 0.06 * want_h.abs().max().item() + 0.02, err


def test_fp8_block_experts_stay_quantised_through_loader_and_engine():
    """A Qwen3-MoE-shaped model declared as fp8 with 128 x 128 blocks keeps its experts in
    fp8 (loader path of quantised checkpoints) and generates through the grouped fp8 GEMMs."""
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    from vllm_gcu_b200.layers.quant.moe import QuantExpertLoader
    llm = LLM("tiny-qwen3-moe", device="cuda", hidden_size=256, intermediate_size=512,
              num_attention_heads=4, num_key_value_heads=2, head_dim=64, num_experts=8,
              num_experts_per_tok=2, moe_intermediate_size=128, dtype="bfloat16",
              quantization="fp8", quant_config={"quant_method": "fp8",
                                                "weight_block_size": [128, 128]},
              max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, num_gpu_blocks=64,
              cuda_graph_sizes=[4])
    moe = llm.engine.model.layers["0"].mlp.experts
    assert moe.fp8_block and moe.w13.dtype == torch.float8_e4m3fn
    # loader: an fp8 projection with its block scale lands in the fp8 tables untouched
    w = (torch.randn(128, 256, device="cuda")).to(torch.float8_e4m3fn)
    sc = torch.rand(1, 2, device="cuda") + 0.5
    ld = QuantExpertLoader("fp8", {"quant_method": "fp8", "weight_block_size": [128, 128]},
                           torch.bfloat16)
    ld.add(moe, "model.layers.0.", 3, "gate", "weight", w)
    ld.add(moe, "model.layers.0.", 3, "gate", "weight_scale_inv", sc)
    assert torch.equal(moe.w13.data[3, :128].view(torch.uint8), w.view(torch.uint8))
    assert torch.equal(moe.w13_scale.data[3, :1], sc)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (20, 9, 33)]
    n0 = _native.launch_count
    outs = llm.generate(prompts, SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True))
    torch.cuda.synchronize()
    _native.check_status()
    assert _native.launch_count > n0 and all(len(o.outputs[0].token_ids) == 5 for o in outs)


@pytest.mark.parametrize("dtype", [torch.int8, torch.float8_e4m3fn])
def test_fused_experts_q8_channel_matches_dequantised_reference(dtype):
    """int8 / fp8 experts with per-channel scales and per-token activation quantisation
    (w8a8 checkpoints) against the fp32 reference on the de-quantised weights."""
    from vllm_gcu_b200.ops import cuda as C
    torch.manual_seed(11)
    dev = "cuda"
    T, E, k, H, I = 150, 8, 2, 256, 192
    w13 = torch.randn(E, 2 * I, H, device=dev) * 0.05
    w2 = torch.randn(E, H, I, device=dev) * 0.05
    qmax = 127.0 if dtype == torch.int8 else 448.0

    def quant(w):
        s = w.abs().amax(-1).clamp_min(1e-8) / qmax
        q = w / s[..., None]
        q = torch.round(q).clamp(-128, 127).to(torch.int8) if dtype == torch.int8 else q.to(dtype)
        return q.contiguous(), s.float().contiguous()

    q13, s13 = quant(w13)
    q2, s2 = quant(w2)
    x = (torch.randn(T, H, device=dev) * 0.5).to(torch.bfloat16)
    tw, ti = torch.topk(torch.softmax(torch.randn(T, E, device=dev), -1), k, dim=-1)
    ti = ti.to(torch.int32)
    got = C.fused_experts_q8(x, q13, s13, q2, s2, tw.float(), ti)
    torch.cuda.synchronize()
    _native.check_status()
    want = ref.fused_experts(x.float(), q13.float() * s13[..., None], q2.float() * s2[..., None],
                             tw.float(), ti).float()
    err = (got.float() - want).abs().max().item()
    tol = (0.03 if dtype == torch.int8 else 0.08) * want.abs().max().item() + 0.02
    assert err < tol, (err, want.abs().max().item())


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("T,k", [(16, 2), (150, 2), (700, 2)])
def test_fused_experts_wna16_packed_matches_dequantised_reference(bits, T, k):
    """Experts kept as packed 4 / 8-bit integers with per-group scales (AWQ / GPTQ layouts):
    the grouped de-quantising GEMM for decode-sized batches and the scratch + bf16 grouped
    GEMM for large ones, against the fp32 reference on the de-quantised weights.  One expert
    gets no token; an expert map hides two experts (expert parallelism)."""
    from vllm_gcu_b200.ops import cuda as C
    torch.manual_seed(13 + bits + T)
    dev = "cuda"
    E, H, I, g = 8, 512, 256, 128
    top = 1 << bits

    def make(n, kk):
        q = torch.randint(0, top, (E, n, kk), device=dev, dtype=torch.uint8)
        s = (torch.rand(E, n, kk // g, device=dev) * (0.4 / top) + 0.1 / top).to(torch.bfloat16)
        z = (torch.randint(0, top, (E, n, kk // g), device=dev).float() * s.float()).to(
            torch.bfloat16)
        w = q.float() * s.float().repeat_interleave(g, -1) - z.float().repeat_interleave(g, -1)
        packed = (q[..., 0::2] | (q[..., 1::2] << 4)).contiguous() if bits == 4 else q
        return packed, s.contiguous(), z.contiguous(), w

    q13, s13, z13, w13 = make(2 * I, H)
    q2, s2, z2, w2 = make(H, I)
    x = (torch.randn(T, H, device=dev) * 0.5).to(torch.bfloat16)
    logits = torch.randn(T, E, device=dev)
    logits[:, 5] = -1e9                                  # expert 5 gets nothing
    tw, ti = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    ti = ti.to(torch.int32)
    fused = T * k <= C.WNA16_GROUPED_MAX_ROWS_PER_EXPERT * E
    assert fused == (T <= 150)
    for emap in (None, torch.tensor([0, 1, -1, 2, 3, 4, -1, 5], device=dev, dtype=torch.int32)):
        if emap is None:
            args = (q13, s13, z13, q2, s2, z2)
            w13_r, w2_r = w13, w2
        else:
            keep = (emap >= 0).nonzero().flatten()
            args = tuple(t[keep].contiguous() for t in (q13, s13, z13, q2, s2, z2))
            w13_r, w2_r = w13[keep], w2[keep]
        add = torch.randn(T, H, device=dev).to(torch.bfloat16)
        got = C.fused_experts_wna16(x, *args, g, bits, tw.float(), ti, emap, add=add)
        torch.cuda.synchronize()
        _native.check_status()
        want = ref.fused_experts(x.float(), w13_r, w2_r, tw.float(), ti, emap).float() \
            + add.float()
        err = (got.float() - want).abs().max().item()
        assert err < 0.03 * want.abs().max().item() + 0.03, (bits, T, emap is None, err,
                                                             want.abs().max().item())


def test_packed_wna16_experts_through_the_moe_layer():
    """``FusedMoE.enable_wna16`` on the GPU: the packed layer equals the same experts
    de-quantised into a bf16 layer."""
    from vllm_gcu_b200.layers.moe import FusedMoE
    torch.manual_seed(21)
    dev = "cuda"
    E, H, I, g, bits = 4, 256, 128, 64, 4
    packed = FusedMoE(E, H, I, torch.bfloat16, dev, False)
    plain = FusedMoE(E, H, I, torch.bfloat16, dev, False)
    assert packed.enable_wna16(bits, g)
    for e in range(E):
        for which, (n, kk) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
            q = torch.randint(0, 16, (n, kk), device=dev, dtype=torch.uint8)
            s = (torch.rand(n, kk // g, device=dev) * 0.02 + 0.005).to(torch.bfloat16)
            zs = (torch.randint(0, 16, (n, kk // g), device=dev).float() * s.float()).to(
                torch.bfloat16)
            w = q.float() * s.float().repeat_interleave(g, 1) - zs.float().repeat_interleave(g, 1)
            assert packed.load_expert_weight_wna16(e, which, q, s, zs)
            plain.load_expert_weight(e, which, w.to(torch.bfloat16))
    plain.finalize()
    packed.finalize()
    x = (torch.randn(33, H, device=dev) * 0.5).to(torch.bfloat16)
    tw, ti = torch.topk(torch.softmax(torch.randn(33, E, device=dev), -1), 2, dim=-1)
    a = packed(x, tw.float(), ti.to(torch.int32)).float()
    b = plain(x, tw.float(), ti.to(torch.int32)).float()
    torch.cuda.synchronize()
    assert (a - b).abs().max().item() < 0.03 * b.abs().max().item() + 0.02
