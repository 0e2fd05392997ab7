"""End-to-end engine checks on a GPU: native kernels + CUDA graphs vs the CPU reference."""
import pytest
import torch

from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams
from vllm_gcu_b200.ops import _native

pytestmark = pytest.mark.gpu


def _prompts(n, lens, vocab, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (lens[i % len(lens)],), generator=g).tolist()
            for i in range(n)]


def test_llama_bf16_gpu_matches_cpu_reference():
    kw = dict(num_hidden_layers=2, hidden_size=512, intermediate_size=1024,
              num_attention_heads=8, num_key_value_heads=2, head_dim=64, vocab_size=2048,
              max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256, num_gpu_blocks=128)
    sp = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    prompts = _prompts(5, [17, 40, 64, 3, 90], 2048)
    gpu = LLM("llama-3-8b", device="cuda", cuda_graph_sizes=[1, 2, 4, 8], **kw)
    n0 = _native.launch_count
    out_gpu = gpu.generate(prompts, sp)
    assert _native.launch_count > n0
    # same weights on the CPU reference path
    cpu = LLM("llama-3-8b", device="cpu", **kw)
    sd = {k: v.detach().cpu() for k, v in gpu.engine.model.state_dict().items()}
    # the GPU model keeps gate_up interleaved for the fused epilogue: undo it for the CPU copy
    for name, mod in gpu.engine.model.named_modules():
        if getattr(mod, "_interleaved", False):
            w = sd[name + ".weight"]
            I = w.shape[0] // 2
            w4 = w.view(I // 32, 2, 32, w.shape[1])
            sd[name + ".weight"] = torch.cat([w4[:, 0].reshape(I, -1), w4[:, 1].reshape(I, -1)])
    cpu.engine.model.load_state_dict(sd, strict=False)
    out_cpu = cpu.generate(prompts, sp)
    for a, b in zip(out_gpu, out_cpu):
        ta, tb = a.outputs[0].token_ids, b.outputs[0].token_ids
        assert len(ta) == len(tb) == 12
        assert ta[0] == tb[0]
    # numerics: logits of one prefill step, GPU kernels vs the torch reference
    one = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
    gpu.engine.runner.keep_logits = True
    cpu.engine.runner.keep_logits = True
    p2 = _prompts(3, [70, 33, 128], 2048, seed=5)
    gpu.engine.runner.graphs = {}            # logits are only kept on the eager path
    gpu.generate(p2, one)
    cpu.generate(p2, one)
    lg, lc = gpu.engine.runner.last_logits, cpu.engine.runner.last_logits
    assert lg.shape == lc.shape == (3, 2048)
    err = (lg - lc).abs().max().item()
    assert err < 0.05 * lc.std().item() + 0.02, (err, lc.std().item())
    _native.check_status()


@pytest.mark.parametrize("async_sched", [False, True])
def test_graphs_async_and_eager_agree(async_sched):
    kw = dict(num_hidden_layers=2, max_num_seqs=16, max_num_batched_tokens=512,
              max_model_len=512, num_gpu_blocks=512)
    sp = SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True)
    prompts = _prompts(20, [33, 100, 7, 250], 128256, seed=3)
    a = LLM("llama-3-8b", device="cuda", enforce_eager=True, **kw).generate(prompts, sp)
    b = LLM("llama-3-8b", device="cuda", cuda_graph_sizes=[1, 2, 4, 8, 16],
            async_scheduling=async_sched, **kw).generate(prompts, sp)
    same = sum(x.outputs[0].token_ids == y.outputs[0].token_ids for x, y in zip(a, b))
    assert same >= 18, same
    _native.check_status()


def test_smoke_entry():
    import __graft_entry__ as g
    g.smoke()


@pytest.mark.parametrize("kvd", ["fp8", "int8"])
def test_engine_with_8bit_kv_cache_tracks_bf16(kvd):
    """The engine with an fp8 / int8 KV cache: logits of a step that reads a long cached
    prefix stay close to the bf16-cache engine; sampling extras work on the GPU path."""
    kw = dict(num_hidden_layers=2, max_num_seqs=8, max_num_batched_tokens=256,
              max_model_len=512, num_gpu_blocks=256, enforce_eager=True)
    prompts = _prompts(3, [200, 33, 120], 128256, seed=9)
    sp = SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True, logprobs=2)
    base = LLM("llama-3-8b", device="cuda", **kw)
    base.engine.runner.keep_logits = True
    ob = base.generate(prompts, sp)
    lb = base.engine.runner.last_logits
    q8 = LLM("llama-3-8b", device="cuda", kv_cache_dtype=kvd, **kw)
    assert q8.engine.runner.kv_caches[0].element_size() == 1
    q8.engine.runner.keep_logits = True
    oq = q8.generate(prompts, sp)
    lq = q8.engine.runner.last_logits
    assert lb.shape == lq.shape
    cos = torch.nn.functional.cosine_similarity(lb.flatten(), lq.flatten(), dim=0).item()
    rms = ((lb - lq).pow(2).mean().sqrt() / lb.std()).item()
    assert cos > 0.97 and rms < 0.25, (cos, rms)
    for o in ob + oq:
        assert len(o.outputs[0].logprobs) == 3 and o.outputs[0].cumulative_logprob <= 0
    _native.check_status()


def test_oracle_mode_checks_every_step(monkeypatch):
    """With VLLM_B200_ORACLE=all the GEMM and attention wrappers recompute their result with
    the torch reference and raise on a mismatch; a short eager run must pass all checks."""
    from vllm_gcu_b200.ops import cuda as C
    monkeypatch.setenv("VLLM_B200_ORACLE", "all")
    assert C.oracle_enabled("gemm_bf16") and C.oracle_enabled("paged_decode")
    kw = dict(num_hidden_layers=2, hidden_size=512, intermediate_size=1024,
              num_attention_heads=8, num_key_value_heads=2, head_dim=128, vocab_size=2048,
              max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256, num_gpu_blocks=128,
              enforce_eager=True)
    llm = LLM("llama-3-8b", device="cuda", **kw)
    out = llm.generate(_prompts(4, [40, 7, 150, 64], 2048, seed=11),
                       SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))
    assert all(len(o.outputs[0].token_ids) == 4 for o in out)
    with pytest.raises(C.OracleMismatch):
        C.oracle_compare("probe", torch.ones(4, device="cuda"), torch.zeros(4))
    _native.check_status()


def test_swap_preemption_on_gpu_reproduces_unpreempted_tokens():
    """Too few KV blocks for the batch: victims are swapped to pinned host blocks
    (b200_swap_blocks on the step's stream) and resume without recomputing."""
    kw = dict(num_hidden_layers=2, hidden_size=512, intermediate_size=1024,
              num_attention_heads=8, num_key_value_heads=2, head_dim=64, vocab_size=2048,
              max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256,
              enable_prefix_caching=False, enforce_eager=True)
    sp = SamplingParams(max_tokens=30, temperature=0.0, ignore_eos=True)
    prompts = _prompts(3, [50, 44, 37], 2048, seed=9)
    ample = LLM("llama-3-8b", device="cuda", num_gpu_blocks=64, **kw)
    want = [o.outputs[0].token_ids for o in ample.generate(prompts, sp)]
    tight = LLM("llama-3-8b", device="cuda", num_gpu_blocks=12, num_cpu_blocks=16, **kw)
    got = [o.outputs[0].token_ids for o in tight.generate(prompts, sp)]
    torch.cuda.synchronize()
    _native.check_status()
    assert tight.engine.scheduler.num_swaps > 0
    assert got == want


def test_gemma_head_dim_256_gpu_tracks_cpu_reference():
    """Gemma-shaped model (head size 256, GeGLU, tied scaled embedding): decode runs on the
    256-wide paged kernel, prefill on the torch formulation; logits follow the CPU path."""
    from vllm_gcu_b200.config import ModelConfig
    d = dict(architectures=["GemmaForCausalLM"], vocab_size=2048, hidden_size=512,
             intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=1, head_dim=256, rms_norm_eps=1e-6,
             hidden_act="gelu_pytorch_tanh", max_position_embeddings=512)
    kw = dict(max_num_seqs=4, max_num_batched_tokens=128, max_model_len=256, num_gpu_blocks=64)
    gpu = LLM(ModelConfig.from_hf_dict(d, dtype=torch.bfloat16), device="cuda",
              cuda_graph_sizes=[4], **kw)
    cpu = LLM(ModelConfig.from_hf_dict(d, dtype=torch.bfloat16), device="cpu", **kw)
    sd = {k: v.detach().cpu() for k, v in gpu.engine.model.state_dict().items()}
    cpu.engine.model.load_state_dict(sd, strict=False)
    prompts = _prompts(3, [40, 9, 77], 2048, seed=3)
    sp = SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True)
    og = gpu.generate(prompts, sp)
    oc = cpu.generate(prompts, sp)
    torch.cuda.synchronize()
    _native.check_status()
    assert [o.outputs[0].token_ids[0] for o in og] == [o.outputs[0].token_ids[0] for o in oc]
    one = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
    gpu.engine.runner.keep_logits = cpu.engine.runner.keep_logits = True
    gpu.engine.runner.graphs = {}
    gpu.generate(prompts, one)
    cpu.generate(prompts, one)
    lg, lc = gpu.engine.runner.last_logits, cpu.engine.runner.last_logits
    err = (lg - lc).abs().max().item()
    assert err < 0.06 * lc.std().item() + 0.03, (err, lc.std().item())


def test_same_batch_twice_is_bitwise_identical():
    """Determinism run (surfaces races in flag protocols and reductions): the same batch
    through the same engine twice gives bitwise equal logits and tokens, eager and graphs."""
    kw = dict(num_hidden_layers=2, hidden_size=512, intermediate_size=1024,
              num_attention_heads=8, num_key_value_heads=2, head_dim=64, vocab_size=2048,
              max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256, num_gpu_blocks=128,
              enable_prefix_caching=False)
    llm = LLM("llama-3-8b", device="cuda", cuda_graph_sizes=[4, 8], **kw)
    prompts = _prompts(6, [17, 40, 64, 3, 90, 33], 2048, seed=21)
    sp = SamplingParams(max_tokens=8, temperature=0.7, top_k=20, top_p=0.9, seed=5,
                        ignore_eos=True)
    llm.engine.runner.keep_logits = True
    runs = []
    for _ in range(2):
        outs = llm.generate(prompts, sp)
        torch.cuda.synchronize()
        runs.append(([o.outputs[0].token_ids for o in outs],
                     llm.engine.runner.last_logits.clone()
                     if llm.engine.runner.last_logits is not None else None))
    assert runs[0][0] == runs[1][0]
    if runs[0][1] is not None:
        assert torch.equal(runs[0][1], runs[1][1])
    _native.check_status()


@pytest.mark.parametrize("scheme", ["fp8_token", "fp8_block", "fp8_static"])
def test_norm_and_activation_kernels_emit_quantised_rows(scheme, monkeypatch):
    """8-bit linear layers: the RMSNorm in front of qkv / gate_up and the gated activation in
    front of down_proj write fp8 rows and scales themselves.  Same logits as with separate
    quantisation kernels (both quantise the same fp32 values up to the 16-bit rounding of the
    intermediate), with fewer launches."""
    qc = {"fp8_token": {}, "fp8_block": {"weight_block_size": [128, 128]},
          "fp8_static": {"activation_scheme": "static"}}[scheme]
    kw = dict(num_hidden_layers=2, hidden_size=512, intermediate_size=1024,
              num_attention_heads=8, num_key_value_heads=2, head_dim=64, vocab_size=2048,
              max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256, num_gpu_blocks=128,
              quantization="fp8", quant_config=qc, enforce_eager=True, seed=0)
    one = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
    prompts = _prompts(3, [70, 33, 128], 2048, seed=5)
    logits, launches = {}, {}
    for fuse in ("1", "0"):
        monkeypatch.setenv("VLLM_B200_FUSE_ACT_QUANT", fuse)
        llm = LLM("llama-3-8b", device="cuda", **kw)
        if scheme == "fp8_static":
            for m in llm.engine.model.modules():
                if hasattr(m, "input_scale"):
                    m.input_scale.data.fill_(0.05)
        llm.engine.runner.keep_logits = True
        n0 = _native.launch_count
        llm.generate(prompts, one)
        launches[fuse] = _native.launch_count - n0
        logits[fuse] = llm.engine.runner.last_logits.float().clone()
        _native.check_status()
    # per layer: the two norms absorb their quantisation kernels; the gated activation absorbs
    # its one for group and static scales (it has no per-token mode)
    saved = 2 if scheme == "fp8_token" else 3
    assert launches["1"] <= launches["0"] - 2 * saved, launches
    err = (logits["1"] - logits["0"]).abs().max().item()
    spread = logits["0"].std().item()
    assert err < 0.1 * spread + 0.02, (err, spread)
    assert logits["1"].isfinite().all()


@pytest.mark.parametrize("method,model", [("ngram", "llama"), ("eagle", "llama"),
                                          ("medusa", "llama"), ("mtp", "tiny-deepseek")])
def test_speculative_decoding_on_gpu(method, model):
    """Draft proposers on the GPU path (n-gram on the host; EAGLE / MTP drafters with their own
    KV cache; Medusa heads): drafts are proposed and verified, every request gets its tokens,
    and the output starts like the greedy output without drafts (later tokens may differ where
    two logits are nearly tied: verification scores several positions in one pass)."""
    if model == "llama":
        name = "llama-3-8b"
        kw = dict(num_hidden_layers=2, hidden_size=512, intermediate_size=1024,
                  num_attention_heads=8, num_key_value_heads=2, head_dim=64, vocab_size=2048)
    else:
        name, kw = model, dict(dtype="bfloat16")
    kw.update(max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256, num_gpu_blocks=128,
              seed=0)
    V = kw.get("vocab_size", 1024)
    g = torch.Generator().manual_seed(2)
    base = torch.randint(0, V, (12,), generator=g).tolist()
    prompts = [base * 3 + base[:5], base[::-1] * 2 + base[:3], base * 2]
    sp = SamplingParams(max_tokens=16, temperature=0.0, ignore_eos=True)
    plain = LLM(name, device="cuda", enforce_eager=True, **kw).generate(prompts, sp)
    k = 3 if method in ("ngram", "medusa") else 1
    llm = LLM(name, device="cuda", enforce_eager=True, speculative_method=method,
              num_speculative_tokens=k, **kw)
    outs = llm.generate(prompts, sp)
    torch.cuda.synchronize()
    _native.check_status()
    m = llm.engine.spec_metrics
    assert m.num_drafts > 0 and m.num_draft_tokens > 0
    for a, b in zip(outs, plain):
        ta, tb = a.outputs[0].token_ids, b.outputs[0].token_ids
        assert len(ta) == len(tb) == 16
        assert ta[:2] == tb[:2], (method, ta, tb)
