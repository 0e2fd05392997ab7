"""Dense decoder families that differ from Llama only in checkpoint layout or small maths:
InternLM2 (fused ``wqkv``, renamed modules), Baichuan2-7B (``W_pack``, normalised LM head) and
Gemma (GeGLU, ``1 + weight`` norms, scaled embeddings).  The oracle is the HuggingFace
implementation of the same mathematics on a tiny random model."""
import pytest
import torch

tr = pytest.importorskip("transformers")

from vllm_gcu_b200.config import ModelConfig  # noqa: E402
from vllm_gcu_b200.engine.llm import LLM  # noqa: E402
from vllm_gcu_b200.engine.request import SamplingParams  # noqa: E402

IDS = [5, 17, 99, 3, 250, 42, 7, 7, 81, 120, 33]


def _engine_logits(arch, hf_cfg_dict, weights):
    d = dict(hf_cfg_dict)
    d["architectures"] = [arch]
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    llm = LLM(mc, device="cpu", max_num_seqs=2, max_num_batched_tokens=32, max_model_len=64,
              num_gpu_blocks=16, load_format="none")
    llm.engine.model.load_weights(weights)
    llm.engine.runner.keep_logits = True
    out = llm.generate([IDS], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
    return llm.engine.runner.last_logits[0], out[0].outputs[0].token_ids[0]


def _tiny_llama(vocab=300, kv=2):
    cfg = tr.LlamaConfig(vocab_size=vocab, hidden_size=64, intermediate_size=128,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=kv,
                         max_position_embeddings=128, rms_norm_eps=1e-6, tie_word_embeddings=False)
    torch.manual_seed(0)
    return cfg, tr.LlamaForCausalLM(cfg).eval().float()


def _hf_last_logits(model):
    with torch.inference_mode():
        return model(input_ids=torch.tensor([IDS])).logits[0, -1]


def test_internlm2_layout_loads_into_the_llama_mathematics():
    cfg, hf = _tiny_llama()
    kvh, g, d = 2, 2, 16
    sd = {}
    for k, v in hf.state_dict().items():
        k = (k.replace("model.embed_tokens.", "model.tok_embeddings.").replace("lm_head.", "output.")
             .replace(".self_attn.o_proj.", ".attention.wo.")
             .replace(".input_layernorm.", ".attention_norm.")
             .replace(".post_attention_layernorm.", ".ffn_norm.")
             .replace(".mlp.gate_proj.", ".feed_forward.w1.").replace(".mlp.up_proj.", ".feed_forward.w3.")
             .replace(".mlp.down_proj.", ".feed_forward.w2."))
        sd[k] = v
    for i in range(2):
        p = f"model.layers.{i}.self_attn."
        q = sd.pop(p + "q_proj.weight").view(kvh, g, d, -1)
        k = sd.pop(p + "k_proj.weight").view(kvh, 1, d, -1)
        v = sd.pop(p + "v_proj.weight").view(kvh, 1, d, -1)
        sd[f"model.layers.{i}.attention.wqkv.weight"] = torch.cat([q, k, v], 1).reshape(-1, 64)
    got, tok = _engine_logits("InternLM2ForCausalLM", cfg.to_dict(), sd.items())
    want = _hf_last_logits(hf)
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()
    assert tok == int(want.argmax())


def test_baichuan2_w_pack_and_normalised_head():
    cfg, hf = _tiny_llama(vocab=125696, kv=4)       # Baichuan: as many KV heads as query heads
    sd = dict(hf.state_dict())
    for i in range(2):
        p = f"model.layers.{i}.self_attn."
        sd[p + "W_pack.weight"] = torch.cat([sd.pop(p + "q_proj.weight"), sd.pop(p + "k_proj.weight"),
                                             sd.pop(p + "v_proj.weight")], 0)
    d = cfg.to_dict()
    d["position_embedding"] = "ROPE"     # a 7B checkpoint (hidden size 4096) selects this itself
    got, tok = _engine_logits("BaichuanForCausalLM", d, sd.items())
    with torch.inference_mode():
        h = hf.model(input_ids=torch.tensor([IDS])).last_hidden_state[0, -1]
        want = torch.nn.functional.normalize(hf.lm_head.weight) @ h
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()
    assert tok == int(want.argmax())


def test_baichuan_13b_alibi_positions():
    """Baichuan 13B: no rotary embedding, ALiBi biases slope_h * (j - i) on the scores.  The
    oracle is the dense mathematics written out here on the weights of a tiny Llama; the engine
    runs it through the paged KV cache, chunked (prefill of 8 tokens, then the rest)."""
    from vllm_gcu_b200.layers.attention import alibi_slopes
    cfg, hf = _tiny_llama(vocab=300, kv=4)
    sd = dict(hf.state_dict())
    for i in range(2):
        p = f"model.layers.{i}.self_attn."
        sd[p + "W_pack.weight"] = torch.cat([sd[p + "q_proj.weight"], sd[p + "k_proj.weight"],
                                             sd[p + "v_proj.weight"]], 0)
    d = cfg.to_dict()
    d["architectures"] = ["BaichuanForCausalLM"]     # hidden size != 4096: the ALiBi variant
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    llm = LLM(mc, device="cpu", max_num_seqs=2, max_num_batched_tokens=8, max_model_len=64,
              num_gpu_blocks=16, load_format="none")
    assert llm.engine.model.layers["0"].self_attn.attn.alibi is not None
    assert llm.engine.model.layers["0"].self_attn.attn.rotary is None
    llm.engine.model.load_weights((k, v) for k, v in sd.items()
                                  if not k.endswith(("q_proj.weight", "k_proj.weight",
                                                     "v_proj.weight")))
    llm.engine.runner.keep_logits = True
    out = llm.generate([IDS], SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True))
    toks = out[0].outputs[0].token_ids

    def rms(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w

    def dense(ids):
        n, H, D = len(ids), 4, 16
        x = sd["model.embed_tokens.weight"][torch.tensor(ids)]
        pos = torch.arange(n)
        bias = alibi_slopes(H)[:, None, None] * (pos[None, :] - pos[:, None]).float()[None]
        causal = pos[None, :] <= pos[:, None]
        for i in range(2):
            p = f"model.layers.{i}."
            h = rms(x, sd[p + "input_layernorm.weight"])
            q = (h @ sd[p + "self_attn.q_proj.weight"].t()).view(n, H, D).transpose(0, 1)
            k = (h @ sd[p + "self_attn.k_proj.weight"].t()).view(n, H, D).transpose(0, 1)
            v = (h @ sd[p + "self_attn.v_proj.weight"].t()).view(n, H, D).transpose(0, 1)
            s_ = q @ k.transpose(1, 2) * D ** -0.5 + bias
            s_ = s_.masked_fill(~causal[None], float("-inf"))
            a = (torch.softmax(s_, -1) @ v).transpose(0, 1).reshape(n, H * D)
            x = x + a @ sd[p + "self_attn.o_proj.weight"].t()
            h = rms(x, sd[p + "post_attention_layernorm.weight"])
            g = torch.nn.functional.silu(h @ sd[p + "mlp.gate_proj.weight"].t())
            x = x + (g * (h @ sd[p + "mlp.up_proj.weight"].t())) @ sd[p + "mlp.down_proj.weight"].t()
        return rms(x, sd["model.norm.weight"])[-1] @ sd["lm_head.weight"].t()

    seq = list(IDS)
    with torch.inference_mode():
        for t in toks:
            want = dense(seq)
            assert t == int(want.argmax())
            seq.append(t)
    got = llm.engine.runner.last_logits[0]
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()


def test_gemma_matches_transformers():
    cfg = tr.GemmaConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=1, head_dim=16,
                         max_position_embeddings=128, rms_norm_eps=1e-6)
    torch.manual_seed(1)
    hf = tr.GemmaForCausalLM(cfg).eval().float()
    with torch.no_grad():                      # non-trivial norm weights (initialised to zero)
        for n, p in hf.named_parameters():
            if n.endswith("norm.weight"):
                p.copy_(torch.randn_like(p) * 0.1)
    got, tok = _engine_logits("GemmaForCausalLM", cfg.to_dict(), hf.state_dict().items())
    want = _hf_last_logits(hf)
    assert torch.allclose(got, want, atol=3e-4), (got - want).abs().max()
    assert tok == int(want.argmax())


def test_chatglm_layout_matches_the_glm_mathematics():
    """ChatGLM3 / GLM-4-9B original checkpoints: the oracle is transformers' ``GlmForCausalLM``
    (same mathematics in the HF layout), its weights renamed into the ChatGLM layout."""
    cfg = tr.GlmConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                       partial_rotary_factor=0.5, attention_bias=True, rms_norm_eps=1e-5,
                       max_position_embeddings=128, tie_word_embeddings=False, pad_token_id=0)
    torch.manual_seed(2)
    hf = tr.GlmForCausalLM(cfg).eval().float()
    src = hf.state_dict()
    sd = {"transformer.embedding.word_embeddings.weight": src["model.embed_tokens.weight"],
          "transformer.encoder.final_layernorm.weight": src["model.norm.weight"],
          "transformer.output_layer.weight": src["lm_head.weight"],
          "transformer.rotary_pos_emb.inv_freq": torch.zeros(4)}
    for i in range(2):
        a, b = f"model.layers.{i}.", f"transformer.encoder.layers.{i}."
        for kind in ("weight", "bias"):
            sd[b + "self_attention.query_key_value." + kind] = torch.cat(
                [src[a + f"self_attn.{p}_proj.{kind}"] for p in "qkv"], 0)
        sd[b + "self_attention.dense.weight"] = src[a + "self_attn.o_proj.weight"]
        sd[b + "mlp.dense_h_to_4h.weight"] = src[a + "mlp.gate_up_proj.weight"]
        sd[b + "mlp.dense_4h_to_h.weight"] = src[a + "mlp.down_proj.weight"]
        sd[b + "input_layernorm.weight"] = src[a + "input_layernorm.weight"]
        sd[b + "post_attention_layernorm.weight"] = src[a + "post_attention_layernorm.weight"]
    chatglm_cfg = {"model_type": "chatglm", "num_layers": 2, "hidden_size": 64,
                   "ffn_hidden_size": 128, "num_attention_heads": 4, "kv_channels": 16,
                   "multi_query_attention": True, "multi_query_group_num": 2,
                   "layernorm_epsilon": 1e-5, "padded_vocab_size": 300, "seq_length": 128,
                   "add_qkv_bias": True, "rmsnorm": True}
    got, tok = _engine_logits("ChatGLMModel", chatglm_cfg, sd.items())
    want = _hf_last_logits(hf)
    assert torch.allclose(got, want, atol=3e-4), (got - want).abs().max()
    assert tok == int(want.argmax())


def test_gpt_bigcode_matches_transformers():
    """StarCoder / WizardCoder architecture: learnt positions, LayerNorm, multi-query
    attention, plain GELU MLP with biases, tied LM head."""
    cfg = tr.GPTBigCodeConfig(vocab_size=300, n_positions=128, n_embd=64, n_layer=2, n_head=4,
                              n_inner=128, activation_function="gelu_pytorch_tanh",
                              multi_query=True, layer_norm_epsilon=1e-5, resid_pdrop=0.0,
                              embd_pdrop=0.0, attn_pdrop=0.0)
    torch.manual_seed(3)
    hf = tr.GPTBigCodeForCausalLM(cfg).eval().float()
    with torch.no_grad():                      # biases and norm offsets start at zero
        for n, p in hf.named_parameters():
            if n.endswith(".bias"):
                p.copy_(torch.randn_like(p) * 0.05)
    got, tok = _engine_logits("GPTBigCodeForCausalLM", cfg.to_dict(), hf.state_dict().items())
    want = _hf_last_logits(hf)
    assert torch.allclose(got, want, atol=3e-4), (got - want).abs().max()
    assert tok == int(want.argmax())
    # decode steps through the paged cache agree with a full recompute
    from vllm_gcu_b200.config import ModelConfig as MC
    from vllm_gcu_b200.engine.llm import LLM as L
    d = cfg.to_dict()
    d["architectures"] = ["GPTBigCodeForCausalLM"]
    llm = L(MC.from_hf_dict(d, dtype=torch.float32), device="cpu", max_num_seqs=2,
            max_num_batched_tokens=8, max_model_len=64, num_gpu_blocks=16, load_format="none")
    llm.engine.model.load_weights(hf.state_dict().items())
    toks = llm.generate([IDS], SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True)
                        )[0].outputs[0].token_ids
    seq = list(IDS)
    for t in toks:
        with torch.inference_mode():
            assert t == int(hf(input_ids=torch.tensor([seq])).logits[0, -1].argmax())
        seq.append(t)


def test_qwen2_embedding_checkpoint_matches_transformers():
    """gte-Qwen2 style embedding: bare ``Qwen2Model`` tensor names, last-token pooling,
    L2-normalised; prompts of different lengths run through the scheduler together."""
    cfg = tr.Qwen2Config(vocab_size=300, hidden_size=64, intermediate_size=128,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         max_position_embeddings=128, rms_norm_eps=1e-6)
    torch.manual_seed(3)
    hf = tr.Qwen2Model(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("bias") or n.endswith("norm.weight"):
                p.copy_(torch.randn_like(p) * 0.2 + (1.0 if "norm" in n else 0.0))
    d = cfg.to_dict()
    d["architectures"] = ["Qwen2Model"]
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    llm = LLM(mc, device="cpu", max_num_seqs=4, max_num_batched_tokens=16, max_model_len=64,
              num_gpu_blocks=32, load_format="none")
    loaded = llm.engine.model.load_weights(hf.state_dict().items())
    assert "model.layers.0.self_attn.q_proj.bias" in loaded and "model.norm.weight" in loaded
    prompts = [IDS, IDS[:4], IDS[2:] + [9, 9, 200, 1, 4, 77, 12, 13]]   # last one is chunked
    got = llm.embed(prompts)
    assert got.shape == (3, 64)
    for g, p in zip(got, prompts):
        with torch.inference_mode():
            want = hf(input_ids=torch.tensor([p])).last_hidden_state[0, -1]
        want = torch.nn.functional.normalize(want, dim=-1)
        assert torch.allclose(g, want, atol=2e-4), (g - want).abs().max()
    # pooling and generating requests share a batch; only the pooling one carries a vector
    out = llm.generate([IDS, IDS[:4]],
                       [SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True),
                        SamplingParams(max_tokens=8, pooling=True)])
    assert len(out[0].outputs[0].token_ids) == 3 and out[0].embedding is None
    assert len(out[1].outputs[0].token_ids) == 1
    e = torch.nn.functional.normalize(out[1].embedding, dim=-1)
    assert torch.allclose(e, got[1], atol=1e-5)


@pytest.mark.parametrize("rope", [
    {"rope_type": "llama3", "rope_theta": 10000.0, "factor": 8.0, "low_freq_factor": 1.0,
     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    {"rope_type": "yarn", "rope_theta": 10000.0, "factor": 8.0,
     "original_max_position_embeddings": 64},
    {"rope_type": "linear", "rope_theta": 10000.0, "factor": 2.0},
    {"rope_type": "default", "rope_theta": 50000.0}], ids=lambda r: r["rope_type"])
def test_rope_scaling_variants_match_transformers(rope):
    """Llama-3.1 frequency scaling, YaRN, linear scaling and a plain base, on a prompt longer
    than the original context."""
    cfg = tr.LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=128,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         max_position_embeddings=512, rms_norm_eps=1e-6,
                         tie_word_embeddings=False, rope_parameters=rope)
    torch.manual_seed(0)
    hf = tr.LlamaForCausalLM(cfg).eval().float()
    d = cfg.to_dict()
    d["architectures"] = ["LlamaForCausalLM"]
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    llm = LLM(mc, device="cpu", max_num_seqs=2, max_num_batched_tokens=512, max_model_len=512,
              num_gpu_blocks=64, load_format="none")
    llm.engine.model.load_weights(hf.state_dict().items())
    ids = torch.randint(0, 320, (200,), generator=torch.Generator().manual_seed(1)).tolist()
    llm.engine.runner.keep_logits = True
    llm.generate([ids], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
    got = llm.engine.runner.last_logits[0]
    with torch.inference_mode():
        want = hf(input_ids=torch.tensor([ids])).logits[0, -1]
    assert torch.allclose(got, want, atol=1e-4), (got - want).abs().max()


@pytest.mark.parametrize("kind", ["qwen2_mixed", "qwen2_off", "mistral"])
def test_sliding_window_layers_follow_the_checkpoint_config(kind):
    """Qwen2 checkpoints switch the window on per layer (``use_sliding_window`` with
    ``max_window_layers``) or carry a value that is not in force; Mistral windows every layer.
    Logits of a prompt longer than the window against transformers."""
    common = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=3,
                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                  rms_norm_eps=1e-6, tie_word_embeddings=False)
    torch.manual_seed(0)
    if kind == "mistral":
        cfg = tr.MistralConfig(sliding_window=16, **common)
        hf, arch, want_windows = tr.MistralForCausalLM(cfg), "MistralForCausalLM", [16, 16, 16]
        d = cfg.to_dict()
    else:
        on = kind == "qwen2_mixed"
        cfg = tr.Qwen2Config(use_sliding_window=on, sliding_window=16, max_window_layers=1,
                             **common)
        hf, arch = tr.Qwen2ForCausalLM(cfg), "Qwen2ForCausalLM"
        want_windows = [0, 16, 16] if on else [0, 0, 0]
        d = cfg.to_dict()
        if not on:      # as such checkpoints are on disk: the value is there, the switch is off
            d.update(sliding_window=16, use_sliding_window=False)
            d.pop("layer_types", None)
    hf = hf.eval().float()
    d["architectures"] = [arch]
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    assert [mc.window_for_layer(i) for i in range(3)] == want_windows
    llm = LLM(mc, device="cpu", max_num_seqs=2, max_num_batched_tokens=32, max_model_len=256,
              num_gpu_blocks=64, load_format="none")
    llm.engine.model.load_weights(hf.state_dict().items())
    ids = torch.randint(0, 320, (70,), generator=torch.Generator().manual_seed(1)).tolist()
    llm.engine.runner.keep_logits = True
    out = llm.generate([ids], SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True))[0]
    with torch.inference_mode():
        t = torch.tensor([ids])
        want = hf.generate(t, attention_mask=torch.ones_like(t), max_new_tokens=3,
                           do_sample=False, pad_token_id=0)[0, len(ids):].tolist()
    assert out.outputs[0].token_ids == want


def _random_norms_and_biases(hf):
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.copy_(torch.randn_like(p) * 0.2 + 1.0)
            elif n.endswith("bias"):
                p.copy_(torch.randn_like(p) * 0.2)
    return hf.eval().float()


@pytest.mark.parametrize("kind", ["qwen3", "qwen2", "glm4", "mistral", "llama_biases",
                                  "llama_gelu_mha"])
def test_families_with_their_own_config_classes(kind):
    """Each family built from its HuggingFace config class with non-default options: explicit
    head sizes, tied embeddings, biases on q / k / v only (Qwen2, GLM-4) or on all four
    attention projections and the MLP (Llama ``attention_bias`` / ``mlp_bias``), GELU."""
    common = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                  rms_norm_eps=1e-6)
    torch.manual_seed(0)
    if kind == "qwen3":
        c, cls, arch = tr.Qwen3Config(**common, head_dim=32, tie_word_embeddings=True), \
            tr.Qwen3ForCausalLM, "Qwen3ForCausalLM"
    elif kind == "qwen2":
        c, cls, arch = tr.Qwen2Config(**common, tie_word_embeddings=False), \
            tr.Qwen2ForCausalLM, "Qwen2ForCausalLM"
    elif kind == "glm4":
        c, cls, arch = tr.Glm4Config(**common, head_dim=16, tie_word_embeddings=False,
                                     attention_bias=True, pad_token_id=0), \
            tr.Glm4ForCausalLM, "Glm4ForCausalLM"
    elif kind == "mistral":
        c, cls, arch = tr.MistralConfig(**common, head_dim=32, tie_word_embeddings=False,
                                        sliding_window=None), \
            tr.MistralForCausalLM, "MistralForCausalLM"
    elif kind == "llama_biases":
        c, cls, arch = tr.LlamaConfig(**common, tie_word_embeddings=False, attention_bias=True,
                                      mlp_bias=True), tr.LlamaForCausalLM, "LlamaForCausalLM"
    else:
        c, cls, arch = tr.LlamaConfig(**{**common, "num_key_value_heads": 4},
                                      tie_word_embeddings=False, hidden_act="gelu"), \
            tr.LlamaForCausalLM, "LlamaForCausalLM"
    hf = _random_norms_and_biases(cls(c))
    got, tok = _engine_logits(arch, c.to_dict(), hf.state_dict().items())
    want = _hf_last_logits(hf)
    assert torch.allclose(got, want, atol=2e-5), (got - want).abs().max()
    assert tok == int(want.argmax())
