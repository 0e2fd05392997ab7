"""Checkpoint loading: HF-named safetensors -> stacked / sharded parameters."""
import json
import os

import pytest
import torch

from vllm_gcu_b200.config import ModelConfig, preset
from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams
from vllm_gcu_b200.models import build_model
from vllm_gcu_b200.utils.weights import iter_safetensors, write_safetensors


def _hf_state_dict(model):
    """Exports a DecoderLM's parameters under HuggingFace names (un-stacking qkv / gate_up)."""
    cfg = model.cfg
    D, Hq, Hkv, I = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, \
        cfg.intermediate_size
    out = {}
    for name, p in model.state_dict().items():
        if name.startswith(("layers.", "embed_tokens.", "norm.")):
            name = "model." + name
        if ".qkv_proj.weight" in name:
            q, k, v = p.split([Hq * D, Hkv * D, Hkv * D], 0)
            for n, t in (("q_proj", q), ("k_proj", k), ("v_proj", v)):
                out[name.replace("qkv_proj", n)] = t.clone()
        elif ".gate_up_proj.weight" in name:
            g, u = p.split([I, I], 0)
            out[name.replace("gate_up_proj", "gate_proj")] = g.clone()
            out[name.replace("gate_up_proj", "up_proj")] = u.clone()
        else:
            out[name] = p.clone()
    return out


def test_safetensors_roundtrip_and_engine_load(tmp_path):
    cfg = preset("tiny-llama")
    src = build_model(cfg, "cpu")
    src.init_random(0)
    sd = _hf_state_dict(src)
    items = list(sd.items())
    half = len(items) // 2
    write_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), dict(items[:half]))
    write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), dict(items[half:]))
    wm = {k: "model-00001-of-00002.safetensors" for k, _ in items[:half]}
    wm.update({k: "model-00002-of-00002.safetensors" for k, _ in items[half:]})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    hf_cfg = {"architectures": ["LlamaForCausalLM"], "vocab_size": cfg.vocab_size,
              "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
              "num_hidden_layers": cfg.num_hidden_layers,
              "num_attention_heads": cfg.num_attention_heads,
              "num_key_value_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
              "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope_theta,
              "max_position_embeddings": cfg.max_position_embeddings, "torch_dtype": "float32"}
    (tmp_path / "config.json").write_text(json.dumps(hf_cfg))
    back = dict(iter_safetensors(str(tmp_path)))
    assert set(back) == set(sd) and all(torch.equal(back[k], sd[k]) for k in sd)
    llm = LLM(str(tmp_path), device="cpu", max_num_seqs=4, max_num_batched_tokens=64,
              max_model_len=128, num_gpu_blocks=32)
    got = llm.engine.model.state_dict()
    want = src.state_dict()
    assert all(torch.equal(got[k], want[k]) for k in want)
    outs = llm.generate([[1, 2, 3, 4, 5]], SamplingParams(max_tokens=4))
    assert len(outs[0].outputs[0].token_ids) == 4


def test_kv_cache_scales_from_checkpoint_and_parameter_file(tmp_path):
    """Scales of an 8-bit KV cache: ``k_scale`` / ``v_scale`` / ``kv_scale`` tensors of a
    checkpoint, and the quantisation-parameter file (scaling_factor[tp_rank][layer]) in its
    three value forms."""
    cfg = preset("tiny-llama")
    model = build_model(cfg, "cpu")
    model.init_random(0)
    loaded = model.load_weights([("model.layers.0.self_attn.k_scale", torch.tensor(0.03)),
                                 ("model.layers.0.self_attn.v_scale", torch.tensor([0.05])),
                                 ("model.layers.1.self_attn.attn.kv_scale", torch.tensor(0.07))])
    assert len(loaded) == 3
    a0, a1 = model.layers["0"].self_attn.attn, model.layers["1"].self_attn.attn
    assert (a0.k_scale, a0.v_scale) == (pytest.approx(0.03), pytest.approx(0.05))
    assert (a1.k_scale, a1.v_scale) == (pytest.approx(0.07), pytest.approx(0.07))
    path = tmp_path / "int8_kv_cache.json"
    path.write_text(json.dumps({"model_type": "llama", "kv_cache": {
        "dtype": "int8", "scaling_factor": {"0": {"0": 0.011, "1": [0.02, 0.04]},
                                            "1": {"0": 9.0, "1": 9.0}}}}))
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=2, max_num_batched_tokens=32,
              max_model_len=64, num_gpu_blocks=16, quantization_param_path=str(path))
    l0 = llm.engine.model.layers["0"].self_attn.attn
    l1 = llm.engine.model.layers["1"].self_attn.attn
    assert (l0.k_scale, l0.v_scale) == (pytest.approx(0.011), pytest.approx(0.011))
    assert (l1.k_scale, l1.v_scale) == (pytest.approx(0.02), pytest.approx(0.04))
    path.write_text(json.dumps({"kv_cache": {"scaling_factor": {"0": {
        "1": {"k_scale": 0.5, "v_scale": 0.25}}}}}))
    assert llm.engine.model.load_kv_cache_scales(str(path)) == 1
    assert (l1.k_scale, l1.v_scale) == (0.5, 0.25)


def test_sharded_safetensors_and_pickled_checkpoints_load(tmp_path):
    """Checkpoint directories in the layouts found in the wild: several safetensors shards with
    an index and tied embeddings, and a pickled ``pytorch_model.bin``."""
    import pytest
    tr = pytest.importorskip("transformers")
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    hc = tr.LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=128,
                        num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                        max_position_embeddings=128, rms_norm_eps=1e-6, tie_word_embeddings=True)
    torch.manual_seed(0)
    hf = tr.LlamaForCausalLM(hc).eval().float()
    ids = [5, 17, 99, 3, 250, 42, 7]
    want = hf.generate(torch.tensor([ids]), attention_mask=torch.ones(1, len(ids), dtype=torch.long),
                       max_new_tokens=5, do_sample=False, pad_token_id=0)[0, len(ids):].tolist()
    a, b = tmp_path / "shards", tmp_path / "pickled"
    hf.save_pretrained(str(a), safe_serialization=True, max_shard_size="100KB")
    assert (a / "model.safetensors.index.json").exists()
    b.mkdir()
    (b / "config.json").write_text((a / "config.json").read_text())
    torch.save(hf.state_dict(), str(b / "pytorch_model.bin"))
    for d in (a, b):
        llm = LLM(str(d), device="cpu", max_num_seqs=4, max_num_batched_tokens=64,
                  max_model_len=128, num_gpu_blocks=64, dtype="float32")
        got = llm.generate([ids], SamplingParams(max_tokens=5, temperature=0.0,
                                                 ignore_eos=True))[0].outputs[0].token_ids
        assert got == want
