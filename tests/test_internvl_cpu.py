"""InternVL2 / 2.5 against the HuggingFace implementation (tiny random model, CPU): tile
features (InternViT, neighbourhood folding, projector) in both checkpoint layouts and the logits
of a prompt with an image, served through the engine."""
import pytest
import torch

tr = pytest.importorskip("transformers")


def _hf_model(norm_type="layer_norm", qk_norm=False):
    from transformers import InternVLConfig, InternVLForConditionalGeneration
    cfg = InternVLConfig(
        text_config=dict(model_type="qwen2", vocab_size=200, hidden_size=64,
                         intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=256,
                         tie_word_embeddings=False, rms_norm_eps=1e-6),
        vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=3,
                           num_attention_heads=2, image_size=[28, 28], patch_size=[7, 7],
                           norm_type=norm_type, use_qk_norm=qk_norm, attention_bias=True,
                           layer_scale_init_value=0.1, hidden_act="gelu", layer_norm_eps=1e-6,
                           use_absolute_position_embeddings=True, use_mean_pooling=True),
        image_token_id=190, downsample_ratio=0.5, vision_feature_layer=-1,
        vision_feature_select_strategy="default", image_seq_length=4)
    torch.manual_seed(0)
    hf = InternVLForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "vision_tower" in n and ("lambda_" in n or "cls_token" in n
                                        or "position_embeddings" in n or "norm.weight" in n):
                p.copy_(torch.randn_like(p) * 0.3 + (1.0 if "norm" in n else 0.0))
    return cfg, hf


def _build(cfg_dict, arch):
    from vllm_gcu_b200.config import ModelConfig
    from vllm_gcu_b200.engine.llm import LLM
    d = dict(cfg_dict)
    d["architectures"] = [arch]
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    return LLM(mc, device="cpu", max_num_seqs=4, max_num_batched_tokens=16, max_model_len=128,
               num_gpu_blocks=64, load_format="none")


def _hf_features(hf, pixels):
    with torch.inference_mode():
        out = hf.model.get_image_features(pixels, vision_feature_layer=-1,
                                          vision_feature_select_strategy="default")
    out = out.pooler_output if hasattr(out, "pooler_output") else out
    return out.reshape(-1, out.shape[-1])


@pytest.mark.parametrize("norm_type,qk_norm", [("layer_norm", False), ("rms_norm", True)])
def test_features_and_logits_match_transformers(norm_type, qk_norm):
    from vllm_gcu_b200.engine.request import SamplingParams
    cfg, hf = _hf_model(norm_type, qk_norm)
    llm = _build(cfg.to_dict(), "InternVLForConditionalGeneration")
    model = llm.engine.model
    assert type(model).__mro__[2].__name__ == "Qwen2ForCausalLM"
    loaded = model.load_weights(hf.state_dict().items())
    missing = [n for n in hf.state_dict() if n not in loaded]
    assert not missing, missing
    assert model.tokens_per_tile == 4
    pixels = torch.randn(2, 3, 28, 28)
    want_img = _hf_features(hf, pixels)
    got_img = model.encode_images(pixels)
    assert got_img.shape == (8, 64)
    assert torch.allclose(got_img, want_img, atol=2e-4), (got_img - want_img).abs().max()
    ids = [3, 4] + [190] * 8 + [5, 6, 7, 8, 9]
    with torch.inference_mode():
        want = hf(input_ids=torch.tensor([ids]), pixel_values=pixels).logits[0, -1]
    llm.engine.runner.keep_logits = True
    llm.generate([{"prompt_token_ids": ids, "multi_modal_data": {"pixel_values": pixels}}],
                 SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
    got = llm.engine.runner.last_logits[0]
    assert torch.allclose(got, want, atol=2e-3), (got - want).abs().max()


def test_original_checkpoint_layout_loads_to_the_same_features():
    """``InternVLChatModel`` checkpoints: fused ``attn.qkv``, ``ls1`` / ``ls2``, ``mlp1.{0,1,3}``,
    the language model below ``language_model.`` and its class named by ``llm_config``."""
    cfg, hf = _hf_model()
    sd = hf.state_dict()
    orig = {}
    ren = {"layernorm_before": "norm1", "layernorm_after": "norm2", "lambda_1": "ls1",
           "lambda_2": "ls2", "attention.projection_layer": "attn.proj"}
    for n, t in sd.items():
        if n.startswith("model.vision_tower.encoder.layer."):
            rest = n[len("model.vision_tower.encoder.layer."):]
            idx, _, rest = rest.partition(".")
            if rest.startswith(("attention.q_proj", "attention.k_proj", "attention.v_proj")):
                continue
            for a, b in ren.items():
                rest = rest.replace(a, b)
            orig[f"vision_model.encoder.layers.{idx}.{rest}"] = t
        elif n.startswith("model.vision_tower.embeddings."):
            rest = n[len("model.vision_tower.embeddings."):]
            rest = {"cls_token": "class_embedding", "position_embeddings": "position_embedding",
                    "patch_embeddings.projection.weight": "patch_embedding.weight",
                    "patch_embeddings.projection.bias": "patch_embedding.bias"}[rest]
            orig["vision_model.embeddings." + rest] = t
        elif n.startswith("model.multi_modal_projector."):
            rest = n[len("model.multi_modal_projector."):]
            for a, b in (("layer_norm", "0"), ("linear_1", "1"), ("linear_2", "3")):
                rest = rest.replace(a, b)
            orig["mlp1." + rest] = t
        elif n.startswith("model.language_model."):
            orig["language_model.model." + n[len("model.language_model."):]] = t
        elif n == "lm_head.weight":
            orig["language_model.lm_head.weight"] = t
    for i in range(3):
        pre = f"model.vision_tower.encoder.layer.{i}.attention."
        for kind in ("weight", "bias"):
            orig[f"vision_model.encoder.layers.{i}.attn.qkv.{kind}"] = torch.cat(
                [sd[pre + f"{p}_proj.{kind}"] for p in "qkv"], dim=0)
    d = cfg.to_dict()
    vc = d["vision_config"]
    cfg_orig = {"llm_config": {**d["text_config"], "architectures": ["Qwen2ForCausalLM"]},
                "vision_config": {"hidden_size": 32, "intermediate_size": 64,
                                  "num_hidden_layers": 3, "num_attention_heads": 2,
                                  "image_size": 28, "patch_size": 7, "norm_type": "layer_norm",
                                  "qkv_bias": True, "qk_normalization": False,
                                  "layer_norm_eps": vc["layer_norm_eps"], "hidden_act": "gelu"},
                "downsample_ratio": 0.5, "select_layer": -1, "ps_version": "v2",
                "img_context_token_id": 190}
    llm = _build(cfg_orig, "InternVLChatModel")
    model = llm.engine.model
    loaded = model.load_weights(orig.items())
    assert set(orig) == loaded
    pixels = torch.randn(2, 3, 28, 28)
    got = model.encode_images(pixels)
    want = _hf_features(hf, pixels)
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()


def test_tile_grid_and_dynamic_tiles():
    from vllm_gcu_b200.models.internvl import dynamic_tiles, fold_neighbourhoods, tile_grid
    assert tile_grid(448, 448, 1, 12) == (1, 1)
    assert tile_grid(1344, 448, 1, 12) == (3, 1)
    assert tile_grid(448, 896, 1, 12) == (1, 2)
    assert tile_grid(2000, 2000, 1, 12) == (3, 3)      # equal distance: the larger grid wins
    t = dynamic_tiles(torch.rand(3, 100, 290), tile=28, max_tiles=6)
    assert t.shape == (4, 3, 28, 28)                   # 3 x 1 grid + thumbnail
    assert dynamic_tiles(torch.rand(3, 50, 50), tile=28, max_tiles=1).shape[0] == 1
    x = torch.arange(16.0).reshape(1, 4, 4, 1)
    y = fold_neighbourhoods(x, 2)
    assert y.shape == (1, 2, 2, 4) and y[0, 0, 1].tolist() == [2.0, 3.0, 6.0, 7.0]
    assert fold_neighbourhoods(x, 2, transposed=False)[0, 1, 0].tolist() == [2.0, 3.0, 6.0, 7.0]
