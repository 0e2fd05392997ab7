"""LLaVA-1.5 against the HuggingFace implementation (tiny random model, CPU): image features
(CLIP tower up to the second-to-last layer, class token dropped, projector) and the logits of
a prompt that contains an image, served through the engine."""
import pytest
import torch

tr = pytest.importorskip("transformers")


def test_image_features_and_logits_match_transformers():
    from transformers import LlavaConfig, LlavaForConditionalGeneration
    from vllm_gcu_b200.config import ModelConfig
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    cfg = LlavaConfig(
        text_config=dict(model_type="llama", vocab_size=200, hidden_size=64,
                         intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=256,
                         tie_word_embeddings=False, rms_norm_eps=1e-6),
        vision_config=dict(model_type="clip_vision_model", hidden_size=32, intermediate_size=64,
                           num_hidden_layers=3, num_attention_heads=2, image_size=28,
                           patch_size=14, hidden_act="quick_gelu", projection_dim=16),
        image_token_index=190, vision_feature_layer=-2, vision_feature_select_strategy="default",
        image_seq_length=4)
    torch.manual_seed(0)
    hf = LlavaForConditionalGeneration(cfg).eval().float()
    d = cfg.to_dict()
    d["architectures"] = ["LlavaForConditionalGeneration"]
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    llm = LLM(mc, device="cpu", max_num_seqs=4, max_num_batched_tokens=8, max_model_len=128,
              num_gpu_blocks=64, load_format="none")
    model = llm.engine.model
    loaded = model.load_weights(hf.state_dict().items())
    assert any("vision_tower" in n for n in loaded) and any("projector" in n for n in loaded)
    assert model.tokens_per_image == 4 and len(model.vision_tower.layers) == 2
    pixels = torch.randn(1, 3, 28, 28)
    with torch.inference_mode():
        want_img = hf.model.get_image_features(pixels)
        want_img = want_img.pooler_output if hasattr(want_img, "pooler_output") else want_img
        if isinstance(want_img, (list, tuple)):
            want_img = torch.cat(list(want_img), dim=0)
    got_img = model.encode_images(pixels)
    assert got_img.shape == (4, 64)
    assert torch.allclose(got_img, want_img.reshape(4, 64), atol=2e-4), \
        (got_img - want_img.reshape(4, 64)).abs().max()
    ids = [3, 4] + [190] * 4 + [5, 6, 7, 8, 9]
    with torch.inference_mode():
        want = hf(input_ids=torch.tensor([ids]), pixel_values=pixels).logits[0, -1]
    llm.engine.runner.keep_logits = True
    llm.generate([{"prompt_token_ids": ids,
                   "multi_modal_data": {"pixel_values": pixels, "image_grid_thw": None}}],
                 SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
    got = llm.engine.runner.last_logits[0]
    assert torch.allclose(got, want, atol=2e-3), (got - want).abs().max()


@pytest.mark.parametrize("size", [(40, 56), (56, 30), (28, 28)])
def test_llava_next_any_resolution_matches_transformers(size):
    """LLaVA-NeXT: base view + tile grid, padding rows cut, ``image_newline`` per row; the
    packed image rows and the logits of the served prompt against transformers."""
    from transformers import LlavaNextConfig, LlavaNextForConditionalGeneration
    from vllm_gcu_b200.config import ModelConfig
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    from vllm_gcu_b200.models.llava import anyres_grid
    pin = [[28, 56], [56, 28], [56, 56]]
    cfg = LlavaNextConfig(
        text_config=dict(model_type="llama", vocab_size=200, hidden_size=64,
                         intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=256,
                         tie_word_embeddings=False, rms_norm_eps=1e-6),
        vision_config=dict(model_type="clip_vision_model", hidden_size=32, intermediate_size=64,
                           num_hidden_layers=3, num_attention_heads=2, image_size=28,
                           patch_size=7, hidden_act="quick_gelu", projection_dim=16),
        image_token_index=190, vision_feature_layer=-2, vision_feature_select_strategy="default",
        image_grid_pinpoints=pin, image_seq_length=16)
    torch.manual_seed(0)
    hf = LlavaNextForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        hf.model.image_newline.copy_(torch.randn(64) * 0.5)
    d = cfg.to_dict()
    d["architectures"] = ["LlavaNextForConditionalGeneration"]
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    llm = LLM(mc, device="cpu", max_num_seqs=4, max_num_batched_tokens=32, max_model_len=256,
              num_gpu_blocks=64, load_format="none")
    model = llm.engine.model
    loaded = model.load_weights(hf.state_dict().items())
    assert "model.image_newline" in loaded
    gh, gw = anyres_grid(size, pin, 28)
    views = 1 + gh * gw
    torch.manual_seed(1)
    pixels = torch.randn(views, 3, 28, 28)
    sizes = torch.tensor([list(size)])
    n_tok = model.num_image_tokens(size, views)
    ids = [3, 4] + [190] * n_tok + [5, 6, 7]
    with torch.inference_mode():
        want = hf(input_ids=torch.tensor([ids]), pixel_values=pixels[None],
                  image_sizes=sizes).logits[0, -1]
    got_img = model.encode_images(pixels, sizes)
    assert got_img.shape == (n_tok, 64)
    llm.engine.runner.keep_logits = True
    llm.generate([{"prompt_token_ids": ids,
                   "multi_modal_data": {"pixel_values": pixels, "image_sizes": sizes}}],
                 SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
    got = llm.engine.runner.last_logits[0]
    assert torch.allclose(got, want, atol=2e-3), (got - want).abs().max()
