"""GOT-OCR-2.0 against the HuggingFace implementation (tiny random model, CPU)."""
import pytest
import torch

tr = pytest.importorskip("transformers")


def test_image_tokens_and_logits_match_transformers():
    from transformers import GotOcr2Config, GotOcr2ForConditionalGeneration
    from vllm_gcu_b200.config import ModelConfig
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    cfg = GotOcr2Config(
        text_config=dict(model_type="qwen2", vocab_size=200, hidden_size=64,
                         intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=256,
                         tie_word_embeddings=False),
        vision_config=dict(hidden_size=32, output_channels=16, num_hidden_layers=3,
                           num_attention_heads=2, image_size=128, patch_size=16, window_size=3,
                           global_attn_indexes=[1], mlp_dim=64),
        image_token_index=190, image_seq_length=4)
    torch.manual_seed(0)
    hf = GotOcr2ForConditionalGeneration(cfg).eval().float()
    for n, p in hf.named_parameters():          # rel-pos tables and pos_embed start at zero
        if "rel_pos" in n or "pos_embed" in n:
            torch.nn.init.normal_(p, std=0.05)
    d = cfg.to_dict()
    d["architectures"] = ["GotOcr2ForConditionalGeneration"]
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    llm = LLM(mc, device="cpu", max_num_seqs=4, max_num_batched_tokens=8, max_model_len=128,
              num_gpu_blocks=64, load_format="none")
    model = llm.engine.model
    loaded = model.load_weights(hf.state_dict().items())
    assert any("vision_tower" in n for n in loaded) and any("projector" in n for n in loaded)
    pixels = torch.randn(1, 3, 128, 128)
    with torch.inference_mode():
        want_img = hf.model.get_image_features(pixels)
        want_img = want_img.pooler_output if hasattr(want_img, "pooler_output") else want_img
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
