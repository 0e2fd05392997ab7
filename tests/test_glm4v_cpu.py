"""GLM-4.1V against the HuggingFace implementation (tiny random model, CPU): the vision tower
(interpolated position table, 2-D rotary attention, strided-convolution merge, merger) and the
logits of a prompt that contains an image, served through the engine."""
import pytest
import torch

tr = pytest.importorskip("transformers")


def test_vision_tower_and_logits_match_transformers():
    from transformers import Glm4vConfig, Glm4vForConditionalGeneration
    from vllm_gcu_b200.config import ModelConfig
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    from vllm_gcu_b200.models.qwen2_5_vl import get_rope_index
    text = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512,
                rms_norm_eps=1e-6, tie_word_embeddings=False, attention_bias=True,
                rope_parameters={"rope_type": "default", "rope_theta": 10000.0,
                                 "mrope_section": [2, 1, 1], "partial_rotary_factor": 0.5})
    vision = dict(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, in_channels=3,
                  image_size=56, patch_size=14, spatial_merge_size=2, temporal_patch_size=2,
                  out_hidden_size=64, rms_norm_eps=1e-5, attention_bias=True, hidden_act="silu")
    cfg = Glm4vConfig(text_config=text, vision_config=vision, image_token_id=290,
                      video_token_id=291, image_start_token_id=288, image_end_token_id=289)
    torch.manual_seed(0)
    hf = Glm4vForConditionalGeneration(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "visual" in n and ("norm" in n or "position_embedding" in n or n.endswith("bias")):
                p.copy_(torch.randn_like(p) * 0.3 + (1.0 if "norm.weight" in n or
                                                     "norm1" in n or "norm2" in n else 0.0))
    d = cfg.to_dict()
    d["architectures"] = ["Glm4vForConditionalGeneration"]
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    assert mc.sandwich_norm and not mc.rope_is_neox and mc.partial_rotary_factor == 0.5
    llm = LLM(mc, device="cpu", max_num_seqs=4, max_num_batched_tokens=16, max_model_len=256,
              num_gpu_blocks=64, load_format="none")
    model = llm.engine.model
    loaded = model.load_weights(hf.state_dict().items())
    missing = [n for n in hf.state_dict() if n not in loaded]
    assert not missing, missing
    # a 6 x 4 patch grid: not the square grid of the position table, so it is interpolated
    grid = torch.tensor([[1, 6, 4]])
    pixels = torch.randn(24, 3 * 2 * 14 * 14, generator=torch.Generator().manual_seed(1))
    with torch.inference_mode():
        want_v = hf.model.visual(pixels, grid_thw=grid)
        want_v = want_v.pooler_output if hasattr(want_v, "pooler_output") else want_v
    got_v = model.encode_images(pixels, grid)
    assert got_v.shape == (6, 64)
    assert torch.allclose(got_v, want_v, atol=3e-4), (got_v - want_v).abs().max()
    ids = [5, 6, 288] + [290] * 6 + [289, 7, 8, 9, 10]
    mpos, delta = get_rope_index(ids, [(1, 6, 4)], 290, 2)
    import inspect
    kw = {}
    if "mm_token_type_ids" in inspect.signature(hf.forward).parameters:
        kw["mm_token_type_ids"] = torch.tensor([[1 if t == 290 else 0 for t in ids]],
                                               dtype=torch.int32)
    with torch.inference_mode():
        want = hf(input_ids=torch.tensor([ids]), pixel_values=pixels, image_grid_thw=grid,
                  position_ids=mpos[:, None, :], **kw).logits[0, -1]
    llm.engine.runner.keep_logits = True
    out = llm.generate([{"prompt_token_ids": ids,
                         "multi_modal_data": {"pixel_values": pixels, "image_grid_thw": grid}}],
                       SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True))
    assert len(out[0].outputs[0].token_ids) == 3
    llm2 = LLM(mc, device="cpu", max_num_seqs=4, max_num_batched_tokens=16, max_model_len=256,
               num_gpu_blocks=64, load_format="none")
    llm2.engine.model.load_weights(hf.state_dict().items())
    llm2.engine.runner.keep_logits = True
    llm2.generate([{"prompt_token_ids": ids,
                    "multi_modal_data": {"pixel_values": pixels, "image_grid_thw": grid}}],
                  SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
    got = llm2.engine.runner.last_logits[0]
    assert torch.allclose(got, want, atol=2e-3), (got - want).abs().max()
