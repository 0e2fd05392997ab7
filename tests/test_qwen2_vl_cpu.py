"""Qwen2-VL against the HuggingFace implementation (tiny random model, CPU): the vision tower
(LayerNorm blocks, quick-GELU MLP, full attention per frame) and the logits of a prompt that
contains an image, served through the engine."""
import pytest
import torch

tr = pytest.importorskip("transformers")


def test_vision_tower_and_logits_match_transformers():
    from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration
    from vllm_gcu_b200.config import ModelConfig
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    from vllm_gcu_b200.models.qwen2_5_vl import get_rope_index
    text = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512,
                rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]})
    vision = dict(depth=2, embed_dim=32, hidden_size=64, mlp_ratio=2, num_heads=2,
                  in_channels=3, patch_size=14, spatial_merge_size=2, temporal_patch_size=2)
    cfg = Qwen2VLConfig(text_config=text, vision_config=vision, image_token_id=290,
                        video_token_id=291, vision_start_token_id=288, vision_end_token_id=289)
    torch.manual_seed(0)
    hf = Qwen2VLForConditionalGeneration(cfg).eval().float()
    d = cfg.to_dict()
    d["architectures"] = ["Qwen2VLForConditionalGeneration"]
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    llm = LLM(mc, device="cpu", max_num_seqs=4, max_num_batched_tokens=16, max_model_len=256,
              num_gpu_blocks=64, load_format="none")
    model = llm.engine.model
    assert type(model).__name__ == "Qwen2VLForConditionalGeneration"
    loaded = model.load_weights(hf.state_dict().items())
    assert any("visual" in n for n in loaded)
    grid = torch.tensor([[1, 6, 4]])
    pixels = torch.randn(24, 3 * 2 * 14 * 14, generator=torch.Generator().manual_seed(1))
    with torch.inference_mode():
        want_v = hf.model.visual(pixels, grid_thw=grid)
        want_v = want_v.pooler_output if hasattr(want_v, "pooler_output") else want_v
    got_v = model.encode_images(pixels, grid)
    assert got_v.shape == (6, 64)
    assert torch.allclose(got_v, want_v, atol=2e-4), (got_v - want_v).abs().max()
    ids = [5, 6, 288] + [290] * 6 + [289, 7, 8, 9, 10]
    mpos, delta = get_rope_index(ids, [(1, 6, 4)], 290, 2, second_per_grid=[1.0],
                                 tokens_per_second=1.0)
    types = torch.tensor([[1 if t == 290 else 0 for t in ids]], dtype=torch.int32)

    def hf_logits(seq):
        n_new = len(seq) - len(ids)
        tail = torch.arange(n_new)[None, :].expand(3, n_new) + len(ids) + delta
        pos = torch.cat([mpos, tail], dim=1)[:, None, :]
        kw = {}
        import inspect
        if "mm_token_type_ids" in inspect.signature(hf.forward).parameters:
            kw["mm_token_type_ids"] = torch.cat(
                [types, torch.zeros(1, n_new, dtype=torch.int32)], dim=1)
        with torch.inference_mode():
            return hf(input_ids=torch.tensor([seq]), pixel_values=pixels, image_grid_thw=grid,
                      position_ids=pos, **kw).logits[0, -1]

    llm.engine.runner.keep_logits = True
    res = llm.generate([{"prompt_token_ids": ids,
                         "multi_modal_data": {"pixel_values": pixels, "image_grid_thw": grid}}],
                       SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True))
    toks = res[0].outputs[0].token_ids
    seq = list(ids)
    for t in toks:
        want = hf_logits(seq)
        assert int(want.argmax()) == t, (int(want.argmax()), t)
        seq.append(t)
    got = llm.engine.runner.last_logits[0]
    want = hf_logits(list(ids) + toks[:2])
    assert torch.allclose(got, want, atol=2e-3), (got - want).abs().max()
