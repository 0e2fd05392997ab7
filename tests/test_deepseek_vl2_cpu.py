"""DeepSeek-VL2 on CPU (tiny random model): the SigLIP tower against the HuggingFace
implementation of the same encoder, the down-sampling projector against an unfold formulation,
the tile layout against explicit loops, and the merge of image rows into the prompt against a
text-only engine whose embedding table carries the image rows as extra tokens."""
import pytest
import torch
import torch.nn.functional as F

tr = pytest.importorskip("transformers")

from vllm_gcu_b200.config import ModelConfig  # noqa: E402
from vllm_gcu_b200.engine.llm import LLM  # noqa: E402
from vllm_gcu_b200.engine.request import SamplingParams  # noqa: E402
from vllm_gcu_b200.models import deepseek_vl2 as M  # noqa: E402

IMG = 9999          # placeholder id outside the text vocabulary range used below


def _hf_config(mla: bool):
    lang = dict(vocab_size=320, hidden_size=64, intermediate_size=96, moe_intermediate_size=32,
                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
                n_routed_experts=4, num_experts_per_tok=2, n_shared_experts=1,
                first_k_dense_replace=1, max_position_embeddings=512, rms_norm_eps=1e-6,
                norm_topk_prob=False, tie_word_embeddings=False)
    if mla:
        lang.update(kv_lora_rank=16, q_lora_rank=0, qk_nope_head_dim=16, qk_rope_head_dim=8,
                    v_head_dim=16)
    return {"architectures": ["DeepseekVLV2ForCausalLM"], "tile_tag": "2D",
            "global_view_pos": "head", "image_token_id": 300,
            "vision_config": dict(image_size=56, patch_size=14, width=32, layers=2, heads=2,
                                  mlp_ratio=2.0),
            "projector_config": dict(projector_type="downsample_mlp_gelu", input_dim=32,
                                     n_embed=64, depth=2, mlp_ratio=1, downsample_ratio=2),
            "language_config": lang}


def test_siglip_tower_matches_transformers():
    c = M.SiglipConfig(image_size=56, patch_size=14, width=32, layers=2, heads=2, mlp_ratio=2.0)
    hc = tr.SiglipVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                               num_attention_heads=2, image_size=56, patch_size=14,
                               hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6)
    torch.manual_seed(0)
    hf = tr.SiglipVisionModel(hc).eval().float()
    ours = M.SiglipVisionTransformer(c, torch.float32, "cpu")
    sd = hf.state_dict()
    pre = "vision_model."
    own = dict(ours.named_parameters())
    own["patch_embed.proj.weight"].data.copy_(sd[pre + "embeddings.patch_embedding.weight"])
    own["patch_embed.proj.bias"].data.copy_(sd[pre + "embeddings.patch_embedding.bias"])
    own["pos_embed"].data.copy_(sd[pre + "embeddings.position_embedding.weight"][None])
    own["norm.weight"].data.copy_(sd[pre + "post_layernorm.weight"])
    own["norm.bias"].data.copy_(sd[pre + "post_layernorm.bias"])
    for i in range(2):
        p = f"{pre}encoder.layers.{i}."
        for wb in ("weight", "bias"):
            own[f"blocks.{i}.attn.qkv.{wb}"].data.copy_(torch.cat(
                [sd[p + f"self_attn.{n}_proj.{wb}"] for n in "qkv"], 0))
            own[f"blocks.{i}.attn.proj.{wb}"].data.copy_(sd[p + f"self_attn.out_proj.{wb}"])
            own[f"blocks.{i}.norm1.{wb}"].data.copy_(sd[p + f"layer_norm1.{wb}"])
            own[f"blocks.{i}.norm2.{wb}"].data.copy_(sd[p + f"layer_norm2.{wb}"])
            own[f"blocks.{i}.mlp.fc1.{wb}"].data.copy_(sd[p + f"mlp.fc1.{wb}"])
            own[f"blocks.{i}.mlp.fc2.{wb}"].data.copy_(sd[p + f"mlp.fc2.{wb}"])
    x = torch.randn(3, 3, 56, 56)
    with torch.inference_mode():
        want = hf(pixel_values=x).last_hidden_state
        got = ours(x)
    assert got.shape == (3, 16, 32)
    assert torch.allclose(got, want, atol=2e-5), (got - want).abs().max()


def test_projector_and_tile_layout():
    pc = M.ProjectorConfig(input_dim=8, n_embed=12, depth=3, mlp_ratio=2, downsample_ratio=2)
    torch.manual_seed(1)
    proj = M.MlpProjector(pc, torch.float32, "cpu")
    x = torch.randn(2, 9, 8)                        # 3 x 3 grid: padded to 4 x 4
    with torch.inference_mode():
        got = proj(x)
        g = F.pad(x.view(2, 3, 3, 8), (0, 0, 0, 1, 0, 1)).permute(0, 3, 1, 2)
        want = proj.layers(F.unfold(g, kernel_size=2, stride=2).permute(0, 2, 1))
    assert got.shape == (2, 4, 12) and torch.allclose(got, want, atol=1e-6)
    # two images: 2 x 1 local tiles (num_w = 2, num_h = 1) and no local tiles... every image
    # has at least one local tile in practice; (1, 2) covers the other orientation
    h, D = 2, 5
    crops = [(2, 1), (1, 2)]
    feats = torch.randn(sum(1 + a * b for a, b in crops), h * h, D)
    nl, sep = torch.randn(D), torch.randn(D)
    got = M.tile_embeddings(feats, crops, nl, sep, True)
    rows, t = [], 0
    for num_w, num_h in crops:
        for r in range(h):
            rows += [feats[t, r * h + c] for c in range(h)] + [nl]
        rows.append(sep)
        for R in range(num_h * h):
            for Cc in range(num_w * h):
                tile = (R // h) * num_w + (Cc // h)
                rows.append(feats[t + 1 + tile, (R % h) * h + (Cc % h)])
            rows.append(nl)
        t += 1 + num_w * num_h
    want = torch.stack(rows)
    assert got.shape == want.shape and torch.equal(got, want)


@pytest.mark.parametrize("mla", [False, True])
def test_image_rows_merge_like_extra_tokens(mla):
    d = _hf_config(mla)
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    assert mc.is_mla == mla and mc.hidden_size == 64
    kw = dict(device="cpu", max_num_seqs=2, max_num_batched_tokens=16, max_model_len=256,
              num_gpu_blocks=64)
    llm = LLM(mc, **kw, seed=0)
    model = llm.engine.model
    assert type(model).__name__ == "DeepseekVLV2ForCausalLM"
    assert model.vision is not None and model.projector is not None
    crops = [(2, 1)]
    n_img = model.num_image_tokens(crops[0])        # 2*(2+1) + 1 + 2*(4+1) = 17
    assert n_img == 17
    pixels = torch.randn(3, 3, 56, 56)
    with torch.inference_mode():
        emb = model.encode_images(pixels, crops)
    assert emb.shape == (n_img, 64)
    # checkpoint names: language.*, vision.*, projector.*, the two learnt vectors
    sd = {}
    for n, p_ in model.state_dict().items():
        if n.startswith(("vision.", "projector.")) or n in ("image_newline", "view_seperator"):
            sd[n] = p_.clone() + 0.01
    loaded = model.load_weights(list(sd.items()) + [("vision.attn_pool.q.weight", torch.zeros(1))])
    assert set(sd) <= loaded
    with torch.inference_mode():
        emb2 = model.encode_images(pixels, crops)
    assert not torch.allclose(emb, emb2)
    ids = [5, 6] + [300] * n_img + [7, 8, 9, 10]
    llm.engine.runner.keep_logits = True
    out = llm.generate([{"prompt_token_ids": ids,
                         "multi_modal_data": {"pixel_values": pixels,
                                              "images_spatial_crop": crops}}],
                       SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
    got = llm.engine.runner.last_logits[0].clone()
    # text-only twin: same language weights, the image rows appended to the embedding table
    lang = dict(d["language_config"], vocab_size=320 + n_img,
                architectures=["DeepseekV2ForCausalLM" if mla else "DeepseekForCausalLM"])
    twin = LLM(ModelConfig.from_hf_dict(lang, dtype=torch.float32), **kw, seed=0)
    tsd, msd = twin.engine.model.state_dict(), model.state_dict()
    for n, p_ in tsd.items():
        src = msd[n]
        if p_.shape == src.shape:
            p_.copy_(src)
        else:                                        # embedding table / LM head: more rows
            p_.zero_()
            p_[:src.shape[0]].copy_(src)
    tsd["embed_tokens.weight"][320:320 + n_img].copy_(emb2)
    twin.engine.runner.keep_logits = True
    ids2 = [5, 6] + list(range(320, 320 + n_img)) + [7, 8, 9, 10]
    twin.generate([ids2], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
    want = twin.engine.runner.last_logits[0]
    assert torch.allclose(got[:320], want[:320], atol=1e-4), (got[:320] - want[:320]).abs().max()
    assert out[0].outputs[0].token_ids[0] == int(got.argmax())


def test_image_tiling_and_placeholder_expansion():
    """The processor side: best candidate resolution, global view + local tiles, and one
    placeholder per embedding row."""
    cands = [[56, 56], [112, 56], [56, 112], [112, 112], [168, 56]]
    assert M.select_best_resolution((200, 100), cands) == (112, 56)
    assert M.select_best_resolution((50, 50), cands) == (56, 56)
    assert M.select_best_resolution((60, 300), cands) == (56, 112)
    img = torch.rand(3, 100, 200)
    px, crops = M.process_images([img, torch.rand(3, 40, 40)], cands, image_size=56)
    assert crops == [(2, 1), (1, 1)] and px.shape == (1 + 2 + 1 + 1, 3, 56, 56)
    assert float(px.min()) >= -1.0 - 1e-6 and float(px.max()) <= 1.0 + 1e-6
    # the wide image fills the 112 x 56 canvas: its two local tiles are its left and right half
    left = torch.nn.functional.interpolate(img[None], size=(56, 112), mode="bicubic",
                                           align_corners=False, antialias=True)[0].clamp(0, 1)
    assert torch.allclose(px[1], (left[:, :, :56] - 0.5) / 0.5, atol=1e-5)
    assert torch.allclose(px[2], (left[:, :, 56:] - 0.5) / 0.5, atol=1e-5)
    # the global view letter-boxes the image with the mean colour (0 after normalisation)
    assert torch.allclose(px[0][:, 0], torch.zeros(3, 56), atol=1e-6)
    d = _hf_config(False)
    d["candidate_resolutions"] = cands
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    llm = LLM(mc, device="cpu", max_num_seqs=2, max_num_batched_tokens=64, max_model_len=256,
              num_gpu_blocks=64, seed=0)
    model = llm.engine.model
    ids, mm = model.prepare_images([img, torch.rand(3, 40, 40)], [5, 300, 6, 300, 7])
    n0, n1 = model.num_image_tokens((2, 1)), model.num_image_tokens((1, 1))
    assert ids == [5] + [300] * n0 + [6] + [300] * n1 + [7]
    out = llm.generate([{"prompt_token_ids": ids, "multi_modal_data": mm}],
                       SamplingParams(max_tokens=2, temperature=0.0, ignore_eos=True))
    assert len(out[0].outputs[0].token_ids) == 2
