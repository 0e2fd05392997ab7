"""Vision-language throughput benchmark: requests with one synthetic image each through one of
the multimodal families of this package (the reference ships
benchmarks/benchmark_vision_language.py plus a ``vision_language/`` folder with one adapter per
model; there is no dataset on this machine, so images are random tensors and weights random).

``--family`` selects the model family; each family contributes a configuration of the given
sizes and the way one request is built (pixel layout, placeholder count):

  qwen2_5_vl   Qwen2.5-VL   windowed vision transformer, M-RoPE; ``--grid h w`` patches
  qwen2_vl     Qwen2-VL / QVQ  full-attention vision transformer, M-RoPE; ``--grid h w``
  glm4v        GLM-4.1V     interpolated positions, convolution merge, M-RoPE; ``--grid h w``
  llava        LLaVA-1.5    CLIP tower, one ``--image-size`` view
  llava_next   LLaVA-NeXT   CLIP tower, base view + 2 x 2 tiles
  internvl     InternVL2 / 2.5  InternViT, ``--tiles`` tiles of ``--image-size``
  deepseek_vl2 DeepSeek-VL2 SigLIP tower, global view + 2 x 1 local tiles

Reports requests/s, prompt (text + image placeholder) tokens/s and output tokens/s, with the
vision tower inside the timed region.

  python benchmarks/benchmark_vision_language.py --family internvl --device cpu --layers 2 \
      --hidden 64 --vision-layers 2 --vision-hidden 32 --image-size 28 --num-prompts 4 \
      --output-len 4 --dtype float32
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from vllm_gcu_b200.config import ModelConfig  # noqa: E402
from vllm_gcu_b200.engine.llm import LLM  # noqa: E402
from vllm_gcu_b200.engine.request import SamplingParams  # noqa: E402

IMG, VSTART, VEND = 290, 288, 289


def _text(a, **extra) -> dict:
    heads = max(a.hidden // 64, 2)
    return dict(vocab_size=a.vocab, hidden_size=a.hidden, intermediate_size=a.hidden * 3,
                num_hidden_layers=a.layers, num_attention_heads=heads,
                num_key_value_heads=max(heads // 4, 1), max_position_embeddings=8192,
                rms_norm_eps=1e-6, tie_word_embeddings=False, **extra)


def _mrope(a) -> dict:
    hd = a.hidden // max(a.hidden // 64, 2)
    sec = [hd // 8, (hd // 2 - hd // 8) // 2, hd // 2 - hd // 8 - (hd // 2 - hd // 8) // 2]
    return {"type": "mrope", "mrope_section": sec}


def _vheads(a) -> int:
    return max(a.vision_hidden // 64, 2)


# -- one (config, request) pair per family ---------------------------------------------------
def qwen2_5_vl(a):
    d = {"architectures": ["Qwen2_5_VLForConditionalGeneration"],
         "text_config": _text(a, rope_theta=1e6, rope_scaling=_mrope(a)),
         "vision_config": dict(depth=a.vision_layers, hidden_size=a.vision_hidden,
                               intermediate_size=a.vision_hidden * 2, num_heads=_vheads(a),
                               in_channels=3, patch_size=14, spatial_merge_size=2,
                               temporal_patch_size=2, window_size=112, out_hidden_size=a.hidden,
                               fullatt_block_indexes=[a.vision_layers - 1]),
         "image_token_id": IMG, "video_token_id": 291, "vision_start_token_id": VSTART,
         "vision_end_token_id": VEND}
    return d, _qwen_request


def qwen2_vl(a):
    d = {"architectures": ["Qwen2VLForConditionalGeneration"],
         "text_config": _text(a, rope_theta=1e6, rope_scaling=_mrope(a)),
         "vision_config": dict(depth=a.vision_layers, embed_dim=a.vision_hidden,
                               hidden_size=a.hidden, mlp_ratio=2, num_heads=_vheads(a),
                               in_channels=3, patch_size=14, spatial_merge_size=2,
                               temporal_patch_size=2),
         "image_token_id": IMG, "video_token_id": 291, "vision_start_token_id": VSTART,
         "vision_end_token_id": VEND}
    return d, _qwen_request


def glm4v(a):
    hd = a.hidden // max(a.hidden // 64, 2)
    quarter = hd // 4                       # rotary pairs on half of the head, split t / h / w
    sec = [quarter - 2 * (quarter // 3), quarter // 3, quarter // 3]
    d = {"architectures": ["Glm4vForConditionalGeneration"],
         "text_config": _text(a, attention_bias=True, rope_parameters={
             "rope_type": "default", "rope_theta": 10000.0, "mrope_section": sec,
             "partial_rotary_factor": 0.5}),
         "vision_config": dict(depth=a.vision_layers, hidden_size=a.vision_hidden,
                               intermediate_size=a.vision_hidden * 2, num_heads=_vheads(a),
                               in_channels=3, image_size=a.image_size, patch_size=14,
                               spatial_merge_size=2, temporal_patch_size=2,
                               out_hidden_size=a.hidden),
         "image_token_id": IMG, "image_start_token_id": VSTART, "image_end_token_id": VEND}
    return d, _qwen_request


def _qwen_request(a, model, text, g):
    gh, gw = a.grid
    assert gh % 2 == 0 and gw % 2 == 0, "the patch grid must be even (2 x 2 merge)"
    n_img = gh * gw // 4
    ids = text[:len(text) // 2] + [VSTART] + [IMG] * n_img + [VEND] + text[len(text) // 2:]
    pixels = torch.randn(gh * gw, 3 * 2 * 14 * 14, generator=g)
    return ids, {"pixel_values": pixels, "image_grid_thw": torch.tensor([[1, gh, gw]])}


def _clip(a) -> dict:
    return dict(model_type="clip_vision_model", hidden_size=a.vision_hidden,
                intermediate_size=a.vision_hidden * 2, num_hidden_layers=a.vision_layers,
                num_attention_heads=_vheads(a), image_size=a.image_size, patch_size=a.patch_size,
                hidden_act="quick_gelu")


def llava(a):
    d = {"architectures": ["LlavaForConditionalGeneration"], "text_config": _text(a),
         "vision_config": _clip(a), "image_token_index": IMG, "vision_feature_layer": -2,
         "vision_feature_select_strategy": "default"}

    def request(a, model, text, g):
        n = model.tokens_per_image
        ids = text[:len(text) // 2] + [IMG] * n + text[len(text) // 2:]
        return ids, {"pixel_values": torch.randn(1, 3, a.image_size, a.image_size, generator=g)}
    return d, request


def llava_next(a):
    s = a.image_size
    d = {"architectures": ["LlavaNextForConditionalGeneration"], "text_config": _text(a),
         "vision_config": _clip(a), "image_token_index": IMG, "vision_feature_layer": -2,
         "vision_feature_select_strategy": "default",
         "image_grid_pinpoints": [[s, 2 * s], [2 * s, s], [2 * s, 2 * s]]}

    def request(a, model, text, g):
        size = (2 * s - 3, 2 * s)                 # slightly wide: one padded row is cut
        n = model.num_image_tokens(size, 5)
        ids = text[:len(text) // 2] + [IMG] * n + text[len(text) // 2:]
        return ids, {"pixel_values": torch.randn(5, 3, s, s, generator=g),
                     "image_sizes": torch.tensor([list(size)])}
    return d, request


def internvl(a):
    d = {"architectures": ["InternVLChatModel"],
         "llm_config": {**_text(a), "architectures": ["Qwen2ForCausalLM"]},
         "vision_config": dict(hidden_size=a.vision_hidden, intermediate_size=a.vision_hidden * 2,
                               num_hidden_layers=a.vision_layers,
                               num_attention_heads=_vheads(a), image_size=a.image_size,
                               patch_size=a.patch_size, norm_type="layer_norm", qkv_bias=True),
         "downsample_ratio": 0.5, "select_layer": -1, "ps_version": "v2",
         "img_context_token_id": IMG}

    def request(a, model, text, g):
        n = a.tiles * model.tokens_per_tile
        ids = text[:len(text) // 2] + [IMG] * n + text[len(text) // 2:]
        return ids, {"pixel_values": torch.randn(a.tiles, 3, a.image_size, a.image_size,
                                                 generator=g)}
    return d, request


def deepseek_vl2(a):
    lang = _text(a, moe_intermediate_size=a.hidden, n_routed_experts=8, num_experts_per_tok=2,
                 n_shared_experts=1, first_k_dense_replace=1, norm_topk_prob=False)
    lang["num_key_value_heads"] = lang["num_attention_heads"]
    d = {"architectures": ["DeepseekVLV2ForCausalLM"], "tile_tag": "2D",
         "global_view_pos": "head", "image_token_id": IMG,
         "vision_config": dict(image_size=a.image_size, patch_size=a.patch_size,
                               width=a.vision_hidden, layers=a.vision_layers, heads=_vheads(a),
                               mlp_ratio=2.0),
         "projector_config": dict(projector_type="downsample_mlp_gelu",
                                  input_dim=a.vision_hidden, n_embed=a.hidden, depth=2,
                                  mlp_ratio=1, downsample_ratio=2),
         "language_config": lang}

    def request(a, model, text, g):
        crop = (2, 1)                             # local tiles: 2 wide, 1 high
        n = model.num_image_tokens(crop)
        ids = text[:len(text) // 2] + [IMG] * n + text[len(text) // 2:]
        return ids, {"pixel_values": torch.randn(3, 3, a.image_size, a.image_size, generator=g),
                     "images_spatial_crop": [crop]}
    return d, request


FAMILIES = {f.__name__: f for f in (qwen2_5_vl, qwen2_vl, glm4v, llava, llava_next, internvl,
                                    deepseek_vl2)}


def run(a) -> dict:
    dtype = getattr(torch, a.dtype)
    d, request = FAMILIES[a.family](a)
    mc = ModelConfig.from_hf_dict(d, dtype=dtype)
    llm = LLM(mc, device=a.device, max_model_len=a.max_model_len,
              max_num_batched_tokens=max(2048, a.max_model_len), load_format="dummy")
    model = llm.engine.model
    dev = getattr(llm.engine.runner, "device", "cpu")
    g = torch.Generator().manual_seed(0)
    reqs = []
    for _ in range(a.num_prompts):
        text = torch.randint(300, a.vocab, (a.text_len,), generator=g).tolist()
        ids, mm = request(a, model, text, g)
        mm = {k: (v.to(device=dev, dtype=dtype) if k == "pixel_values" else v)
              for k, v in mm.items()}
        reqs.append({"prompt_token_ids": ids, "multi_modal_data": mm})
    longest = max(len(r["prompt_token_ids"]) for r in reqs)
    assert longest + a.output_len < a.max_model_len, \
        f"--max-model-len must exceed {longest + a.output_len}"
    sp = SamplingParams(max_tokens=a.output_len, temperature=0.0, ignore_eos=True)
    llm.generate(reqs[:1], sp)                         # warm-up
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = llm.generate(reqs, sp)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    n_in = sum(len(r["prompt_token_ids"]) for r in reqs)
    n_out = sum(len(o.outputs[0].token_ids) for o in outs)
    n_img = sum(t == IMG for t in reqs[0]["prompt_token_ids"])
    return {"family": a.family, "requests_per_s": len(reqs) / dt, "prompt_tokens_per_s": n_in / dt,
            "output_tokens_per_s": n_out / dt, "image_tokens_per_request": n_img, "seconds": dt}


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--family", default="qwen2_5_vl", choices=sorted(FAMILIES))
    ap.add_argument("--device", default="auto")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--vision-layers", type=int, default=8)
    ap.add_argument("--vision-hidden", type=int, default=1280)
    ap.add_argument("--num-prompts", type=int, default=32)
    ap.add_argument("--text-len", type=int, default=32)
    ap.add_argument("--grid", type=int, nargs=2, default=[32, 32],
                    help="image patches h w (Qwen families)")
    ap.add_argument("--image-size", type=int, default=448, help="pixels per view / tile")
    ap.add_argument("--patch-size", type=int, default=14)
    ap.add_argument("--tiles", type=int, default=5, help="tiles per image (InternVL)")
    ap.add_argument("--output-len", type=int, default=32)
    ap.add_argument("--max-model-len", type=int, default=4096)
    res = run(ap.parse_args(argv))
    print(json.dumps(res, indent=1))
    return res


if __name__ == "__main__":
    main()
