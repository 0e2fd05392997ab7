"""Vision-language throughput benchmark: requests with one synthetic image each through
Qwen2.5-VL (the reference ships benchmarks/benchmark_vision_language.py, which feeds dataset
images to its multimodal models; there is no dataset on this machine, so images are random
patch tensors of a fixed grid and the weights are random).

Reports requests/s, prompt (text + image placeholder) tokens/s and output tokens/s, with the
vision tower inside the timed region.

  python benchmarks/benchmark_vision_language.py --device cpu --layers 2 --hidden 64 \
      --num-prompts 4 --grid 6 4 --output-len 4 --dtype float32
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


def config(a) -> ModelConfig:
    heads = max(a.hidden // 64, 2)
    hd = a.hidden // heads
    sec = [hd // 8, (hd // 2 - hd // 8) // 2, hd // 2 - hd // 8 - (hd // 2 - hd // 8) // 2]
    d = {
        "architectures": ["Qwen2_5_VLForConditionalGeneration"],
        "text_config": dict(vocab_size=a.vocab, hidden_size=a.hidden,
                            intermediate_size=a.hidden * 3, num_hidden_layers=a.layers,
                            num_attention_heads=heads, num_key_value_heads=max(heads // 4, 1),
                            max_position_embeddings=8192, rope_theta=1e6, rms_norm_eps=1e-6,
                            tie_word_embeddings=False,
                            rope_scaling={"type": "mrope", "mrope_section": sec}),
        "vision_config": dict(depth=a.vision_layers, hidden_size=a.vision_hidden,
                              intermediate_size=a.vision_hidden * 2,
                              num_heads=max(a.vision_hidden // 64, 2), in_channels=3,
                              patch_size=14, spatial_merge_size=2, temporal_patch_size=2,
                              window_size=112, out_hidden_size=a.hidden,
                              fullatt_block_indexes=[a.vision_layers - 1]),
        "image_token_id": IMG, "video_token_id": 291, "vision_start_token_id": VSTART,
        "vision_end_token_id": VEND,
    }
    return ModelConfig.from_hf_dict(d, dtype=getattr(torch, a.dtype))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="auto")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--vision-layers", type=int, default=8)
    ap.add_argument("--vision-hidden", type=int, default=1280)
    ap.add_argument("--num-prompts", type=int, default=32)
    ap.add_argument("--text-len", type=int, default=32)
    ap.add_argument("--grid", type=int, nargs=2, default=[32, 32], help="image patches h w")
    ap.add_argument("--output-len", type=int, default=32)
    a = ap.parse_args()
    gh, gw = a.grid
    assert gh % 2 == 0 and gw % 2 == 0, "the patch grid must be even (2 x 2 merge)"
    n_img = gh * gw // 4
    llm = LLM(config(a), device=a.device, max_model_len=a.text_len + n_img + a.output_len + 16,
              max_num_batched_tokens=max(2048, a.text_len + n_img + 8), load_format="dummy")
    dev = llm.engine.runner.device if hasattr(llm.engine.runner, "device") else "cpu"
    g = torch.Generator().manual_seed(0)
    reqs = []
    for _ in range(a.num_prompts):
        text = torch.randint(300, a.vocab, (a.text_len,), generator=g).tolist()
        ids = text[: a.text_len // 2] + [VSTART] + [IMG] * n_img + [VEND] + text[a.text_len // 2:]
        pixels = torch.randn(gh * gw, 3 * 2 * 14 * 14, generator=g).to(
            device=dev, dtype=getattr(torch, a.dtype))
        reqs.append({"prompt_token_ids": ids,
                     "multi_modal_data": {"pixel_values": pixels,
                                          "image_grid_thw": torch.tensor([[1, gh, gw]])}})
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
    print(json.dumps({"requests_per_s": len(reqs) / dt, "prompt_tokens_per_s": n_in / dt,
                      "output_tokens_per_s": n_out / dt, "image_tokens_per_request": n_img,
                      "seconds": dt}, indent=1))


if __name__ == "__main__":
    main()
