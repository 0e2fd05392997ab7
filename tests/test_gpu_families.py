"""Model families whose special paths only matter on the GPU: ALiBi slopes through the
attention kernels (Baichuan 13B layout) and the DeepSeek-VL2 vision side in bf16."""
import pytest
import torch

from vllm_gcu_b200.config import ModelConfig
from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams
from vllm_gcu_b200.ops import _native

pytestmark = pytest.mark.gpu


def _copy_weights(src, dst):
    sd = {k: v.detach().cpu() for k, v in src.state_dict().items()}
    for name, mod in src.named_modules():
        if getattr(mod, "_interleaved", False) and name + ".weight" in sd:
            w = sd[name + ".weight"]
            I = w.shape[0] // 2
            w4 = w.view(I // 32, 2, 32, w.shape[1])
            sd[name + ".weight"] = torch.cat([w4[:, 0].reshape(I, -1), w4[:, 1].reshape(I, -1)])
    dst.load_state_dict({k: v.to(dst.state_dict()[k].dtype) for k, v in sd.items()
                         if k in dst.state_dict()}, strict=False)


def test_alibi_model_gpu_tracks_cpu_reference():
    d = {"architectures": ["BaichuanForCausalLM"], "vocab_size": 2048, "hidden_size": 512,
         "intermediate_size": 1024, "num_hidden_layers": 2, "num_attention_heads": 8,
         "num_key_value_heads": 8, "head_dim": 64, "rms_norm_eps": 1e-6,
         "max_position_embeddings": 512, "tie_word_embeddings": False}
    kw = dict(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256, num_gpu_blocks=64,
              load_format="dummy", seed=0)
    gpu = LLM(ModelConfig.from_hf_dict(d, dtype=torch.bfloat16), device="cuda",
              enforce_eager=True, **kw)
    assert gpu.engine.model.layers["0"].self_attn.attn.alibi is not None
    cpu = LLM(ModelConfig.from_hf_dict(d, dtype=torch.float32), device="cpu", **kw)
    _copy_weights(gpu.engine.model, cpu.engine.model)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (100, 33, 7)]
    one = SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True)
    gpu.engine.runner.keep_logits = True
    cpu.engine.runner.keep_logits = True
    og = gpu.generate(prompts, one)         # chunked prefill (64 tokens per step), then decode
    oc = cpu.generate(prompts, one)
    torch.cuda.synchronize()
    _native.check_status()
    lg, lc = gpu.engine.runner.last_logits.float().cpu(), cpu.engine.runner.last_logits.float()
    err = (lg - lc).abs().max().item()
    assert err < 0.06 * lc.std().item() + 0.03, (err, lc.std().item())
    assert [o.outputs[0].token_ids[0] for o in og] == [o.outputs[0].token_ids[0] for o in oc]


def test_deepseek_vl2_vision_side_on_gpu():
    lang = dict(vocab_size=320, hidden_size=256, intermediate_size=256, moe_intermediate_size=128,
                num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
                n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1,
                first_k_dense_replace=1, max_position_embeddings=512, rms_norm_eps=1e-6,
                norm_topk_prob=False, tie_word_embeddings=False)
    d = {"architectures": ["DeepseekVLV2ForCausalLM"], "tile_tag": "2D",
         "global_view_pos": "head", "image_token_id": 300,
         "vision_config": dict(image_size=56, patch_size=14, width=32, layers=2, heads=2,
                               mlp_ratio=2.0),
         "projector_config": dict(projector_type="downsample_mlp_gelu", input_dim=32,
                                  n_embed=256, depth=2, mlp_ratio=1, downsample_ratio=2),
         "language_config": lang}
    kw = dict(max_num_seqs=2, max_num_batched_tokens=64, max_model_len=256, num_gpu_blocks=64,
              seed=0)
    gpu = LLM(ModelConfig.from_hf_dict(d, dtype=torch.bfloat16), device="cuda",
              enforce_eager=True, **kw)
    cpu = LLM(ModelConfig.from_hf_dict(d, dtype=torch.float32), device="cpu", **kw)
    _copy_weights(gpu.engine.model, cpu.engine.model)
    pixels = torch.randn(3, 3, 56, 56)
    crops = [(2, 1)]
    with torch.inference_mode():
        eg = gpu.engine.model.encode_images(pixels.cuda(), crops).float().cpu()
        ec = cpu.engine.model.encode_images(pixels, crops)
    assert eg.shape == ec.shape == (17, 256)
    assert (eg - ec).abs().max().item() < 0.05 * ec.abs().max().item() + 0.02
    ids = [5, 6] + [300] * 17 + [7, 8, 9, 10]
    out = gpu.generate([{"prompt_token_ids": ids,
                         "multi_modal_data": {"pixel_values": pixels.cuda(),
                                              "images_spatial_crop": crops}}],
                       SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))
    torch.cuda.synchronize()
    _native.check_status()
    assert len(out[0].outputs[0].token_ids) == 4


def test_gpt_bigcode_gpu_tracks_cpu_reference():
    """LayerNorm (+ residual) and plain GELU kernels, learnt positions, multi-query attention."""
    d = {"architectures": ["GPTBigCodeForCausalLM"], "vocab_size": 2048, "n_positions": 512,
         "n_embd": 512, "n_layer": 2, "n_head": 8, "n_inner": 1024, "multi_query": True}
    kw = dict(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256, num_gpu_blocks=64,
              load_format="dummy", seed=0)
    gpu = LLM(ModelConfig.from_hf_dict(d, dtype=torch.bfloat16), device="cuda",
              enforce_eager=True, **kw)
    cpu = LLM(ModelConfig.from_hf_dict(d, dtype=torch.float32), device="cpu", **kw)
    _copy_weights(gpu.engine.model, cpu.engine.model)
    with torch.no_grad():                      # non-trivial biases on both sides
        for (n, pg), (_, pc) in zip(sorted(gpu.engine.model.named_parameters()),
                                    sorted(cpu.engine.model.named_parameters())):
            if n.endswith(".bias"):
                b = torch.randn(pg.shape, generator=torch.Generator().manual_seed(len(n))) * 0.05
                pg.copy_(b.to(pg.dtype))
                pc.copy_(pg.float().cpu())
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (100, 33, 7)]
    one = SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True)
    gpu.engine.runner.keep_logits = True
    cpu.engine.runner.keep_logits = True
    og = gpu.generate(prompts, one)
    oc = cpu.generate(prompts, one)
    torch.cuda.synchronize()
    _native.check_status()
    lg, lc = gpu.engine.runner.last_logits.float().cpu(), cpu.engine.runner.last_logits.float()
    err = (lg - lc).abs().max().item()
    assert err < 0.06 * lc.std().item() + 0.03, (err, lc.std().item())
    assert [o.outputs[0].token_ids[0] for o in og] == [o.outputs[0].token_ids[0] for o in oc]
