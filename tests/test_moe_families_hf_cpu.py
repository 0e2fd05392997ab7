"""Mixture-of-experts families against the HuggingFace implementations with the field names and
options of real ``config.json`` files: Qwen3-MoE with dense layers in between
(``decoder_sparse_step``, ``mlp_only_layers``, unnormalised routing weights), Mixtral, and
DeepSeek-V3 (latent attention, group-limited sigmoid routing with a selection bias, shared
experts, YaRN given as ``type: yarn`` with ``mscale`` / ``mscale_all_dim``).  The state dicts
carry all experts of a layer in one tensor, as newer library versions write them."""
import pytest
import torch

tr = pytest.importorskip("transformers")

from vllm_gcu_b200.config import ModelConfig  # noqa: E402
from vllm_gcu_b200.engine.llm import LLM  # noqa: E402
from vllm_gcu_b200.engine.request import SamplingParams  # noqa: E402

COMMON = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_attention_heads=4,
              max_position_embeddings=256, rms_norm_eps=1e-6, tie_word_embeddings=False)


def _check(hf, cfg_dict, arch, prompt_len=23):
    d = dict(cfg_dict)
    d["architectures"] = [arch]
    mc = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    llm = LLM(mc, device="cpu", max_num_seqs=2, max_num_batched_tokens=256, max_model_len=256,
              num_gpu_blocks=64, load_format="none")
    loaded = llm.engine.model.load_weights(hf.state_dict().items())
    missing = [n for n in hf.state_dict() if n not in loaded and "rotary" not in n]
    assert not missing, missing
    ids = torch.randint(0, 320, (prompt_len,), generator=torch.Generator().manual_seed(1)).tolist()
    llm.engine.runner.keep_logits = True
    llm.generate([ids], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
    got = llm.engine.runner.last_logits[0]
    with torch.inference_mode():
        want = hf(input_ids=torch.tensor([ids])).logits[0, -1]
    assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())
    return mc


@pytest.mark.parametrize("step,dense,norm", [(2, [], True), (1, [1], False)])
def test_qwen3_moe_layer_layout_and_routing(step, dense, norm):
    torch.manual_seed(0)
    c = tr.Qwen3MoeConfig(**COMMON, num_hidden_layers=4, num_key_value_heads=2, head_dim=16,
                          moe_intermediate_size=32, num_experts=8, num_experts_per_tok=2,
                          norm_topk_prob=norm, decoder_sparse_step=step, mlp_only_layers=dense)
    mc = _check(tr.Qwen3MoeForCausalLM(c).eval().float(), c.to_dict(), "Qwen3MoeForCausalLM")
    want = [(i + 1) % step == 0 and i not in dense for i in range(4)]
    assert [mc.is_moe_layer(i) for i in range(4)] == want


def test_mixtral():
    torch.manual_seed(0)
    c = tr.MixtralConfig(**COMMON, num_hidden_layers=2, num_key_value_heads=2,
                         num_local_experts=4, num_experts_per_tok=2)
    _check(tr.MixtralForCausalLM(c).eval().float(), c.to_dict(), "MixtralForCausalLM")


@pytest.mark.parametrize("rope", [
    {"rope_type": "default", "rope_theta": 10000.0},
    {"rope_type": "yarn", "rope_theta": 10000.0, "factor": 4.0,
     "original_max_position_embeddings": 64, "mscale": 1.0, "mscale_all_dim": 1.0,
     "beta_fast": 32, "beta_slow": 1}], ids=lambda r: r["rope_type"])
def test_deepseek_v3(rope):
    torch.manual_seed(0)
    c = tr.DeepseekV3Config(**COMMON, num_hidden_layers=3, num_key_value_heads=4,
                            moe_intermediate_size=32, n_routed_experts=8, n_shared_experts=1,
                            num_experts_per_tok=2, n_group=2, topk_group=1,
                            routed_scaling_factor=2.5, norm_topk_prob=True,
                            first_k_dense_replace=1, kv_lora_rank=32, q_lora_rank=48,
                            qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                            rope_parameters=rope)
    hf = tr.DeepseekV3ForCausalLM(c).eval().float()
    with torch.no_grad():                         # a selection bias that changes the routing
        for n, t in list(hf.named_parameters()) + list(hf.named_buffers()):
            if "e_score_correction_bias" in n:
                t.copy_(torch.randn_like(t) * 0.1)
    mc = _check(hf, c.to_dict(), "DeepseekV3ForCausalLM", prompt_len=150)
    assert mc.scoring_func == "sigmoid" and mc.topk_method == "noaux_tc"


@pytest.mark.parametrize("q_lora,scale", [(None, 1.0), (None, 16.0), (48, 1.0)])
def test_deepseek_v2(q_lora, scale):
    """DeepSeek-V2 / V2-Lite: plain softmax top-k routing with a scaling factor, two shared
    experts, and (Lite) no query down-projection: ``q_proj`` is a layer of its own."""
    torch.manual_seed(0)
    c = tr.DeepseekV2Config(**COMMON, num_hidden_layers=3, num_key_value_heads=4,
                            moe_intermediate_size=32, n_routed_experts=8, n_shared_experts=2,
                            num_experts_per_tok=2, first_k_dense_replace=1, kv_lora_rank=32,
                            q_lora_rank=q_lora, qk_nope_head_dim=16, qk_rope_head_dim=8,
                            v_head_dim=16, topk_method="greedy", n_group=1, topk_group=1,
                            routed_scaling_factor=scale, norm_topk_prob=False)
    _check(tr.DeepseekV2ForCausalLM(c).eval().float(), c.to_dict(), "DeepseekV2ForCausalLM")
