"""Model registry: HuggingFace architecture name -> implementation.

The reference registers its model classes with vLLM's ``ModelRegistry``
(vllm_gcu/models/__init__.py:20-40); this table is the same idea for the built-in engine
and is also what the vLLM plugin entry point registers.
"""
from __future__ import annotations

import importlib
from typing import Callable

_REGISTRY: dict[str, str] = {
    "LlamaForCausalLM": "vllm_gcu_b200.models.llama:LlamaForCausalLM",
    "MistralForCausalLM": "vllm_gcu_b200.models.llama:LlamaForCausalLM",
    "Qwen2ForCausalLM": "vllm_gcu_b200.models.llama:Qwen2ForCausalLM",
    "Qwen2Model": "vllm_gcu_b200.models.llama:Qwen2EmbeddingModel",
    "Qwen2EmbeddingModel": "vllm_gcu_b200.models.llama:Qwen2EmbeddingModel",
    "Qwen3ForCausalLM": "vllm_gcu_b200.models.llama:Qwen3ForCausalLM",
    "Glm4ForCausalLM": "vllm_gcu_b200.models.llama:Glm4ForCausalLM",
    "InternLM2ForCausalLM": "vllm_gcu_b200.models.llama:InternLM2ForCausalLM",
    "BaichuanForCausalLM": "vllm_gcu_b200.models.llama:BaichuanForCausalLM",
    "BaiChuanForCausalLM": "vllm_gcu_b200.models.llama:BaichuanForCausalLM",
    "GemmaForCausalLM": "vllm_gcu_b200.models.llama:GemmaForCausalLM",
    "ChatGLMModel": "vllm_gcu_b200.models.llama:ChatGLMForCausalLM",
    "ChatGLMForConditionalGeneration": "vllm_gcu_b200.models.llama:ChatGLMForCausalLM",
    "YiForCausalLM": "vllm_gcu_b200.models.llama:LlamaForCausalLM",
    # the reference registers this name for a customer's Llama variant
    # (vllm_gcu/models/__init__.py:29-31); the architecture is Llama's
    "CustomerLlaMAForCausalLM": "vllm_gcu_b200.models.llama:LlamaForCausalLM",
    "GPTBigCodeForCausalLM": "vllm_gcu_b200.models.gpt_bigcode:GPTBigCodeForCausalLM",
    "Qwen3MoeForCausalLM": "vllm_gcu_b200.models.moe_models:Qwen3MoeForCausalLM",
    "MixtralForCausalLM": "vllm_gcu_b200.models.moe_models:MixtralForCausalLM",
    "QuantMixtralForCausalLM": "vllm_gcu_b200.models.moe_models:MixtralForCausalLM",
    "Qwen2_5_VLForConditionalGeneration":
        "vllm_gcu_b200.models.qwen2_5_vl:Qwen2_5_VLForConditionalGeneration",
    "Qwen2VLForConditionalGeneration":
        "vllm_gcu_b200.models.qwen2_vl:Qwen2VLForConditionalGeneration",
    "LlavaForConditionalGeneration": "vllm_gcu_b200.models.llava:LlavaForConditionalGeneration",
    "LlavaNextForConditionalGeneration":
        "vllm_gcu_b200.models.llava:LlavaNextForConditionalGeneration",
    "Glm4vForConditionalGeneration":
        "vllm_gcu_b200.models.glm4v:Glm4vForConditionalGeneration",
    "InternVLChatModel": "vllm_gcu_b200.models.internvl:InternVLChatModel",
    "InternVLForConditionalGeneration": "vllm_gcu_b200.models.internvl:InternVLChatModel",
    "GotOcr2ForConditionalGeneration":
        "vllm_gcu_b200.models.got_ocr2:GotOcr2ForConditionalGeneration",
    "GOTQwenForCausalLM": "vllm_gcu_b200.models.got_ocr2:GotOcr2ForConditionalGeneration",
    "DeepseekForCausalLM": "vllm_gcu_b200.models.moe_models:DeepseekMoeForCausalLM",
    "QuantDeepseekForCausalLM": "vllm_gcu_b200.models.moe_models:DeepseekMoeForCausalLM",
    "DeepseekV2ForCausalLM": "vllm_gcu_b200.models.deepseek:DeepseekV3ForCausalLM",
    "DeepseekV3ForCausalLM": "vllm_gcu_b200.models.deepseek:DeepseekV3ForCausalLM",
    "DeepseekVLV2ForCausalLM": "vllm_gcu_b200.models.deepseek_vl2:DeepseekVLV2ForCausalLM",
    "DeepSeekMTPModel": "vllm_gcu_b200.models.deepseek_mtp:DeepSeekMTP",
    # pooling models (no KV cache; built by build_pooling_model)
    "XLMRobertaForSequenceClassification":
        "vllm_gcu_b200.models.roberta:XLMRobertaForSequenceClassification",
    "XLMRobertaModel": "vllm_gcu_b200.models.roberta:RobertaEmbeddingModel",
    "RobertaModel": "vllm_gcu_b200.models.roberta:RobertaEmbeddingModel",
}

POOLING_ARCHITECTURES = {"XLMRobertaForSequenceClassification", "XLMRobertaModel", "RobertaModel"}


def register_model(arch: str, target: str) -> None:
    """``target`` is ``"module.path:ClassName"``."""
    _REGISTRY[arch] = target


def supported_architectures() -> list[str]:
    return sorted(_REGISTRY)


def get_model_class(arch: str) -> Callable:
    try:
        target = _REGISTRY[arch]
    except KeyError:
        raise ValueError(f"unsupported architecture {arch!r}; known: {supported_architectures()}")
    mod, _, cls = target.partition(":")
    return getattr(importlib.import_module(mod), cls)


def build_model(cfg, device):
    return get_model_class(cfg.architecture)(cfg, device)


def build_pooling_model(hf_config: dict, device="cpu", dtype=None):
    """Cross-encoder / embedding model from a HuggingFace ``config.json`` dict, wrapped in a
    ``PoolingRunner`` (``run`` for embeddings or logits, ``score`` for query-document pairs)."""
    from .roberta import PoolingRunner, RobertaConfig
    arch = (hf_config.get("architectures") or ["XLMRobertaModel"])[0]
    if arch not in POOLING_ARCHITECTURES:
        raise ValueError(f"{arch!r} is not a pooling architecture")
    over = {"dtype": dtype} if dtype is not None else {}
    cfg = RobertaConfig.from_hf_dict(hf_config, **over)
    return PoolingRunner(get_model_class(arch)(cfg, device), device)
