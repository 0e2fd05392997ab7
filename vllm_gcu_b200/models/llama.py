"""Dense decoder families on the generic :class:`DecoderLM`.

``LlamaForCausalLM`` covers Llama 2/3/3.1, Mistral, Yi and InternLM2-style
checkpoints; ``Qwen2ForCausalLM`` adds q/k/v biases; ``Qwen3ForCausalLM`` adds
per-head QK RMSNorm (vllm_gcu/models/qwen3/qwen3.py:437); ``Glm4ForCausalLM`` is the
GLM-4-0414 variant with four norms per layer, GPT-J rotary on half of the head and a
fused ``gate_up_proj`` checkpoint tensor (vllm_gcu/models/glm4/glm4.py:82-231).
"""
from __future__ import annotations

import dataclasses

from ..config import ModelConfig
from .decoder import DecoderLM


class LlamaForCausalLM(DecoderLM):
    pass


class Qwen2ForCausalLM(DecoderLM):
    def __init__(self, cfg: ModelConfig, device="cpu"):
        if not cfg.attention_bias:
            cfg = dataclasses.replace(cfg, attention_bias=True)
        super().__init__(cfg, device)


class Qwen3ForCausalLM(DecoderLM):
    def __init__(self, cfg: ModelConfig, device="cpu"):
        if not cfg.qk_norm:
            cfg = dataclasses.replace(cfg, qk_norm=True)
        super().__init__(cfg, device)


class Glm4ForCausalLM(DecoderLM):
    def __init__(self, cfg: ModelConfig, device="cpu"):
        cfg = dataclasses.replace(cfg, sandwich_norm=True, rope_is_neox=False,
                                  partial_rotary_factor=cfg.partial_rotary_factor
                                  if cfg.partial_rotary_factor < 1.0 else 0.5)
        super().__init__(cfg, device)
