"""Mixture-of-experts decoder families on :class:`DecoderLM`.

``Qwen3MoeForCausalLM``: QK-RMSNorm attention, softmax top-k router, routed experts only
(vllm_gcu/models/qwen3_moe/qwen3_moe.py:132-238).  ``MixtralForCausalLM``: Mixtral naming
(``block_sparse_moe.gate``, experts ``w1`` / ``w3`` / ``w2``); the reference's
``QuantMixtralForCausalLM`` loads the same layout with per-expert quantised linears
(vllm_gcu/models/... deepseek_moe_quant.py:487 ``load_kv_cache_scales``).
"""
from __future__ import annotations

import dataclasses
import re

import torch

from ..config import ModelConfig
from .decoder import DecoderLM

_EXPERT_RE = re.compile(r"^(model\.layers\.\d+\.)(mlp|block_sparse_moe)\.experts\.(\d+)\."
                        r"(gate_proj|up_proj|down_proj|w1|w2|w3)\.weight$")
# quantised checkpoints: the same expert projections with format-specific tensor suffixes
_QEXPERT_RE = re.compile(r"^(model\.layers\.\d+\.)(mlp|block_sparse_moe)\.experts\.(\d+)\."
                         r"(gate_proj|up_proj|down_proj|w1|w2|w3)\."
                         r"(weight|qweight|qzeros|scales|g_idx|weight_scale|weight_scale_inv|"
                         r"out_scales|input_scale|in_scales)$")
_WHICH = {"gate_proj": "gate", "up_proj": "up", "down_proj": "down",
          "w1": "gate", "w3": "up", "w2": "down"}
_FUSED_EXPERTS_RE = re.compile(
    r"^model\.layers\.(\d+)\.(?:mlp|block_sparse_moe)\.experts\.(gate_up_proj|down_proj)$")


class MoeDecoderLM(DecoderLM):
    def _expert_loader(self):
        ld = getattr(self, "_qexpert_loader", None)
        if ld is None:
            from ..layers.quant.moe import QuantExpertLoader
            ld = QuantExpertLoader(self.cfg.quantization, self.cfg.quant_config, self.cfg.dtype)
            self._qexpert_loader = ld
        return ld

    def finish_loading(self) -> None:
        """Called after the last checkpoint tensor: flushes buffered quantised experts."""
        ld = getattr(self, "_qexpert_loader", None)
        if ld is not None:
            ld.flush(lambda key: self.layers[key.split(".")[2]].mlp.experts)

    def load_special(self, name, tensor, owners) -> bool:
        if self.cfg.quantization:
            mq = _QEXPERT_RE.match(name)
            if mq is not None:
                layer = int(mq.group(1).split(".")[2])
                if not (self.start_layer <= layer < self.end_layer):
                    return True
                if mq.group(5) in ("input_scale", "in_scales"):
                    return True                 # activations stay bf16 on this path
                moe = self.layers[str(layer)].mlp.experts
                self._expert_loader().add(moe, mq.group(1), int(mq.group(3)), _WHICH[mq.group(4)],
                                          mq.group(5), tensor.to(moe.w13.device))
                return True
        m = _EXPERT_RE.match(name)
        if m is not None:
            layer = int(m.group(1).split(".")[2])
            if not (self.start_layer <= layer < self.end_layer):
                return True
            moe = self.layers[str(layer)].mlp.experts
            moe.load_expert_weight(int(m.group(3)), _WHICH[m.group(4)], tensor)
            return True
        mf = _FUSED_EXPERTS_RE.match(name)
        if mf is not None:
            # all experts of a layer in one tensor (checkpoints written by newer transformers):
            # gate_up_proj [E, 2I, H] with the gate rows first, down_proj [E, H, I]
            layer = int(mf.group(1))
            if self.start_layer <= layer < self.end_layer:
                moe = self.layers[str(layer)].mlp.experts
                for e in range(tensor.shape[0]):
                    if mf.group(2) == "gate_up_proj":
                        half = tensor.shape[1] // 2
                        moe.load_expert_weight(e, "gate", tensor[e, :half])
                        moe.load_expert_weight(e, "up", tensor[e, half:])
                    else:
                        moe.load_expert_weight(e, "down", tensor[e])
            return True
        if ".block_sparse_moe.gate." in name:
            return self._load_renamed(name.replace(".block_sparse_moe.gate.", ".mlp.gate."),
                                      tensor, owners)
        if name.endswith(".mlp.gate.e_score_correction_bias"):
            owner = name[: -len(".gate.e_score_correction_bias")]
            mod = owners.get(owner)
            if mod is not None:
                mod.load_weight("e_score_correction_bias", tensor)
            return True
        return False

    def _load_renamed(self, name, tensor, owners) -> bool:
        m = self.map_weight_name(name)
        if m is None:
            return True
        owner, pname, sid = m
        mod = owners.get(owner)
        if mod is not None:
            mod.load_weight(pname, tensor, sid)
        return True


class Qwen3MoeForCausalLM(MoeDecoderLM):
    def __init__(self, cfg: ModelConfig, device="cpu"):
        if not cfg.qk_norm:
            cfg = dataclasses.replace(cfg, qk_norm=True)
        super().__init__(cfg, device)


class MixtralForCausalLM(MoeDecoderLM):
    def __init__(self, cfg: ModelConfig, device="cpu"):
        if cfg.moe_intermediate_size == 0:
            cfg = dataclasses.replace(cfg, moe_intermediate_size=cfg.intermediate_size)
        super().__init__(cfg, device)


class DeepseekMoeForCausalLM(MoeDecoderLM):
    """DeepSeek-MoE (v1, e.g. deepseek-moe-16b): multi-head attention without MLA, softmax
    top-k routing without groups, shared experts, the first ``first_k_dense_replace`` layers
    dense.  The reference's ``QuantDeepseekForCausalLM`` serves it from per-expert quantised
    linears (vllm_gcu/models/deepseek_moe_quant.py:487); here the quantised expert tensors go
    through ``layers.quant.moe``."""
