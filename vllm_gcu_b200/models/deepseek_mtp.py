"""DeepSeek multi-token-prediction (MTP) drafter.

One MTP module = ``enorm`` / ``hnorm`` -> concat -> ``eh_proj`` -> one decoder block ->
``shared_head`` (norm + LM head), vllm_gcu/models/deepseek_mtp/deepseek_mtp.py:47-102.  The
module predicts token ``t + 2`` from the target's hidden state at ``t`` and the embedding of
token ``t + 1``; its decoder block has its own KV cache that shares the target's block
tables.  Checkpoint names ``model.layers.{num_hidden_layers + i}.*`` are re-homed onto
``mtp.{i}.*`` (deepseek_mtp.py:291-316).
"""
from __future__ import annotations

import dataclasses
import re
from typing import Iterable, Optional

import torch
import torch.nn as nn

from ..config import ModelConfig
from ..layers.attention import AttentionMetadata
from ..layers.basic import ParallelLMHead, RMSNorm, VocabParallelEmbedding
from ..layers.linear import ReplicatedLinear
from .decoder import DecoderLayer
from .deepseek import DeepseekV3ForCausalLM


class MTPLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device, prefix: str):
        super().__init__()
        H = cfg.hidden_size
        self.enorm = RMSNorm(H, cfg.rms_norm_eps, cfg.dtype, device)
        self.hnorm = RMSNorm(H, cfg.rms_norm_eps, cfg.dtype, device)
        self.eh_proj = ReplicatedLinear(2 * H, H, bias=False, dtype=cfg.dtype, device=device,
                                        prefix=prefix + ".eh_proj")
        # the MTP block is a MoE layer like the last body layers
        self.block = DecoderLayer(cfg, layer_idx, device, prefix)
        self.shared_head_norm = RMSNorm(H, cfg.rms_norm_eps, cfg.dtype, device)

    def forward(self, embeds: torch.Tensor, prev_hidden: torch.Tensor, positions: torch.Tensor,
                kv_cache: Optional[torch.Tensor], md: AttentionMetadata) -> torch.Tensor:
        # position 0 has no preceding token to condition on (deepseek_mtp.py:66-70)
        embeds = torch.where((positions == 0)[:, None], torch.zeros_like(embeds), embeds)
        x = self.eh_proj(torch.cat([self.enorm(embeds), self.hnorm(prev_hidden)], dim=-1))
        h, residual = self.block(x, None, kv_cache, md)
        out, _ = self.shared_head_norm(h, residual)
        return out


class DeepSeekMTP(nn.Module):
    """Holds ``num_nextn_predict_layers`` MTP modules; embeddings and LM head are shared with
    (or loaded like) the target model's."""

    def __init__(self, cfg: ModelConfig, device="cpu", target: Optional[nn.Module] = None):
        super().__init__()
        self.cfg = cfg
        n = max(1, cfg.num_nextn_predict_layers)
        self.num_mtp_layers = n
        L = cfg.num_hidden_layers
        # every MTP block is a sparse layer: make the layer index look like a MoE layer
        self.layers = nn.ModuleDict({str(i): MTPLayer(cfg, L + i, device, f"model.layers.{L + i}")
                                     for i in range(n)})
        self._shared = target is not None
        if target is not None:
            self.embed_tokens = target.embed_tokens
            self.lm_head = target.lm_head
        else:
            self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype,
                                                       device)
            self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype, device)
        self.device = torch.device(device)

    def kv_cache_spec(self) -> dict:
        cfg = self.cfg
        if cfg.is_mla:
            return {"type": "mla", "layers": self.num_mtp_layers,
                    "width": cfg.kv_lora_rank + cfg.qk_rope_head_dim}
        from ..parallel.state import tp_size
        return {"type": "gqa", "layers": self.num_mtp_layers,
                "kv_heads": max(1, cfg.num_key_value_heads // tp_size()), "head_dim": cfg.head_dim}

    def forward(self, input_ids: torch.Tensor, prev_hidden: torch.Tensor, md: AttentionMetadata,
                kv_caches: list, spec_step_idx: int = 0) -> torch.Tensor:
        i = spec_step_idx % self.num_mtp_layers
        emb = self.embed_tokens(input_ids)
        return self.layers[str(i)](emb, prev_hidden, md.positions, kv_caches[i], md)

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.lm_head.logits(hidden)

    # -- weights ---------------------------------------------------------------------
    _RENAME = [("embed_tokens", None), ("shared_head.norm", "shared_head_norm"),
               ("shared_head.head", None)]

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        """Accepts the full DeepSeek checkpoint stream; only ``model.layers.{L + i}.*`` is
        consumed."""
        cfg = self.cfg
        L = cfg.num_hidden_layers
        helper = _MtpLoader(self)
        loaded: set[str] = set()
        for name, t in weights:
            m = re.match(r"^model\.layers\.(\d+)\.(.*)$", name)
            if m is None or int(m.group(1)) < L:
                continue
            i = int(m.group(1)) - L
            if i >= self.num_mtp_layers:
                continue
            rest = m.group(2)
            layer = self.layers[str(i)]
            if rest.startswith("embed_tokens."):
                self.embed_tokens.load_weight("weight", t)
            elif rest.startswith("shared_head.head."):
                self.lm_head.load_weight("weight", t)
            elif rest.startswith("shared_head.norm."):
                layer.shared_head_norm.load_weight("weight", t)
            elif rest.startswith(("enorm.", "hnorm.")):
                getattr(layer, rest.split(".")[0]).load_weight("weight", t)
            elif rest.startswith("eh_proj."):
                layer.eh_proj.load_weight(rest.split(".")[-1], t)
            else:
                helper.load_block(i, f"model.layers.{L + i}.{rest}", t)
            loaded.add(name)
        for mod in self.modules():
            fin = getattr(mod, "finalize", None)
            if fin is not None and mod is not self:
                fin()
        return loaded

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        import zlib
        for name, p in sorted(self.named_parameters()):
            if name.startswith(("embed_tokens.", "lm_head.")) and self._shared:
                continue        # owned (and initialised) by the target model
            if "norm" in name and name.endswith("weight"):
                p.data.fill_(1.0)
            elif name.endswith(".bias") or "e_score_correction_bias" in name:
                p.data.zero_()
            elif p.dtype in (torch.float32, torch.bfloat16, torch.float16):
                g = torch.Generator(device=p.device)
                g.manual_seed(zlib.crc32(("mtp." + name).encode()) ^ seed)
                tmp = torch.empty(p.shape, dtype=torch.float32, device=p.device)
                tmp.normal_(0.0, std, generator=g)
                p.data.copy_(tmp)
        for mod in self.modules():
            fin = getattr(mod, "finalize", None)
            if fin is not None and mod is not self:
                fin()


class _MtpLoader(DeepseekV3ForCausalLM):
    """Reuses the DeepSeek name mapping for the decoder block inside an MTP layer."""

    def __init__(self, mtp: DeepSeekMTP):  # noqa: D401 - deliberately skips the parent ctor
        nn.Module.__init__(self)
        object.__setattr__(self, "_mtp", mtp)
        object.__setattr__(self, "cfg", dataclasses.replace(
            mtp.cfg, num_hidden_layers=mtp.cfg.num_hidden_layers + mtp.num_mtp_layers))
        self.start_layer = mtp.cfg.num_hidden_layers
        self.end_layer = self.cfg.num_hidden_layers

    def load_block(self, i: int, name: str, t: torch.Tensor) -> None:
        mtp = self._mtp
        L = mtp.cfg.num_hidden_layers
        block = mtp.layers[str(i)].block
        owners = {}
        prefix = f"model.layers.{L + i}"
        for n, mod in block.named_modules():
            if hasattr(mod, "load_weight"):
                owners[prefix + ("." + n if n else "")] = mod
        # stacked experts
        from .moe_models import _EXPERT_RE, _WHICH
        m = _EXPERT_RE.match(name)
        if m is not None:
            block.mlp.experts.load_expert_weight(int(m.group(3)), _WHICH[m.group(4)], t)
            return
        if name.endswith(".mlp.gate.e_score_correction_bias"):
            block.mlp.load_weight("e_score_correction_bias", t)
            return
        mapped = self.map_weight_name(name)
        if mapped is None:
            return
        owner, pname, sid = mapped
        mod = owners.get(owner)
        if mod is not None:
            mod.load_weight(pname, t, sid)
