"""EAGLE draft head for dense decoder models (Llama family).

The draft model is one decoder layer on top of ``fc(concat(embedding of token t + 1, target
hidden state at t))``; its output goes through the target's LM head and proposes token
``t + 2``.  It has its own KV cache (one layer) that shares the target's block tables, so it
plugs into the model runner exactly like the DeepSeek MTP module (``runner.drafter``).  The
reference reaches EAGLE / multi-step draft models through vLLM's spec-decode worker
(vllm_gcu/worker/spec_decode/spec_decode_worker.py:135-212).

Checkpoint layout (EAGLE-1 heads): ``embed_tokens.weight`` (a copy of the target's, ignored
when the target's embedding is shared), ``fc.weight`` (+ ``fc.bias``), ``layers.0.self_attn.*``,
``layers.0.mlp.*``, ``layers.0.post_attention_layernorm.weight``; the first layer has no input
layer norm.  An optional ``model.`` prefix is accepted.
"""
from __future__ import annotations

import dataclasses
import zlib
from typing import Iterable, Optional

import torch
import torch.nn as nn

from ..config import ModelConfig
from ..layers.attention import AttentionMetadata
from ..layers.linear import ReplicatedLinear
from ..parallel.state import tp_size


class EagleDrafter(nn.Module):
    def __init__(self, cfg: ModelConfig, device="cpu", target: Optional[nn.Module] = None,
                 fc_bias: bool = True):
        super().__init__()
        from ..models.decoder import DecoderLayer
        if cfg.is_mla or cfg.is_moe:
            raise ValueError("the EAGLE drafter covers dense decoder models; DeepSeek models "
                             "use their MTP module")
        if target is None:
            raise ValueError("the EAGLE drafter shares the embedding and LM head of its target")
        self.cfg = dataclasses.replace(cfg, num_hidden_layers=1, quantization=None,
                                       quant_config=None)
        H = cfg.hidden_size
        self.fc = ReplicatedLinear(2 * H, H, bias=fc_bias, dtype=cfg.dtype, device=device,
                                   prefix="fc")
        self.layers = nn.ModuleDict({"0": DecoderLayer(self.cfg, 0, device, "layers.0")})
        # shared with the target, not registered as sub-modules (their weights are the target's)
        object.__setattr__(self, "_embed", target.embed_tokens)
        object.__setattr__(self, "_head", target._head())
        self.device = torch.device(device)

    def kv_cache_spec(self) -> dict:
        return {"type": "gqa", "layers": 1,
                "kv_heads": max(1, self.cfg.num_key_value_heads // tp_size()),
                "head_dim": self.cfg.head_dim}

    def forward(self, input_ids: torch.Tensor, prev_hidden: torch.Tensor, md: AttentionMetadata,
                kv_caches: list, spec_step_idx: int = 0) -> torch.Tensor:
        layer = self.layers["0"]
        x = self.fc(torch.cat([self._embed(input_ids), prev_hidden], dim=-1))
        # the first (only) layer has no input layer norm: attention reads x as it is
        h = layer.self_attn(x, kv_caches[0], md)
        h, residual = layer.post_attention_layernorm(h, x.clone())
        h = layer.mlp(h)
        return h + residual

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return self._head.logits(hidden)

    # -- weights ---------------------------------------------------------------------
    _STACKED = (("qkv_proj", "q_proj", "q"), ("qkv_proj", "k_proj", "k"),
                ("qkv_proj", "v_proj", "v"), ("gate_up_proj", "gate_proj", 0),
                ("gate_up_proj", "up_proj", 1))

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        owners = {n: m for n, m in self.named_modules() if hasattr(m, "load_weight")}
        loaded: set[str] = set()
        for name, t in weights:
            n = name[len("model."):] if name.startswith("model.") else name
            if n.startswith(("embed_tokens.", "lm_head.")) or "input_layernorm" in n:
                continue
            owner, _, pname = n.rpartition(".")
            sid = None
            for stacked, part, shard in self._STACKED:
                if owner.endswith("." + part):
                    owner, sid = owner[:-len(part)] + stacked, shard
                    break
            mod = owners.get(owner)
            if mod is None:
                continue
            mod.load_weight(pname, t, sid)
            loaded.add(name)
        self._finalize()
        return loaded

    def _finalize(self) -> None:
        for mod in self.modules():
            fin = getattr(mod, "finalize", None)
            if fin is not None and mod is not self:
                fin()

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        for name, p in sorted(self.named_parameters()):
            if "norm" in name and name.endswith("weight"):
                p.data.fill_(1.0)
            elif name.endswith(".bias"):
                p.data.zero_()
            elif p.dtype in (torch.float32, torch.bfloat16, torch.float16):
                g = torch.Generator(device=p.device)
                g.manual_seed(zlib.crc32(("eagle." + name).encode()) ^ seed)
                tmp = torch.empty(p.shape, dtype=torch.float32, device=p.device)
                tmp.normal_(0.0, std, generator=g)
                p.data.copy_(tmp)
        self._finalize()
