"""GPT-BigCode (StarCoder, WizardCoder-15B): learnt absolute positions, LayerNorm, multi-query
attention (one key / value head), a plain GELU MLP, biases everywhere, LM head tied to the
token embedding.  The reference lists WizardCoder in its support matrix and serves it through
vLLM's upstream class (docs/source/user_guide/support_matrix/supported_models.md).

Checkpoint names: ``transformer.wte / wpe``, ``transformer.h.N.{ln_1, attn.c_attn,
attn.c_proj, ln_2, mlp.c_fc, mlp.c_proj}``, ``transformer.ln_f``; ``c_attn`` packs
``[q (hidden) | k (head_dim) | v (head_dim)]`` rows.
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config import ModelConfig
from ..layers.attention import AttentionMetadata, PagedAttention
from ..layers.basic import ParallelLMHead
from ..layers.linear import ColumnParallelLinear, QKVParallelLinear, RowParallelLinear
from ..ops import cuda as C
from ..parallel.state import get_state
from .decoder import DecoderLM


class LayerNormR(nn.Module):
    """LayerNorm with the ``(x)`` / ``(x, residual)`` contract of ``layers.basic.RMSNorm``:
    with a residual it returns ``(norm(x + residual), x + residual)``."""

    def __init__(self, hidden: int, eps: float, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden, dtype=dtype, device=device),
                                   requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(hidden, dtype=dtype, device=device),
                                 requires_grad=False)
        self.eps = eps

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        if x.numel() == 0:
            return x if residual is None else (x, residual)
        if ops.use_native(x) and x.dtype in (torch.bfloat16, torch.float16) \
                and x.shape[-1] % 8 == 0:
            out = C.norm(x, self.weight, self.eps, residual=residual, bias=self.bias,
                         layer_norm=True)
            return out if residual is None else (out, residual)
        if residual is not None:
            x = x + residual
        y = F.layer_norm(x.float(), (x.shape[-1],), self.weight.float(), self.bias.float(),
                         self.eps).to(x.dtype)
        return y if residual is None else (y, x)

    def load_weight(self, name: str, full: torch.Tensor, shard_id=None) -> None:
        getattr(self, name).data.copy_(full)


class BigCodeAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, device, prefix: str):
        super().__init__()
        D = cfg.head_dim
        self.c_attn = QKVParallelLinear(cfg.hidden_size, D, cfg.num_attention_heads,
                                        cfg.num_key_value_heads, bias=True, dtype=cfg.dtype,
                                        device=device, prefix=prefix + ".c_attn")
        self.c_proj = RowParallelLinear(cfg.num_attention_heads * D, cfg.hidden_size, bias=True,
                                        dtype=cfg.dtype, device=device, prefix=prefix + ".c_proj")
        self.attn = PagedAttention(self.c_attn.num_heads, self.c_attn.num_kv_heads, D,
                                   D ** -0.5, None)

    def forward(self, x, kv_cache, md: AttentionMetadata):
        return self.c_proj(self.attn(self.c_attn(x), kv_cache, md))


class BigCodeMLP(nn.Module):
    def __init__(self, cfg: ModelConfig, device, prefix: str):
        super().__init__()
        self.c_fc = ColumnParallelLinear(cfg.hidden_size, cfg.intermediate_size, bias=True,
                                         dtype=cfg.dtype, device=device, prefix=prefix + ".c_fc")
        self.c_proj = RowParallelLinear(cfg.intermediate_size, cfg.hidden_size, bias=True,
                                        dtype=cfg.dtype, device=device, prefix=prefix + ".c_proj")
        self.tanh = cfg.hidden_act in ("gelu_pytorch_tanh", "gelu_tanh", "gelu_new", "gelu_fast")

    def forward(self, x):
        h = self.c_fc(x)
        if ops.use_native(h) and h.dtype in (torch.bfloat16, torch.float16):
            h = C.activation(h, "gelu_tanh" if self.tanh else "gelu", mode="plain")
        else:
            h = F.gelu(h, approximate="tanh" if self.tanh else "none")
        return self.c_proj(h)


class BigCodeBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, device, prefix: str):
        super().__init__()
        H = cfg.hidden_size
        self.ln_1 = LayerNormR(H, cfg.rms_norm_eps, cfg.dtype, device)
        self.attn = BigCodeAttention(cfg, device, prefix + ".attn")
        self.ln_2 = LayerNormR(H, cfg.rms_norm_eps, cfg.dtype, device)
        self.mlp = BigCodeMLP(cfg, device, prefix + ".mlp")

    def forward(self, x, residual, kv_cache, md):
        if residual is None:
            residual = x
            h = self.ln_1(x)
        else:
            h, residual = self.ln_1(x, residual)
        h = self.attn(h, kv_cache, md)
        h, residual = self.ln_2(h, residual)
        return self.mlp(h), residual


class GPTBigCodeForCausalLM(DecoderLM):
    def __init__(self, cfg: ModelConfig, device="cpu"):
        nn.Module.__init__(self)
        if cfg.num_key_value_heads != 1:
            raise ValueError("GPT-BigCode checkpoints without multi-query attention pack q, k, v "
                             "per head and are not supported")
        self.cfg = cfg
        self.device = torch.device(device)
        st = get_state()
        pp, pp_rank = st.pp.world_size, st.pp.rank_in_group
        L = cfg.num_hidden_layers
        per = -(-L // pp)
        self.start_layer, self.end_layer = min(L, pp_rank * per), min(L, (pp_rank + 1) * per)
        self.is_first_stage, self.is_last_stage = pp_rank == 0, pp_rank == pp - 1
        self.sequence_parallel = False
        if self.is_first_stage or self.is_last_stage:
            self.embed_tokens = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype, device)
        if self.is_first_stage:
            self.wpe = nn.Embedding(cfg.max_position_embeddings, cfg.hidden_size,
                                    dtype=cfg.dtype, device=device)
        self.layers = nn.ModuleDict({str(i): BigCodeBlock(cfg, i, device, f"transformer.h.{i}")
                                     for i in range(self.start_layer, self.end_layer)})
        if self.is_last_stage:
            self.norm = LayerNormR(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)
        self.lm_head = None                               # tied to the token embedding

    def forward(self, input_ids, md: AttentionMetadata, kv_caches, intermediate=None,
                inputs_embeds=None):
        if self.is_first_stage:
            x = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
            x = x + self.wpe(md.positions[: x.shape[0]])
            residual = None
        else:
            x, residual = intermediate
        for j, i in enumerate(range(self.start_layer, self.end_layer)):
            x, residual = self.layers[str(i)](x, residual, kv_caches[j], md)
        if not self.is_last_stage:
            return x, residual
        x, _ = self.norm(x, residual) if residual is not None else (self.norm(x), None)
        return x

    # -- weights ---------------------------------------------------------------------
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        cfg = self.cfg
        H, D = cfg.hidden_size, cfg.head_dim
        loaded: set[str] = set()
        for name, t in weights:
            n = name[len("transformer."):] if name.startswith("transformer.") else name
            if n == "lm_head.weight":
                loaded.add(name)                          # tied
                continue
            if n == "wte.weight":
                if hasattr(self, "embed_tokens"):
                    self.embed_tokens.load_weight("weight", t)
                loaded.add(name)
                continue
            if n == "wpe.weight":
                if self.is_first_stage:
                    self.wpe.weight.data.copy_(t[: self.wpe.weight.shape[0]])
                loaded.add(name)
                continue
            if n.startswith("ln_f."):
                if self.is_last_stage:
                    self.norm.load_weight(n.split(".")[-1], t)
                loaded.add(name)
                continue
            if not n.startswith("h."):
                continue
            _, idx, rest = n.split(".", 2)
            if idx not in self.layers:
                continue
            block = self.layers[idx]
            owner, _, pname = rest.rpartition(".")
            if owner == "attn.c_attn":
                q, k, v = t.split([H, D, D], dim=0)
                for part, sid in ((q, "q"), (k, "k"), (v, "v")):
                    block.attn.c_attn.load_weight(pname, part, sid)
            else:
                mod = block.get_submodule(owner)
                mod.load_weight(pname, t, None)
            loaded.add(name)
        self.finalize_weights()
        return loaded
