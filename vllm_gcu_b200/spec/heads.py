"""Draft heads that propose tokens from the target model's last hidden state: Medusa heads
and the MLP speculator.  Both run inside the model runner right after the target step, on the
hidden row of the last accepted token of every request, and their drafts are verified by the
rejection sampler in the next step (the reference builds vLLM's Medusa / MLPSpeculator
workers into its spec-decode worker, vllm_gcu/worker/spec_decode/spec_decode_worker.py:135-173).

Checkpoint layouts follow the public ones: Medusa ``blocks.{i}.layers.{j}.{weight,bias}`` +
``lm_heads.{i}.weight``; MLP speculator ``emb.{i}.weight``, ``proj.{i}.weight``,
``ln.{i}.{weight,bias}``, ``head.{i}.weight``.
"""
from __future__ import annotations

import math
from typing import Iterable

import torch
import torch.nn as nn
import torch.nn.functional as F


class MedusaProposer(nn.Module):
    """``k`` independent heads; head i predicts the token ``i + 1`` positions after the one
    the target model has just produced: ``lm_head_i(h + SiLU(W_i h + b_i))`` (one residual
    block per head by default)."""

    def __init__(self, hidden_size: int, vocab_size: int, num_heads: int, num_layers: int = 1,
                 dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.k = num_heads
        kw = dict(dtype=dtype, device=device)
        self.blocks = nn.ModuleList([
            nn.ModuleList([nn.Linear(hidden_size, hidden_size, **kw) for _ in range(num_layers)])
            for _ in range(num_heads)])
        self.lm_heads = nn.ModuleList([nn.Linear(hidden_size, vocab_size, bias=False, **kw)
                                       for _ in range(num_heads)])

    @torch.inference_mode()
    def propose(self, hidden: torch.Tensor, last_tokens: torch.Tensor) -> torch.Tensor:
        """hidden ``[n, H]`` (final-norm output of the last accepted position), returns
        ``[n, k]`` int64 draft ids (greedy per head)."""
        outs = []
        for blocks, head in zip(self.blocks, self.lm_heads):
            h = hidden
            for lin in blocks:
                h = h + F.silu(lin(h))
            outs.append(head(h).float().argmax(-1))
        return torch.stack(outs, dim=1)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            tgt = name.replace("blocks.", "blocks.").replace(".layers.", ".")
            if tgt in params and params[tgt].shape == w.shape:
                params[tgt].data.copy_(w)
                loaded.add(name)
        return loaded

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        g = torch.Generator(device="cpu").manual_seed(seed)
        for p in self.parameters():
            p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))


class MLPSpeculatorProposer(nn.Module):
    """Chain of ``k`` small predictors: ``state_i = act(LN_i(w_s * proj_i(state_{i-1}) +
    w_e * emb_i(token_{i-1})))``, ``token_i = argmax head_i(state_i)``; the first state is the
    target's hidden state and the first token the one it has just produced."""

    def __init__(self, hidden_size: int, vocab_size: int, num_predict: int, inner_dim: int = 0,
                 dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.k = num_predict
        inner = inner_dim or hidden_size
        kw = dict(dtype=dtype, device=device)
        self.emb = nn.ModuleList([nn.Embedding(vocab_size, inner, **kw) for _ in range(num_predict)])
        self.proj = nn.ModuleList([nn.Linear(hidden_size if i == 0 else inner, inner, bias=False,
                                             **kw) for i in range(num_predict)])
        self.ln = nn.ModuleList([nn.LayerNorm(inner, **kw) for _ in range(num_predict)])
        self.head = nn.ModuleList([nn.Linear(inner, vocab_size, bias=False, **kw)
                                   for _ in range(num_predict)])
        self.state_weight = 0.5 ** (0.5 / num_predict)
        self.emb_weight = math.sqrt((1 - self.state_weight ** 2) * (inner / 2))

    @torch.inference_mode()
    def propose(self, hidden: torch.Tensor, last_tokens: torch.Tensor) -> torch.Tensor:
        state, tok = hidden, last_tokens.long()
        outs = []
        for i in range(self.k):
            z = self.emb[i](tok)
            state = self.proj[i](state)
            state = torch.add(state, z, alpha=self.emb_weight / self.state_weight)
            state = F.gelu(self.ln[i](state))
            tok = self.head[i](state).float().argmax(-1)
            outs.append(tok)
        return torch.stack(outs, dim=1)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        params = dict(self.named_parameters())
        loaded = set()
        for name, w in weights:
            tgt = name[len("speculator."):] if name.startswith("speculator.") else name
            if tgt in params and params[tgt].shape == w.shape:
                params[tgt].data.copy_(w)
                loaded.add(name)
        return loaded

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        g = torch.Generator(device="cpu").manual_seed(seed)
        for n, p in self.named_parameters():
            if n.startswith("ln.") and n.endswith("weight"):
                p.fill_(1.0)
            elif n.startswith("ln."):
                p.zero_()
            else:
                p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
