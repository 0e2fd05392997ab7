"""XLM-RoBERTa cross-encoder / reranker and embedding models (pooling models).

Covers what the reference adds on top of upstream BERT
(vllm_gcu/models/roberta.py:73-216): position ids recomputed per sequence from
``padding_idx`` (RoBERTa numbers real tokens from ``padding_idx + 1``), a classification head
applied on the ``<s>`` token, an embedding variant that returns the pooled hidden state, and
the jina-reranker weight-name mapping.

Pooling models have no KV cache: a batch of variable-length sequences is packed, every
sequence attends only to itself (bidirectional), and one vector or score per sequence is
returned.  ``PoolingRunner`` gives the ``LLM.encode`` / ``LLM.score`` calls.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class RobertaConfig:
    vocab_size: int = 250002
    hidden_size: int = 1024
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    intermediate_size: int = 4096
    max_position_embeddings: int = 514
    type_vocab_size: int = 1
    layer_norm_eps: float = 1e-5
    pad_token_id: int = 1
    num_labels: int = 1
    hidden_act: str = "gelu"
    dtype: torch.dtype = torch.bfloat16

    @classmethod
    def from_hf_dict(cls, d: dict, **over) -> "RobertaConfig":
        kw = {f: d[f] for f in cls.__dataclass_fields__ if f in d and f != "dtype"}
        kw.update(over)
        return cls(**kw)


def roberta_position_ids(input_ids: torch.Tensor, seq_starts: Sequence[int],
                         padding_idx: int) -> torch.Tensor:
    """Per-sequence positions ``padding_idx + 1 + i`` over the non-pad tokens; pad tokens keep
    ``padding_idx`` (vllm_gcu/models/roberta.py:73-119)."""
    pos = torch.full_like(input_ids, padding_idx)
    for s, e in zip(seq_starts[:-1], seq_starts[1:]):
        ids = input_ids[s:e]
        mask = (ids != padding_idx).long()
        pos[s:e] = torch.cumsum(mask, 0) * mask + padding_idx
    return pos


class RobertaLayer(nn.Module):
    def __init__(self, c: RobertaConfig, device):
        super().__init__()
        H, I = c.hidden_size, c.intermediate_size
        kw = dict(dtype=c.dtype, device=device)
        self.qkv = nn.Linear(H, 3 * H, **kw)
        self.attn_out = nn.Linear(H, H, **kw)
        self.attn_norm = nn.LayerNorm(H, eps=c.layer_norm_eps, **kw)
        self.fc1 = nn.Linear(H, I, **kw)
        self.fc2 = nn.Linear(I, H, **kw)
        self.out_norm = nn.LayerNorm(H, eps=c.layer_norm_eps, **kw)
        self.heads = c.num_attention_heads
        self.act = c.hidden_act

    def forward(self, x: torch.Tensor, seq_starts: Sequence[int]) -> torch.Tensor:
        T, H = x.shape
        D = H // self.heads
        qkv = self.qkv(x).view(T, 3, self.heads, D)
        outs = []
        for s, e in zip(seq_starts[:-1], seq_starts[1:]):        # block-diagonal attention
            q, k, v = (qkv[s:e, i].transpose(0, 1) for i in range(3))
            outs.append(F.scaled_dot_product_attention(q, k, v).transpose(0, 1).reshape(e - s, H))
        a = torch.cat(outs, 0) if outs else x.new_zeros(0, H)
        x = self.attn_norm(x + self.attn_out(a))
        h = self.fc1(x)
        h = F.gelu(h) if self.act == "gelu" else F.gelu(h, approximate="tanh")
        return self.out_norm(x + self.fc2(h))


class RobertaModel(nn.Module):
    def __init__(self, c: RobertaConfig, device="cpu"):
        super().__init__()
        self.cfg = c
        kw = dict(dtype=c.dtype, device=device)
        self.word_embeddings = nn.Embedding(c.vocab_size, c.hidden_size,
                                            padding_idx=c.pad_token_id, **kw)
        self.position_embeddings = nn.Embedding(c.max_position_embeddings, c.hidden_size,
                                                padding_idx=c.pad_token_id, **kw)
        self.token_type_embeddings = nn.Embedding(c.type_vocab_size, c.hidden_size, **kw)
        self.emb_norm = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps, **kw)
        self.layers = nn.ModuleList([RobertaLayer(c, device) for _ in range(c.num_hidden_layers)])

    def forward(self, input_ids: torch.Tensor, seq_starts: Sequence[int],
                token_type_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        pos = roberta_position_ids(input_ids, seq_starts, self.cfg.pad_token_id)
        tt = token_type_ids if token_type_ids is not None else torch.zeros_like(input_ids)
        x = self.word_embeddings(input_ids) + self.position_embeddings(pos) \
            + self.token_type_embeddings(tt)
        x = self.emb_norm(x)
        for layer in self.layers:
            x = layer(x, seq_starts)
        return x


_HF_LAYER_MAP = {
    "attention.output.dense": "attn_out", "attention.output.LayerNorm": "attn_norm",
    "intermediate.dense": "fc1", "output.dense": "fc2", "output.LayerNorm": "out_norm",
}


class _PoolingBase(nn.Module):
    def __init__(self, c: RobertaConfig, device="cpu"):
        super().__init__()
        self.cfg = c
        self.roberta = RobertaModel(c, device)

    def _map_name(self, name: str) -> Optional[str]:
        """HuggingFace (and jina-reranker, vllm_gcu/models/roberta.py:206-216) names ->
        parameters of this module; q / k / v are merged by ``load_weights``."""
        for pre in ("roberta.", "bert.", "model."):
            if name.startswith(pre):
                name = name[len(pre):]
        name = name.replace("emb_ln", "embeddings.LayerNorm").replace("mixer.Wqkv", "attention.qkv")
        if name.startswith("embeddings."):
            n = name[len("embeddings."):]
            n = n.replace("LayerNorm", "emb_norm")
            if n.startswith("position_ids"):
                return None
            return "roberta." + n
        if name.startswith("encoder.layer.") or name.startswith("encoder.layers."):
            parts = name.split(".")
            idx, rest = parts[2], ".".join(parts[3:])
            for k, v in _HF_LAYER_MAP.items():
                if rest.startswith(k + "."):
                    return f"roberta.layers.{idx}.{v}.{rest[len(k) + 1:]}"
            return f"roberta.layers.{idx}.{rest}"
        return name

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        params = dict(self.named_parameters())
        loaded: set[str] = set()
        H = self.cfg.hidden_size
        for name, w in weights:
            m = self._map_name(name)
            if m is None or "pooler" in m:
                continue
            done = False
            for i, proj in enumerate(("query", "key", "value")):
                tag = f"attention.self.{proj}."
                if tag in m:
                    tgt = m.replace(tag, "qkv.")
                    params[tgt].data[i * H:(i + 1) * H].copy_(w)
                    loaded.add(tgt)
                    done = True
            if done:
                continue
            m = m.replace("attention.qkv.", "qkv.")
            if m in params:
                params[m].data.copy_(w)
                loaded.add(m)
        return loaded


class XLMRobertaForSequenceClassification(_PoolingBase):
    """Cross-encoder: score = head(hidden of ``<s>``) (vllm_gcu/models/roberta.py:147-160)."""

    def __init__(self, c: RobertaConfig, device="cpu"):
        super().__init__(c, device)
        kw = dict(dtype=c.dtype, device=device)
        self.classifier = nn.ModuleDict({
            "dense": nn.Linear(c.hidden_size, c.hidden_size, **kw),
            "out_proj": nn.Linear(c.hidden_size, c.num_labels, **kw)})

    def forward(self, input_ids, seq_starts, token_type_ids=None) -> torch.Tensor:
        h = self.roberta(input_ids, seq_starts, token_type_ids)
        first = h[torch.as_tensor(list(seq_starts[:-1]), device=h.device, dtype=torch.long)]
        x = torch.tanh(self.classifier["dense"](first))
        return self.classifier["out_proj"](x).float()


class RobertaEmbeddingModel(_PoolingBase):
    """Sentence embedding: hidden state of the first token (CLS pooling), L2-normalised."""

    def forward(self, input_ids, seq_starts, token_type_ids=None) -> torch.Tensor:
        h = self.roberta(input_ids, seq_starts, token_type_ids)
        first = h[torch.as_tensor(list(seq_starts[:-1]), device=h.device, dtype=torch.long)]
        return F.normalize(first.float(), dim=-1)


class PoolingRunner:
    """Batches token-id sequences through a pooling model (``encode`` / ``score``)."""

    def __init__(self, model: _PoolingBase, device="cpu", max_batch_tokens: int = 8192):
        self.model = model.eval()
        self.device = torch.device(device)
        self.max_batch_tokens = max_batch_tokens

    @torch.inference_mode()
    def run(self, seqs: Sequence[Sequence[int]]) -> torch.Tensor:
        outs = []
        i = 0
        while i < len(seqs):
            j, tok = i, 0
            while j < len(seqs) and (j == i or tok + len(seqs[j]) <= self.max_batch_tokens):
                tok += len(seqs[j])
                j += 1
            starts = [0]
            flat: list[int] = []
            for s in seqs[i:j]:
                flat.extend(s)
                starts.append(len(flat))
            ids = torch.tensor(flat, dtype=torch.long, device=self.device)
            outs.append(self.model(ids, starts))
            i = j
        return torch.cat(outs, 0)

    def score(self, query: Sequence[int], docs: Sequence[Sequence[int]], sep_token_id: int = 2
              ) -> list[float]:
        """Cross-encoder scores of (query, doc) pairs: ``<s> q </s></s> d </s>``."""
        pairs = [list(query) + [sep_token_id] + list(d) for d in docs]
        return self.run(pairs)[:, 0].tolist()
