"""Ranking metrics, an Okapi BM25 first-stage retriever and a loader for retrieval datasets
in the common ``corpus.jsonl`` / ``queries.jsonl`` / ``qrels/<split>.tsv`` layout, shared by
``evaluate_embeddings.py`` and ``evaluate_reranking.py``.  Self-contained: the reference's
evaluators delegate these to the mteb / beir / rank_bm25 packages
(benchmarks/evaluate_datasets/evaluate_embeddings.py:108-120, evaluate_reranking.py:72-123),
which need network access for their datasets."""
from __future__ import annotations

import csv
import json
import math
import os
from collections import Counter
from typing import Iterable, Mapping, Sequence

import numpy as np


def load_retrieval_dataset(directory: str, split: str = "test"):
    """(corpus {id: text}, queries {id: text}, qrels {query id: {doc id: relevance}})."""
    def rows(path):
        with open(path, encoding="utf-8") as f:
            for line in f:
                if line.strip():
                    yield json.loads(line)

    corpus = {str(r["_id"]): ((r.get("title") or "") + " " + r.get("text", "")).strip()
              for r in rows(os.path.join(directory, "corpus.jsonl"))}
    queries = {str(r["_id"]): r["text"] for r in rows(os.path.join(directory, "queries.jsonl"))}
    qrels: dict[str, dict[str, int]] = {}
    with open(os.path.join(directory, "qrels", split + ".tsv"), encoding="utf-8") as f:
        for i, row in enumerate(csv.reader(f, delimiter="\t")):
            if i == 0 and not row[-1].lstrip("-").isdigit():
                continue                                  # header line
            qrels.setdefault(str(row[0]), {})[str(row[1])] = int(row[-1])
    queries = {q: t for q, t in queries.items() if q in qrels}
    return corpus, queries, qrels


def ndcg_at_k(ranked: Sequence[str], rel: Mapping[str, int], k: int) -> float:
    dcg = sum((2 ** rel.get(d, 0) - 1) / math.log2(i + 2) for i, d in enumerate(ranked[:k]))
    ideal = sorted(rel.values(), reverse=True)[:k]
    idcg = sum((2 ** r - 1) / math.log2(i + 2) for i, r in enumerate(ideal))
    return dcg / idcg if idcg > 0 else 0.0


def mrr_at_k(ranked: Sequence[str], rel: Mapping[str, int], k: int) -> float:
    for i, d in enumerate(ranked[:k]):
        if rel.get(d, 0) > 0:
            return 1.0 / (i + 1)
    return 0.0


def recall_at_k(ranked: Sequence[str], rel: Mapping[str, int], k: int) -> float:
    pos = {d for d, r in rel.items() if r > 0}
    return len(pos & set(ranked[:k])) / len(pos) if pos else 0.0


def average_precision(ranked: Sequence[str], rel: Mapping[str, int]) -> float:
    pos = {d for d, r in rel.items() if r > 0}
    hits, total = 0, 0.0
    for i, d in enumerate(ranked):
        if d in pos:
            hits += 1
            total += hits / (i + 1)
    return total / len(pos) if pos else 0.0


def evaluate_rankings(results: Mapping[str, Mapping[str, float]],
                      qrels: Mapping[str, Mapping[str, int]], ks: Iterable[int] = (1, 10, 100)
                      ) -> dict[str, float]:
    """Means over the queries of ``qrels`` (a query without results scores zero)."""
    ks = list(ks)
    sums: Counter = Counter()
    for q, rel in qrels.items():
        scored = results.get(q, {})
        ranked = [d for d, _ in sorted(scored.items(), key=lambda kv: (-kv[1], kv[0]))]
        for k in ks:
            sums[f"ndcg@{k}"] += ndcg_at_k(ranked, rel, k)
            sums[f"recall@{k}"] += recall_at_k(ranked, rel, k)
        sums["mrr@10"] += mrr_at_k(ranked, rel, 10)
        sums["map"] += average_precision(ranked, rel)
    n = max(1, len(qrels))
    return {k: v / n for k, v in sorted(sums.items())}


def spearman(a: Sequence[float], b: Sequence[float]) -> float:
    """Rank correlation with average ranks for ties."""
    def ranks(x):
        x = np.asarray(x, dtype=np.float64)
        order = np.argsort(x, kind="stable")
        r = np.empty(len(x))
        i = 0
        while i < len(x):
            j = i
            while j + 1 < len(x) and x[order[j + 1]] == x[order[i]]:
                j += 1
            r[order[i:j + 1]] = (i + j) / 2.0 + 1.0
            i = j + 1
        return r
    ra, rb = ranks(a), ranks(b)
    ra, rb = ra - ra.mean(), rb - rb.mean()
    den = math.sqrt(float((ra * ra).sum() * (rb * rb).sum()))
    return float((ra * rb).sum() / den) if den > 0 else 0.0


class BM25:
    """Okapi BM25 over whitespace tokens (lower-cased)."""

    def __init__(self, docs: Mapping[str, str], k1: float = 1.5, b: float = 0.75):
        self.ids = list(docs)
        toks = [docs[d].lower().split() for d in self.ids]
        self.len = np.array([len(t) for t in toks], dtype=np.float64)
        self.avg = float(self.len.mean()) if len(toks) else 0.0
        self.k1, self.b = k1, b
        self.postings: dict[str, list[tuple[int, int]]] = {}
        for i, t in enumerate(toks):
            for w, c in Counter(t).items():
                self.postings.setdefault(w, []).append((i, c))
        n = len(toks)
        self.idf = {w: math.log(1.0 + (n - len(p) + 0.5) / (len(p) + 0.5))
                    for w, p in self.postings.items()}

    def scores(self, query: str) -> np.ndarray:
        out = np.zeros(len(self.ids))
        for w in set(query.lower().split()):
            post = self.postings.get(w)
            if not post:
                continue
            idx = np.array([i for i, _ in post])
            tf = np.array([c for _, c in post], dtype=np.float64)
            norm = tf + self.k1 * (1.0 - self.b + self.b * self.len[idx] / max(self.avg, 1e-9))
            out[idx] += self.idf[w] * tf * (self.k1 + 1.0) / norm
        return out

    def top(self, query: str, k: int) -> dict[str, float]:
        s = self.scores(query)
        order = np.argsort(-s, kind="stable")[:k]
        return {self.ids[i]: float(s[i]) for i in order}


def save_csv(path: str, args: Mapping[str, object], metrics: Mapping[str, float]) -> None:
    """Appends one row with the arguments and the metrics (header on first use)."""
    row = {**{f"arg_{k}": v for k, v in args.items()},
           **{f"metric_{k}": f"{v:.4f}" for k, v in metrics.items()}}
    new = not os.path.exists(path)
    with open(path, "a", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(row))
        if new:
            w.writeheader()
        w.writerow(row)
