"""Embedding / reranking quality on a local BEIR-style dataset (the reference's
``evaluate_embeddings.py`` / ``evaluate_reranking.py``: nDCG@k, MRR@k, recall@k over corpus,
queries and relevance judgements; benchmarks/evaluate_datasets/evaluate_reranking.py:56-192).

Files (JSON lines): corpus ``{"_id", "text"}``, queries ``{"_id", "text"}``, qrels
``{"query_id", "corpus_id", "score"}``.

    python benchmarks/evaluate_datasets/retrieval.py --model /ckpt/bge-m3 --task embed \
        --corpus corpus.jsonl --queries queries.jsonl --qrels qrels.jsonl --k 10

``--task embed``: cosine similarity of pooled embeddings ranks the whole corpus.
``--task rerank``: a cross-encoder checkpoint scores (query, document) pairs for the
``--candidates`` documents a lexical first stage (token-overlap BM25) retrieved.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
from collections import Counter, defaultdict
from typing import Optional, Sequence

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def ndcg_at_k(ranked: Sequence[str], rel: dict[str, int], k: int) -> float:
    dcg = sum((2 ** rel.get(d, 0) - 1) / math.log2(i + 2) for i, d in enumerate(ranked[:k]))
    ideal = sorted(rel.values(), reverse=True)[:k]
    idcg = sum((2 ** r - 1) / math.log2(i + 2) for i, r in enumerate(ideal))
    return dcg / idcg if idcg > 0 else 0.0


def mrr_at_k(ranked: Sequence[str], rel: dict[str, int], k: int) -> float:
    for i, d in enumerate(ranked[:k]):
        if rel.get(d, 0) > 0:
            return 1.0 / (i + 1)
    return 0.0


def recall_at_k(ranked: Sequence[str], rel: dict[str, int], k: int) -> float:
    pos = {d for d, r in rel.items() if r > 0}
    return len(pos & set(ranked[:k])) / len(pos) if pos else 0.0


def bm25_rank(query: str, docs: dict[str, str], n: int, k1: float = 1.5, b: float = 0.75
              ) -> list[str]:
    toks = {d: t.lower().split() for d, t in docs.items()}
    avg = sum(len(t) for t in toks.values()) / max(1, len(toks))
    df = Counter(w for t in toks.values() for w in set(t))
    N = len(toks)
    scores = {}
    for d, t in toks.items():
        tf = Counter(t)
        s = 0.0
        for w in query.lower().split():
            if w in tf:
                idf = math.log(1 + (N - df[w] + 0.5) / (df[w] + 0.5))
                s += idf * tf[w] * (k1 + 1) / (tf[w] + k1 * (1 - b + b * len(t) / avg))
        scores[d] = s
    return sorted(scores, key=scores.get, reverse=True)[:n]


def summarise(rankings: dict[str, list[str]], qrels: dict[str, dict[str, int]], k: int) -> dict:
    qs = [q for q in rankings if q in qrels]
    n = max(1, len(qs))
    return {f"ndcg@{k}": sum(ndcg_at_k(rankings[q], qrels[q], k) for q in qs) / n,
            f"mrr@{k}": sum(mrr_at_k(rankings[q], qrels[q], k) for q in qs) / n,
            f"recall@{k}": sum(recall_at_k(rankings[q], qrels[q], k) for q in qs) / n,
            "queries": len(qs)}


def _jsonl(path: str) -> list[dict]:
    return [json.loads(line) for line in open(path) if line.strip()]


def main(argv: Optional[Sequence[str]] = None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", required=True)
    ap.add_argument("--task", choices=["embed", "rerank"], default="embed")
    ap.add_argument("--corpus", required=True)
    ap.add_argument("--queries", required=True)
    ap.add_argument("--qrels", required=True)
    ap.add_argument("--k", type=int, default=10)
    ap.add_argument("--candidates", type=int, default=100)
    ap.add_argument("--device", default="auto")
    args = ap.parse_args(argv)
    import torch
    from vllm_gcu_b200.entrypoints.api_server import load_tokenizer
    from vllm_gcu_b200.models import build_pooling_model
    from vllm_gcu_b200.utils.weights import iter_safetensors
    hf = json.load(open(os.path.join(args.model, "config.json")))
    dev = ("cuda" if torch.cuda.is_available() else "cpu") if args.device == "auto" else args.device
    runner = build_pooling_model(hf, dev)
    runner.model.load_weights(iter_safetensors(args.model))
    tok = load_tokenizer(args.model, int(hf.get("vocab_size", 0)))
    corpus = {r["_id"]: r["text"] for r in _jsonl(args.corpus)}
    queries = {r["_id"]: r["text"] for r in _jsonl(args.queries)}
    qrels: dict[str, dict[str, int]] = defaultdict(dict)
    for r in _jsonl(args.qrels):
        qrels[r["query_id"]][r["corpus_id"]] = int(r["score"])
    rankings: dict[str, list[str]] = {}
    if args.task == "embed":
        ids = list(corpus)
        dv = torch.nn.functional.normalize(
            runner.run([list(tok.encode(corpus[d])) for d in ids]).float(), dim=-1)
        for q, text in queries.items():
            qv = torch.nn.functional.normalize(runner.run([list(tok.encode(text))]).float(), dim=-1)
            order = (dv @ qv[0]).argsort(descending=True)[: args.k].tolist()
            rankings[q] = [ids[i] for i in order]
    else:
        for q, text in queries.items():
            cand = bm25_rank(text, corpus, args.candidates)
            scores = runner.score(list(tok.encode(text)), [list(tok.encode(corpus[d])) for d in cand])
            order = sorted(range(len(cand)), key=lambda i: float(scores[i]), reverse=True)
            rankings[q] = [cand[i] for i in order]
    out = summarise(rankings, qrels, args.k)
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
