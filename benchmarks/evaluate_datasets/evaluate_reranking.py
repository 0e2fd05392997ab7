"""Accuracy of a cross-encoder reranker on a retrieval dataset (``corpus.jsonl``,
``queries.jsonl``, ``qrels/<split>.tsv``): BM25 retrieves ``--initial-top-k`` documents per
query, the reranker re-orders the first ``--rerank-top-k`` of them, and the ranking metrics are
reported before and after (the flow of benchmarks/evaluate_datasets/evaluate_reranking.py:96-123
of the reference).

The reranker is a checkpoint directory of this package (XLM-RoBERTa sequence classification,
e.g. jina-reranker-v2 / bge-reranker) or, with ``--base-url``, a running server's ``/rerank``.

    python benchmarks/evaluate_datasets/evaluate_reranking.py --model /ckpt/bge-reranker \
        --dataset-dir /data/scifact --rerank-top-k 100 [--csv results.csv]
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Callable, Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import ir_metrics  # noqa: E402

Reranker = Callable[[str, Sequence[str]], Sequence[float]]


def local_reranker(model_dir: str, device: str = "auto", max_len: int = 512) -> Reranker:
    import torch
    from transformers import AutoTokenizer
    from vllm_gcu_b200.models import build_pooling_model
    from vllm_gcu_b200.utils.weights import iter_safetensors
    tok = AutoTokenizer.from_pretrained(model_dir)
    hf = json.load(open(os.path.join(model_dir, "config.json")))
    dev = ("cuda" if torch.cuda.is_available() else "cpu") if device == "auto" else device
    runner = build_pooling_model(hf, dev)
    runner.model.load_weights(iter_safetensors(model_dir))

    def rerank(query, docs):
        pairs = [tok.encode(query, d, truncation=True, max_length=max_len) for d in docs]
        return runner.run(pairs)[:, 0].float().tolist()
    return rerank


def remote_reranker(base_url: str, model: str = "") -> Reranker:
    import requests

    def rerank(query, docs):
        r = requests.post(base_url.rstrip("/") + "/rerank",
                          json={"model": model, "query": query, "documents": list(docs)},
                          timeout=3600)
        r.raise_for_status()
        scores = [0.0] * len(docs)
        for item in r.json()["results"]:
            scores[item["index"]] = float(item["relevance_score"])
        return scores
    return rerank


def evaluate(rerank: Reranker, corpus: dict, queries: dict, qrels: dict,
             initial_top_k: int = 1000, rerank_top_k: int = 100) -> tuple[dict, dict]:
    bm25 = ir_metrics.BM25(corpus)
    initial, reranked = {}, {}
    for qid, text in queries.items():
        first = bm25.top(text, initial_top_k)
        initial[qid] = first
        ids = list(first)[:rerank_top_k]
        scores = rerank(text, [corpus[d] for d in ids]) if ids else []
        reranked[qid] = {d: float(s) for d, s in zip(ids, scores)}
    return (ir_metrics.evaluate_rankings(initial, qrels),
            ir_metrics.evaluate_rankings(reranked, qrels))


def main(argv: Optional[Sequence[str]] = None) -> tuple[dict, dict]:
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default=None)
    ap.add_argument("--base-url", default=None, help="use a running server's /rerank")
    ap.add_argument("--dataset-dir", required=True)
    ap.add_argument("--eval-split", default="test")
    ap.add_argument("--initial-top-k", type=int, default=1000)
    ap.add_argument("--rerank-top-k", type=int, default=100)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--csv", default=None)
    a = ap.parse_args(argv)
    rerank = remote_reranker(a.base_url, a.model or "") if a.base_url else \
        local_reranker(a.model, a.device)
    first, second = evaluate(rerank, *ir_metrics.load_retrieval_dataset(a.dataset_dir,
                                                                        a.eval_split),
                             initial_top_k=a.initial_top_k, rerank_top_k=a.rerank_top_k)
    print(json.dumps({"bm25": first, "reranked": second}, indent=1))
    if a.csv:
        ir_metrics.save_csv(a.csv, vars(a), second)
    return first, second


if __name__ == "__main__":
    main()
