"""Accuracy of an embedding model on local datasets.

Two tasks (the reference runs MTEB tasks of the same two kinds through the mteb package,
benchmarks/evaluate_datasets/evaluate_embeddings.py:87-122):

* ``--task sts``: JSON-lines rows ``{"sentence1", "sentence2", "score"}``; the metric is the
  Spearman correlation between the cosine similarity of the two embeddings and the gold score.
* ``--task retrieval``: a directory with ``corpus.jsonl``, ``queries.jsonl`` and
  ``qrels/<split>.tsv``; documents are ranked by the dot product of normalised embeddings;
  NDCG / recall / MRR / MAP.

The model is a checkpoint directory of this package (an XLM-RoBERTa style encoder, or a decoder
such as gte-Qwen2, whose last-token state is the embedding) or, with ``--base-url``, a running
server's ``/v1/embeddings``.

    python benchmarks/evaluate_datasets/evaluate_embeddings.py --model /ckpt/gte-qwen2 \
        --task retrieval --dataset-dir /data/scifact [--batch-size 64] [--csv results.csv]
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Callable, Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import ir_metrics  # noqa: E402

Encoder = Callable[[Sequence[str]], np.ndarray]


def local_encoder(model_dir: str, device: str = "auto", max_len: int = 512) -> Encoder:
    """Embeds texts with a checkpoint of this package (encoder or decoder architecture)."""
    import torch
    from transformers import AutoTokenizer
    from vllm_gcu_b200.models import POOLING_ARCHITECTURES
    tok = AutoTokenizer.from_pretrained(model_dir)
    hf = json.load(open(os.path.join(model_dir, "config.json")))
    arch = (hf.get("architectures") or [""])[0]
    dev = ("cuda" if torch.cuda.is_available() else "cpu") if device == "auto" else device
    if arch in POOLING_ARCHITECTURES:
        from vllm_gcu_b200.models import build_pooling_model
        from vllm_gcu_b200.utils.weights import iter_safetensors
        runner = build_pooling_model(hf, dev)
        runner.model.load_weights(iter_safetensors(model_dir))

        def encode(texts):
            ids = [tok.encode(t, truncation=True, max_length=max_len) for t in texts]
            v = runner.run(ids).float()
            return torch.nn.functional.normalize(v, dim=-1).cpu().numpy()
        return encode
    from vllm_gcu_b200.engine.llm import LLM
    llm = LLM(model_dir, device=dev, max_model_len=max_len + 8)

    def encode(texts):
        ids = [tok.encode(t, truncation=True, max_length=max_len) for t in texts]
        return llm.embed(ids).numpy()
    return encode


def remote_encoder(base_url: str, model: str = "") -> Encoder:
    import requests

    def encode(texts):
        r = requests.post(base_url.rstrip("/") + "/v1/embeddings",
                          json={"model": model, "input": list(texts)}, timeout=3600)
        r.raise_for_status()
        data = sorted(r.json()["data"], key=lambda d: d["index"])
        v = np.asarray([d["embedding"] for d in data], dtype=np.float32)
        return v / np.maximum(np.linalg.norm(v, axis=-1, keepdims=True), 1e-12)
    return encode


def batched(encode: Encoder, texts: Sequence[str], batch_size: int) -> np.ndarray:
    out = [encode(texts[i:i + batch_size]) for i in range(0, len(texts), batch_size)]
    return np.concatenate(out, axis=0) if out else np.zeros((0, 1), dtype=np.float32)


def evaluate_sts(encode: Encoder, rows: Sequence[dict], batch_size: int = 64) -> dict:
    a = batched(encode, [r["sentence1"] for r in rows], batch_size)
    b = batched(encode, [r["sentence2"] for r in rows], batch_size)
    cos = (a * b).sum(-1) / np.maximum(np.linalg.norm(a, axis=-1) * np.linalg.norm(b, axis=-1),
                                       1e-12)
    return {"cosine_spearman": ir_metrics.spearman(cos, [float(r["score"]) for r in rows]),
            "pairs": float(len(rows))}


def evaluate_retrieval(encode: Encoder, corpus: dict, queries: dict, qrels: dict,
                       batch_size: int = 64, top_k: int = 100) -> dict:
    doc_ids, q_ids = list(corpus), list(queries)
    d = batched(encode, [corpus[i] for i in doc_ids], batch_size)
    q = batched(encode, [queries[i] for i in q_ids], batch_size)
    sims = q @ d.T
    results = {}
    for qi, row in zip(q_ids, sims):
        top = np.argsort(-row, kind="stable")[:top_k]
        results[qi] = {doc_ids[j]: float(row[j]) for j in top}
    return ir_metrics.evaluate_rankings(results, qrels)


def main(argv: Optional[Sequence[str]] = None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default=None)
    ap.add_argument("--base-url", default=None, help="use a running server's /v1/embeddings")
    ap.add_argument("--task", choices=["sts", "retrieval"], required=True)
    ap.add_argument("--dataset", default=None, help="JSON-lines file (sts)")
    ap.add_argument("--dataset-dir", default=None, help="retrieval dataset directory")
    ap.add_argument("--eval-split", default="test")
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--csv", default=None)
    ap.add_argument("--save-output", default=None)
    a = ap.parse_args(argv)
    encode = remote_encoder(a.base_url, a.model or "") if a.base_url else \
        local_encoder(a.model, a.device)
    if a.task == "sts":
        rows = [json.loads(x) for x in open(a.dataset) if x.strip()]
        metrics = evaluate_sts(encode, rows, a.batch_size)
    else:
        metrics = evaluate_retrieval(encode, *ir_metrics.load_retrieval_dataset(
            a.dataset_dir, a.eval_split), batch_size=a.batch_size)
    print(json.dumps(metrics, indent=1))
    if a.csv:
        ir_metrics.save_csv(a.csv, vars(a), metrics)
    if a.save_output:
        with open(a.save_output, "w") as f:
            json.dump(metrics, f, indent=1)
    return metrics


if __name__ == "__main__":
    main()
