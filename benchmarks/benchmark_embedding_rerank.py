"""Embedding / rerank throughput of the pooling models (the reference ships
benchmarks/benchmark_embedding_rerank.py): sequences per second for ``encode`` and pairs per
second for ``score``.

  python benchmarks/benchmark_embedding_rerank.py --task rerank --num-docs 64 --doc-len 128
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from vllm_gcu_b200.models import build_pooling_model  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--task", choices=["embed", "rerank"], default="rerank")
    ap.add_argument("--config", default=None, help="HF config.json of the pooling model")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--num-docs", type=int, default=256)
    ap.add_argument("--doc-len", type=int, default=256)
    ap.add_argument("--query-len", type=int, default=16)
    ap.add_argument("--layers", type=int, default=0)
    a = ap.parse_args()
    if a.config:
        cfg = json.load(open(a.config))
    else:
        cfg = {"architectures": ["XLMRobertaForSequenceClassification" if a.task == "rerank"
                                 else "XLMRobertaModel"], "vocab_size": 250002,
               "hidden_size": 1024, "num_hidden_layers": 24, "num_attention_heads": 16,
               "intermediate_size": 4096, "max_position_embeddings": 8194}
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    dtype = torch.bfloat16 if a.device == "cuda" else torch.float32
    runner = build_pooling_model(cfg, a.device, dtype)
    g = torch.Generator().manual_seed(0)
    V = cfg["vocab_size"]
    docs = torch.randint(5, V, (a.num_docs, a.doc_len), generator=g).tolist()
    query = torch.randint(5, V, (a.query_len,), generator=g).tolist()
    fn = (lambda: runner.score(query, docs)) if a.task == "rerank" else (lambda: runner.run(docs))
    fn()
    if a.device == "cuda":
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    fn()
    if a.device == "cuda":
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    print(json.dumps({"task": a.task, "sequences": a.num_docs, "seconds": dt,
                      "sequences_per_s": a.num_docs / dt}))


if __name__ == "__main__":
    main()
