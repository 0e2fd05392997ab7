"""Small-dataset accuracy harness for the built-in engine.

What the reference's ``benchmarks/evaluate_datasets/run.py`` does through OpenCompass (MMLU /
C-Eval style multiple choice scored by perplexity, HumanEval / GSM8K style generation scored
by a post-processed match; ``evaluate_datasets/README.md:5-13``), reduced to what runs without
network access: datasets are local JSON-lines files, the model is any checkpoint directory or
architecture preset of this package.

Dataset rows:
  multiple choice  {"question": "...", "choices": ["...", ...], "answer": 2}
  generation       {"prompt": "...", "reference": "..."}

    python benchmarks/evaluate_datasets/run.py --model /ckpt/qwen3 --dataset mmlu.jsonl \
        --mode ppl [--limit 200] [--csv results.csv]

``--mode ppl``: every choice is appended to the question and scored by the mean
log-probability of its tokens (``prompt_logprobs``); the best-scoring choice is the prediction.
``--mode gen``: greedy generation; a row counts when the normalised reference occurs in the
normalised output (``--match exact`` demands equality).  Results are appended to a CSV with the
arguments, as the reference's evaluators do (evaluate_reranking.py:24-53).
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import re
import sys
import time
from typing import Optional, Sequence

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def load_rows(path: str, limit: Optional[int] = None) -> list[dict]:
    rows = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line:
                rows.append(json.loads(line))
            if limit and len(rows) >= limit:
                break
    return rows


def normalise(text: str) -> str:
    return re.sub(r"\s+", " ", re.sub(r"[^\w\s]", " ", text.lower())).strip()


def score_choices(llm, tokenizer, question: str, choices: Sequence[str]) -> list[float]:
    """Mean log-probability of each choice's tokens given the question."""
    from vllm_gcu_b200.engine.request import SamplingParams
    q_ids = list(tokenizer.encode(question))
    prompts, spans = [], []
    for c in choices:
        c_ids = list(tokenizer.encode(" " + c))
        prompts.append(q_ids + c_ids)
        spans.append((len(q_ids), len(q_ids) + len(c_ids)))
    sp = SamplingParams(max_tokens=1, temperature=0.0, prompt_logprobs=0, ignore_eos=True)
    outs = llm.generate(prompts, sp)
    scores = []
    for o, ids, (a, b) in zip(outs, prompts, spans):
        lps = o.prompt_logprobs or []
        tot = 0.0
        for pos in range(a, b):
            d = lps[pos] if pos < len(lps) and lps[pos] is not None else {}
            tot += d.get(ids[pos], -1e4)
        scores.append(tot / max(1, b - a))
    return scores


def evaluate(llm, tokenizer, rows: list[dict], mode: str, max_tokens: int = 64,
             match: str = "contains") -> dict:
    from vllm_gcu_b200.engine.request import SamplingParams
    correct = 0
    t0 = time.time()
    if mode == "ppl":
        for r in rows:
            sc = score_choices(llm, tokenizer, r["question"], r["choices"])
            correct += int(max(range(len(sc)), key=sc.__getitem__) == int(r["answer"]))
    else:
        sp = SamplingParams(max_tokens=max_tokens, temperature=0.0)
        outs = llm.generate([list(tokenizer.encode(r["prompt"])) for r in rows], sp)
        for r, o in zip(rows, outs):
            text = normalise(tokenizer.decode(list(o.outputs[0].token_ids)))
            ref = normalise(r["reference"])
            correct += int(text == ref if match == "exact" else ref in text)
    n = max(1, len(rows))
    return {"accuracy": correct / n, "correct": correct, "total": len(rows),
            "seconds": round(time.time() - t0, 2)}


def save_csv(path: str, args: argparse.Namespace, metrics: dict) -> None:
    row = {"timestamp": time.strftime("%Y-%m-%d %H:%M:%S")}
    row.update({f"arg_{k}": str(v) for k, v in vars(args).items()})
    row.update({f"metric_{k}": v for k, v in metrics.items()})
    new = not os.path.isfile(path)
    with open(path, "a", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(row.keys()))
        if new:
            w.writeheader()
        w.writerow(row)


def main(argv: Optional[Sequence[str]] = None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", required=True)
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--mode", choices=["ppl", "gen"], default="ppl")
    ap.add_argument("--match", choices=["contains", "exact"], default="contains")
    ap.add_argument("--limit", type=int, default=0)
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--max-model-len", type=int, default=2048)
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--device", default="auto")
    ap.add_argument("--csv", default="")
    args = ap.parse_args(argv)
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.entrypoints.api_server import load_tokenizer
    llm = LLM(args.model, tensor_parallel_size=args.tensor_parallel_size, device=args.device,
              max_model_len=args.max_model_len, max_num_seqs=64,
              max_num_batched_tokens=min(8192, args.max_model_len * 4))
    tok = load_tokenizer(args.model if os.path.isdir(args.model) else None,
                         llm.engine.cfg.model.vocab_size)
    metrics = evaluate(llm, tok, load_rows(args.dataset, args.limit or None), args.mode,
                       args.max_tokens, args.match)
    print(json.dumps(metrics))
    if args.csv:
        save_csv(args.csv, args, metrics)
    return metrics


if __name__ == "__main__":
    main()
