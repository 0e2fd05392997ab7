"""Performance + accuracy tool with fixed request shapes (the role of the reference's
benchmarks/benchmark_test.py: ``--perf`` prefill / decode latency per token, :547-589;
``--acc`` ROUGE-L of the outputs against references, :592-621; CSV export).

  python benchmarks/benchmark_test.py --model tiny-llama --device cpu --perf \
      --input-len 64 --output-len 16 --num-prompts 8 --save-output out.csv
  python benchmarks/benchmark_test.py --model tiny-llama --device cpu --acc \
      --reference-file refs.jsonl        # lines: {"prompt_token_ids": [...], "reference": [...]}
"""
import argparse
import csv
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from vllm_gcu_b200.engine.llm import LLM  # noqa: E402
from vllm_gcu_b200.engine.request import SamplingParams  # noqa: E402


def rouge_l(hyp, ref) -> float:
    """F-measure of the longest common subsequence of two token sequences."""
    if not hyp or not ref:
        return 0.0
    prev = [0] * (len(ref) + 1)
    for h in hyp:
        cur = [0]
        for j, r in enumerate(ref):
            cur.append(prev[j] + 1 if h == r else max(prev[j + 1], cur[j]))
        prev = cur
    lcs = prev[-1]
    if lcs == 0:
        return 0.0
    p, r = lcs / len(hyp), lcs / len(ref)
    return 2 * p * r / (p + r)


def run_perf(llm, a):
    V = llm.engine.cfg.model.vocab_size
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, V, (a.num_prompts, a.input_len), generator=g).tolist()
    sync = torch.cuda.synchronize if torch.cuda.is_available() else (lambda: None)
    one = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
    full = SamplingParams(max_tokens=a.output_len, temperature=0.0, ignore_eos=True)
    llm.generate(prompts[:1], one)                       # warm-up
    sync()
    t0 = time.perf_counter()
    llm.generate(prompts, one)
    sync()
    t_prefill = time.perf_counter() - t0
    llm.engine.scheduler.kv.pool.reset_prefix_cache()
    t0 = time.perf_counter()
    outs = llm.generate(prompts, full)
    sync()
    t_total = time.perf_counter() - t0
    n_out = sum(len(o.outputs[0].token_ids) for o in outs)
    decode_s = max(t_total - t_prefill, 1e-9)
    return {"num_prompts": a.num_prompts, "input_len": a.input_len, "output_len": a.output_len,
            "prefill_latency_per_token_ms": t_prefill / (a.num_prompts * a.input_len) * 1e3,
            "decode_latency_per_token_ms": decode_s / max(a.output_len - 1, 1) * 1e3,
            "output_tokens_per_s": n_out / t_total, "total_s": t_total}, outs


def run_acc(llm, a):
    rows = [json.loads(l) for l in open(a.reference_file) if l.strip()]
    sp = SamplingParams(max_tokens=a.output_len, temperature=0.0)
    outs = llm.generate([r["prompt_token_ids"] for r in rows], sp)
    scores = [rouge_l(o.outputs[0].token_ids, r["reference"]) for o, r in zip(outs, rows)]
    return {"rouge_l": sum(scores) / max(len(scores), 1), "samples": len(scores)}, outs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=128)
    ap.add_argument("--num-prompts", type=int, default=8)
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--perf", action="store_true")
    ap.add_argument("--acc", action="store_true")
    ap.add_argument("--reference-file", default=None)
    ap.add_argument("--dump-reference", default=None,
                    help="write this run's greedy outputs as a reference file for --acc (e.g. "
                         "from the unquantised model, to score a quantised or sharded one)")
    ap.add_argument("--save-output", default=None, help="CSV file for the metrics")
    ap.add_argument("--dtype", default=None)
    a = ap.parse_args()
    llm = LLM(a.model, device=a.device, tensor_parallel_size=a.tensor_parallel_size,
              max_num_seqs=a.max_num_seqs, dtype=a.dtype,
              max_model_len=a.input_len + a.output_len + 16)
    res = {}
    if a.perf or not (a.acc or a.dump_reference):
        res.update(run_perf(llm, a)[0])
    if a.dump_reference:
        import torch
        g = torch.Generator().manual_seed(0)
        vocab = llm.engine.cfg.model.vocab_size
        prompts = torch.randint(10, vocab, (a.num_prompts, a.input_len), generator=g).tolist()
        outs = llm.generate(prompts, SamplingParams(max_tokens=a.output_len, temperature=0.0))
        with open(a.dump_reference, "w") as f:
            for p_, o in zip(prompts, outs):
                f.write(json.dumps({"prompt_token_ids": p_,
                                    "reference": o.outputs[0].token_ids}) + "\n")
        res["reference_rows"] = len(prompts)
    if a.acc:
        assert a.reference_file, "--acc needs --reference-file"
        res.update(run_acc(llm, a)[0])
    print(json.dumps(res, indent=1))
    if a.save_output:
        with open(a.save_output, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(list(res))
            w.writerow(list(res.values()))


if __name__ == "__main__":
    main()
