"""Every benchmark / example tool runs from its command line on the CPU engine (tiny models)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CASES = {
    "latency": ["benchmark_latency.py", "--model", "tiny-llama", "--device", "cpu", "--batch-size",
                "2", "--input-len", "16", "--output-len", "4", "--num-iters-warmup", "1",
                "--num-iters", "2"],
    "prefix_caching": ["benchmark_prefix_caching.py", "--model", "tiny-llama", "--device", "cpu",
                       "--prefix-len", "32", "--suffix-len", "8", "--num-prompts", "4",
                       "--output-len", "2", "--dtype", "float32"],
    "perf_tool": ["benchmark_test.py", "--model", "tiny-llama", "--device", "cpu", "--input-len",
                  "16", "--output-len", "4", "--num-prompts", "2", "--perf", "--dtype", "float32"],
    "embed": ["benchmark_embedding_rerank.py", "--task", "embed", "--device", "cpu", "--num-docs",
              "4", "--doc-len", "16", "--query-len", "8", "--layers", "1"],
    "rerank": ["benchmark_embedding_rerank.py", "--task", "rerank", "--device", "cpu",
               "--num-docs", "4", "--doc-len", "16", "--query-len", "8", "--layers", "1"],
    "example_spec": ["offline_inference_examples.py", "--model", "tiny-llama", "--device", "cpu",
                     "spec"],
    "example_lora": ["offline_inference_examples.py", "--model", "tiny-llama", "--device", "cpu",
                     "lora"],
    "throughput": ["benchmark_throughput.py", "--model", "tiny-llama", "--device", "cpu",
                   "--num-prompts", "4", "--input-len", "16", "--output-len", "4",
                   "--max-num-seqs", "4", "--max-num-batched-tokens", "64"],
    "offline_dp": ["dpllm.py", "--model", "tiny-qwen3-moe", "--dp", "2", "--device", "cpu",
                   "--num-prompts", "4", "--input-len", "8", "--output-len", "3",
                   "--expert-parallel"],
}


@pytest.mark.timeout(300)
def test_accuracy_mode_scores_against_a_dumped_reference(tmp_path):
    """``benchmark_test.py``: outputs dumped by one configuration are the ROUGE-L reference of
    another (here the same one: score 1)."""
    ref = str(tmp_path / "ref.jsonl")
    common = ["--model", "tiny-llama", "--device", "cpu", "--input-len", "16", "--output-len",
              "6", "--num-prompts", "3", "--dtype", "float32"]
    tool = os.path.join(ROOT, "benchmarks", "benchmark_test.py")
    r = subprocess.run([sys.executable, tool, *common, "--dump-reference", ref],
                       capture_output=True, text=True, timeout=280, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    r = subprocess.run([sys.executable, tool, *common, "--acc", "--reference-file", ref],
                       capture_output=True, text=True, timeout=280, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout[r.stdout.index("{"):])
    assert out["rouge_l"] == 1.0 and out["samples"] == 3


@pytest.mark.timeout(300)
@pytest.mark.parametrize("name", sorted(CASES))
def test_tool_runs(name):
    argv = CASES[name]
    res = subprocess.run([sys.executable, os.path.join(ROOT, "benchmarks", argv[0]), *argv[1:]],
                         capture_output=True, text=True, timeout=280, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    out = res.stdout.strip()
    assert out, "the tool printed nothing"
    if out.lstrip().startswith("{"):
        json.loads(out[out.index("{"):])
