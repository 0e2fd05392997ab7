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
