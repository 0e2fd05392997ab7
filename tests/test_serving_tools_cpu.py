"""The serving benchmark tools against live HTTP servers on the CPU engine (tiny model):
``benchmark_serving.py`` over two servers with a concurrency cap and goodput objectives,
``benchmark_serving_prioritization.py`` with its lowest-priority background load, and the
data-parallel router in front of both servers."""
import argparse
import asyncio
import importlib.util
import os
import socket
import sys
import threading
import time

import pytest

pytest.importorskip("aiohttp")
uvicorn = pytest.importorskip("uvicorn")

from vllm_gcu_b200.config import CacheConfig, EngineConfig, SchedulerConfig, preset  # noqa: E402
from vllm_gcu_b200.engine.async_llm import AsyncLLM  # noqa: E402
from vllm_gcu_b200.entrypoints.api_server import ByteTokenizer, build_app  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    path = os.path.join(ROOT, "benchmarks", name + ".py")
    sys.path.insert(0, os.path.dirname(path))
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _Server:
    def __init__(self, app):
        self.port = _free_port()
        self.server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=self.port,
                                                    log_level="error"))
        self.thread = threading.Thread(target=self.server.run, daemon=True)
        self.thread.start()
        t_end = time.monotonic() + 30
        while not self.server.started and time.monotonic() < t_end:
            time.sleep(0.02)
        assert self.server.started

    def stop(self):
        self.server.should_exit = True
        self.thread.join(10)


@pytest.fixture(scope="module")
def servers():
    engines, srv = [], []
    for _ in range(2):
        cfg = EngineConfig(model=preset("tiny-llama"), cache=CacheConfig(num_gpu_blocks=128),
                           scheduler=SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=64,
                                                     max_model_len=128, policy="priority"),
                           device="cpu")
        eng = AsyncLLM(cfg)
        engines.append(eng)
        srv.append(_Server(build_app(eng, ByteTokenizer(32000), "tiny-llama")))
    yield srv
    for s in srv:
        s.stop()
    for e in engines:
        e.shutdown()


@pytest.mark.timeout(180)
def test_serving_benchmark_over_two_servers(servers):
    bs = _load("benchmark_serving")
    args = argparse.Namespace(
        host="127.0.0.1", port=servers[0].port, ports=[s.port for s in servers],
        backend="openai", num_prompts=6, request_rate=float("inf"), burstiness=1.0,
        input_len_range=[4, 12], output_len_range=[3, 6], vocab_size=32000, temperature=0.0,
        extra_body=None, seed=0, output_json=None, max_concurrency=3,
        goodput=["ttft:60000", "tpot:60000"], dataset_name="random",
        metric_percentiles="50,99", profile=False)
    res = asyncio.run(bs.run(args))
    assert res["completed"] == 6 and res["failed"] == 0
    assert res["ttft"]["p50_ms"] <= res["ttft"]["p99_ms"] and "std_ms" in res["e2el"]
    assert res["good_requests"] == 6 and res["request_goodput"] > 0
    assert res["output_token_throughput"] > 0 and res["ttft"]["median_ms"] > 0
    strict = bs.summarise([{"ok": True, "ttft": 0.5, "e2e": 1.0, "itl": [0.1], "n_out": 6,
                            "n_in": 4}], 1.0, bs.parse_goodput(["ttft:100"]))
    assert strict["good_requests"] == 0 and strict["tpot"]["mean_ms"] == pytest.approx(100.0)
    with pytest.raises(ValueError):
        bs.parse_goodput(["latency:5"])


@pytest.mark.timeout(180)
def test_prioritization_benchmark_keeps_background_load(servers):
    bp = _load("benchmark_serving_prioritization")
    res = bp.main(["--ports", *[str(s.port) for s in servers], "--num-prompts", "5",
                   "--input-len-range", "4", "10", "--output-len-range", "3", "5",
                   "--background-tokens", "4", "--goodput", "e2el:60000"])
    assert res["completed"] == 5 and res["failed"] == 0
    assert res["background_requests"] >= 2 and res["good_requests"] == 5


@pytest.mark.timeout(180)
def test_router_spreads_requests_and_forwards_streams(servers):
    rt = _load("router")
    router = rt.Router([f"127.0.0.1:{s.port}" for s in servers])
    front = _Server(router.app())
    try:
        bs = _load("benchmark_serving")
        args = argparse.Namespace(
            host="127.0.0.1", port=front.port, ports=None, backend="openai", num_prompts=4,
            request_rate=float("inf"), burstiness=1.0, input_len_range=[4, 8],
            output_len_range=[3, 4], vocab_size=32000, temperature=0.0, extra_body=None,
            seed=1, output_json=None, max_concurrency=None, goodput=None, dataset_name="random")
        res = asyncio.run(bs.run(args))
        assert res["completed"] == 4 and res["failed"] == 0
        assert router.active == [0, 0]
    finally:
        front.stop()


@pytest.mark.timeout(180)
def test_serving_benchmark_with_dataset_files(servers, tmp_path):
    """ShareGPT-style conversations and a text file of lines as prompt sources (text prompts
    are tokenised by the server)."""
    import json as _json
    bs = _load("benchmark_serving")
    share = [{"conversations": [{"from": "human", "value": f"question number {i} " * 3},
                                {"from": "gpt", "value": "an answer " * (2 + i)}]}
             for i in range(6)]
    share.append({"conversations": [{"from": "human", "value": "too short"}]})
    (tmp_path / "share.json").write_text(_json.dumps(share))
    (tmp_path / "poem.txt").write_text("\n".join(f"line {i} of the poem" for i in range(20)))
    base = dict(host="127.0.0.1", port=servers[0].port, ports=None, backend="openai",
                num_prompts=4, request_rate=float("inf"), burstiness=1.0,
                input_len_range=[4, 8], output_len_range=[3, 4], vocab_size=32000,
                temperature=0.0, extra_body=None, seed=0, output_json=None,
                max_concurrency=None, goodput=None, tokenizer=None, max_input_len=100,
                max_output_len=100, fixed_output_len=None, sonnet_input_len=12,
                sonnet_output_len=5, sonnet_prefix_len=4)
    a = argparse.Namespace(**base, dataset_name="sharegpt", dataset_path=str(tmp_path / "share.json"))
    reqs = bs.load_dataset_requests(a, __import__("random").Random(0))
    assert len(reqs) == 4 and all(isinstance(p, str) and n >= 4 for p, n in reqs)
    res = asyncio.run(bs.run(a))
    assert res["completed"] == 4 and res["failed"] == 0
    b = argparse.Namespace(**base, dataset_name="sonnet", dataset_path=str(tmp_path / "poem.txt"))
    res = asyncio.run(bs.run(b))
    assert res["completed"] == 4 and res["output_token_throughput"] > 0
    # a prompt the server refuses counts as a failed request, not as an empty success
    c = argparse.Namespace(**{**base, "sonnet_input_len": 400}, dataset_name="sonnet",
                           dataset_path=str(tmp_path / "poem.txt"))
    res = asyncio.run(bs.run(c))
    assert res["completed"] == 0 and res["failed"] == 4
