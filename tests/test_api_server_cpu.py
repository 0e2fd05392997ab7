"""OpenAI-compatible server on the CPU engine, driven through the ASGI app in-process."""
import asyncio
import json

import pytest
import torch

from vllm_gcu_b200.config import CacheConfig, EngineConfig, SchedulerConfig, preset
from vllm_gcu_b200.engine.async_llm import AsyncLLM
from vllm_gcu_b200.entrypoints.api_server import ByteTokenizer, build_app


@pytest.mark.timeout(120)
def test_completions_and_streaming():
    httpx = pytest.importorskip("httpx")
    cfg = EngineConfig(model=preset("tiny-llama"), cache=CacheConfig(num_gpu_blocks=64),
                       scheduler=SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=64,
                                                 max_model_len=128), device="cpu")
    eng = AsyncLLM(cfg)
    app = build_app(eng, ByteTokenizer(32000), "tiny-llama")

    async def run():
        transport = httpx.ASGITransport(app=app)
        async with httpx.AsyncClient(transport=transport, base_url="http://t") as c:
            r = await c.get("/health")
            assert r.json()["status"] == "ok"
            body = {"prompt": [[1, 2, 3, 4], [9, 8, 7]], "max_tokens": 5, "temperature": 0.0,
                    "ignore_eos": True}
            r = await c.post("/v1/completions", json=body)
            js = r.json()
            assert len(js["choices"]) == 2
            assert all(len(ch["token_ids"]) == 5 for ch in js["choices"])
            assert js["usage"]["completion_tokens"] == 10
            # streaming returns the same tokens as the blocking call
            body1 = {"prompt": [1, 2, 3, 4], "max_tokens": 5, "temperature": 0.0,
                     "ignore_eos": True, "stream": True}
            toks = []
            async with c.stream("POST", "/v1/completions", json=body1) as resp:
                async for line in resp.aiter_lines():
                    if line.startswith("data: ") and "[DONE]" not in line:
                        toks += json.loads(line[6:])["choices"][0]["token_ids"]
            assert toks == js["choices"][0]["token_ids"]
            m = await c.get("/metrics")
            assert "vllm_b200_generation_tokens_total" in m.text
            # chat endpoint: blocking and streaming give the same text; tokenize round trip
            chat = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
                    "temperature": 0.0, "ignore_eos": True}
            r = await c.post("/v1/chat/completions", json=chat)
            cj = r.json()
            assert cj["object"] == "chat.completion" and cj["usage"]["completion_tokens"] == 4
            text = ""
            async with c.stream("POST", "/v1/chat/completions", json={**chat, "stream": True}) as resp:
                async for line in resp.aiter_lines():
                    if line.startswith("data: ") and "[DONE]" not in line:
                        text += json.loads(line[6:])["choices"][0]["delta"].get("content", "")
            assert text == cj["choices"][0]["message"]["content"]
            tk = (await c.post("/tokenize", json={"prompt": "abc"})).json()
            assert tk["count"] == 3
            dt = (await c.post("/detokenize", json={"tokens": tk["tokens"]})).json()
            assert dt["prompt"] == "abc"
            assert "version" in (await c.get("/version")).json()
            # prompts the scheduler would refuse are answered with 400, not queued
            r = await c.post("/v1/completions", json={"prompt": [[]], "max_tokens": 2})
            assert r.status_code == 400
            r = await c.post("/v1/completions", json={"prompt": [[1] * 500], "max_tokens": 2})
            assert r.status_code == 400
            r = await c.post("/v1/completions", json={"prompt": [1, 2], "max_tokens": 2,
                                                      "temperature": 0.0, "ignore_eos": True})
            assert r.status_code == 200 and len(r.json()["choices"][0]["token_ids"]) == 2
            bad = await c.post("/v1/chat/completions", json={"max_tokens": 2})
            assert bad.status_code == 400
            # requests that must be refused before they reach the engine (an id outside the
            # vocabulary would index past the embedding table)
            for body_, word in (({"prompt": [1, 999999], "max_tokens": 2}, "vocabulary"),
                                ({"prompt": [1, -4], "max_tokens": 2}, "vocabulary"),
                                ({"prompt": [1, 2], "max_tokens": 0}, "max_tokens"),
                                ({"prompt": [1, 2], "max_tokens": 2, "logprobs": 1000}, "logprobs"),
                                ({"prompt": [1, 2], "max_tokens": 2, "guided_regex": "([a-z"},
                                 "]"),
                                ({"prompt": [1, 2], "max_tokens": 2, "temperature": "hot"},
                                 "float")):
                r = await c.post("/v1/completions", json=body_)
                assert r.status_code == 400 and word in r.json()["error"], (body_, r.text)
            assert (await c.get("/health")).json()["status"] == "ok"
            bad = await c.post("/v1/completions", content=b"{not json",
                               headers={"Content-Type": "application/json"})
            assert bad.status_code == 400 and "JSON" in bad.json()["error"]
            # n / best_of: seeded samples, the best n by cumulative log-probability; logprobs
            many = {"prompt": [1, 2, 3, 4], "max_tokens": 4, "temperature": 1.0, "seed": 3,
                    "ignore_eos": True, "n": 2, "best_of": 4, "logprobs": 1}
            r1 = (await c.post("/v1/completions", json=many)).json()
            r2 = (await c.post("/v1/completions", json=many)).json()
            assert [ch["index"] for ch in r1["choices"]] == [0, 1]
            assert [ch["token_ids"] for ch in r1["choices"]] == \
                [ch["token_ids"] for ch in r2["choices"]]
            lp = [sum(ch["logprobs"]["token_logprobs"]) for ch in r1["choices"]]
            assert lp[0] >= lp[1] and len(r1["choices"][0]["logprobs"]["top_logprobs"]) == 4
            assert r1["usage"]["completion_tokens"] == 8 and r1["usage"]["prompt_tokens"] == 4
            for bad_body in ({**many, "stream": True}, {**many, "best_of": 1},
                             {**many, "use_beam_search": True}):
                assert (await c.post("/v1/completions", json=bad_body)).status_code == 400
            # a decoder engine answers /v1/embeddings with last-token vectors of unit length
            e = (await c.post("/v1/embeddings", json={"input": [[1, 2, 3, 4], [9, 8, 7]]})).json()
            assert len(e["data"]) == 2 and e["usage"]["prompt_tokens"] == 7
            v0, v1 = (e["data"][i]["embedding"] for i in (0, 1))
            assert len(v0) == cfg.model.hidden_size
            assert abs(sum(x * x for x in v0) - 1.0) < 1e-3 and v0 != v1
            again = (await c.post("/v1/embeddings", json={"input": [[1, 2, 3, 4]]})).json()
            assert max(abs(a - b) for a, b in zip(again["data"][0]["embedding"], v0)) < 1e-4
    try:
        asyncio.run(run())
    finally:
        eng.shutdown()


@pytest.mark.timeout(120)
def test_pooling_endpoints_embed_score_rerank():
    """/v1/embeddings, /score and /rerank on a tiny XLM-RoBERTa cross-encoder."""
    httpx = pytest.importorskip("httpx")
    from vllm_gcu_b200.models import build_pooling_model
    hf = {"architectures": ["XLMRobertaForSequenceClassification"], "vocab_size": 400,
          "hidden_size": 32, "num_hidden_layers": 2, "num_attention_heads": 2,
          "intermediate_size": 64, "max_position_embeddings": 130, "pad_token_id": 1,
          "num_labels": 1, "type_vocab_size": 1, "layer_norm_eps": 1e-5}
    import torch
    torch.manual_seed(0)
    pooler = build_pooling_model(hf, dtype=torch.float32)
    for p in pooler.model.parameters():
        torch.nn.init.normal_(p, std=0.05)
    app = build_app(None, ByteTokenizer(400), "tiny-reranker", pooler=pooler)

    async def run():
        transport = httpx.ASGITransport(app=app)
        async with httpx.AsyncClient(transport=transport, base_url="http://t") as c:
            e = (await c.post("/v1/embeddings", json={"input": ["ab", "cde"]})).json()
            assert len(e["data"]) == 2 and e["usage"]["prompt_tokens"] == 5
            body = {"query": "q", "documents": ["aa", "bbbb", "c"]}
            sc = (await c.post("/score", json=body)).json()["data"]
            assert [d["index"] for d in sc] == [0, 1, 2]
            rr = (await c.post("/rerank", json={**body, "top_n": 2})).json()["results"]
            want = sorted(sc, key=lambda d: -d["score"])[:2]
            assert [r["index"] for r in rr] == [d["index"] for d in want]
            assert rr[0]["relevance_score"] >= rr[1]["relevance_score"]
    asyncio.run(run())
    # a generation-only server declines
    app2 = build_app(None, ByteTokenizer(400), "x")

    async def run2():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app2), base_url="http://t") as c:
            assert (await c.post("/score", json={"query": "a", "documents": ["b"]})).status_code == 400
    asyncio.run(run2())


@pytest.mark.timeout(180)
def test_lora_adapters_are_loaded_and_selected_by_model_name(tmp_path):
    """``/v1/load_lora_adapter`` reads a PEFT-layout directory; a request whose ``model`` is
    the adapter's name runs with it (same tokens as the offline engine with that adapter),
    other requests run the base model; unloading makes the name unknown again."""
    httpx = pytest.importorskip("httpx")
    import sys
    import os
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_lora_cpu import _adapter
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    from vllm_gcu_b200.lora import LoRARequest
    from vllm_gcu_b200.utils.weights import write_safetensors
    cfg = EngineConfig(model=preset("tiny-llama"), cache=CacheConfig(num_gpu_blocks=64),
                       scheduler=SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=64,
                                                 max_model_len=128), device="cpu")
    cfg.additional_config["lora"] = {"max_loras": 2, "max_lora_rank": 8}
    tensors, conf = _adapter(cfg.model, 1)
    tensors = {k: v * 6.0 for k, v in tensors.items()}
    adir = tmp_path / "adapter"
    adir.mkdir()
    (adir / "adapter_config.json").write_text(json.dumps(conf))
    write_safetensors(str(adir / "adapter_model.safetensors"), tensors)
    prompt = list(range(100, 120))
    off = LLM("tiny-llama", device="cpu", max_num_seqs=4, max_num_batched_tokens=64,
              max_model_len=128, num_gpu_blocks=32, enable_lora=True, max_loras=2,
              max_lora_rank=8)
    off.engine.add_lora(LoRARequest("a", 1, str(adir)))
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    rid = off.engine.add_request(prompt, sp, lora_id=1)
    rid0 = off.engine.add_request(prompt, sp)
    want = {}
    while off.engine.has_unfinished():
        for o in off.engine.step():
            if o.finished:
                want[o.request_id] = o.outputs[0].token_ids
    assert want[rid] != want[rid0]
    eng = AsyncLLM(cfg)
    app = build_app(eng, ByteTokenizer(32000), "tiny-llama")

    async def run():
        transport = httpx.ASGITransport(app=app)
        async with httpx.AsyncClient(transport=transport, base_url="http://t") as c:
            body = {"prompt": prompt, "max_tokens": 6, "temperature": 0.0, "ignore_eos": True}
            r = await c.post("/v1/load_lora_adapter", json={"lora_name": "sql"})
            assert r.status_code == 400
            r = await c.post("/v1/load_lora_adapter",
                             json={"lora_name": "bad", "lora_path": str(tmp_path / "none")})
            assert r.status_code == 400
            r = await c.post("/v1/load_lora_adapter",
                             json={"lora_name": "sql", "lora_path": str(adir)})
            assert r.status_code == 200 and r.json()["lora_int_id"] == 1
            ms = (await c.get("/v1/models")).json()["data"]
            assert [m["id"] for m in ms] == ["tiny-llama", "sql"]
            with_a = (await c.post("/v1/completions", json={**body, "model": "sql"})).json()
            base = (await c.post("/v1/completions", json={**body, "model": "tiny-llama"})).json()
            assert with_a["choices"][0]["token_ids"] == want[rid]
            assert base["choices"][0]["token_ids"] == want[rid0]
            chat = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
                    "temperature": 0.0, "ignore_eos": True}
            ca = (await c.post("/v1/chat/completions", json={**chat, "model": "sql"})).json()
            cb = (await c.post("/v1/chat/completions", json=chat)).json()
            assert ca["model"] == "sql" and ca["choices"][0]["message"]["content"] != \
                cb["choices"][0]["message"]["content"]
            r = await c.post("/v1/unload_lora_adapter", json={"lora_name": "sql"})
            assert r.status_code == 200
            again = (await c.post("/v1/completions", json={**body, "model": "sql"})).json()
            assert again["choices"][0]["token_ids"] == want[rid0]
            assert (await c.post("/v1/unload_lora_adapter",
                                 json={"lora_name": "sql"})).status_code == 404
    try:
        asyncio.run(run())
    finally:
        eng.shutdown()


def _server_args(*argv):
    import argparse
    from vllm_gcu_b200.entrypoints.api_server import add_engine_arguments
    ap = argparse.ArgumentParser()
    add_engine_arguments(ap)
    return ap.parse_args(list(argv))


def test_server_command_line_reaches_the_engine_configuration():
    from vllm_gcu_b200.entrypoints.api_server import engine_config
    a = _server_args("--model", "tiny-qwen3-moe", "--device", "cpu", "-dp", "2", "-tp", "2",
                     "--enable-expert-parallel", "--num-scheduler-steps", "4",
                     "--scheduling-policy", "priority", "--num-cpu-blocks", "8",
                     "--no-enable-prefix-caching", "--kv-cache-dtype", "int8",
                     "--speculative-method", "ngram", "--num-speculative-tokens", "3",
                     "--additional-config", '{"cascade_min_tokens": 64}', "--seed", "5",
                     "--enable-lora", "--max-loras", "2", "--dtype", "float32",
                     "--comm-backend", "nccl")
    c = engine_config(a)
    assert c.parallel.world_size == 4 and c.parallel.enable_expert_parallel
    assert c.parallel.comm_backend == "nccl" and c.model.extra["dp_attention"] is True
    assert c.scheduler.num_scheduler_steps == 4 and c.scheduler.policy == "priority"
    assert c.cache.num_cpu_blocks == 8 and not c.cache.enable_prefix_caching
    assert c.model.kv_cache_dtype == "int8" and c.model.dtype == torch.float32
    assert c.speculative.method == "ngram" and c.speculative.num_speculative_tokens == 3
    assert c.additional_config["cascade_min_tokens"] == 64 and c.seed == 5
    assert c.additional_config["lora"] == {"max_loras": 2, "max_lora_rank": 16}
    q = engine_config(_server_args("--model", "tiny-llama", "--device", "cpu",
                                   "--quantization", "fp8_block"))
    assert q.model.quantization == "fp8" and q.model.quant_config["weight_block_size"] == [128, 128]


@pytest.mark.timeout(300)
def test_server_on_a_data_parallel_expert_parallel_engine():
    """``-dp 2 --enable-expert-parallel`` starts one worker process per replica behind the same
    HTTP front end; concurrent requests are spread over the replicas and all finish."""
    httpx = pytest.importorskip("httpx")
    from vllm_gcu_b200.entrypoints.api_server import make_engine
    a = _server_args("--model", "tiny-qwen3-moe", "--device", "cpu", "-dp", "2",
                     "--enable-expert-parallel", "--comm-backend", "nccl", "--num-gpu-blocks",
                     "64", "--max-num-seqs", "8", "--max-num-batched-tokens", "64",
                     "--max-model-len", "128", "--dtype", "float32")
    a.host, a.kv_port = "127.0.0.1", 0
    eng, mc = make_engine(a)
    app = build_app(eng, ByteTokenizer(mc.vocab_size), "tiny-qwen3-moe")

    async def run():
        transport = httpx.ASGITransport(app=app)
        async with httpx.AsyncClient(transport=transport, base_url="http://t", timeout=120) as c:
            body = {"prompt": [[1, 2, 3, 4], [9, 8, 7], [5, 6, 7, 8, 9, 10]], "max_tokens": 5,
                    "temperature": 0.0, "ignore_eos": True}
            js = (await c.post("/v1/completions", json=body)).json()
            assert [len(ch["token_ids"]) for ch in js["choices"]] == [5, 5, 5]
            one = (await c.post("/v1/completions", json={**body, "prompt": [1, 2, 3, 4]})).json()
            assert one["choices"][0]["token_ids"] == js["choices"][0]["token_ids"]
            assert (await c.get("/health")).json()["status"] == "ok"
            # the workers report their scheduler counters to the front end
            for _ in range(40):
                m = (await c.get("/metrics")).text
                if "vllm_b200_kv_cache_usage" in m:
                    break
                await asyncio.sleep(0.1)
            assert "vllm_b200_num_running" in m and "vllm_b200_kv_cache_usage" in m
    try:
        asyncio.run(run())
    finally:
        eng.shutdown()
