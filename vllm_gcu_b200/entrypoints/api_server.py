"""Minimal OpenAI-compatible completion server on the built-in engine.

Endpoints: ``POST /v1/completions`` (``prompt`` as a list of token ids, a list of such lists,
or a string tokenised byte-wise when no tokenizer directory is given; ``stream`` for server
sent events; per-request ``extra_args`` are forwarded into the sampling parameters, which is
how the router marks keep-alive requests, vllm_gcu/patch/patch_0_9_2/entrypoints.py:7-68),
``GET /v1/models``, ``GET /health``, ``GET /metrics`` (Prometheus text),
``POST /start_profile`` / ``POST /stop_profile`` (torch profiler, as used by the reference's
benchmark tools, benchmarks/benchmark_test.py:352-353).

Run: ``python -m vllm_gcu_b200.entrypoints.api_server --model llama-3-8b --port 8000``
"""
from __future__ import annotations

import argparse
import asyncio
import json
import time
import uuid
from typing import Any, Optional

from ..config import (CacheConfig, EngineConfig, ModelConfig, ParallelConfig, SchedulerConfig,
                      SpeculativeConfig,
                      preset)
from ..engine.llm import decode_text
from ..engine.request import SamplingParams

try:        # module level so that FastAPI can resolve the handler annotations
    from fastapi import FastAPI, Request
    from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse
except Exception:   # pragma: no cover - the server needs fastapi, the helpers do not
    FastAPI = Request = JSONResponse = PlainTextResponse = StreamingResponse = None


class ByteTokenizer:
    """Fallback when no tokenizer files are available: UTF-8 bytes offset into the vocabulary."""

    def __init__(self, vocab_size: int):
        self.vocab_size = vocab_size

    def encode(self, text: str) -> list[int]:
        return [3 + b for b in text.encode("utf-8")] or [3]

    def decode(self, ids: list[int]) -> str:
        return bytes((i - 3) % 256 for i in ids).decode("utf-8", errors="replace")


def load_tokenizer(path: Optional[str], vocab_size: int):
    if path:
        try:
            from transformers import AutoTokenizer
            return AutoTokenizer.from_pretrained(path)
        except Exception:
            pass
    return ByteTokenizer(vocab_size)


def sampling_from_body(body: dict, default_max: int = 16,
                       defaults: Optional[dict] = None) -> SamplingParams:
    """``defaults``: the checkpoint's recommended sampling values (``generation_config.json``),
    used for the fields a request leaves out."""
    if defaults:
        body = {**defaults, **body}
    extra = dict(body.get("extra_args") or {})
    if int(body.get("max_tokens", default_max)) < 1:
        raise ValueError("max_tokens must be at least 1")
    lp = body.get("logprobs")
    if lp is not None and not isinstance(lp, bool) and not 0 <= int(lp) <= 20:
        raise ValueError("logprobs must be between 0 and 20")
    stop_ids = tuple(body.get("stop_token_ids") or ())
    return SamplingParams(
        max_tokens=int(body.get("max_tokens", default_max)),
        min_tokens=int(body.get("min_tokens", 0)),
        temperature=float(body.get("temperature", 1.0)),
        top_k=int(body.get("top_k", 0) or 0), top_p=float(body.get("top_p", 1.0)),
        presence_penalty=float(body.get("presence_penalty", 0.0)),
        frequency_penalty=float(body.get("frequency_penalty", 0.0)),
        repetition_penalty=float(body.get("repetition_penalty", 1.0)),
        seed=body.get("seed"), ignore_eos=bool(body.get("ignore_eos", False)),
        stop_token_ids=stop_ids, stop=_stop_strings(body),
        include_stop_str_in_output=bool(body.get("include_stop_str_in_output", False)),
        logprobs=body.get("logprobs"),
        prompt_logprobs=body.get("prompt_logprobs"),
        allowed_token_ids=(tuple(int(t) for t in body["allowed_token_ids"])
                           if body.get("allowed_token_ids") else None),
        guided_choice=(tuple(tuple(int(t) for t in c) for c in body["guided_choice_token_ids"])
                       if body.get("guided_choice_token_ids") else None),
        guided_regex=_guided_pattern(body), guided_json=_guided_schema(body),
        extra_args=extra)


def _stop_strings(body: dict) -> tuple:
    stop = body.get("stop")
    if not stop:
        return ()
    return (str(stop),) if isinstance(stop, str) else tuple(str(t) for t in stop if t)


def cut_at_stop(text: str, sp: SamplingParams) -> tuple[str, bool]:
    """``text`` up to its first stop string (kept with ``include_stop_str_in_output``)."""
    cut = min((text.find(t) + (len(t) if sp.include_stop_str_in_output else 0)
               for t in sp.stop if t in text), default=-1)
    return (text[:cut], True) if cut >= 0 else (text, False)


def _guided_pattern(body: dict) -> Optional[str]:
    """``guided_regex`` as given; ``guided_choice`` (strings) as an alternation."""
    if body.get("guided_regex"):
        return str(body["guided_regex"])
    choice = body.get("guided_choice")
    if choice:
        import re
        return "(" + "|".join(re.escape(str(c)) for c in choice) + ")"
    return None


def _guided_schema(body: dict):
    """``guided_json`` or the OpenAI form ``response_format = {"type": "json_schema", ...}``."""
    if body.get("guided_json"):
        return body["guided_json"]
    rf = body.get("response_format") or {}
    if rf.get("type") == "json_schema":
        js = rf.get("json_schema") or {}
        return js.get("schema", js) or None
    return None


def build_app(engine: Any, tokenizer: Any, model_name: str, pooler: Any = None,
              lora_modules: Optional[dict] = None, mm_processor: Any = None):
    """``mm_processor(messages, images) -> (prompt_token_ids, multi_modal_data)`` turns chat
    messages with image parts into engine inputs (``entrypoints/multimodal.py``)."""
    if FastAPI is None:
        raise RuntimeError("the API server needs the fastapi package")
    app = FastAPI()

    @app.exception_handler(json.JSONDecodeError)
    async def _bad_json(request: Request, exc: json.JSONDecodeError):
        return JSONResponse({"error": f"the request body is not valid JSON: {exc}"},
                            status_code=400)

    state = {"profiler": None, "requests": 0, "tokens_out": 0, "t0": time.time()}

    inner_engine = getattr(engine, "engine", None)
    if inner_engine is not None and hasattr(inner_engine, "_apply_stop_strings"):
        # stop strings end a request inside the engine; engines in worker processes generate
        # on and the text is cut here
        inner_engine.detokenizer = lambda ids: decode_text(tokenizer, ids)

    model_cfg = getattr(getattr(inner_engine, "cfg", None) or getattr(engine, "cfg", None),
                        "model", None)
    gen_defaults = dict(getattr(model_cfg, "extra", {}).get("generation_defaults") or {}) \
        if model_cfg is not None else {}

    def text_of(comp, sp_: SamplingParams) -> tuple[str, Optional[str]]:
        """(text, finish reason) of a finished completion with the stop strings applied."""
        if comp.text is not None:
            return comp.text, comp.finish_reason
        text = decode_text(tokenizer, comp.token_ids)
        if sp_.stop:
            text, hit = cut_at_stop(text, sp_)
            if hit:
                return text, "stop"
        return text, comp.finish_reason

    def to_ids(p) -> list[int]:
        if isinstance(p, str):
            return list(tokenizer.encode(p))
        return [int(t) for t in p]

    @app.get("/health")
    async def health():
        err = getattr(engine, "error", None) or getattr(engine, "dead", None)
        if err:
            return JSONResponse({"status": "dead", "detail": str(err)}, status_code=503)
        return {"status": "ok"}

    # LoRA adapters by name: a request selects one through its "model" field (the way the
    # reference's multi-LoRA serving example addresses adapters, benchmarks/multilora_inference.py)
    adapters: dict[str, int] = {}
    state["next_lora_id"] = 1
    for name_, path_ in (lora_modules or {}).items():
        from ..lora import LoRARequest
        engine.add_lora(LoRARequest(name_, state["next_lora_id"], path_))
        adapters[name_] = state["next_lora_id"]
        state["next_lora_id"] += 1

    def lora_of(body: dict) -> int:
        name = body.get("model")
        if name in adapters:
            return adapters[name]
        return -1

    def gen_kwargs(body: dict) -> dict:
        lid = lora_of(body)
        return {"lora_id": lid} if lid >= 0 else {}

    @app.get("/v1/models")
    async def models():
        data = [{"id": model_name, "object": "model"}]
        data += [{"id": n, "object": "model", "parent": model_name} for n in adapters]
        return {"object": "list", "data": data}

    @app.post("/v1/load_lora_adapter")
    async def load_lora_adapter(request: Request):
        body = await request.json()
        name, path = body.get("lora_name"), body.get("lora_path")
        if not name or not path:
            return JSONResponse({"error": "lora_name and lora_path are required"}, status_code=400)
        if name in adapters:
            return JSONResponse({"error": f"adapter {name!r} is already loaded"}, status_code=400)
        if not hasattr(engine, "add_lora"):
            return JSONResponse({"error": "this engine cannot load adapters"}, status_code=400)
        from ..lora import LoRARequest
        lid = state["next_lora_id"]
        try:
            await asyncio.get_running_loop().run_in_executor(
                None, engine.add_lora, LoRARequest(name, lid, path))
        except Exception as e:  # noqa: BLE001  (bad path, rank too large, LoRA not enabled)
            return JSONResponse({"error": f"loading {name!r} failed: {e}"}, status_code=400)
        state["next_lora_id"] = lid + 1
        adapters[name] = lid
        return {"status": "ok", "lora_name": name, "lora_int_id": lid}

    @app.post("/v1/unload_lora_adapter")
    async def unload_lora_adapter(request: Request):
        body = await request.json()
        name = body.get("lora_name")
        if name not in adapters:
            return JSONResponse({"error": f"adapter {name!r} is not loaded"}, status_code=404)
        # the slot is reused by least-recently-used eviction; the name stops resolving now
        del adapters[name]
        return {"status": "ok", "lora_name": name}

    def _ensure_vocabulary() -> None:
        """Guided requests need the text of every token; built on first use."""
        if state.get("vocab_set"):
            return
        inner = getattr(engine, "engine", engine)
        if not hasattr(inner, "set_vocabulary"):
            raise ValueError("guided decoding is not available on this engine")
        from ..engine.guided import vocabulary_of
        inner.set_vocabulary(vocabulary_of(tokenizer, inner.cfg.model.vocab_size))
        state["vocab_set"] = True

    @app.get("/metrics")
    async def metrics():
        lines = [f"vllm_b200_requests_total {state['requests']}",
                 f"vllm_b200_generation_tokens_total {state['tokens_out']}"]
        st = engine.stats() if hasattr(engine, "stats") else {}
        for k, v in st.items():
            try:
                lines.append(f"vllm_b200_{k} {float(v)}")
            except (TypeError, ValueError):
                pass
        return PlainTextResponse("\n".join(lines) + "\n")

    @app.post("/start_profile")
    async def start_profile():
        import torch
        if state["profiler"] is None:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            state["profiler"] = torch.profiler.profile(activities=acts)
            state["profiler"].__enter__()
        return {"status": "started"}

    @app.post("/stop_profile")
    async def stop_profile():
        prof = state["profiler"]
        if prof is not None:
            prof.__exit__(None, None, None)
            path = f"/tmp/vllm_b200_trace_{int(time.time())}.json"
            prof.export_chrome_trace(path)
            state["profiler"] = None
            return {"status": "stopped", "trace": path}
        return {"status": "idle"}

    @app.post("/v1/completions")
    async def completions(request: Request):
        body = await request.json()
        prompt = body.get("prompt")
        if prompt is None:
            return JSONResponse({"error": "prompt is required"}, status_code=400)
        batch = prompt if (isinstance(prompt, list) and prompt and
                           isinstance(prompt[0], (list, str))) else [prompt]
        try:
            sp = sampling_from_body(body, defaults=gen_defaults)
            if sp.guided_regex is not None or sp.guided_json is not None:
                from ..engine.guided import check_guided
                check_guided(sp.guided_regex, sp.guided_json)
                _ensure_vocabulary()
        except ValueError as e:
            return JSONResponse({"error": str(e)}, status_code=400)
        try:
            batch_ids = [to_ids(p) for p in batch]
            for ids_ in batch_ids:
                engine.validate_prompt(ids_)
        except (ValueError, TypeError) as e:
            return JSONResponse({"error": str(e)}, status_code=400)
        n = int(body.get("n") or 1)
        best_of = int(body.get("best_of") or n)
        if body.get("use_beam_search"):
            return JSONResponse({"error": "beam search is offered by the offline LLM class "
                                          "(LLM.beam_search), not by the server"}, status_code=400)
        if n < 1 or best_of < n:
            return JSONResponse({"error": "best_of must be at least n >= 1"}, status_code=400)
        if best_of > 1 and body.get("stream", False):
            return JSONResponse({"error": "n / best_of > 1 cannot be streamed"}, status_code=400)
        rid = "cmpl-" + uuid.uuid4().hex[:16]
        created = int(time.time())
        state["requests"] += len(batch)
        priority = int(body.get("priority", 0))
        # disaggregated prefill: the proxy names the request and the peer instance
        kvp = body.get("kv_transfer_params")
        gen_kw = gen_kwargs(body)
        if kvp:
            gen_kw["kv_transfer_params"] = kvp
            if body.get("request_id") and len(batch) == 1:
                gen_kw["request_id"] = str(body["request_id"])

        def chunk(idx: int, toks: list[int], finish: Optional[str]) -> dict:
            return {"id": rid, "object": "text_completion", "created": created,
                    "model": model_name,
                    "choices": [{"index": idx, "text": decode_text(tokenizer, toks),
                                 "token_ids": toks, "finish_reason": finish}]}

        if body.get("stream", False):
            async def sse():
                ids = batch_ids[0]
                sent = 0
                async for out in engine.generate_stream(ids, sp, priority=priority, **gen_kw):
                    toks = out.outputs[0].token_ids
                    new = toks[sent:]
                    sent = len(toks)
                    state["tokens_out"] += len(new)
                    yield "data: " + json.dumps(chunk(0, new, out.outputs[0].finish_reason)) + "\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")

        import dataclasses

        def with_logprobs(c: dict, comp) -> dict:
            if sp.logprobs is not None and comp.logprobs:
                c["logprobs"] = {
                    "tokens": [tokenizer.decode([t]) for t in comp.token_ids],
                    "token_logprobs": [d.get(t) for t, d in zip(comp.token_ids, comp.logprobs)],
                    "top_logprobs": [{tokenizer.decode([k]): v for k, v in d.items()}
                                     for d in comp.logprobs]}
            return c

        async def sample(ids, sp_c):
            last = None
            async for out in engine.generate_stream(ids, sp_c, priority=priority, **gen_kw):
                last = out
            return last

        async def one(idx: int, ids) -> list[dict]:
            """The ``n`` choices of one prompt: ``best_of`` seeded samples ranked by their
            cumulative log-probability when more were asked for than are returned."""
            if best_of == 1:
                lasts = [await sample(ids, sp)]
            else:
                base = (sp.seed if sp.seed is not None else 0) * 7919
                need_lp = sp.logprobs if sp.logprobs is not None else (0 if best_of > n else None)
                lasts = list(await asyncio.gather(*[
                    sample(ids, dataclasses.replace(sp, seed=base + c + 1, logprobs=need_lp))
                    for c in range(best_of)]))
                if best_of > n:
                    lasts.sort(key=lambda o: -(o.outputs[0].cumulative_logprob or 0.0))
                    lasts = lasts[:n]
            out = []
            for j, last in enumerate(lasts):
                comp = last.outputs[0]
                state["tokens_out"] += len(comp.token_ids)
                c = chunk(idx * n + j, comp.token_ids, comp.finish_reason)["choices"][0]
                c["text"], c["finish_reason"] = text_of(comp, sp)
                c["prompt_tokens"] = len(ids) if j == 0 else 0
                c["kv_transfer_params"] = getattr(last, "kv_transfer_params", None)
                out.append(with_logprobs(c, comp))
            return out

        groups = await asyncio.gather(*[one(i, p) for i, p in enumerate(batch_ids)])
        choices = [c for g in groups for c in g]
        usage = {"prompt_tokens": sum(c.pop("prompt_tokens") for c in choices),
                 "completion_tokens": sum(len(c["token_ids"]) for c in choices)}
        usage["total_tokens"] = usage["prompt_tokens"] + usage["completion_tokens"]
        resp = {"id": rid, "object": "text_completion", "created": created, "model": model_name,
                "choices": list(choices), "usage": usage}
        kv_out = [c.pop("kv_transfer_params") for c in choices]
        if kv_out and kv_out[0]:
            # prefill instance of a disaggregated pair: what the proxy passes on to the decode
            # instance (peer address, request id, first token)
            resp["kv_transfer_params"] = kv_out[0]
        return resp

    def render_chat(messages: list) -> list[int]:
        """Conversation -> prompt ids: the tokenizer's chat template when it has one, else a
        plain ``<role>: content`` transcript."""
        if hasattr(tokenizer, "apply_chat_template") and getattr(tokenizer, "chat_template", None):
            from ..engine.llm import chat_template_ids
            return chat_template_ids(tokenizer, messages)
        text = "".join(f"{m.get('role', 'user')}: {m.get('content', '')}\n" for m in messages)
        return list(tokenizer.encode(text + "assistant: "))

    @app.post("/v1/chat/completions")
    async def chat_completions(request: Request):
        body = await request.json()
        messages = body.get("messages")
        if not messages:
            return JSONResponse({"error": "messages is required"}, status_code=400)
        try:
            sp = sampling_from_body(body, default_max=int(body.get("max_completion_tokens", 256)),
                                    defaults=gen_defaults)
            if sp.guided_regex is not None or sp.guided_json is not None:
                from ..engine.guided import check_guided
                check_guided(sp.guided_regex, sp.guided_json)
                _ensure_vocabulary()
        except ValueError as e:
            return JSONResponse({"error": str(e)}, status_code=400)
        mm_kw: dict = {}
        try:
            from .multimodal import split_messages
            messages, images = split_messages(messages)
            if images:
                if mm_processor is None:
                    raise ValueError("this server was not started with a multimodal processor")
                ids, mm = mm_processor(messages, images)
                mm_kw = {"multi_modal_data": mm}
            else:
                ids = render_chat([{**m, "content": "".join(p.get("text", "") for p in m["content"])}
                                   if isinstance(m.get("content"), list) else m for m in messages])
            engine.validate_prompt(ids, multimodal=bool(images))
        except (ValueError, KeyError, OSError) as e:
            return JSONResponse({"error": str(e)}, status_code=400)
        rid = "chatcmpl-" + uuid.uuid4().hex[:16]
        created = int(time.time())
        state["requests"] += 1
        priority = int(body.get("priority", 0))
        base = {"id": rid, "created": created, "model": body.get("model") or model_name}
        lora_kw = {**gen_kwargs(body), **mm_kw}

        if body.get("stream", False):
            async def sse():
                sent = 0
                first = {"index": 0, "delta": {"role": "assistant", "content": ""},
                         "finish_reason": None}
                yield "data: " + json.dumps({**base, "object": "chat.completion.chunk",
                                             "choices": [first]}) + "\n\n"
                async for out in engine.generate_stream(ids, sp, priority=priority, **lora_kw):
                    toks = out.outputs[0].token_ids
                    new, sent = toks[sent:], len(toks)
                    state["tokens_out"] += len(new)
                    ch = {"index": 0, "delta": {"content": decode_text(tokenizer, new)},
                          "finish_reason": out.outputs[0].finish_reason}
                    yield "data: " + json.dumps({**base, "object": "chat.completion.chunk",
                                                 "choices": [ch]}) + "\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")

        last = None
        async for out in engine.generate_stream(ids, sp, priority=priority, **lora_kw):
            last = out
        toks = last.outputs[0].token_ids
        state["tokens_out"] += len(toks)
        content, reason = text_of(last.outputs[0], sp)
        choice = {"index": 0, "finish_reason": reason,
                  "message": {"role": "assistant", "content": content}}
        usage = {"prompt_tokens": len(ids), "completion_tokens": len(toks),
                 "total_tokens": len(ids) + len(toks)}
        return {**base, "object": "chat.completion", "choices": [choice], "usage": usage}

    @app.post("/tokenize")
    async def tokenize(request: Request):
        body = await request.json()
        ids = render_chat(body["messages"]) if body.get("messages") else to_ids(body.get("prompt", ""))
        return {"tokens": ids, "count": len(ids)}

    @app.post("/detokenize")
    async def detokenize(request: Request):
        body = await request.json()
        return {"prompt": tokenizer.decode([int(t) for t in body.get("tokens", [])])}

    # -- pooling models (embedding / cross-encoder): ``pooler`` is a models.roberta.PoolingRunner
    def _need_pooler():
        if pooler is None:
            return JSONResponse({"error": "this server was not started with a pooling model"},
                                status_code=400)
        return None

    def _as_ids(x) -> list[int]:
        return [int(t) for t in x] if isinstance(x, list) and x and isinstance(x[0], int) \
            else list(tokenizer.encode(str(x)))

    async def _decoder_embedding(ids: list[int]) -> list[float]:
        """Last-token embedding from the generation engine (decoder checkpoints published as
        embedding models): one pooling request through the same scheduler as completions."""
        import torch
        final = None
        async for out in engine.generate_stream(ids, SamplingParams(max_tokens=1, pooling=True)):
            final = out
        vec = final.embedding.float()
        return torch.nn.functional.normalize(vec, dim=-1).tolist()

    @app.post("/v1/embeddings")
    async def embeddings(request: Request):
        body = await request.json()
        inp = body.get("input")
        items = inp if isinstance(inp, list) and inp and not isinstance(inp[0], int) else [inp]
        seqs = [_as_ids(x) for x in items]
        if pooler is None and engine is not None and hasattr(engine, "generate_stream"):
            try:
                for q in seqs:
                    engine.validate_prompt(q)
            except ValueError as e:
                return JSONResponse({"error": str(e)}, status_code=400)
            vecs = list(await asyncio.gather(*[_decoder_embedding(q) for q in seqs]))
        else:
            err = _need_pooler()
            if err is not None:
                return err
            vecs = pooler.run(seqs).float().tolist()
        return {"object": "list", "model": model_name,
                "data": [{"object": "embedding", "index": i, "embedding": v}
                         for i, v in enumerate(vecs)],
                "usage": {"prompt_tokens": sum(len(q) for q in seqs)}}

    async def _scores(request: Request):
        body = await request.json()
        query = body.get("query", body.get("text_1"))
        docs = body.get("documents", body.get("text_2"))
        docs = docs if isinstance(docs, list) and docs and not isinstance(docs[0], int) else [docs]
        q = _as_ids(query)
        d = [_as_ids(x) for x in docs]
        sep = int(body.get("sep_token_id", getattr(tokenizer, "sep_token_id", None) or 2))
        return body, docs, pooler.score(q, d, sep)

    @app.post("/score")
    async def score(request: Request):
        err = _need_pooler()
        if err is not None:
            return err
        _, _, sc = await _scores(request)
        return {"object": "list", "model": model_name,
                "data": [{"object": "score", "index": i, "score": v} for i, v in enumerate(sc)]}

    @app.post("/rerank")
    async def rerank(request: Request):
        err = _need_pooler()
        if err is not None:
            return err
        body, docs, sc = await _scores(request)
        order = sorted(range(len(sc)), key=lambda i: -sc[i])[: int(body.get("top_n", len(sc)))]
        return {"model": model_name,
                "results": [{"index": i, "relevance_score": sc[i], "document": docs[i]}
                            for i in order]}

    @app.get("/version")
    async def version():
        from .. import __version__
        return {"version": __version__}

    return app


def engine_config(args) -> EngineConfig:
    """``EngineConfig`` from the server's command line (the options of ``vllm serve`` that the
    reference's tutorials use: parallel sizes, expert parallelism, scheduler steps and policy,
    quantisation, KV-cache dtype, swap space, speculative decoding, ``--additional-config``)."""
    import os
    overrides: dict = {}
    if args.num_hidden_layers:
        overrides["num_hidden_layers"] = args.num_hidden_layers
    if getattr(args, "kv_cache_dtype", "auto") != "auto":
        overrides["kv_cache_dtype"] = args.kv_cache_dtype
    quant = getattr(args, "quantization", None)
    if quant == "fp8_block":
        overrides.update(quantization="fp8", quant_config={"quant_method": "fp8",
                                                           "weight_block_size": [128, 128]})
    elif quant and not os.path.isdir(args.model):
        overrides.update(quantization=quant, quant_config={"quant_method": quant})
    if os.path.isdir(args.model):
        mc = ModelConfig.from_pretrained(args.model, **overrides)
        path, fmt = args.model, "safetensors"
    else:
        mc = preset(args.model, **overrides)
        path, fmt = None, "dummy"
    if getattr(args, "dtype", None):
        from ..config import to_dtype
        mc.dtype = to_dtype(args.dtype)
    dp = int(getattr(args, "data_parallel_size", 1))
    if dp > 1:
        mc.extra["dp_attention"] = True
    extra_cfg = json.loads(args.additional_config) if getattr(args, "additional_config", None) \
        else {}
    if getattr(args, "enable_lora", False):
        extra_cfg["lora"] = {"max_loras": args.max_loras, "max_lora_rank": args.max_lora_rank}
    spec = SpeculativeConfig()
    if getattr(args, "speculative_method", None):
        spec = SpeculativeConfig(args.speculative_method, int(args.num_speculative_tokens),
                                 draft_model=getattr(args, "speculative_model", None))
    return EngineConfig(
        model=mc,
        cache=CacheConfig(block_size=args.block_size,
                          gpu_memory_utilization=args.gpu_memory_utilization,
                          num_gpu_blocks=args.num_gpu_blocks,
                          num_cpu_blocks=int(getattr(args, "num_cpu_blocks", 0)),
                          enable_prefix_caching=not getattr(args, "no_enable_prefix_caching",
                                                            False)),
        scheduler=SchedulerConfig(max_num_seqs=args.max_num_seqs,
                                  max_num_batched_tokens=args.max_num_batched_tokens,
                                  max_model_len=args.max_model_len or mc.max_position_embeddings,
                                  policy=args.scheduling_policy,
                                  async_scheduling=not args.no_async_scheduling,
                                  num_scheduler_steps=int(getattr(args, "num_scheduler_steps", 1))),
        parallel=ParallelConfig(tensor_parallel_size=args.tensor_parallel_size,
                                pipeline_parallel_size=int(getattr(args, "pipeline_parallel_size",
                                                                   1)),
                                data_parallel_size=dp,
                                enable_expert_parallel=bool(getattr(args, "enable_expert_parallel",
                                                                    False)),
                                comm_backend=getattr(args, "comm_backend", "fused")),
        speculative=spec, device=args.device, seed=int(getattr(args, "seed", 0)),
        enforce_eager=args.enforce_eager, load_format=fmt, model_path=path,
        additional_config=extra_cfg)


def make_engine(args) -> tuple[Any, ModelConfig]:
    cfg = engine_config(args)
    mc = cfg.model
    sc, pc = cfg.scheduler, cfg.parallel
    if sc.async_scheduling and (sc.num_scheduler_steps > 1 or pc.pipeline_parallel_size > 1
                                or cfg.speculative.method):
        sc.async_scheduling = False        # the platform policy's exclusions
    if pc.world_size > 1:
        from ..engine.executor import AsyncMultiprocExecutor
        if getattr(args, "kv_port", 0):
            # every worker opens its own connector on kv_port + rank
            cfg.additional_config["kv_connector"] = {"host": args.host, "port": args.kv_port,
                                                     "send_type": args.kv_send_type}
        return AsyncMultiprocExecutor(cfg), mc
    from ..engine.async_llm import AsyncLLM
    eng = AsyncLLM(cfg)
    if getattr(args, "kv_port", 0):
        # disaggregated prefill / decode: requests that carry kv_transfer_params exchange
        # their KV with the peer instance through this connector
        from ..parallel.kv_transfer import P2PKVConnector
        conn = P2PKVConnector(host=args.host, port=args.kv_port, send_type=args.kv_send_type,
                              device=str(eng.engine.device))
        eng.engine.attach_kv_connector(conn)
    return eng, mc


def add_engine_arguments(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--tensor-parallel-size", "-tp", type=int, default=1)
    ap.add_argument("--pipeline-parallel-size", "-pp", type=int, default=1)
    ap.add_argument("--data-parallel-size", "-dp", type=int, default=1,
                    help="replicas with their own attention and KV cache (one process per GPU)")
    ap.add_argument("--enable-expert-parallel", action="store_true",
                    help="experts spread over all dp x tp ranks instead of sharded")
    ap.add_argument("--comm-backend", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--max-model-len", type=int, default=0)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--num-gpu-blocks", type=int, default=None)
    ap.add_argument("--num-cpu-blocks", type=int, default=0,
                    help="host blocks for swapping pre-empted requests (0: recompute)")
    ap.add_argument("--no-enable-prefix-caching", action="store_true")
    ap.add_argument("--scheduling-policy", default="fcfs", choices=["fcfs", "priority"])
    ap.add_argument("--num-scheduler-steps", type=int, default=1)
    ap.add_argument("--no-async-scheduling", action="store_true")
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--dtype", default=None)
    ap.add_argument("--kv-cache-dtype", default="auto", choices=["auto", "fp8", "int8"])
    ap.add_argument("--quantization", default=None,
                    help="for architecture presets with random weights: fp8, fp8_block, w8a8; "
                         "checkpoints carry their own quantization_config")
    ap.add_argument("--speculative-method", default=None,
                    choices=[None, "ngram", "mtp", "eagle", "medusa", "mlp_speculator"])
    ap.add_argument("--num-speculative-tokens", type=int, default=1)
    ap.add_argument("--speculative-model", default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--additional-config", default=None,
                    help='JSON, e.g. \'{"cascade_min_tokens": 512}\'')
    ap.add_argument("--num-hidden-layers", type=int, default=0)
    ap.add_argument("--enable-lora", action="store_true")
    ap.add_argument("--max-loras", type=int, default=4)
    ap.add_argument("--max-lora-rank", type=int, default=16)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    add_engine_arguments(ap)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--kv-port", type=int, default=0,
                    help="port of the point-to-point KV connector (disaggregated prefill)")
    ap.add_argument("--kv-send-type", default="PUT_ASYNC", choices=["PUT", "PUT_ASYNC", "GET"])
    ap.add_argument("--lora-modules", nargs="*", default=[], metavar="NAME=PATH",
                    help="adapters loaded at start-up; requests select one by model name")
    args = ap.parse_args()
    import os
    cfg_path = os.path.join(args.model, "config.json") if os.path.isdir(args.model) else None
    if cfg_path and os.path.exists(cfg_path):
        # embedding / reranker checkpoints are served by the pooling runner (no KV cache)
        from ..models import POOLING_ARCHITECTURES, build_pooling_model
        hf = json.load(open(cfg_path))
        if (hf.get("architectures") or [""])[0] in POOLING_ARCHITECTURES:
            import torch
            dev = "cuda" if (args.device == "auto" and torch.cuda.is_available()) else \
                ("cpu" if args.device == "auto" else args.device)
            pooler = build_pooling_model(hf, dev)
            from ..utils.weights import iter_safetensors
            pooler.model.load_weights(iter_safetensors(args.model))
            tok = load_tokenizer(args.tokenizer or args.model, int(hf.get("vocab_size", 0)))
            import uvicorn
            uvicorn.run(build_app(None, tok, args.model, pooler=pooler), host=args.host,
                        port=args.port, log_level="warning")
            return
    engine, mc = make_engine(args)
    tok = load_tokenizer(args.tokenizer or (args.model if "/" in args.model else None),
                         mc.vocab_size)
    import uvicorn
    from .multimodal import default_processor
    import os as _os
    inner = getattr(getattr(engine, "engine", None), "model", None)
    app = build_app(engine, tok, args.model, lora_modules=dict(
        m.split("=", 1) for m in args.lora_modules),
        mm_processor=default_processor(args.model if _os.path.isdir(args.model) else None,
                                       inner, tok))
    try:
        uvicorn.run(app, host=args.host, port=args.port, log_level="warning")
    finally:
        engine.shutdown()          # worker processes / the engine thread end with the server


if __name__ == "__main__":
    main()
