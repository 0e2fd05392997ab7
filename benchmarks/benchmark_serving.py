"""Online serving benchmark against an OpenAI-compatible ``/v1/completions`` (or, with
``--backend openai-chat``, ``/v1/chat/completions``) endpoint.

Poisson (gamma with configurable burstiness) arrivals, random token-id prompts with uniform
input / output lengths, streaming responses; reports request and token throughput and
mean / median / p99 of TTFT, TPOT, ITL and end-to-end latency
(benchmarks/benchmark_serving.py:414-562 of the reference, including its ``--extra-body``
and ``--strict-in-out-len`` conveniences).  ``--goodput ttft:200 tpot:50`` counts the requests
that met every given service-level objective (milliseconds); ``--max-concurrency`` caps the
requests in flight; several ``--ports`` spread the requests over as many servers.

Example:
  python -m vllm_gcu_b200.entrypoints.api_server --model llama-3-8b --port 8000 &
  python benchmarks/benchmark_serving.py --port 8000 --num-prompts 1000 --request-rate 8 \
      --input-len-range 256 2048 --output-len-range 64 512
"""
import argparse
import asyncio
import json
import random
import time

import numpy as np


async def one_request(session, url, body, result):
    t0 = time.perf_counter()
    ttft = None
    last = t0
    itl = []
    n_out = 0
    try:
        async with session.post(url, json=body) as resp:
            if resp.status != 200:
                raise RuntimeError(f"HTTP {resp.status}: {(await resp.text())[:200]}")
            async for raw in resp.content:
                line = raw.decode().strip()
                if not line.startswith("data: ") or line.endswith("[DONE]"):
                    continue
                now = time.perf_counter()
                choice = json.loads(line[6:])["choices"][0]
                if "delta" in choice:            # chat endpoint: one chunk per engine step
                    n_new = 1 if choice["delta"].get("content") else 0
                else:
                    n_new = len(choice.get("token_ids", [1]))
                if n_new == 0:
                    continue
                if ttft is None:
                    ttft = now - t0
                else:
                    itl.append(now - last)
                last = now
                n_out += n_new
        result.append({"ok": True, "ttft": ttft, "e2e": last - t0, "itl": itl, "n_out": n_out,
                       "n_in": (len(body["prompt"]) if not isinstance(body["prompt"], str)
                                else max(1, len(body["prompt"]) // 4)) if "prompt" in body
                       else sum(len(m["content"]) for m in body["messages"])})
    except Exception as e:  # noqa: BLE001
        result.append({"ok": False, "error": repr(e)})


def _count(tokenizer, text: str) -> int:
    """Token count of ``text`` (about four characters per token without a tokenizer)."""
    if tokenizer is not None:
        return len(tokenizer.encode(text))
    return max(1, len(text) // 4)


def load_dataset_requests(args, rng) -> list:
    """(prompt, output length) pairs from a dataset file, as the reference's load generator
    samples them (benchmarks/benchmark_serving.py:100-220 of the reference): ``sharegpt`` takes
    the first two turns of each conversation (the reply's length is the output length),
    ``sonnet`` builds prompts from randomly chosen lines of a text file."""
    tokenizer = None
    if getattr(args, "tokenizer", None):
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(args.tokenizer)
    out = []
    if args.dataset_name == "sharegpt":
        with open(args.dataset_path, encoding="utf-8") as f:
            data = json.load(f)
        convs = [d["conversations"] for d in data if len(d.get("conversations", [])) >= 2]
        rng.shuffle(convs)
        for c in convs:
            prompt, reply = c[0]["value"], c[1]["value"]
            n_in, n_out = _count(tokenizer, prompt), _count(tokenizer, reply)
            if n_in < 4 or n_out < 4 or n_in > args.max_input_len or \
                    n_in + n_out > args.max_input_len + args.max_output_len:
                continue                          # the reference prunes the same extremes
            out.append((prompt, args.fixed_output_len or n_out))
            if len(out) == args.num_prompts:
                break
    elif args.dataset_name == "sonnet":
        with open(args.dataset_path, encoding="utf-8") as f:
            lines = [ln.strip() for ln in f if ln.strip()]
        per_line = sum(_count(tokenizer, ln) for ln in lines) / max(1, len(lines))
        n_lines = max(1, int(args.sonnet_input_len / per_line))
        n_prefix = min(n_lines, int(args.sonnet_prefix_len / per_line))
        prefix = lines[:n_prefix]
        for _ in range(args.num_prompts):
            body = [rng.choice(lines) for _ in range(n_lines - n_prefix)]
            text = "Pick as many lines as you can from these poem lines:\n" + \
                "\n".join(prefix + body)
            out.append((text, args.fixed_output_len or args.sonnet_output_len))
    else:
        raise ValueError(f"unknown dataset {args.dataset_name!r}")
    if len(out) < args.num_prompts:
        out = (out * (args.num_prompts // max(1, len(out)) + 1))[:args.num_prompts]
    return out


async def run(args):
    import aiohttp
    rng = random.Random(args.seed)
    nprng = np.random.default_rng(args.seed)
    chat = args.backend == "openai-chat"
    path = "/v1/" + ("chat/completions" if chat else "completions")
    urls = [f"http://{args.host}:{p}{path}" for p in (args.ports or [args.port])]
    gate = asyncio.Semaphore(args.max_concurrency) if args.max_concurrency else None

    async def limited(session, url, body, results):
        if gate is None:
            return await one_request(session, url, body, results)
        async with gate:
            return await one_request(session, url, body, results)
    extra = json.loads(args.extra_body) if args.extra_body else {}
    results: list = []
    tasks = []
    timeout = aiohttp.ClientTimeout(total=6 * 3600)
    dataset = load_dataset_requests(args, rng) \
        if getattr(args, "dataset_name", "random") != "random" else None
    async with aiohttp.ClientSession(timeout=timeout) as session:
        bases = [u[:u.index("/v1/")] for u in urls]
        if getattr(args, "profile", False):        # the servers' profiler brackets the run
            for b in bases:
                async with session.post(b + "/start_profile") as r:
                    await r.read()
        t_start = time.perf_counter()
        for i in range(args.num_prompts):
            n_in = rng.randint(*args.input_len_range)
            n_out = rng.randint(*args.output_len_range)
            if dataset is not None:
                n_out = dataset[i][1]
            body = {"max_tokens": n_out, "temperature": args.temperature, "stream": True,
                    "ignore_eos": True}
            if dataset is not None:
                if chat:
                    body["messages"] = [{"role": "user", "content": dataset[i][0]}]
                else:
                    body["prompt"] = dataset[i][0]
            elif chat:     # random printable text of about n_in characters
                text = "".join(chr(rng.randrange(97, 123)) for _ in range(n_in))
                body["messages"] = [{"role": "user", "content": text}]
            else:
                body["prompt"] = [rng.randrange(10, args.vocab_size) for _ in range(n_in)]
            body.update(extra)
            tasks.append(asyncio.create_task(
                limited(session, urls[i % len(urls)], body, results)))
            if args.request_rate != float("inf"):
                theta = 1.0 / (args.request_rate * args.burstiness)
                await asyncio.sleep(float(nprng.gamma(shape=args.burstiness, scale=theta)))
        await asyncio.gather(*tasks)
        dur = time.perf_counter() - t_start
        if getattr(args, "profile", False):
            for b in bases:
                async with session.post(b + "/stop_profile") as r:
                    await r.read()
    pcts = tuple(float(p) for p in str(getattr(args, "metric_percentiles", "99")).split(","))
    res = summarise(results, dur, parse_goodput(args.goodput), pcts)
    print(json.dumps(res, indent=1))
    if args.output_json:
        with open(args.output_json, "w") as f:
            json.dump(res, f)
    return res


def parse_goodput(pairs) -> dict:
    """``["ttft:200", "tpot:50"]`` -> ``{"ttft": 0.2, "tpot": 0.05}`` (seconds)."""
    out = {}
    for p in pairs or ():
        name, _, ms = p.partition(":")
        if name not in ("ttft", "tpot", "e2el"):
            raise ValueError(f"unknown service-level objective {name!r} (ttft, tpot, e2el)")
        out[name] = float(ms) / 1e3
    return out


def summarise(results: list, dur: float, slo: dict | None = None,
              percentiles: tuple = (99,)) -> dict:
    """Throughput and latency statistics of finished requests; with ``slo`` also the rate of
    requests that met every objective."""
    ok = [r for r in results if r["ok"]]
    if not ok:
        return {"completed": 0, "failed": len(results),
                "errors": [r.get("error") for r in results][:3]}
    for r in ok:
        r["tpot"] = ((r["e2e"] - r["ttft"]) / max(1, r["n_out"] - 1)
                     if r["ttft"] is not None and r["n_out"] > 1 else None)
    ttft = np.array([r["ttft"] for r in ok if r["ttft"] is not None] or [0.0])
    e2e = np.array([r["e2e"] for r in ok])
    tpot = np.array([r["tpot"] for r in ok if r["tpot"] is not None] or [0.0])
    itl = np.array([x for r in ok for x in r["itl"]] or [0.0])

    def st(x):
        d = {"mean_ms": float(x.mean() * 1e3), "median_ms": float(np.median(x) * 1e3),
             "std_ms": float(x.std() * 1e3)}
        for p in percentiles:
            d[f"p{p:g}_ms"] = float(np.percentile(x, p) * 1e3)
        return d

    res = {"completed": len(ok), "failed": len(results) - len(ok), "duration_s": dur,
           "request_throughput": len(ok) / dur,
           "output_token_throughput": sum(r["n_out"] for r in ok) / dur,
           "total_token_throughput": sum(r["n_out"] + r["n_in"] for r in ok) / dur,
           "ttft": st(ttft), "tpot": st(tpot), "itl": st(itl), "e2el": st(e2e)}
    if slo:
        good = sum(1 for r in ok
                   if ("ttft" not in slo or (r["ttft"] is not None and r["ttft"] <= slo["ttft"]))
                   and ("tpot" not in slo or r["tpot"] is None or r["tpot"] <= slo["tpot"])
                   and ("e2el" not in slo or r["e2e"] <= slo["e2el"]))
        res["request_goodput"] = good / dur
        res["good_requests"] = good
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--ports", type=int, nargs="+", default=None,
                    help="several servers: requests are spread over them in turn")
    ap.add_argument("--max-concurrency", type=int, default=None)
    ap.add_argument("--goodput", nargs="+", default=None,
                    help="service-level objectives in ms, e.g. ttft:200 tpot:50 e2el:5000")
    ap.add_argument("--backend", default="openai", choices=["openai", "openai-chat"],
                    help="/v1/completions with token-id prompts, or /v1/chat/completions")
    ap.add_argument("--num-prompts", type=int, default=1000)
    ap.add_argument("--request-rate", type=float, default=float("inf"))
    ap.add_argument("--burstiness", type=float, default=1.0)
    ap.add_argument("--input-len-range", type=int, nargs=2, default=[256, 2048])
    ap.add_argument("--output-len-range", type=int, nargs=2, default=[64, 512])
    ap.add_argument("--vocab-size", type=int, default=32000)
    ap.add_argument("--dataset-name", default="random", choices=["random", "sharegpt", "sonnet"])
    ap.add_argument("--dataset-path", default=None)
    ap.add_argument("--tokenizer", default=None,
                    help="tokenizer directory for counting dataset tokens (else 4 chars / token)")
    ap.add_argument("--max-input-len", type=int, default=1024)
    ap.add_argument("--max-output-len", type=int, default=1024)
    ap.add_argument("--fixed-output-len", type=int, default=None)
    ap.add_argument("--sonnet-input-len", type=int, default=550)
    ap.add_argument("--sonnet-output-len", type=int, default=150)
    ap.add_argument("--sonnet-prefix-len", type=int, default=200)
    ap.add_argument("--metric-percentiles", default="99",
                    help="comma-separated percentiles of every latency metric, e.g. 50,90,99")
    ap.add_argument("--profile", action="store_true",
                    help="call the servers' /start_profile and /stop_profile around the run")
    ap.add_argument("--strict-in-out-len", action="store_true",
                    help="accepted for compatibility: requests always run to max_tokens "
                         "(ignore_eos) and token-id prompts have exact lengths")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--extra-body", default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--output-json", default=None)
    asyncio.run(run(ap.parse_args()))


if __name__ == "__main__":
    main()
