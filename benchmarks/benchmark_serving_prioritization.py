"""Serving benchmark with request priorities over one or several servers.

The measured requests are sent with a high priority (``--priority``, default 1; smaller runs
first) to a randomly chosen server, while every server is kept busy by one background request
of the lowest priority (100) at a time: as soon as one of them finishes, the next is sent to the
same server.  On servers started with ``--scheduling-policy priority`` the measured requests
overtake that background load; the report is the one of ``benchmark_serving.py`` plus the number
of background requests that ran (benchmarks/benchmark_serving_prioritization.py:651-755 of the
reference keeps its servers stepping the same way).

Example:
  python -m vllm_gcu_b200.entrypoints.api_server --model llama-3-8b --port 8000 \
      --scheduling-policy priority &
  python benchmarks/benchmark_serving_prioritization.py --ports 8000 --num-prompts 200 \
      --request-rate 8 --goodput ttft:500
"""
import argparse
import asyncio
import json
import os
import random
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from benchmark_serving import one_request, parse_goodput, summarise  # noqa: E402

BACKGROUND_PRIORITY = 100


async def background_request(session, url: str, vocab_size: int, tokens: int, seed: int) -> str:
    """One lowest-priority request; returns its server's url when it is over."""
    rng = random.Random(seed)
    body = {"prompt": [rng.randrange(10, vocab_size) for _ in range(8)], "max_tokens": tokens,
            "temperature": 0.0, "stream": True, "ignore_eos": True,
            "priority": BACKGROUND_PRIORITY}
    try:
        async with session.post(url, json=body) as resp:
            async for _ in resp.content:
                pass
    except Exception:  # noqa: BLE001 - the background load never fails the benchmark
        await asyncio.sleep(0.05)
    return url


async def run(args) -> dict:
    import aiohttp
    rng = random.Random(args.seed)
    nprng = np.random.default_rng(args.seed)
    urls = [f"http://{args.host}:{p}/v1/completions" for p in args.ports]
    extra = json.loads(args.extra_body) if args.extra_body else {}
    results: list = []
    timeout = aiohttp.ClientTimeout(total=6 * 3600)
    n_background = 0
    async with aiohttp.ClientSession(timeout=timeout) as session:
        background = {asyncio.create_task(background_request(
            session, u, args.vocab_size, args.background_tokens, i)) for i, u in enumerate(urls)}
        n_background = len(background)
        t_start = time.perf_counter()
        tasks = []
        for i in range(args.num_prompts):
            n_in = rng.randint(*args.input_len_range)
            n_out = rng.randint(*args.output_len_range)
            body = {"prompt": [rng.randrange(10, args.vocab_size) for _ in range(n_in)],
                    "max_tokens": n_out, "temperature": 0.0, "stream": True,
                    "ignore_eos": True, "priority": args.priority, **extra}
            tasks.append(asyncio.create_task(
                one_request(session, rng.choice(urls), body, results)))
            if args.request_rate != float("inf"):
                theta = 1.0 / (args.request_rate * args.burstiness)
                await asyncio.sleep(float(nprng.gamma(shape=args.burstiness, scale=theta)))
        # a new background request for a server as soon as its last one is over
        while any(not t.done() for t in tasks):
            done, _ = await asyncio.wait(background | {t for t in tasks if not t.done()},
                                         return_when=asyncio.FIRST_COMPLETED)
            for d in done & background:
                background.remove(d)
                background.add(asyncio.create_task(background_request(
                    session, d.result(), args.vocab_size, args.background_tokens,
                    n_background)))
                n_background += 1
        await asyncio.gather(*tasks)
        dur = time.perf_counter() - t_start
        for b in background:
            b.cancel()
        await asyncio.gather(*background, return_exceptions=True)
    res = summarise(results, dur, parse_goodput(args.goodput))
    res["background_requests"] = n_background
    res["priority"] = args.priority
    print(json.dumps(res, indent=1))
    if args.output_json:
        with open(args.output_json, "w") as f:
            json.dump(res, f)
    return res


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--ports", type=int, nargs="+", default=[8000])
    ap.add_argument("--num-prompts", type=int, default=200)
    ap.add_argument("--request-rate", type=float, default=float("inf"))
    ap.add_argument("--burstiness", type=float, default=1.0)
    ap.add_argument("--input-len-range", type=int, nargs=2, default=[256, 2048])
    ap.add_argument("--output-len-range", type=int, nargs=2, default=[64, 512])
    ap.add_argument("--vocab-size", type=int, default=32000)
    ap.add_argument("--priority", type=int, default=1)
    ap.add_argument("--background-tokens", type=int, default=64,
                    help="output length of the lowest-priority background requests")
    ap.add_argument("--goodput", nargs="+", default=None)
    ap.add_argument("--extra-body", default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--output-json", default=None)
    return asyncio.run(run(ap.parse_args(argv)))


if __name__ == "__main__":
    main()
