"""Guided-decoding benchmark: throughput and validity of regex / JSON-schema requests against
the same requests without a grammar (the reference ships benchmarks/benchmark_guided.py, which
sends structured-output requests and reports throughput and the fraction of valid outputs).

Without tokenizer files the vocabulary is synthetic: printable ASCII characters plus common
multi-character pieces, the rest of the ids unusable for guided requests.

  python benchmarks/benchmark_guided.py --model tiny-llama --device cpu --num-prompts 8
"""
import argparse
import json
import os
import re
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from vllm_gcu_b200.engine.guided import json_schema_to_regex  # noqa: E402
from vllm_gcu_b200.engine.llm import LLM  # noqa: E402
from vllm_gcu_b200.engine.request import SamplingParams  # noqa: E402

SCHEMA = {"type": "object",
          "properties": {"name": {"type": "string", "maxLength": 12},
                         "age": {"type": "integer"},
                         "skills": {"type": "array", "items": {"type": "string", "maxLength": 8},
                                    "maxItems": 3},
                         "active": {"type": "boolean"}}}
REGEX = r"(\d{1,3}\.){3}\d{1,3}"


def synthetic_vocab(n: int) -> list:
    vocab = [None] * n
    for c in range(32, 127):
        vocab[c] = chr(c)
    pieces = ['{"', '":', '", "', '"}', "true", "false", "null", "name", "age", "skills",
              "active", " ", "10", "192", "168", ".1", "[]", '["', '"]', ": "]
    for i, t in enumerate(pieces):
        if 200 + i < n:
            vocab[200 + i] = t
    return vocab


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--tokenizer", default=None, help="directory with tokenizer files")
    ap.add_argument("--device", default="auto")
    ap.add_argument("--num-prompts", type=int, default=64)
    ap.add_argument("--input-len", type=int, default=64)
    ap.add_argument("--output-len", type=int, default=96)
    ap.add_argument("--dtype", default=None)
    ap.add_argument("--structure", default="json", choices=["json", "regex"])
    a = ap.parse_args()
    llm = LLM(a.model, device=a.device, dtype=a.dtype,
              max_model_len=a.input_len + a.output_len + 16)
    V = llm.engine.cfg.model.vocab_size
    if a.tokenizer:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(a.tokenizer)
        from vllm_gcu_b200.engine.guided import vocabulary_of
        vocab, eos = vocabulary_of(tok, V), tok.eos_token_id
    else:
        vocab, eos = synthetic_vocab(V), 2
    llm.set_vocabulary(vocab)
    pattern = json_schema_to_regex(SCHEMA) if a.structure == "json" else REGEX
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(300, V, (a.input_len,), generator=g).tolist()
               for _ in range(a.num_prompts)]
    res = {"structure": a.structure, "num_prompts": a.num_prompts}
    for name, extra in (("unguided", {}), ("guided", {"guided_regex": pattern})):
        sp = SamplingParams(max_tokens=a.output_len, temperature=0.8, seed=1, **extra)
        t0 = time.perf_counter()
        rids = [llm.engine.add_request(p, sp, eos_token_id=eos) for p in prompts]
        final = {}
        while llm.engine.has_unfinished():
            for ro in llm.engine.step():
                if ro.finished:
                    final[ro.request_id] = ro
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        outs = [final[r].outputs[0] for r in rids]
        n_tok = sum(len(o.token_ids) for o in outs)
        row = {"seconds": dt, "output_tokens": n_tok, "tokens_per_s": n_tok / max(dt, 1e-9)}
        if extra:
            texts = ["".join(vocab[t] or "" for t in o.token_ids if t != eos) for o in outs]
            done = [t for t, o in zip(texts, outs) if o.finish_reason == "stop"]
            row["finished"] = len(done)
            row["valid"] = sum(re.fullmatch(pattern, t) is not None for t in done)
            if a.structure == "json":
                row["parsed"] = sum(_parses(t) for t in done)
        res[name] = row
    print(json.dumps(res, indent=1))


def _parses(text: str) -> bool:
    try:
        json.loads(text)
        return True
    except ValueError:
        return False


if __name__ == "__main__":
    main()
