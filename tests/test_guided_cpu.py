"""Grammar-guided decoding (engine/guided.py): the pattern compiler against Python's ``re``,
token masks over a multi-character vocabulary, JSON schemas, and requests through the engine
(the reference benchmarks this feature with benchmarks/benchmark_guided.py)."""
import json
import re

import pytest
import torch

from vllm_gcu_b200.engine.guided import (GuideCursor, RegexGuide, RegexSyntaxError,
                                         json_schema_to_regex)
from vllm_gcu_b200.engine.llm import LLM
from vllm_gcu_b200.engine.request import SamplingParams

PATTERNS = [
    r"abc", r"a|b|cd", r"(ab)+c?", r"[a-c]{2,4}x", r"\d{3}-\d{4}", r"[^0-9]+",
    r"(yes|no)(, (yes|no))*", r"-?(0|[1-9][0-9]*)(\.[0-9]+)?", r"a.c", r"\w+@\w+\.(com|org)",
    r"(a|b)*abb", r"x{0,2}y{2}", r"[\]\-a]+", r"\s*\S+\s*", r"(?:ab|a)(?:bc|c)?",
]
STRINGS = ["", "abc", "a", "cd", "ababc", "abab", "abcx", "aabbx", "555-1234", "55-1234", "hello",
           "h3llo", "yes, no, yes", "yes,no", "-12.50", "012", "0", "a\nc", "axc", "me@site.org",
           "me@site.net", "babb", "abba", "xyy", "xxxyy", "yy", "]-a", " word ", "two words", "abc",
           "ac", "abbc", "aa"]


@pytest.mark.parametrize("pattern", PATTERNS)
def test_automaton_accepts_the_same_strings_as_re(pattern):
    g = RegexGuide(pattern, [], None)
    for s in STRINGS:
        assert g.matches(s) == (re.fullmatch(pattern, s) is not None), (pattern, s)


def test_syntax_errors_are_reported():
    for bad in ["(ab", "a{3,1}", "*a", "[abc", "(?=a)b"]:
        with pytest.raises(RegexSyntaxError):
            RegexGuide(bad, [], None)


def test_token_moves_over_multi_character_tokens():
    vocab = ["a", "b", "ab", "abc", "c", "1", "12", "123", " ", None, "<eos>"]
    eos = 10
    g = RegexGuide(r"(ab)+c?\d{2}", vocab, eos)
    tok = {t: i for i, t in enumerate(vocab) if t}
    assert set(g.allowed(g.start)) == {tok["a"], tok["ab"], tok["abc"]}
    s = g.advance(g.start, tok["abc"])                       # "abc": only two digits may follow
    assert set(g.allowed(s)) == {tok["1"], tok["12"]}         # "123" would be one digit too many
    s2 = g.advance(s, tok["12"])
    assert g.accepting(s2) and g.exhausted(s2) and g.allowed(s2) == [eos]
    s3 = g.advance(g.start, tok["ab"])                       # "ab": another "ab", "c" or digits
    assert set(g.allowed(s3)) == {tok["a"], tok["ab"], tok["abc"], tok["c"], tok["1"], tok["12"]}
    # a cursor follows the output incrementally and survives a roll-back
    cur = GuideCursor(g)
    assert set(cur.allowed_next([tok["ab"]])) == set(g.allowed(s3))
    assert cur.allowed_next([tok["ab"], tok["1"]]) == [tok["1"]]
    assert not cur.finished([tok["ab"], tok["1"]])
    assert cur.finished([tok["ab"], tok["1"], tok["1"]])
    assert set(cur.allowed_next([])) == set(g.allowed(g.start))


SCHEMA = {
    "type": "object",
    "properties": {
        "name": {"type": "string", "maxLength": 8},
        "age": {"type": "integer"},
        "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "maxItems": 3},
        "score": {"type": ["number", "null"]},
        "nick": {"type": "string"},
    },
    "required": ["name", "age", "tags", "score"],
}


def test_json_schema_pattern_accepts_valid_documents_only():
    pat = json_schema_to_regex(SCHEMA)
    g = RegexGuide(pat, [], None)
    good = [
        {"name": "Ada", "age": 36, "tags": [], "score": 1.5},
        {"name": "", "age": -1, "tags": ["a", "b", "a"], "score": None, "nick": "x\"y"},
        {"name": "Bob", "age": 0, "tags": ["b"], "score": 2e3},
    ]
    for doc in good:
        for text in (json.dumps(doc), json.dumps(doc, separators=(",", ":"))):
            assert g.matches(text), text
            assert re.fullmatch(pat, text), text
    bad = [
        '{"name": "Ada"}',                                               # required keys missing
        '{"name": "waytoolongname", "age": 1, "tags": [], "score": 1}',  # maxLength
        '{"name": "Ada", "age": 1.5, "tags": [], "score": 1}',           # not an integer
        '{"name": "Ada", "age": 1, "tags": ["c"], "score": 1}',          # not in the enum
        '{"name": "Ada", "age": 1, "tags": ["a","a","a","a"], "score": 1}',
        '{"age": 1, "name": "Ada", "tags": [], "score": 1}',             # declaration order
    ]
    for text in bad:
        assert not g.matches(text), text


def _char_vocab(n):
    # token id = code point for printable ASCII, a few multi-character tokens above them
    vocab = [None] * n
    for c in range(32, 127):
        vocab[c] = chr(c)
    extra = ["yes", "no", "true", "false", '":', '", "', "{\"", "null", "10", "2024"]
    for i, t in enumerate(extra):
        vocab[200 + i] = t
    return vocab


def _decode(vocab, ids, eos):
    return "".join(vocab[t] for t in ids if t != eos)


def test_engine_regex_and_json_requests_match_their_grammar():
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=8, max_num_batched_tokens=64,
              max_model_len=256, num_gpu_blocks=256, dtype="float32")
    V = llm.engine.cfg.model.vocab_size
    vocab = _char_vocab(V)
    eos = 2
    llm.set_vocabulary(vocab)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(300, V, (9 + i,), generator=g).tolist() for i in range(4)]
    pattern = r"(yes|no)(, (yes|no)){1,2}!"
    small = {"type": "object", "properties": {"ok": {"type": "boolean"},
                                              "n": {"type": "integer"},
                                              "s": {"type": "string", "maxLength": 4}}}
    sps = [SamplingParams(max_tokens=64, temperature=1.0, seed=11, guided_regex=pattern),
           SamplingParams(max_tokens=64, temperature=0.0, guided_regex=pattern),
           SamplingParams(max_tokens=120, temperature=0.8, seed=5, top_k=50, guided_json=small),
           SamplingParams(max_tokens=16, temperature=0.0)]                 # unguided neighbour
    rids = [llm.engine.add_request(p, sp, eos_token_id=eos) for p, sp in zip(prompts, sps)]
    final = {}
    while llm.engine.has_unfinished():
        for ro in llm.engine.step():
            if ro.finished:
                final[ro.request_id] = ro
    outs = [final[r] for r in rids]
    for o in outs[:2]:
        text = _decode(vocab, o.outputs[0].token_ids, eos)
        assert re.fullmatch(pattern, text), text
        assert o.outputs[0].finish_reason == "stop"
    text = _decode(vocab, outs[2].outputs[0].token_ids, eos)
    if outs[2].outputs[0].finish_reason == "stop":
        doc = json.loads(text)
        assert isinstance(doc["ok"], bool) and isinstance(doc["n"], int) and len(doc["s"]) <= 4
    else:                                   # ran into max_tokens: still a prefix of the grammar
        assert text.startswith("{")
    assert len(outs[3].outputs[0].token_ids) == 16

    # without a vocabulary the request is refused, not silently unguided
    llm2 = LLM("tiny-llama", device="cpu", max_num_seqs=2, max_num_batched_tokens=32,
               max_model_len=64, num_gpu_blocks=32, dtype="float32")
    with pytest.raises(ValueError):
        llm2.engine.add_request(prompts[0], SamplingParams(guided_regex="a+"))
