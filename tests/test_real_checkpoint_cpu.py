"""A checkpoint directory as users have it (config.json, generation_config.json, safetensors,
tokenizer files with a chat template), built here with a small trained BPE tokenizer: text in /
text out against transformers, chat template, end-of-sequence stopping, guided decoding over the
real vocabulary, embeddings, and the same through the server."""
import asyncio

import pytest
import torch

tr = pytest.importorskip("transformers")
tokenizers = pytest.importorskip("tokenizers")


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    d = str(tmp_path_factory.mktemp("ckpt"))
    tok = Tokenizer(models.BPE(unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    corpus = ["the quick brown fox jumps over the lazy dog", "hello world, how are you today?",
              "0123456789 - phone 555-1234", '{"name": "x", "age": 3}',
              "user: hi assistant: hello"] * 20
    tok.train_from_iterator(corpus, trainers.BpeTrainer(
        vocab_size=400, special_tokens=["<unk>", "<s>", "</s>"],
        initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    fast = tr.PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>",
                                      unk_token="<unk>")
    fast.chat_template = ("{% for m in messages %}{{ m['role'] }}: {{ m['content'] }}\n"
                          "{% endfor %}{% if add_generation_prompt %}assistant: {% endif %}")
    fast.save_pretrained(d)
    cfg = tr.LlamaConfig(vocab_size=len(fast), hidden_size=64, intermediate_size=128,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         max_position_embeddings=256, rms_norm_eps=1e-6,
                         tie_word_embeddings=False, bos_token_id=1, eos_token_id=2)
    torch.manual_seed(0)
    tr.LlamaForCausalLM(cfg).save_pretrained(d, safe_serialization=True)
    return d


def _llm(ckpt):
    from vllm_gcu_b200 import LLM
    return LLM(ckpt, device="cpu", max_num_seqs=32, max_num_batched_tokens=128,
               max_model_len=128, num_gpu_blocks=128, dtype="float32")


def test_text_chat_eos_guided_and_embeddings(ckpt):
    from vllm_gcu_b200 import SamplingParams
    llm = _llm(ckpt)
    hf = tr.AutoModelForCausalLM.from_pretrained(ckpt).eval().float()
    tok = tr.AutoTokenizer.from_pretrained(ckpt)
    assert llm.engine.cfg.model.eos_token_ids == (2,)
    sp = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
    out = llm.generate("the quick brown fox", sp)[0]
    ids = tok.encode("the quick brown fox")
    want = hf.generate(torch.tensor([ids]), attention_mask=torch.ones(1, len(ids), dtype=torch.long),
                       max_new_tokens=8, do_sample=False, pad_token_id=0)[0, len(ids):].tolist()
    assert out.prompt_token_ids == ids and out.outputs[0].token_ids == want
    assert out.outputs[0].text == tok.decode(want, skip_special_tokens=True)
    chat = llm.chat([{"role": "user", "content": "hello world"}], sp)[0]
    assert tok.decode(chat.prompt_token_ids) == "user: hello world\nassistant: "
    # sampled requests stop at the checkpoint's end-of-sequence id, which stays out of the text
    outs = llm.generate(["hello"] * 24, [SamplingParams(max_tokens=60, temperature=1.5, seed=i)
                                         for i in range(24)])
    stopped = [o.outputs[0] for o in outs if o.outputs[0].finish_reason == "stop"]
    assert stopped and all(c.token_ids[-1] == 2 and "</s>" not in c.text for c in stopped)
    assert not any(2 in o.outputs[0].token_ids[:-1] for o in outs)
    same = llm.generate(["hello"], SamplingParams(max_tokens=60, temperature=1.5, seed=0,
                                                  ignore_eos=True))[0]
    assert len(same.outputs[0].token_ids) == 60
    # guided decoding over a real byte-level BPE vocabulary
    import json
    import re
    g = llm.generate("phone ", SamplingParams(max_tokens=12, temperature=0.0,
                                              guided_regex=r"\d{3}-\d{4}"))[0].outputs[0]
    assert re.fullmatch(r"\d{3}-\d{4}", g.text) and g.finish_reason == "stop"
    schema = {"type": "object", "properties": {"age": {"type": "integer"}}, "required": ["age"]}
    j = llm.generate("json ", SamplingParams(max_tokens=60, temperature=0.0,
                                             guided_json=schema))[0].outputs[0]
    assert isinstance(json.loads(j.text)["age"], int)
    e = llm.embed(["hello world", "the lazy dog"])
    assert e.shape == (2, 64) and torch.allclose(e.norm(dim=-1), torch.ones(2), atol=1e-5)


@pytest.mark.timeout(180)
def test_server_on_the_checkpoint(ckpt):
    httpx = pytest.importorskip("httpx")
    import argparse
    from vllm_gcu_b200.entrypoints.api_server import (add_engine_arguments, build_app,
                                                      load_tokenizer, make_engine)
    ap = argparse.ArgumentParser()
    add_engine_arguments(ap)
    a = ap.parse_args(["--model", ckpt, "--device", "cpu", "--max-num-seqs", "8",
                       "--max-num-batched-tokens", "64", "--max-model-len", "128",
                       "--num-gpu-blocks", "64", "--dtype", "float32"])
    a.host, a.kv_port = "127.0.0.1", 0
    eng, mc = make_engine(a)
    tok = load_tokenizer(ckpt, mc.vocab_size)
    app = build_app(eng, tok, "tiny")

    async def run():
        transport = httpx.ASGITransport(app=app)
        async with httpx.AsyncClient(transport=transport, base_url="http://t") as c:
            r = (await c.post("/v1/chat/completions", json={
                "messages": [{"role": "user", "content": "hello world"}], "max_tokens": 6,
                "temperature": 0.0, "ignore_eos": True})).json()
            assert r["usage"]["prompt_tokens"] == len(tok.encode("user: hello world\nassistant: "))
            assert isinstance(r["choices"][0]["message"]["content"], str)
            g = (await c.post("/v1/completions", json={
                "prompt": "phone ", "max_tokens": 12, "temperature": 0.0,
                "guided_regex": r"\d{3}-\d{4}"})).json()
            import re
            assert re.fullmatch(r"\d{3}-\d{4}", g["choices"][0]["text"])
            assert g["choices"][0]["finish_reason"] == "stop"
            t = (await c.post("/tokenize", json={"prompt": "the lazy dog"})).json()
            assert t["tokens"] == tok.encode("the lazy dog")
    try:
        asyncio.run(run())
    finally:
        eng.shutdown()


def test_stop_strings_offline_and_through_the_server(ckpt):
    """``stop`` strings end a request as soon as its text contains one: the text is cut in front
    of it (or behind it with ``include_stop_str_in_output``) and no further tokens are
    generated; the server honours the OpenAI ``stop`` field the same way."""
    from vllm_gcu_b200 import SamplingParams
    httpx = pytest.importorskip("httpx")
    llm = _llm(ckpt)
    base = SamplingParams(max_tokens=30, temperature=0.0, ignore_eos=True)
    full = llm.generate("the quick brown fox", base)[0].outputs[0]
    assert len(full.token_ids) == 30 and len(full.text) > 8
    needle = full.text[5:8]                              # a piece that will appear
    where = full.text.find(needle)
    import dataclasses
    cut = llm.generate("the quick brown fox", dataclasses.replace(base, stop=(needle,)))[0]
    c = cut.outputs[0]
    assert c.text == full.text[:where] and c.finish_reason == "stop"
    assert len(c.token_ids) < 30 and c.token_ids == full.token_ids[:len(c.token_ids)]
    keep = llm.generate("the quick brown fox", dataclasses.replace(
        base, stop=(needle, "never-there"), include_stop_str_in_output=True))[0].outputs[0]
    assert keep.text == full.text[:where + len(needle)]
    miss = llm.generate("the quick brown fox", dataclasses.replace(base, stop=("@@@@",)))[0]
    assert miss.outputs[0].text == full.text and miss.outputs[0].finish_reason == "length"
    # the server: same cut, and the engine is free again right away
    from vllm_gcu_b200.engine.async_llm import AsyncLLM
    from vllm_gcu_b200.entrypoints.api_server import build_app, load_tokenizer
    eng = AsyncLLM(llm.engine.cfg)
    app = build_app(eng, load_tokenizer(ckpt, 0), "tiny")

    async def run():
        transport = httpx.ASGITransport(app=app)
        async with httpx.AsyncClient(transport=transport, base_url="http://t") as cl:
            body = {"prompt": "the quick brown fox", "max_tokens": 30, "temperature": 0.0,
                    "ignore_eos": True, "stop": [needle]}
            r = (await cl.post("/v1/completions", json=body)).json()["choices"][0]
            assert r["text"] == full.text[:where] and r["finish_reason"] == "stop"
            assert len(r["token_ids"]) < 30
            r2 = (await cl.post("/v1/completions", json={**body, "stop": needle,
                                                         "include_stop_str_in_output": True}))
            assert r2.json()["choices"][0]["text"] == full.text[:where + len(needle)]
    import asyncio as _a
    try:
        _a.run(run())
    finally:
        eng.shutdown()


def test_server_uses_the_checkpoints_sampling_defaults(ckpt, tmp_path):
    """``generation_config.json`` of the checkpoint: its temperature / top-k / top-p /
    repetition penalty apply to requests that do not set them."""
    import json
    import os
    import shutil
    from vllm_gcu_b200.config import ModelConfig
    from vllm_gcu_b200.entrypoints.api_server import sampling_from_body
    d = str(tmp_path / "c")
    shutil.copytree(ckpt, d)
    with open(os.path.join(d, "generation_config.json"), "w") as f:
        json.dump({"do_sample": True, "temperature": 0.7, "top_p": 0.8, "top_k": 20,
                   "repetition_penalty": 1.05, "eos_token_id": [2, 5]}, f)
    mc = ModelConfig.from_pretrained(d)
    gd = mc.extra["generation_defaults"]
    assert gd == {"temperature": 0.7, "top_p": 0.8, "top_k": 20, "repetition_penalty": 1.05}
    assert mc.eos_token_ids == (2, 5)
    sp = sampling_from_body({"max_tokens": 4}, defaults=gd)
    assert (sp.temperature, sp.top_p, sp.top_k, sp.repetition_penalty) == (0.7, 0.8, 20, 1.05)
    sp = sampling_from_body({"max_tokens": 4, "temperature": 0.0, "top_k": 0}, defaults=gd)
    assert sp.temperature == 0.0 and sp.top_k == 0 and sp.top_p == 0.8
