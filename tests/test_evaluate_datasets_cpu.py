"""The small-dataset accuracy harness (benchmarks/evaluate_datasets) on the CPU engine."""
import importlib.util
import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    path = os.path.join(ROOT, "benchmarks", "evaluate_datasets", name + ".py")
    spec = importlib.util.spec_from_file_location("evalds_" + name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_retrieval_metrics():
    r = _load("retrieval")
    rel = {"a": 2, "b": 1}
    assert r.ndcg_at_k(["a", "b", "c"], rel, 3) == 1.0
    assert 0 < r.ndcg_at_k(["c", "b", "a"], rel, 3) < 1.0
    assert r.mrr_at_k(["c", "a"], rel, 5) == 0.5 and r.mrr_at_k(["c"], rel, 5) == 0.0
    assert r.recall_at_k(["a", "x"], rel, 2) == 0.5
    docs = {"d1": "the cat sat on the mat", "d2": "stock markets fell today", "d3": "a cat and a dog"}
    assert r.bm25_rank("cat mat", docs, 2)[0] == "d1"
    s = r.summarise({"q1": ["d1", "d3"], "q2": ["d2"]}, {"q1": {"d1": 1}, "q2": {"d3": 1}}, 2)
    assert s["queries"] == 2 and s["mrr@2"] == 0.5


def test_multiple_choice_and_generation_modes(tmp_path):
    run = _load("run")
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.entrypoints.api_server import ByteTokenizer
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=8, max_num_batched_tokens=128,
              max_model_len=128, num_gpu_blocks=128, dtype="float32")
    tok = ByteTokenizer(32000)
    rows = [{"question": "2 + 2 =", "choices": ["3", "4", "5"], "answer": 1},
            {"question": "sky colour:", "choices": ["blue", "green"], "answer": 0}]
    path = tmp_path / "mc.jsonl"
    path.write_text("\n".join(json.dumps(r) for r in rows))
    loaded = run.load_rows(str(path))
    assert loaded == rows and len(run.load_rows(str(path), 1)) == 1
    sc = run.score_choices(llm, tok, rows[0]["question"], rows[0]["choices"])
    assert len(sc) == 3 and all(s < 0 for s in sc)         # log-probabilities
    m = run.evaluate(llm, tok, rows, "ppl")
    assert m["total"] == 2 and 0.0 <= m["accuracy"] <= 1.0
    # generation mode: the reference text is whatever the (random) model says for the prompt
    from vllm_gcu_b200.engine.request import SamplingParams
    out = llm.generate([list(tok.encode("hello"))], SamplingParams(max_tokens=4, temperature=0.0))
    said = tok.decode(list(out[0].outputs[0].token_ids))
    g = run.evaluate(llm, tok, [{"prompt": "hello", "reference": said}], "gen", max_tokens=4,
                     match="contains")
    assert g["correct"] == (1 if run.normalise(said) else g["correct"])
    run.save_csv(str(tmp_path / "r.csv"), __import__("argparse").Namespace(model="m"), m)
    assert (tmp_path / "r.csv").read_text().count("\n") == 2
