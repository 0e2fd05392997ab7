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


def _write_retrieval_dataset(d):
    import csv as _csv
    corpus = {"d1": "the cat sat on the mat", "d2": "stock markets fell sharply today",
              "d3": "a dog chased the cat", "d4": "central banks raised interest rates",
              "d5": "markets rallied after the banks spoke"}
    queries = {"q1": "cat on a mat", "q2": "banks and interest rates", "q3": "unjudged query"}
    os.makedirs(d / "qrels")
    (d / "corpus.jsonl").write_text("\n".join(
        json.dumps({"_id": k, "title": "", "text": v}) for k, v in corpus.items()))
    (d / "queries.jsonl").write_text("\n".join(
        json.dumps({"_id": k, "text": v}) for k, v in queries.items()))
    with open(d / "qrels" / "test.tsv", "w", newline="") as f:
        w = _csv.writer(f, delimiter="\t")
        w.writerow(["query-id", "corpus-id", "score"])
        w.writerows([["q1", "d1", 2], ["q1", "d3", 1], ["q2", "d4", 1], ["q2", "d5", 1]])
    return corpus, queries


def test_ir_metrics_bm25_and_dataset_loader(tmp_path):
    import sys
    sys.path.insert(0, os.path.join(ROOT, "benchmarks", "evaluate_datasets"))
    m = _load("ir_metrics")
    _write_retrieval_dataset(tmp_path)
    corpus, queries, qrels = m.load_retrieval_dataset(str(tmp_path))
    assert set(queries) == {"q1", "q2"} and qrels["q1"] == {"d1": 2, "d3": 1} and len(corpus) == 5
    rel = {"a": 2, "b": 1}
    assert m.ndcg_at_k(["a", "b"], rel, 10) == 1.0 and m.average_precision(["x", "a", "b"], rel) \
        == (1 / 2 + 2 / 3) / 2
    assert abs(m.spearman([1, 2, 3, 4], [10, 20, 30, 40]) - 1.0) < 1e-12
    assert abs(m.spearman([1, 2, 3, 4], [4, 3, 2, 1]) + 1.0) < 1e-12
    assert abs(m.spearman([1, 2, 2, 3], [1, 2, 2, 3]) - 1.0) < 1e-12      # ties
    bm = m.BM25(corpus)
    assert list(bm.top("cat mat", 2))[0] == "d1" and list(bm.top("interest rates", 1)) == ["d4"]
    perfect = {"q1": {"d1": 2.0, "d3": 1.0}, "q2": {"d4": 1.0, "d5": 0.5}}
    got = m.evaluate_rankings(perfect, qrels, ks=(1, 10))
    assert got["ndcg@10"] == 1.0 and got["mrr@10"] == 1.0 and got["recall@1"] == 0.5
    m.save_csv(str(tmp_path / "r.csv"), {"model": "x"}, got)
    m.save_csv(str(tmp_path / "r.csv"), {"model": "y"}, got)
    assert len((tmp_path / "r.csv").read_text().strip().splitlines()) == 3


def _bag_of_words_encoder(dim=1009):
    import numpy as np

    def encode(texts):
        out = np.zeros((len(texts), dim), dtype=np.float32)
        for i, t in enumerate(texts):
            for w in t.lower().split():
                out[i, sum((j + 1) * 131 * ord(c) for j, c in enumerate(w)) % dim] += 1.0
        return out / np.maximum(np.linalg.norm(out, axis=-1, keepdims=True), 1e-9)
    return encode


def test_embedding_and_reranking_evaluators(tmp_path):
    import sys
    sys.path.insert(0, os.path.join(ROOT, "benchmarks", "evaluate_datasets"))
    m = _load("ir_metrics")
    ee, er = _load("evaluate_embeddings"), _load("evaluate_reranking")
    corpus, _ = _write_retrieval_dataset(tmp_path)
    data = m.load_retrieval_dataset(str(tmp_path))
    enc = _bag_of_words_encoder()
    got = ee.evaluate_retrieval(enc, *data, batch_size=2)
    assert got["recall@10"] == 1.0 and got["ndcg@10"] > 0.6
    rows = [{"sentence1": "a cat on a mat", "sentence2": "the cat sat on the mat", "score": 4.5},
            {"sentence1": "a cat on a mat", "sentence2": "the dog chased a bird", "score": 2.0},
            {"sentence1": "a cat on a mat", "sentence2": "banks raised rates", "score": 0.0}]
    sts = ee.evaluate_sts(enc, rows, batch_size=2)
    assert sts["cosine_spearman"] == 1.0 and sts["pairs"] == 3.0

    def oracle_reranker(query, docs):          # knows the judgements: must lift every metric
        qid = next(q for q, t in data[1].items() if t == query)
        ids = {v: k for k, v in data[0].items()}
        return [float(data[2][qid].get(ids[d], 0)) for d in docs]
    first, second = er.evaluate(oracle_reranker, *data, initial_top_k=5, rerank_top_k=5)
    assert second["ndcg@10"] == 1.0 and second["ndcg@10"] >= first["ndcg@10"]
    assert second["map"] == 1.0
