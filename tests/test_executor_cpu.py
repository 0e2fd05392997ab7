"""Multi-process executor on CPU ranks (gloo): tensor parallelism and failure detection.

Failures are injected on the host (a worker that raises, a worker process that exits); no
device is involved.
"""
import os

import pytest
import torch

from vllm_gcu_b200.config import (CacheConfig, EngineConfig, ParallelConfig, SchedulerConfig,
                                  preset)
from vllm_gcu_b200.engine.executor import EngineDeadError, MultiprocExecutor
from vllm_gcu_b200.engine.llm import LLMEngine
from vllm_gcu_b200.engine.request import SamplingParams


def _cfg(tp):
    return EngineConfig(model=preset("tiny-llama"),
                        cache=CacheConfig(block_size=16, num_gpu_blocks=64),
                        scheduler=SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=64,
                                                  max_model_len=128),
                        parallel=ParallelConfig(tensor_parallel_size=tp, comm_backend="nccl"),
                        device="cpu", seed=0)


def _prompts():
    g = torch.Generator().manual_seed(4)
    return [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (17, 40, 5)]


@pytest.mark.timeout(300)
def test_tp2_executor_matches_single_process():
    sp = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
    ex = MultiprocExecutor(_cfg(2))
    try:
        # commands reach both ranks through one shared-memory ring
        from vllm_gcu_b200.utils import shm_ring
        assert (ex.rings is not None) == shm_ring.available()
        outs = ex.generate(_prompts(), sp)
        ex.check_health()
    finally:
        ex.shutdown()
    assert ex.rings is None
    # The TP workers initialise their shards from per-shard seeds, so compare structure and
    # determinism rather than token identity with a TP=1 engine.
    assert [len(o.outputs[0].token_ids) for o in outs] == [8, 8, 8]
    os.environ["VLLM_B200_SHM_BROADCAST"] = "0"      # same result over pipe-backed queues
    try:
        ex2 = MultiprocExecutor(_cfg(2))
    finally:
        del os.environ["VLLM_B200_SHM_BROADCAST"]
    try:
        assert ex2.rings is None
        outs2 = ex2.generate(_prompts(), sp)
    finally:
        ex2.shutdown()
    assert [o.outputs[0].token_ids for o in outs] == [o.outputs[0].token_ids for o in outs2]


@pytest.mark.timeout(300)
@pytest.mark.parametrize("what", ["raise", "exit"])
def test_worker_failure_is_detected(what):
    ex = MultiprocExecutor(_cfg(2))
    try:
        sp = SamplingParams(max_tokens=64, temperature=0.0, ignore_eos=True)
        ex.add_request(_prompts()[0], sp)
        ex.inject_fault(what, 1)
        with pytest.raises(EngineDeadError) as ei:
            for _ in range(600):
                ex.poll(0.1)
        assert "worker" in str(ei.value)
        with pytest.raises(EngineDeadError):
            ex.add_request([1, 2, 3], sp)
    finally:
        ex.shutdown()


def _dp_cfg():
    mc = preset("tiny-qwen3-moe")
    mc.extra["dp_attention"] = True
    return EngineConfig(model=mc, cache=CacheConfig(block_size=16, num_gpu_blocks=64),
                        scheduler=SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=64,
                                                  max_model_len=128),
                        parallel=ParallelConfig(data_parallel_size=2, enable_expert_parallel=True,
                                                comm_backend="nccl"),
                        device="cpu", seed=0)


@pytest.mark.timeout(300)
def test_dp2_ep_executor_keeps_idle_replica_in_step():
    """Data-parallel attention with expert parallelism: requests are spread over two
    replicas; with a single request one replica is idle and must still join every
    expert-parallel exchange (zero-token forward), otherwise the busy one would stall."""
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 30, 4, 21, 13)]
    ex = MultiprocExecutor(_dp_cfg())
    try:
        one = ex.generate(prompts[:1], sp, timeout_s=120)
        many = ex.generate(prompts, sp, timeout_s=120)
        ex.check_health()
    finally:
        ex.shutdown()
    assert len(one[0].outputs[0].token_ids) == 6
    assert [len(o.outputs[0].token_ids) for o in many] == [6] * 5
    # the first prompt gives the same tokens whether or not the other replica has work:
    # a request only sees its own tokens and the (replicated or expert-sharded) weights
    assert many[0].outputs[0].token_ids == one[0].outputs[0].token_ids


def _moe_checkpoint(path, mc):
    """Random Qwen3-MoE weights under HuggingFace names (one tensor per expert projection)."""
    from vllm_gcu_b200.models import build_model
    from vllm_gcu_b200.utils.weights import write_safetensors
    src = build_model(mc, "cpu")
    src.init_random(3, std=0.05)
    D, Hq, Hkv = mc.head_dim, mc.num_attention_heads, mc.num_key_value_heads
    I = mc.moe_intermediate_size
    out = {}
    for name, p_ in src.state_dict().items():
        if name.startswith(("layers.", "embed_tokens.", "norm.")):
            name = "model." + name
        if ".qkv_proj.weight" in name:
            q, k, v = p_.split([Hq * D, Hkv * D, Hkv * D], 0)
            for n, t in (("q_proj", q), ("k_proj", k), ("v_proj", v)):
                out[name.replace("qkv_proj", n)] = t.clone()
        elif name.endswith(".experts.w13"):
            for e in range(p_.shape[0]):
                base = name[:-len("w13")] + f"{e}."
                out[base + "gate_proj.weight"] = p_[e, :I].clone()
                out[base + "up_proj.weight"] = p_[e, I:].clone()
        elif name.endswith(".experts.w2"):
            for e in range(p_.shape[0]):
                out[name[:-len("w2")] + f"{e}.down_proj.weight"] = p_[e].clone()
        else:
            out[name] = p_.clone()
    write_safetensors(os.path.join(path, "model.safetensors"), out)


@pytest.mark.timeout(300)
def test_dp2_etp_executor_matches_single_process(tmp_path):
    """ETP (data-parallel attention, no expert parallelism): experts are sharded over the two
    replicas, rows are gathered and the sums scattered back every MoE layer.  The tokens are
    those of one unsharded engine, with one replica idle or both busy."""
    from vllm_gcu_b200.engine.llm import LLMEngine
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 30, 4, 21)]
    _moe_checkpoint(str(tmp_path), preset("tiny-qwen3-moe"))
    cfg = _dp_cfg()
    cfg.parallel.enable_expert_parallel = False
    cfg.load_format, cfg.model_path = "safetensors", str(tmp_path)
    ex = MultiprocExecutor(cfg)
    try:
        one = ex.generate(prompts[:1], sp, timeout_s=120)
        many = ex.generate(prompts, sp, timeout_s=120)
        ex.check_health()
    finally:
        ex.shutdown()
    single = _dp_cfg()
    single.parallel = ParallelConfig()
    single.model.extra.pop("dp_attention")
    single.load_format, single.model_path = "safetensors", str(tmp_path)
    eng = LLMEngine(single)
    for i_, p_ in enumerate(prompts):
        eng.add_request(p_, sp, request_id=str(i_))
    want = {}
    while eng.has_unfinished():
        for o in eng.step():
            if o.finished:
                want[int(o.request_id)] = o.outputs[0].token_ids
    assert [o.outputs[0].token_ids for o in many] == [want[i_] for i_ in range(len(prompts))]
    assert one[0].outputs[0].token_ids == want[0]


@pytest.mark.timeout(400)
def test_dp2_tp2_ep_executor_matches_single_process(tmp_path):
    """Expert parallelism over four ranks arranged as two replicas of two tensor-parallel
    ranks: every tensor-parallel rank dispatches its slice of the replica's rows (decode steps
    leave one of them with no row at all); the tokens are those of one unsharded engine."""
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 30, 4, 21)]
    _moe_checkpoint(str(tmp_path), preset("tiny-qwen3-moe"))
    cfg = _dp_cfg()
    cfg.parallel.tensor_parallel_size = 2
    cfg.load_format, cfg.model_path = "safetensors", str(tmp_path)
    ex = MultiprocExecutor(cfg)
    try:
        many = ex.generate(prompts, sp, timeout_s=200)
        ex.check_health()
    finally:
        ex.shutdown()
    single = _dp_cfg()
    single.parallel = ParallelConfig()
    single.model.extra.pop("dp_attention")
    single.load_format, single.model_path = "safetensors", str(tmp_path)
    eng = LLMEngine(single)
    for i_, p_ in enumerate(prompts):
        eng.add_request(p_, sp, request_id=str(i_))
    want = {}
    while eng.has_unfinished():
        for o in eng.step():
            if o.finished:
                want[int(o.request_id)] = o.outputs[0].token_ids
    assert [o.outputs[0].token_ids for o in many] == [want[i_] for i_ in range(len(prompts))]


@pytest.mark.timeout(400)
def test_tp4_with_two_kv_heads_and_a_small_vocabulary_matches_transformers(tmp_path):
    """More tensor-parallel ranks than KV heads (each KV head lives on two ranks) and a
    vocabulary that leaves the last rank's padded shard without a real column: the greedy
    tokens are those of the HuggingFace model with the same weights."""
    tr = pytest.importorskip("transformers")
    from vllm_gcu_b200.config import ModelConfig
    from vllm_gcu_b200.utils.weights import write_safetensors
    hc = tr.LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=128,
                        num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2,
                        max_position_embeddings=128, rms_norm_eps=1e-6,
                        tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = tr.LlamaForCausalLM(hc).eval().float()
    write_safetensors(os.path.join(str(tmp_path), "model.safetensors"),
                      {k: v.clone() for k, v in hf.state_dict().items()})
    d = hc.to_dict()
    d["architectures"] = ["LlamaForCausalLM"]
    cfg = _cfg(4)
    cfg.model = ModelConfig.from_hf_dict(d, dtype=torch.float32)
    cfg.load_format, cfg.model_path = "safetensors", str(tmp_path)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 300, (n,), generator=g).tolist() for n in (17, 40, 5)]
    ex = MultiprocExecutor(cfg)
    try:
        outs = ex.generate(prompts, SamplingParams(max_tokens=8, temperature=0.0,
                                                   ignore_eos=True), timeout_s=300)
    finally:
        ex.shutdown()
    for p, o in zip(prompts, outs):
        with torch.inference_mode():
            ids = torch.tensor([p])
            want = hf.generate(ids, attention_mask=torch.ones_like(ids), max_new_tokens=8,
                               do_sample=False, pad_token_id=299)[0, len(p):].tolist()
        assert o.outputs[0].token_ids == want


def _deepseek_checkpoint(path, mc):
    """Random DeepSeek-V3 style weights under HuggingFace names: separate ``q_a_proj`` /
    ``kv_a_proj_with_mqa``, gate / up halves, one tensor per expert projection, the routing
    bias below ``mlp.gate``."""
    from vllm_gcu_b200.models import build_model
    from vllm_gcu_b200.utils.weights import write_safetensors
    src = build_model(mc, "cpu")
    src.init_random(3, std=0.08)
    out = {}
    for name, p_ in src.state_dict().items():
        if name.startswith(("layers.", "embed_tokens.", "norm.")):
            name = "model." + name
        if name.endswith("qkv_a_proj.weight"):
            out[name.replace("qkv_a_proj", "q_a_proj")] = p_[:mc.q_lora_rank].clone()
            out[name.replace("qkv_a_proj", "kv_a_proj_with_mqa")] = p_[mc.q_lora_rank:].clone()
        elif name.endswith(".experts.w13"):
            half = p_.shape[1] // 2
            for e in range(p_.shape[0]):
                out[name[:-3] + f"{e}.gate_proj.weight"] = p_[e, :half].clone()
                out[name[:-3] + f"{e}.up_proj.weight"] = p_[e, half:].clone()
        elif name.endswith(".experts.w2"):
            for e in range(p_.shape[0]):
                out[name[:-2] + f"{e}.down_proj.weight"] = p_[e].clone()
        elif name.endswith("gate_up_proj.weight"):
            half = p_.shape[0] // 2
            out[name.replace("gate_up_proj", "gate_proj")] = p_[:half].clone()
            out[name.replace("gate_up_proj", "up_proj")] = p_[half:].clone()
        elif name.endswith("mlp.e_score_correction_bias"):
            g = torch.Generator().manual_seed(len(out))
            out[name.replace("mlp.e_score", "mlp.gate.e_score")] = \
                torch.randn(p_.shape, generator=g) * 0.1
        else:
            out[name] = p_.clone()
    write_safetensors(os.path.join(path, "model.safetensors"), out)


@pytest.mark.timeout(400)
@pytest.mark.parametrize("layout", ["tp2", "dp2_tp2_ep"])
def test_deepseek_parallel_layouts_match_single_process(tmp_path, layout):
    """Latent attention, grouped routing with a bias and shared experts, sharded over two
    tensor-parallel ranks, and over two replicas of two tensor-parallel ranks with expert
    parallelism across all four: the tokens of the unsharded engine."""
    sp = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 30, 4, 21)]
    _deepseek_checkpoint(str(tmp_path), preset("tiny-deepseek", dtype="float32"))

    def cfg(par, dp_attention=False):
        mc = preset("tiny-deepseek", dtype="float32")
        if dp_attention:
            mc.extra["dp_attention"] = True
        c = EngineConfig(model=mc, cache=CacheConfig(block_size=16, num_gpu_blocks=64),
                         scheduler=SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=64,
                                                   max_model_len=128),
                         parallel=par, device="cpu", seed=0)
        c.load_format, c.model_path = "safetensors", str(tmp_path)
        return c

    eng = LLMEngine(cfg(ParallelConfig()))
    for i_, p_ in enumerate(prompts):
        eng.add_request(p_, sp, request_id=str(i_))
    want = {}
    while eng.has_unfinished():
        for o in eng.step():
            if o.finished:
                want[int(o.request_id)] = o.outputs[0].token_ids
    par = ParallelConfig(tensor_parallel_size=2, comm_backend="nccl") if layout == "tp2" else \
        ParallelConfig(data_parallel_size=2, tensor_parallel_size=2,
                       enable_expert_parallel=True, comm_backend="nccl")
    ex = MultiprocExecutor(cfg(par, dp_attention=layout != "tp2"))
    try:
        got = ex.generate(prompts, sp, timeout_s=300)
    finally:
        ex.shutdown()
    assert [o.outputs[0].token_ids for o in got] == [want[i_] for i_ in range(len(prompts))]


@pytest.mark.timeout(400)
def test_tp2_multi_lora_matches_single_process(tmp_path):
    """LoRA adapters under tensor parallelism: the executor hands the full adapter tensors to
    every worker, each keeps its shard (B rows of column-parallel layers, A columns of
    row-parallel ones, KV slices by KV-head owner); a batch mixing two adapters and none gives
    the tokens of the unsharded engine with the same adapters."""
    tr = pytest.importorskip("transformers")
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from test_lora_cpu import _adapter
    from vllm_gcu_b200.config import ModelConfig
    from vllm_gcu_b200.lora import LoRARequest
    from vllm_gcu_b200.utils.weights import write_safetensors
    hc = tr.LlamaConfig(vocab_size=512, hidden_size=64, intermediate_size=128,
                        num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                        max_position_embeddings=128, rms_norm_eps=1e-6,
                        tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = tr.LlamaForCausalLM(hc).eval().float()
    write_safetensors(os.path.join(str(tmp_path), "model.safetensors"),
                      {k: v.clone() for k, v in hf.state_dict().items()})
    d = hc.to_dict()
    d["architectures"] = ["LlamaForCausalLM"]

    def cfg(tp):
        c = _cfg(tp)
        c.model = ModelConfig.from_hf_dict(d, dtype=torch.float32)
        c.load_format, c.model_path = "safetensors", str(tmp_path)
        c.additional_config["lora"] = {"max_loras": 2, "max_lora_rank": 8}
        return c

    mc = cfg(1).model
    a1, c1 = _adapter(mc, 1)
    a2, c2 = _adapter(mc, 2, r=8)
    for t in (a1, a2):                      # large enough to change the greedy tokens
        for k in t:
            t[k] = t[k] * 4.0
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, 512, (20,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    eng = LLMEngine(cfg(1))
    eng.add_lora(LoRARequest("a1", 1, ""), a1, c1)
    eng.add_lora(LoRARequest("a2", 2, ""), a2, c2)
    ids = [eng.add_request(p, sp, lora_id=l) for p, l in zip(prompts, (1, -1, 2))]
    want = {}
    while eng.has_unfinished():
        for o in eng.step():
            if o.finished:
                want[o.request_id] = o.outputs[0].token_ids
    plain = [eng.add_request(p, sp) for p in prompts]
    while eng.has_unfinished():
        for o in eng.step():
            if o.finished:
                want[o.request_id] = o.outputs[0].token_ids
    assert want[ids[0]] != want[plain[0]] and want[ids[2]] != want[plain[2]]
    ex = MultiprocExecutor(cfg(2))
    try:
        ex.add_lora(LoRARequest("a1", 1, ""), a1, c1)
        ex.add_lora(LoRARequest("a2", 2, ""), a2, c2)
        rids = [ex.add_request(p, sp, lora_id=l) for p, l in zip(prompts, (1, -1, 2))]
        got = {}
        for _ in range(600):
            for o in ex.poll(0.1):
                if o.finished:
                    got[o.request_id] = o.outputs[0].token_ids
            if len(got) == 3:
                break
    finally:
        ex.shutdown()
    assert [got[r] for r in rids] == [want[i] for i in ids]


@pytest.mark.timeout(400)
def test_pp2_tp2_random_schedule_matches_transformers_weights(tmp_path):
    """Two pipeline stages of two tensor-parallel ranks under a small KV pool with priorities,
    swapping and staggered arrivals: every request gets the tokens of the unsharded engine."""
    import random
    tr = pytest.importorskip("transformers")
    from vllm_gcu_b200.config import ModelConfig
    from vllm_gcu_b200.utils.weights import write_safetensors
    hc = tr.LlamaConfig(vocab_size=512, hidden_size=64, intermediate_size=128,
                        num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                        max_position_embeddings=256, rms_norm_eps=1e-6,
                        tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = tr.LlamaForCausalLM(hc).eval().float()
    write_safetensors(os.path.join(str(tmp_path), "model.safetensors"),
                      {k: v.clone() for k, v in hf.state_dict().items()})
    d = hc.to_dict()
    d["architectures"] = ["LlamaForCausalLM"]

    def cfg(par, blocks, seqs, budget, cpu_blocks=0, policy="fcfs"):
        c = EngineConfig(model=ModelConfig.from_hf_dict(d, dtype=torch.float32),
                         cache=CacheConfig(block_size=16, num_gpu_blocks=blocks,
                                           num_cpu_blocks=cpu_blocks),
                         scheduler=SchedulerConfig(max_num_seqs=seqs, policy=policy,
                                                   max_num_batched_tokens=budget,
                                                   max_model_len=256),
                         parallel=par, device="cpu", seed=0)
        c.load_format, c.model_path = "safetensors", str(tmp_path)
        return c

    rng = random.Random(1)
    g = torch.Generator().manual_seed(1)
    n = 7
    prompts = [torch.randint(0, 512, (rng.randint(3, 70),), generator=g).tolist()
               for _ in range(n)]
    sps = [SamplingParams(max_tokens=rng.randint(1, 20), temperature=0.0, ignore_eos=True)
           for _ in prompts]
    eng = LLMEngine(cfg(ParallelConfig(), 256, 16, 256))
    for i, p in enumerate(prompts):
        eng.add_request(p, sps[i], request_id=str(i))
    want = {}
    while eng.has_unfinished():
        for o in eng.step():
            if o.finished:
                want[int(o.request_id)] = o.outputs[0].token_ids
    par = ParallelConfig(pipeline_parallel_size=2, tensor_parallel_size=2, comm_backend="nccl")
    ex = MultiprocExecutor(cfg(par, 12, 4, 32, cpu_blocks=16, policy="priority"))
    try:
        pending, ids, got = list(range(n)), {}, {}
        for _ in range(3000):
            for _ in range(rng.randint(0, 3)):
                if pending:
                    i = pending.pop()
                    ids[ex.add_request(prompts[i], sps[i], priority=rng.randint(0, 2))] = i
            for o in ex.poll(0.02):
                if o.finished:
                    got[ids[o.request_id]] = o.outputs[0].token_ids
            if len(got) == n:
                break
    finally:
        ex.shutdown()
    assert got == want


def _free_port_pair():
    import socket
    for _ in range(50):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            p = s.getsockname()[1]
        try:
            with socket.socket() as s2:
                s2.bind(("127.0.0.1", p + 1))
            return p
        except OSError:
            continue
    raise RuntimeError("no two adjacent free ports")


@pytest.mark.timeout(400)
def test_disaggregated_prefill_between_two_tensor_parallel_instances():
    """1P1D with both instances sharded over two ranks: every worker opens its own connector
    (base port + rank), rank r of the prefill instance ships its KV shard to rank r of the
    decode instance; the decode instance takes the prompt's KV over, and the tokens are those
    of one instance working alone."""
    g = torch.Generator().manual_seed(8)
    prompt = torch.randint(0, 32000, (37,), generator=g).tolist()
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)

    def cfg(port=None):
        c = _cfg(2)
        if port:
            c.additional_config["kv_connector"] = {"host": "127.0.0.1", "port": port,
                                                   "send_type": "PUT", "recv_timeout_s": 10.0}
        return c

    def finish(ex, rid):
        for _ in range(1200):
            for o in ex.poll(0.05):
                if o.finished and o.request_id == rid:
                    return o
        raise AssertionError("request did not finish")

    alone = MultiprocExecutor(cfg())
    try:
        want = alone.generate([prompt], sp)[0].outputs[0].token_ids
    finally:
        alone.shutdown()
    pp, dp_ = _free_port_pair(), _free_port_pair()
    pre, dec = MultiprocExecutor(cfg(pp)), MultiprocExecutor(cfg(dp_))
    try:
        rid = pre.add_request(prompt, SamplingParams(max_tokens=1, temperature=0.0,
                                                     ignore_eos=True), request_id="r-77",
                              kv_transfer_params={"do_remote_decode": True,
                                                  "remote": f"127.0.0.1:{dp_}"})
        first = finish(pre, rid)
        assert first.outputs[0].token_ids == want[:1]
        handoff = first.kv_transfer_params
        assert handoff["remote"] == f"127.0.0.1:{pp}" and handoff["remote_request_id"] == rid
        did = dec.add_request(prompt, sp, request_id="d-1", kv_transfer_params={
            "do_remote_prefill": True, "remote": handoff["remote"],
            "remote_request_id": handoff["remote_request_id"]})
        out = finish(dec, did)
        assert out.outputs[0].token_ids == want
        assert out.num_cached_tokens == len(prompt) - 1      # taken over, not recomputed
    finally:
        pre.shutdown()
        dec.shutdown()


def _front_end_that_gets_killed(q):
    ex = MultiprocExecutor(_cfg(2))
    q.put([p.pid for p in ex.procs])
    import time
    time.sleep(600)


@pytest.mark.timeout(300)
def test_workers_exit_when_the_front_end_is_killed():
    """A front end that dies without shutting down (SIGKILL) must not leave its workers
    running: they notice the missing parent at their next loop iteration and exit."""
    import multiprocessing as mp
    import signal
    import time
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    front = ctx.Process(target=_front_end_that_gets_killed, args=(q,))
    front.start()
    pids = q.get(timeout=240)
    os.kill(front.pid, signal.SIGKILL)
    front.join(10)

    def alive(pid):
        try:
            os.kill(pid, 0)
        except ProcessLookupError:
            return False
        try:                                    # a zombie waiting for its new parent counts as gone
            with open(f"/proc/{pid}/stat") as f:
                return f.read().split(") ")[-1].split()[0] != "Z"
        except OSError:
            return False
    deadline = time.monotonic() + 30
    while time.monotonic() < deadline and any(alive(p) for p in pids):
        time.sleep(0.2)
    assert not any(alive(p) for p in pids)
