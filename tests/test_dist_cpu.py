"""Collective semantics on CPU ranks (gloo, world size 2 and 3): uneven scatter,
reduce-scatter-v / all-gather-v, sequence-parallel round trip, all-to-all-v and the
expert-parallel dispatch / combine against the single-process reference."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _leave():
    """End of a worker with several process groups: after the last barrier the process exits
    without tearing the groups down (their background threads have aborted the interpreter's
    own shutdown now and then); everything a peer still needs has been sent by then."""
    import time
    dist.barrier()
    time.sleep(0.2)
    os._exit(0)


def _worker(rank, world, port, fn_name):
    sys.path.insert(0, ROOT)
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    from vllm_gcu_b200.parallel.state import init_distributed
    if fn_name in ("_check_ep", "_check_ep_fp8"):
        # data-parallel attention: every rank is a replica of its own with its own tokens
        init_distributed(tp=1, dp=world, backend="gloo", enable_ep=True)
    else:
        init_distributed(tp=world, backend="gloo", enable_ep=True)
    globals()[fn_name](rank, world)
    dist.barrier()
    dist.destroy_process_group()


def _spawn(fn_name, world):
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port, fn_name), nprocs=world, join=True)


def _check_sp(rank, world):
    from vllm_gcu_b200.parallel import sp
    from vllm_gcu_b200.parallel.communicator import get_comm, scatter_sizes
    for T in (7, 8, 1, 0):
        sizes = scatter_sizes(T, world)
        assert sum(sizes) == T and sizes == sorted(sizes)
        g = torch.Generator().manual_seed(T)
        full = [torch.randn(T, 5, generator=g) for _ in range(world)]
        mine = full[rank]
        red = sp.tp_to_sp(mine.clone())
        want = sum(full)
        start = sum(sizes[:rank])
        assert torch.allclose(red, want[start:start + sizes[rank]], atol=1e-6)
        back = sp.sp_to_tp(red, T)
        assert torch.allclose(back, want, atol=1e-6)
        assert torch.equal(sp.slice_tensor_sp(want), want[start:start + sizes[rank]])
    comm = get_comm("tp")
    x = torch.full((rank + 1, 2), float(rank))
    send = [1] * min(world, rank + 1) + [0] * max(0, world - rank - 1)
    send[0] += rank + 1 - sum(send)
    recv = []
    for r in range(world):
        s_r = [1] * min(world, r + 1) + [0] * max(0, world - r - 1)
        s_r[0] += r + 1 - sum(s_r)
        recv.append(s_r[rank])
    out = comm.all_to_all_v(x, send, recv)
    assert out.shape[0] == sum(recv)


def _check_ep(rank, world):
    from vllm_gcu_b200.config import preset
    from vllm_gcu_b200.layers.moe import SparseMoeBlock
    from vllm_gcu_b200.ops import ref
    cfg = preset("tiny-qwen3-moe", num_experts=6 if world == 3 else 8, num_experts_per_tok=2)
    cfg.extra["dp_attention"] = True
    torch.manual_seed(0)
    blk = SparseMoeBlock(cfg, "cpu", "m")
    E, I, H = cfg.num_experts, cfg.moe_intermediate_size, cfg.hidden_size
    g = torch.Generator().manual_seed(1)
    w13 = torch.randn(E, 2 * I, H, generator=g) * 0.05
    w2 = torch.randn(E, H, I, generator=g) * 0.05
    gate = torch.randn(E, H, generator=g) * 0.5
    blk.gate.weight.data.copy_(gate)
    for e in range(E):
        blk.experts.load_expert_weight(e, "gate", w13[e, :I])
        blk.experts.load_expert_weight(e, "up", w13[e, I:])
        blk.experts.load_expert_weight(e, "down", w2[e])
    # every rank owns different tokens (data-parallel attention); rank 1 is idle (T = 0)
    T = 0 if rank == 1 else 5 + rank
    xg = torch.Generator().manual_seed(10 + rank)
    x = torch.randn(T, H, generator=xg)
    got = blk(x)
    logits = x @ gate.t()
    w, ids = ref.topk_softmax(logits, 2, True) if T else (torch.zeros(0, 2), torch.zeros(0, 2, dtype=torch.int32))
    want = ref.fused_experts(x, w13, w2, w, ids) if T else x
    assert got.shape == x.shape
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-4), (got - want).abs().max()


def _check_sp_model(rank, world):
    """Tensor-parallel Llama and Qwen3-MoE with the residual stream sharded by rows
    (sequence parallelism): same logits as the plain tensor-parallel forward."""
    import dataclasses

    from vllm_gcu_b200.config import preset
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    kw = dict(device="cpu", tensor_parallel_size=world, max_num_seqs=4, max_num_batched_tokens=32,
              max_model_len=128, num_gpu_blocks=64, comm_backend="nccl", seed=0)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (19, 7, 40)]
    sp_ = SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True)
    for name in ("tiny-llama", "tiny-qwen3-moe"):
        logits = {}
        for flag in (False, True):
            mc = dataclasses.replace(preset(name), dtype=torch.float32)
            mc.extra = dict(mc.extra, sequence_parallel=flag)
            llm = LLM(mc, **kw)
            assert llm.engine.model.sequence_parallel == flag
            llm.engine.runner.keep_logits = True
            out = llm.generate(prompts, sp_)
            logits[flag] = (llm.engine.runner.last_logits, [o.outputs[0].token_ids for o in out])
        a, b = logits[False], logits[True]
        assert a[1] == b[1], (name, a[1], b[1])
        assert torch.allclose(a[0], b[0], atol=1e-4, rtol=1e-4), (name, (a[0] - b[0]).abs().max())


@pytest.mark.timeout(600)
@pytest.mark.parametrize("world", [2])
def test_sequence_parallel_model_matches_tensor_parallel(world):
    _spawn("_check_sp_model", world)


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world", [2, 3])
def test_sequence_parallel_and_collectives(world):
    _spawn("_check_sp", world)


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world", [2, 3])
def test_expert_parallel_dispatch_combine(world):
    _spawn("_check_ep", world)


def _check_pp(rank, world):
    """Pipeline parallel engine (2 stages) must reproduce the single-stage tokens."""
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (21, 40, 6)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    llm = LLM("tiny-llama", device="cpu", pipeline_parallel_size=world, max_num_seqs=4,
              max_num_batched_tokens=32, max_model_len=128, num_gpu_blocks=32)
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    want = torch.load(os.environ["PP_EXPECT"])
    assert got == want, (got, want)


def _worker_pp(rank, world, port, fn_name):
    sys.path.insert(0, ROOT)
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    from vllm_gcu_b200.parallel.state import init_distributed
    init_distributed(tp=1, pp=world, backend="gloo")
    globals()[fn_name](rank, world)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_pipeline_parallel_matches_single_stage(tmp_path):
    from vllm_gcu_b200.engine.llm import LLM
    from vllm_gcu_b200.engine.request import SamplingParams
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (21, 40, 6)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, max_num_batched_tokens=32,
              max_model_len=128, num_gpu_blocks=32)
    want = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    path = str(tmp_path / "expect.pt")
    torch.save(want, path)
    os.environ["PP_EXPECT"] = path
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker_pp, args=(2, port, "_check_pp"), nprocs=2, join=True)


def _check_etp(rank, world):
    """ETP: data-parallel attention without EP.  Every rank holds a slice of every expert's
    intermediate dimension; rows are gathered over DP and the sums scattered back."""
    from vllm_gcu_b200.config import preset
    from vllm_gcu_b200.layers.moe import SparseMoeBlock
    from vllm_gcu_b200.ops import ref
    from vllm_gcu_b200.parallel.state import get_state
    st = get_state()
    cfg = preset("tiny-qwen3-moe", num_experts=8, num_experts_per_tok=2)
    cfg.extra["dp_attention"] = True
    torch.manual_seed(0)
    blk = SparseMoeBlock(cfg, "cpu", "m")
    assert blk.use_etp and not blk.use_ep
    E, I, H = cfg.num_experts, cfg.moe_intermediate_size, cfg.hidden_size
    assert blk.experts.inter == I // world
    assert blk.experts.shard_index == st.dp.rank_in_group * st.tp.world_size + st.tp.rank_in_group
    g = torch.Generator().manual_seed(1)
    w13 = torch.randn(E, 2 * I, H, generator=g) * 0.05
    w2 = torch.randn(E, H, I, generator=g) * 0.05
    gate = torch.randn(E, H, generator=g) * 0.5
    blk.gate.weight.data.copy_(gate)
    for e in range(E):
        blk.experts.load_expert_weight(e, "gate", w13[e, :I])
        blk.experts.load_expert_weight(e, "up", w13[e, I:])
        blk.experts.load_expert_weight(e, "down", w2[e])
    # ranks of one TP group hold the same rows; replicas hold different ones, one is idle
    d = st.dp.rank_in_group
    for trial in range(2):
        T = 0 if (d == 1 and trial == 0) else 4 + d + trial
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(10 + d + 7 * trial))
        got = blk(x)
        logits = x @ gate.t()
        if T:
            w, ids = ref.topk_softmax(logits, 2, True)
            want = ref.fused_experts(x, w13, w2, w, ids)
        else:
            want = x
        assert got.shape == x.shape
        assert torch.allclose(got, want, atol=1e-5, rtol=1e-4), (got - want).abs().max()


def _worker_etp(rank, world, port, tp):
    sys.path.insert(0, ROOT)
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    from vllm_gcu_b200.parallel.state import init_distributed
    init_distributed(tp=tp, dp=world // tp, backend="gloo", enable_ep=False)
    _check_etp(rank, world)
    _leave()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world,tp", [(2, 1), (4, 2)])
def test_etp_gather_scatter_matches_reference(world, tp):
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker_etp, args=(world, port, tp), nprocs=world, join=True)


def _check_ep_tp(rank, world, shared):
    """Expert parallelism over dp x tp ranks with tensor-parallel attention inside a replica:
    each tensor-parallel rank dispatches its own slice of the replica's rows, so a token
    reaches every destination rank once per replica; with shared experts their partial sums
    and the routed rows leave through one all-reduce."""
    from vllm_gcu_b200.config import preset
    from vllm_gcu_b200.layers.moe import SparseMoeBlock
    from vllm_gcu_b200.ops import ref
    from vllm_gcu_b200.parallel.state import get_state
    st = get_state()
    cfg = preset("tiny-qwen3-moe", num_experts=8, num_experts_per_tok=2,
                 num_shared_experts=shared)
    cfg.extra["dp_attention"] = True
    torch.manual_seed(0)
    blk = SparseMoeBlock(cfg, "cpu", "m")
    assert blk.use_ep and blk.dispatcher is not None
    E, I, H = cfg.num_experts, cfg.moe_intermediate_size, cfg.hidden_size
    Is = I * max(shared, 1)
    g = torch.Generator().manual_seed(1)
    w13 = torch.randn(E, 2 * I, H, generator=g) * 0.05
    w2 = torch.randn(E, H, I, generator=g) * 0.05
    gate = torch.randn(E, H, generator=g) * 0.5
    sw_gu = torch.randn(2 * Is, H, generator=g) * 0.05
    sw_d = torch.randn(H, Is, generator=g) * 0.05
    blk.gate.weight.data.copy_(gate)
    for e in range(E):
        blk.experts.load_expert_weight(e, "gate", w13[e, :I])
        blk.experts.load_expert_weight(e, "up", w13[e, I:])
        blk.experts.load_expert_weight(e, "down", w2[e])
    if shared:
        blk.shared_experts.gate_up_proj.load_weight("weight", sw_gu[:Is], 0)
        blk.shared_experts.gate_up_proj.load_weight("weight", sw_gu[Is:], 1)
        blk.shared_experts.down_proj.load_weight("weight", sw_d, None)
    seen = {"rows": 0}
    inner = blk.experts.forward

    def counting(xr, *a, **kw):
        seen["rows"] += xr.shape[0]
        return inner(xr, *a, **kw)
    blk.experts.forward = counting
    d = st.dp.rank_in_group
    per_rank = E // world
    for trial in range(3):
        # one replica idle in the first trial; a single row (fewer rows than TP ranks) last
        T = 0 if (d == 1 and trial == 0) else (1 if trial == 2 else 4 + d + trial)
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(10 + d + 7 * trial))
        seen["rows"] = 0
        got = blk(x)
        visits = 0
        if T:
            w, ids = ref.topk_softmax(x @ gate.t(), 2, True)
            want = ref.fused_experts(x, w13, w2, w, ids)
            if shared:
                gu = x @ sw_gu.t()
                want = want + (torch.nn.functional.silu(gu[:, :Is]) * gu[:, Is:]) @ sw_d.t()
            assert torch.allclose(got, want, atol=1e-5, rtol=1e-4), (got - want).abs().max()
            visits = sum(len({int(e) // per_rank for e in row}) for row in ids.tolist())
        assert got.shape == x.shape
        # rows that reached any rank's experts = token visits, counted once per replica
        tot = torch.tensor([seen["rows"], visits if st.tp.rank_in_group == 0 else 0])
        dist.all_reduce(tot)
        assert int(tot[0]) == int(tot[1]), tot.tolist()


def _worker_ep_tp(rank, world, port, tp, shared):
    sys.path.insert(0, ROOT)
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    from vllm_gcu_b200.parallel.state import init_distributed
    init_distributed(tp=tp, dp=world // tp, backend="gloo", enable_ep=True)
    _check_ep_tp(rank, world, shared)
    _leave()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("shared", [0, 1])
def test_expert_parallel_with_tensor_parallel_replicas(shared):
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker_ep_tp, args=(4, port, 2, shared), nprocs=4, join=True)


def _check_ep_fp8(rank, world):
    """fp8 dispatch payload: rows cross the exchange quantised in groups of 128 with their
    scales in the same row (about half the bytes); the result is the routed-expert output of
    the de-quantised rows."""
    from vllm_gcu_b200.config import preset
    from vllm_gcu_b200.layers.moe import SparseMoeBlock
    from vllm_gcu_b200.layers.moe_ep import pack_fp8_rows, packed_width, unpack_fp8_rows
    from vllm_gcu_b200.ops import ref
    cfg = preset("tiny-qwen3-moe", num_experts=8, num_experts_per_tok=2)
    cfg.extra["dp_attention"] = True
    H = cfg.hidden_size
    sent = {}
    for mode in (False, True):
        cfg.extra["ep_fp8_dispatch"] = mode
        torch.manual_seed(0)
        blk = SparseMoeBlock(cfg, "cpu", "m")
        assert blk.dispatcher.fp8_payload is mode
        E, I = cfg.num_experts, cfg.moe_intermediate_size
        g = torch.Generator().manual_seed(1)
        w13 = torch.randn(E, 2 * I, H, generator=g) * 0.05
        w2 = torch.randn(E, H, I, generator=g) * 0.05
        gate = torch.randn(E, H, generator=g) * 0.5
        blk.gate.weight.data.copy_(gate)
        for e in range(E):
            blk.experts.load_expert_weight(e, "gate", w13[e, :I])
            blk.experts.load_expert_weight(e, "up", w13[e, I:])
            blk.experts.load_expert_weight(e, "down", w2[e])
        T = 0 if rank == 1 else 6 + rank
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(10 + rank))
        got = blk(x)
        sent[mode] = blk.dispatcher.bytes_sent
        if T:
            w, ids = ref.topk_softmax(x @ gate.t(), 2, True)
            seen = unpack_fp8_rows(pack_fp8_rows(x), H, x.dtype) if mode else x
            want = ref.fused_experts(seen, w13, w2, w, ids)
            assert torch.allclose(got, want, atol=1e-5, rtol=1e-4), (got - want).abs().max()
            exact = ref.fused_experts(x, w13, w2, w, ids)
            assert (got - exact).abs().max() < 0.05 * exact.abs().max() + 1e-3
    if sent[False]:
        # fp32 rows on this path: H * 4 bytes against H + H / 32 bytes
        assert sent[True] * 4 * H == sent[False] * 2 * packed_width(H)


@pytest.mark.timeout(300)
def test_expert_parallel_fp8_dispatch_payload():
    _spawn("_check_ep_fp8", 2)
