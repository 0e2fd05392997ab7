"""Worker of the multi-GPU tests (launched by torch.distributed.run, one rank per GPU).

Checks, on N >= 2 GPUs: the fused GEMM + all-reduce kernel and the stand-alone symmetric
all-reduce against a torch reference, and that a tensor-parallel engine produces the same
greedy tokens as the single-GPU engine when both load the same checkpoint tensors.
NVLS is not needed: the kernels use plain peer loads / stores.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_gcu_b200.config import preset  # noqa: E402
from vllm_gcu_b200.engine.llm import LLM  # noqa: E402
from vllm_gcu_b200.engine.request import SamplingParams  # noqa: E402
from vllm_gcu_b200.ops import _native  # noqa: E402
from vllm_gcu_b200.parallel import symm  # noqa: E402
from vllm_gcu_b200.parallel.communicator import get_comm  # noqa: E402
from vllm_gcu_b200.parallel.state import get_state, init_distributed  # noqa: E402


def full_state_dict(cfg, seed=0):
    """HF-named full (unsharded) random checkpoint, identical on every rank."""
    g = torch.Generator().manual_seed(seed)
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads

    def rnd(*shape):
        return (torch.randn(*shape, generator=g) * 0.02).to(cfg.dtype)

    sd = {"model.embed_tokens.weight": rnd(V, H), "model.norm.weight": torch.ones(H, dtype=cfg.dtype),
          "lm_head.weight": rnd(V, H)}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        sd[p + "self_attn.q_proj.weight"] = rnd(Hq * D, H)
        sd[p + "self_attn.k_proj.weight"] = rnd(Hkv * D, H)
        sd[p + "self_attn.v_proj.weight"] = rnd(Hkv * D, H)
        sd[p + "self_attn.o_proj.weight"] = rnd(H, Hq * D)
        sd[p + "mlp.gate_proj.weight"] = rnd(I, H)
        sd[p + "mlp.up_proj.weight"] = rnd(I, H)
        sd[p + "mlp.down_proj.weight"] = rnd(H, I)
        sd[p + "input_layernorm.weight"] = torch.ones(H, dtype=cfg.dtype)
        sd[p + "post_attention_layernorm.weight"] = torch.ones(H, dtype=cfg.dtype)
    return sd


def dense_last_logits(cfg, sd, prompts, dev, all_positions=False):
    """fp32 no-cache forward of the full (unsharded) checkpoint: logits at the last position
    of every prompt, [len(prompts), V] (``all_positions``: a list of [S, V] tensors).  The
    single-GPU reference of the engine runs."""
    from vllm_gcu_b200.layers.basic import build_cos_sin_cache
    from vllm_gcu_b200.ops import ref
    W = {k: v.to(dev).float() for k, v in sd.items()}
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    cs = build_cos_sin_cache(cfg.rotary_dim, 1024, cfg.rope_theta, cfg.rope_scaling).to(dev)
    rows = []
    for p in prompts:
        ids = torch.tensor(p, device=dev)
        S = ids.shape[0]
        x = W["model.embed_tokens.weight"][ids]
        pos = torch.arange(S, device=dev)
        residual = None
        for i in range(cfg.num_hidden_layers):
            pre = f"model.layers.{i}."
            if residual is None:
                residual, h = x, ref.rms_norm(x, W[pre + "input_layernorm.weight"], cfg.rms_norm_eps)
            else:
                h, residual = ref.fused_add_rms_norm(x, residual, W[pre + "input_layernorm.weight"],
                                                     cfg.rms_norm_eps)
            q = h @ W[pre + "self_attn.q_proj.weight"].t()
            k = h @ W[pre + "self_attn.k_proj.weight"].t()
            v = h @ W[pre + "self_attn.v_proj.weight"].t()
            q, k = ref.rotary_embedding(pos, q, k, D, cs, True)
            o = ref.dense_causal_attention(q.view(S, Hq, D), k.view(S, Hkv, D), v.view(S, Hkv, D),
                                           D ** -0.5).reshape(S, Hq * D)
            h = o @ W[pre + "self_attn.o_proj.weight"].t()
            h, residual = ref.fused_add_rms_norm(h, residual,
                                                 W[pre + "post_attention_layernorm.weight"],
                                                 cfg.rms_norm_eps)
            gu = torch.cat([h @ W[pre + "mlp.gate_proj.weight"].t(),
                            h @ W[pre + "mlp.up_proj.weight"].t()], -1)
            x = ref.silu_and_mul(gu) @ W[pre + "mlp.down_proj.weight"].t()
        x, _ = ref.fused_add_rms_norm(x, residual, W["model.norm.weight"], cfg.rms_norm_eps)
        rows.append((x if all_positions else x[-1]) @ W["lm_head.weight"].t())
    return [r.cpu() for r in rows] if all_positions else torch.stack(rows).cpu()


def check_gemm_ar_norm(fused, world, rank, dev):
    """GEMM + all-reduce + residual + RMSNorm in one kernel against torch, with and without
    the norm, with the new residual on the owner only / on every rank, over plain peer
    accesses and (when the allocation has a multicast view) over multimem."""
    lo_hi = lambda r: (128 * r // world, 128 * (r + 1) // world)
    modes = [(False, 0), (False, 1), (False, 2), (False, 3), (False, None)]
    if fused.buf.multicast_ptr:
        modes.append((True, 0))
    for use_mc, rn_mode in modes:
        fused.use_multimem = use_mc
        fused.force_rn_mode = rn_mode
        fused.row_owner = True if rn_mode is None else None
        for (M, N, K) in [(256, 4096, 512), (7, 1024, 256), (1024, 4096, 1792), (300, 2048, 72)]:
            g = torch.Generator(device="cuda").manual_seed(100 + rank)
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16, generator=g)
            w = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
            g2 = torch.Generator(device="cuda").manual_seed(5)           # same on every rank
            res = torch.randn(M, N, device=dev, generator=g2).to(torch.bfloat16)
            nw = (1.0 + 0.1 * torch.randn(N, device=dev, generator=g2)).to(torch.bfloat16)
            part = (x.float() @ w.float().t()).to(torch.bfloat16).float()
            dist.all_reduce(part)
            z = (part + res.float()).to(torch.bfloat16).float()
            normed = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + 1e-5) * nw.float()
            for rep, bcast in enumerate([True, False, True, False, False]):
                out, nres = fused.gemm_ar_norm(x, w, res, nw, 1e-5, bcast_residual=bcast)
                torch.cuda.synchronize()
                _native.check_status()
                tag = f"gemm_ar_norm mc={use_mc} mode={rn_mode} {M}x{N}x{K} rep {rep}"
                err = (out.float() - normed).abs().max().item()
                assert err < 0.03 * normed.abs().max().item() + 0.03, f"{tag}: out err {err}"
                rows = torch.arange(M, device=dev)
                if not bcast and fused._rn_mode(M, N, 64) != 2:
                    l, h = lo_hi(rank)
                    rows = rows[(rows % 128 >= l) & (rows % 128 < h)]
                rerr = (nres.float()[rows] - z[rows]).abs().max().item() if rows.numel() else 0.0
                assert rerr < 0.03 * z.abs().max().item() + 0.03, f"{tag}: residual err {rerr}"
            out, nres = fused.gemm_ar_norm(x, w, None, None)
            torch.cuda.synchronize()
            _native.check_status()
            assert nres is None
            err = (out.float() - part).abs().max().item()
            assert err < 0.03 * part.abs().max().item() + 0.03, f"plain reduce {M}x{N}x{K}: {err}"
    fused.force_rn_mode = None
    fused.row_owner = None
    # the default policy (may run as GEMM + all-reduce followed by the norm kernel)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    x = torch.randn(256, 512, device=dev, dtype=torch.bfloat16, generator=g)
    w = (torch.randn(4096, 512, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    g2 = torch.Generator(device="cuda").manual_seed(5)
    res = torch.randn(256, 4096, device=dev, generator=g2).to(torch.bfloat16)
    nw = (1.0 + 0.1 * torch.randn(4096, device=dev, generator=g2)).to(torch.bfloat16)
    part = (x.float() @ w.float().t()).to(torch.bfloat16).float()
    dist.all_reduce(part)
    z = (part + res.float()).to(torch.bfloat16).float()
    normed = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + 1e-5) * nw.float()
    out, _ = fused.gemm_ar_norm(x, w, res.clone(), nw, 1e-5, bcast_residual=True)
    torch.cuda.synchronize()
    _native.check_status()
    err = (out.float() - normed).abs().max().item()
    assert err < 0.03 * normed.abs().max().item() + 0.03, f"default policy: out err {err}"
    # greedy tokens from vocabulary-parallel logits
    for B, V in [(256, 16064), (3, 520)]:
        g = torch.Generator(device="cuda").manual_seed(900 + rank)
        lg = torch.randn(B, V, device=dev, generator=g).to(torch.bfloat16)
        valid = V - 8 if rank == world - 1 else V
        parts = [torch.empty_like(lg) for _ in range(world)]
        dist.all_gather(parts, lg)
        parts[-1] = parts[-1][:, :V - 8]
        want = torch.cat([q.float() for q in parts], dim=1).argmax(-1)
        want = want + (want // V) * 0        # ids are global: block r starts at r * V
        for rep in range(3):
            got = fused.greedy_argmax(lg[:, :valid], valid, rank * V)
            torch.cuda.synchronize()
            _native.check_status()
            assert torch.equal(got, want), f"greedy_argmax B={B} rep {rep}"


def main():
    """Runs the checks; a failing rank does not leave while its peers are still inside a
    kernel that waits for it: every rank reaches the final barrier, then all exit together."""
    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    pp_mode = os.environ.get("B200_TEST_ONLY") == "pp"
    st = init_distributed(tp=1, pp=world) if pp_mode else init_distributed(tp=world)
    failed = False
    try:
        if pp_mode:
            run_pp_check(world, rank, st)
        else:
            run_checks(world, rank, st)
    except BaseException:  # noqa: BLE001
        import traceback
        traceback.print_exc()
        failed = True
    try:
        torch.cuda.synchronize()
    except Exception:  # noqa: BLE001
        failed = True
    flag = torch.tensor([int(failed)], device="cuda")
    dist.all_reduce(flag)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(1 if int(flag.item()) else 0)


def run_pp_check(world, rank, st):
    """Pipeline parallelism on GPUs: the stages hand (hidden, residual) over NCCL p2p on a side
    stream; every generated token must be a (near-)maximum of the dense fp32 logits."""
    dev = torch.device("cuda", st.local_rank)
    kw = dict(num_hidden_layers=4, hidden_size=1024, intermediate_size=2048,
              num_attention_heads=8, num_key_value_heads=2, head_dim=128, vocab_size=4096,
              max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256, num_gpu_blocks=128)
    cfg = preset("llama-3-8b", **{k: v for k, v in kw.items() if k in (
        "num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads",
        "num_key_value_heads", "head_dim", "vocab_size")})
    sd = full_state_dict(cfg)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (33, 64, 5, 120)]
    llm = LLM("llama-3-8b", pipeline_parallel_size=world, enforce_eager=True, load_format="none",
              **kw)
    llm.engine.model.load_weights(sd.items())
    outs = llm.generate(prompts, SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
    torch.cuda.synchronize()
    _native.check_status()
    seqs = [o.outputs[0].token_ids for o in outs]
    full = [p_ + t_ for p_, t_ in zip(prompts, seqs)]
    dense = dense_last_logits(cfg, sd, [f[:-1] for f in full], dev, all_positions=True)
    for p_, t_, lg in zip(prompts, seqs, dense):
        tail = lg[len(p_) - 1:]
        assert len(t_) == 8
        gap = tail.max(-1).values - tail.gather(-1, torch.tensor(t_)[:, None]).squeeze(-1)
        assert gap.max().item() < 0.06 * lg.std().item() + 0.03, f"pp{world}: {gap}"
    if rank == 0:
        print(f"pp{world} engine ok", flush=True)


def run_checks(world, rank, st):
    dev = torch.device("cuda", st.local_rank)
    torch.manual_seed(0)

    # ---- fused GEMM + all-reduce ------------------------------------------------------
    fused = symm.FusedTP(max_tokens=1024, max_n=4096, device=dev)
    if os.environ.get("B200_TEST_ONLY") == "ar_norm":
        check_gemm_ar_norm(fused, world, rank, dev)
        if rank == 0:
            print(f"gemm + all-reduce + norm ok (multicast view: "
                  f"{bool(fused.buf.multicast_ptr)})", flush=True)
        return
    for (M, N, K) in [(256, 4096, 512), (7, 1024, 256), (1024, 4096, 1792), (130, 136, 72)]:
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16, generator=g)
        w = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        want = (x.float() @ w.float().t())
        dist.all_reduce(want)
        for rep in range(3):       # several launches exercise the epoch / buffer reuse logic
            got = fused.gemm_all_reduce(x, w)
            assert got is not None
            torch.cuda.synchronize()
            _native.check_status()
            err = (got.float() - want).abs().max().item()
            tol = 0.05 * want.abs().max().item() + 0.05
            assert err < tol, f"gemm_all_reduce {M}x{N}x{K} rep {rep}: err {err} tol {tol}"
    check_gemm_ar_norm(fused, world, rank, dev)
    if rank == 0:
        print("gemm + all-reduce + norm ok", flush=True)
    for n in (8, 4096, 1 << 20):
        x = torch.randn(n, device=dev, dtype=torch.bfloat16)
        want = x.float().clone()
        dist.all_reduce(want)
        got = fused.all_reduce(x.clone())
        torch.cuda.synchronize()
        _native.check_status()
        assert (got.float() - want).abs().max().item() < 0.05 * want.abs().max().item() + 0.05
    # ---- GEMM + all-gather of the output (vocabulary-parallel LM head) ------------------
    fg = symm.FusedGather(dev, out_rows=300, out_cols=4096 * world, sp_tokens=1200, sp_k=1024)
    for (M, N, K) in [(256, 4096, 512), (5, 1024, 256), (300, 520, 72)]:
        g = torch.Generator(device="cuda").manual_seed(7)          # same x on every rank
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16, generator=g)
        g2 = torch.Generator(device="cuda").manual_seed(200 + rank)
        w = (torch.randn(N, K, device=dev, generator=g2) * 0.05).to(torch.bfloat16)
        mine = (x.float() @ w.float().t())
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        want = torch.cat(parts, dim=1)
        for rep in range(3):
            got = fg.gemm_all_gather(x, w)
            assert got is not None
            torch.cuda.synchronize()
            _native.check_status()
            err = (got.float() - want).abs().max().item()
            assert err < 0.02 * want.abs().max().item() + 0.02, \
                f"gemm_all_gather {M}x{N}x{K} rep {rep}: err {err}"
    # ---- all-gather of the input fused into the GEMM (sequence-parallel activations) ----
    from vllm_gcu_b200.parallel.sp import scatter
    for (M, N, K) in [(1024, 2048, 1024), (1200, 512, 1024), (77, 256, 1024), (3, 128, 1024)]:
        sizes = scatter(M, world)
        g = torch.Generator(device="cuda").manual_seed(300 + rank)
        xs = torch.randn(sizes[rank], K, device=dev, dtype=torch.bfloat16, generator=g)
        g2 = torch.Generator(device="cuda").manual_seed(9)
        w = (torch.randn(N, K, device=dev, generator=g2) * 0.05).to(torch.bfloat16)
        full = get_comm("tp").all_gather_v(xs, sizes)
        want = full.float() @ w.float().t()
        for rep in range(3):
            got = fg.all_gather_gemm(xs, w, sizes)
            assert got is not None
            torch.cuda.synchronize()
            _native.check_status()
            err = (got.float() - want).abs().max().item()
            assert err < 0.02 * want.abs().max().item() + 0.02, \
                f"all_gather_gemm {M}x{N}x{K} rep {rep}: err {err}"
    # ---- raw NCCL binding (unique id over the gloo group) ---------------------------------
    from vllm_gcu_b200.parallel.pynccl import PyNcclCommunicator
    pn = PyNcclCommunicator(rank, world, dev, group=st.tp.cpu_group)
    x = torch.full((1000,), float(rank + 1), device=dev, dtype=torch.bfloat16)
    pn.all_reduce(x)
    torch.cuda.synchronize()
    assert torch.all(x == world * (world + 1) / 2)
    y = torch.full((8,), float(rank), device=dev)
    if rank == 0:
        pn.send(y, 1)
    elif rank == 1:
        pn.recv(y, 0)
    torch.cuda.synchronize()
    if rank == 1:
        assert torch.all(y == 0)
    pn.destroy()
    if rank == 0:
        print("fused collectives ok", flush=True)

    # ---- tensor-parallel engine vs single GPU --------------------------------------------
    kw = dict(num_hidden_layers=2, hidden_size=1024, intermediate_size=2048,
              num_attention_heads=max(8, world), num_key_value_heads=max(2, world), head_dim=128,
              vocab_size=4096,
              max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256, num_gpu_blocks=128)
    cfg = preset("llama-3-8b", **{k: v for k, v in kw.items() if k in (
        "num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads",
        "num_key_value_heads", "head_dim", "vocab_size")})
    sd = full_state_dict(cfg)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (33, 64, 5, 120)]
    sp = SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True)
    results = {}
    for comm in ("nccl", "fused", "fused+sp"):
        get_comm("tp").fused = None
        get_comm("tp").fused_gather = None
        extra = {"sequence_parallel": True} if comm.endswith("+sp") else {}
        llm = LLM("llama-3-8b", tensor_parallel_size=world, comm_backend=comm.split("+")[0],
                  enforce_eager=True, load_format="none", extra=extra, **kw)
        llm.engine.model.load_weights(sd.items())
        llm.engine.runner.keep_logits = True
        llm.generate(prompts, sp)
        torch.cuda.synchronize()
        _native.check_status()
        results[comm] = llm.engine.runner.last_logits
    # generation with the greedy shortcut, eagerly and through CUDA graphs.  With random weights
    # the logits are nearly flat, so a rounding difference may pick another token and the
    # sequences part ways; what must hold is that every generated token is a (near-)maximum
    # of the dense fp32 logits given the tokens before it.
    sp8 = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
    bad = []
    for comm, eager in (("nccl", False), ("fused", True), ("fused", False)):
        get_comm("tp").fused = None
        get_comm("tp").fused_gather = None
        llm = LLM("llama-3-8b", tensor_parallel_size=world, comm_backend=comm,
                  async_scheduling=True, enforce_eager=True, load_format="none", **kw)
        llm.engine.model.load_weights(sd.items())
        if not eager:
            # capture only now: loading re-lays-out some weights into new storage, which a
            # graph captured before the load would not see
            llm.engine.cfg.enforce_eager = False
            llm.engine.runner.capture_graphs([4, 8])
        outs = llm.generate(prompts, sp8)
        torch.cuda.synchronize()
        _native.check_status()
        seqs = [o.outputs[0].token_ids for o in outs]
        full = [p_ + t_ for p_, t_ in zip(prompts, seqs)]
        dense = dense_last_logits(cfg, sd, [f[:-1] for f in full], dev, all_positions=True)
        for p_, t_, lg in zip(prompts, seqs, dense):
            tail = lg[len(p_) - 1:]
            assert tail.shape[0] == len(t_) == 8
            gap = tail.max(-1).values - tail.gather(-1, torch.tensor(t_)[:, None]).squeeze(-1)
            tol = 0.06 * lg.std().item() + 0.03
            if gap.max().item() >= tol:
                bad.append((comm, "eager" if eager else "graphs", [round(g_, 3) for g_ in gap.tolist()]))
    get_comm("tp").fused = None
    get_comm("tp").fused_gather = None
    assert not bad, f"generated tokens far from the dense maximum: {bad}"
    # the single-GPU reference: a dense fp32 forward of the same full checkpoint
    want = dense_last_logits(cfg, sd, prompts, dev)
    for name, got in results.items():
        e = (got - want).abs().max().item()
        assert e < 0.06 * want.std().item() + 0.03, f"{name} logits vs dense reference: {e}"
    a, b = results["nccl"], results["fused"]
    err = (a - b).abs().max().item()
    assert err < 0.05 * a.std().item() + 0.02, f"fused vs nccl logits differ: {err}"
    # sequence parallelism: gather fused into the qkv / gate-up GEMMs, reduce-scatter after
    err_sp = (a - results["fused+sp"]).abs().max().item()
    assert err_sp < 0.05 * a.std().item() + 0.02, f"sequence-parallel logits differ: {err_sp}"
    if rank == 0:
        print(f"tp{world} engine ok (nccl vs fused max logit diff {err:.4f})", flush=True)


if __name__ == "__main__":
    main()
