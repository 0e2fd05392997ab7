"""Child process of tests/test_gpu_vllm_plugin.py: vLLM (its own engine, scheduler and model
code) with this package loaded through the ``vllm.platform_plugins`` /
``vllm.general_plugins`` entry points.

Checks: the active platform is ``B200Platform``; vLLM's worker is ``B200Worker``; the
attention backend of every layer is ``B200AttentionBackend``; greedy generation of a small
Llama (weights set to N(0, 0.02) after the dummy load) launches this package's kernels and
every generated token is a (near-)maximum of a dense fp32 forward of the same weights; the
built-in engine of this package, given the same weights, passes the same check; vLLM's kernel
chooser selects this package's fp8 / int8 linear kernels, whose results match an fp32 product,
and an fp8-quantised engine runs on them.
"""
import json
import os
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"      # engine core in this process
os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")

import torch  # noqa: E402

CFG = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 1024,
       "intermediate_size": 2048, "num_hidden_layers": 2, "num_attention_heads": 8,
       "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 4096, "rms_norm_eps": 1e-5,
       "rope_theta": 500000.0, "max_position_embeddings": 2048, "torch_dtype": "bfloat16",
       "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2}


def randomise(model):
    """Overwrites the dummy weights with N(0, 0.02) (norm weights 1) and returns them."""
    import zlib
    out = {}
    with torch.no_grad():
        for name, p in sorted(model.named_parameters()):
            if name.endswith("norm.weight") or "layernorm" in name:
                p.fill_(1.0)
            else:
                g = torch.Generator(device=p.device).manual_seed(zlib.crc32(name.encode()))
                p.copy_((torch.randn(p.shape, device=p.device, generator=g) * 0.02).to(p.dtype))
            out[name] = p.detach().float().cpu()
    return out


def to_hf(sd):
    """vLLM's fused parameters -> the per-projection names of a HuggingFace checkpoint."""
    hf = {}
    Hq, Hkv, D, I = 8, 2, 128, CFG["intermediate_size"]
    for k, v in sd.items():
        if k.endswith("qkv_proj.weight"):
            base = k[: -len("qkv_proj.weight")]
            q, kk, vv = v.split([Hq * D, Hkv * D, Hkv * D], 0)
            hf[base + "q_proj.weight"], hf[base + "k_proj.weight"] = q, kk
            hf[base + "v_proj.weight"] = vv
        elif k.endswith("gate_up_proj.weight"):
            base = k[: -len("gate_up_proj.weight")]
            hf[base + "gate_proj.weight"], hf[base + "up_proj.weight"] = v[:I], v[I:]
        else:
            hf[k] = v
    return {k: v.to(torch.bfloat16) for k, v in hf.items()}


def near_max(cfg, sd, prompts, seqs, dev, tag):
    from _tp_worker import dense_last_logits
    full = [p + t for p, t in zip(prompts, seqs)]
    dense = dense_last_logits(cfg, sd, [f[:-1] for f in full], dev, all_positions=True)
    for p, t, lg in zip(prompts, seqs, dense):
        tail = lg[len(p) - 1:]
        gap = tail.max(-1).values - tail.gather(-1, torch.tensor(t)[:, None]).squeeze(-1)
        tol = 0.06 * lg.std().item() + 0.03
        assert gap.max().item() < tol, f"{tag}: generated token far from the maximum: {gap}"


def check_linear_kernels(dev):
    """The fp8 / int8 kernel classes this package puts at the head of vLLM's kernel lists:
    selected by vLLM's own chooser, results against an fp32 product of the de-quantised
    operands."""
    import vllm.model_executor.kernels.linear as vk
    from vllm.model_executor.layers.quantization.utils.quant_utils import (
        kFp8DynamicTokenSym, kFp8StaticTensorSym)
    from vllm.platforms import PlatformEnum
    assert vk._POSSIBLE_FP8_KERNELS[PlatformEnum.CUDA][0].__name__ == "B200FP8ScaledMMLinearKernel"
    assert vk._POSSIBLE_INT8_KERNELS[PlatformEnum.CUDA][0].__name__ == "B200Int8ScaledMMLinearKernel"
    g = torch.Generator(device=dev).manual_seed(11)
    M, N, K = 77, 768, 512
    x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, device=dev, generator=g) * 0.05
    bias = torch.randn(N, device=dev, generator=g).to(torch.bfloat16)
    f8 = torch.float8_e4m3fn
    for static in (False, True):
        k = vk.init_fp8_linear_kernel(
            activation_quant_key=kFp8StaticTensorSym if static else kFp8DynamicTokenSym,
            weight_quant_key=kFp8StaticTensorSym, input_dtype=torch.bfloat16,
            out_dtype=torch.bfloat16, weight_shape=(N, K), module_name="check")
        assert type(k).__name__ == "B200FP8ScaledMMLinearKernel", type(k)
        # two fused shards with one scale each
        ws = torch.stack([w[:256].abs().max(), w[256:].abs().max()]) / 448.0
        per_row = torch.cat([ws[0].expand(256), ws[1].expand(N - 256)])
        qw = (w / per_row[:, None]).to(f8)
        layer = torch.nn.Module()
        layer.weight = torch.nn.Parameter(qw.t(), requires_grad=False)
        layer.weight_scale = torch.nn.Parameter(ws.clone(), requires_grad=False)
        layer.logical_widths = [256, N - 256]
        layer.input_scale = torch.nn.Parameter(x.float().abs().max() / 448.0,
                                               requires_grad=False) if static else None
        k.process_weights_after_loading(layer)
        y = k.apply_weights(layer, x, bias).float()
        want = x.float() @ (qw.float() * per_row[:, None]).t() + bias.float()
        err = (y - want).abs().max().item()
        assert err < 0.08 * want.abs().max().item(), ("fp8", static, err)
    for static in (False, True):
        k = vk.init_int8_linear_kernel(is_channelwise=True, is_static_input_scheme=static,
                                       input_symmetric=True, module_name="check")
        assert type(k).__name__ == "B200Int8ScaledMMLinearKernel", type(k)
        ws = w.abs().amax(1, keepdim=True) / 127.0
        qw = torch.round(w / ws).clamp(-128, 127).to(torch.int8)
        layer = torch.nn.Module()
        layer.weight = torch.nn.Parameter(qw, requires_grad=False)
        layer.weight_scale = torch.nn.Parameter(ws.clone(), requires_grad=False)
        layer.logical_widths = [N]
        layer.input_scale = torch.nn.Parameter((x.float().abs().max() / 127.0).reshape(1),
                                               requires_grad=False) if static else None
        layer.input_zero_point = None
        layer.azp_adj = None
        k.process_weights_after_loading(layer)
        y = k.apply_weights(layer, x, bias).float()
        want = x.float() @ (qw.float() * ws).t() + bias.float()
        err = (y - want).abs().max().item()
        assert err < 0.05 * want.abs().max().item(), ("int8", static, err)


def check_fp8_engine(d, prompts):
    """vLLM with ``quantization="fp8"`` (weights quantised at load): every linear layer picks
    this package's fp8 kernel and generation launches it."""
    from vllm import LLM, SamplingParams
    from vllm_gcu_b200.ops import _native
    llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16",
              quantization="fp8", enforce_eager=True, max_model_len=256, max_num_seqs=8,
              block_size=16, max_num_batched_tokens=256, gpu_memory_utilization=0.25,
              enable_prefix_caching=False, seed=0)

    def kernels(model):
        return sorted({type(m.quant_method.fp8_linear).__name__ for m in model.modules()
                       if hasattr(getattr(m, "quant_method", None), "fp8_linear")})
    assert llm.apply_model(kernels)[0] == ["B200FP8ScaledMMLinearKernel"], \
        llm.apply_model(kernels)
    sp = SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True, detokenize=False)
    n0 = _native.launch_count
    outs = llm.generate([{"prompt_token_ids": p} for p in prompts], sp, use_tqdm=False)
    torch.cuda.synchronize()
    _native.check_status()
    assert all(len(o.outputs[0].token_ids) == 4 for o in outs)
    return _native.launch_count - n0


def main():
    from vllm import LLM, SamplingParams
    from vllm.platforms import current_platform
    assert type(current_platform).__name__ == "B200Platform", type(current_platform)
    assert current_platform.get_nixl_supported_devices() == {"cuda": ("cuda", "cpu")}
    assert current_platform.get_nixl_memory_type() == "VRAM"
    from vllm_gcu_b200.ops import _native

    d = tempfile.mkdtemp(prefix="tiny_llama_cfg_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(CFG, f)
    if os.environ.get("B200_PLUGIN_CHECK", "base") == "fp8":
        g = torch.Generator().manual_seed(3)
        prompts = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (33, 64, 5, 120)]
        launched_fp8 = check_fp8_engine(d, prompts)
        print(f"vllm fp8 ok: {launched_fp8} native launches with fp8 weights", flush=True)
        sys.stdout.flush()
        os._exit(0)
    llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16",
              enforce_eager=True, max_model_len=256, max_num_seqs=8, block_size=16,
              max_num_batched_tokens=256, gpu_memory_utilization=0.25,
              enable_prefix_caching=False, seed=0)
    vcfg = llm.llm_engine.vllm_config
    assert vcfg.parallel_config.worker_cls.endswith("B200Worker"), vcfg.parallel_config.worker_cls
    sd = llm.apply_model(randomise)[0]

    def backends(model):
        return sorted({type(m.impl).__name__ for m in model.modules() if hasattr(m, "impl")})
    assert llm.apply_model(backends)[0] == ["B200AttentionImpl"], llm.apply_model(backends)

    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (33, 64, 5, 120)]
    sp = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True, detokenize=False)
    n0 = _native.launch_count
    outs = llm.generate([{"prompt_token_ids": p} for p in prompts], sp, use_tqdm=False)
    torch.cuda.synchronize()
    _native.check_status()
    launched = _native.launch_count - n0
    seqs = [list(o.outputs[0].token_ids) for o in outs]
    assert all(len(s) == 8 for s in seqs)
    # 2 layers x (norms, GEMMs, activation, cache write, attention) x 9 engine steps
    assert launched >= 2 * 8 * 9, f"only {launched} native launches"

    from vllm_gcu_b200.config import preset
    keys = ("num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads",
            "num_key_value_heads", "head_dim", "vocab_size", "rms_norm_eps")
    kw = {k: CFG[k] for k in keys}
    cfg = preset("llama-3-8b", **kw)
    hf = to_hf(sd)
    dev = torch.device("cuda")
    near_max(cfg, hf, prompts, seqs, dev, "vllm + plugin")

    # the built-in engine on the same weights
    from vllm_gcu_b200.engine.llm import LLM as OwnLLM
    from vllm_gcu_b200.engine.request import SamplingParams as OwnSP
    own = OwnLLM("llama-3-8b", max_num_seqs=8, max_num_batched_tokens=256, max_model_len=256,
                 num_gpu_blocks=128, enforce_eager=True, load_format="none", **kw)
    own.engine.model.load_weights(hf.items())
    outs2 = own.generate(prompts, OwnSP(max_tokens=8, temperature=0.0, ignore_eos=True))
    seqs2 = [o.outputs[0].token_ids for o in outs2]
    near_max(cfg, hf, prompts, seqs2, dev, "built-in engine")
    same = sum(a == b for s1, s2 in zip(seqs, seqs2) for a, b in zip(s1, s2))
    from vllm.config import set_current_vllm_config
    with set_current_vllm_config(vcfg):              # kernel objects build vLLM custom ops
        check_linear_kernels(dev)
    print(f"vllm plugin ok: {launched} native launches under vLLM, "
          f"{same}/{8 * len(prompts)} tokens equal to the built-in engine; fp8 and int8 "
          f"linear kernels selected and checked", flush=True)
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
