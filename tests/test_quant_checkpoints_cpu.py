"""Quantised checkpoint directories as users have them (``quantization_config`` in
``config.json``, packed tensors under the HuggingFace names of the separate q / k / v / gate / up
projections): GPTQ, AWQ, fp8 with per-tensor scales, fp8 with block scales and compressed-tensors
int8 load through ``LLM(directory)`` and give the logits of the de-quantised dense model."""
import json
import os
import sys

import pytest
import torch

tr = pytest.importorskip("transformers")

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from test_quant_cpu import _awq_pack, _to_i32  # noqa: E402

from vllm_gcu_b200 import LLM, SamplingParams  # noqa: E402
from vllm_gcu_b200.utils.weights import write_safetensors  # noqa: E402


def gptq_pack(w, bits, g):
    # w [N, K] dense -> GPTQ layout: qweight [K/per, N], qzeros [K/g, N/per], scales [K/g, N]
    N, K = w.shape
    per = 32 // bits
    wt = w.t().contiguous()                       # [K, N]
    grp = wt.view(K // g, g, N)
    mx, mn = grp.amax(1), grp.amin(1)
    scale = ((mx - mn) / (2 ** bits - 1)).clamp_min(1e-8)
    zero = torch.round(-mn / scale).clamp(1, 2 ** bits - 1)    # gptq stores zero-1
    q = torch.round(grp / scale[:, None] + zero[:, None]).clamp(0, 2 ** bits - 1).long().view(K, N)
    deq = ((q.view(K // g, g, N).float() - zero[:, None]) * scale[:, None]).view(K, N).t().contiguous()
    qw = torch.zeros(K // per, N, dtype=torch.int64)
    for i in range(per):
        qw |= q[i::per] << (bits * i)
    qz = torch.zeros(K // g, N // per, dtype=torch.int64)
    zi = zero.long() - 1
    for i in range(per):
        qz |= zi[:, i::per] << (bits * i)
    return {"qweight": _to_i32(qw), "qzeros": _to_i32(qz), "scales": scale,
            "g_idx": torch.arange(K, dtype=torch.int32) // g}, deq


def awq_pack(w, g):
    N, K = w.shape
    wt = w.t().contiguous()
    grp = wt.view(K // g, g, N)
    mx, mn = grp.amax(1), grp.amin(1)
    scale = ((mx - mn) / 15).clamp_min(1e-8)
    zero = torch.round(-mn / scale).clamp(0, 15)
    q = torch.round(grp / scale[:, None] + zero[:, None]).clamp(0, 15).view(K, N)
    deq = ((q.view(K // g, g, N) - zero[:, None]) * scale[:, None]).view(K, N).t().contiguous()
    return {"qweight": _awq_pack(q.to(torch.uint8)), "qzeros": _awq_pack(zero.to(torch.uint8)),
            "scales": scale}, deq


def fp8_tensor(w):
    s = w.abs().max() / 448.0
    q = (w / s).clamp(-448, 448).to(torch.float8_e4m3fn)
    return {"weight": q, "weight_scale": s.reshape(())}, q.float() * s


def fp8_block(w):
    N, K = w.shape
    wb = w.view(N // 64, 64, K // 64, 64)
    s = wb.abs().amax(dim=(1, 3)) / 448.0
    q = (wb / s[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    return {"weight": q.view(N, K), "weight_scale_inv": s}, (q.float() * s[:, None, :, None]).view(N, K)


def int8_ct(w):
    s = w.abs().amax(1, keepdim=True) / 127.0
    q = torch.round(w / s).clamp(-128, 127).to(torch.int8)
    return {"weight": q, "weight_scale": s}, q.float() * s


_CT = {"quant_method": "compressed-tensors", "format": "int-quantized", "config_groups": {
    "group_0": {"weights": {"num_bits": 8, "type": "int", "symmetric": True,
                            "strategy": "channel"},
                "input_activations": {"num_bits": 8, "type": "int", "dynamic": True,
                                      "strategy": "token"}, "targets": ["Linear"]}}}

FORMATS = {
    "gptq": (lambda w: gptq_pack(w, 4, 32),
             {"quant_method": "gptq", "bits": 4, "group_size": 32, "desc_act": False,
              "sym": False}, 1e-4),
    "awq": (lambda w: awq_pack(w, 32),
            {"quant_method": "awq", "bits": 4, "group_size": 32, "zero_point": True,
             "version": "gemm"}, 1e-4),
    "fp8_tensor": (fp8_tensor, {"quant_method": "fp8", "activation_scheme": "dynamic"}, 0.08),
    "fp8_block": (fp8_block, {"quant_method": "fp8", "activation_scheme": "dynamic",
                              "weight_block_size": [64, 64]}, 0.08),
    "int8": (int8_ct, _CT, 0.05),
}


@pytest.mark.parametrize("fmt", sorted(FORMATS))
def test_quantised_checkpoint_directory(fmt, tmp_path):
    packer, qcfg, tol = FORMATS[fmt]
    hc = tr.LlamaConfig(vocab_size=320, hidden_size=128, intermediate_size=256,
                        num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                        max_position_embeddings=128, rms_norm_eps=1e-6,
                        tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = tr.LlamaForCausalLM(hc).eval().float()
    out, sd = {}, hf.state_dict()
    for name, w in sd.items():
        if name.endswith("proj.weight"):
            tensors, deq = packer(w)
            sd[name].copy_(deq)                  # the oracle runs the de-quantised weights
            for k, v in tensors.items():
                out[name[:-len("weight")] + k] = v
        else:
            out[name] = w.clone()
    write_safetensors(str(tmp_path / "model.safetensors"), out)
    cfg = hc.to_dict()
    cfg["architectures"] = ["LlamaForCausalLM"]
    cfg["quantization_config"] = qcfg
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    llm = LLM(str(tmp_path), device="cpu", max_num_seqs=4, max_num_batched_tokens=64,
              max_model_len=128, num_gpu_blocks=64, dtype="float32")
    ids = [5, 17, 99, 3, 250, 42, 7, 7, 81, 120, 33]
    llm.engine.runner.keep_logits = True
    llm.generate([ids], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
    got = llm.engine.runner.last_logits[0]
    with torch.inference_mode():
        want = hf(input_ids=torch.tensor([ids])).logits[0, -1]
    assert float((got - want).abs().max()) < tol
    assert int(got.argmax()) == int(want.argmax())
