"""Quantised linear methods on the CPU reference path: checkpoint formats, load-time
re-packing and numerics against the de-quantised weights."""
import torch

from vllm_gcu_b200.layers import quant as Q
from vllm_gcu_b200.layers.linear import (ColumnParallelLinear, MergedColumnParallelLinear,
                                         RowParallelLinear)
from vllm_gcu_b200.ops import ref


def _to_i32(x: torch.Tensor) -> torch.Tensor:
    x = x & 0xFFFFFFFF
    return torch.where(x >= 2 ** 31, x - 2 ** 32, x).to(torch.int32)


def test_awq_linear_matches_dequantised():
    torch.manual_seed(0)
    K, N, g = 256, 128, 64
    q = torch.randint(0, 16, (K, N), dtype=torch.uint8)
    z = torch.randint(0, 16, (K // g, N), dtype=torch.uint8)
    s = (torch.rand(K // g, N) * 0.02 + 0.01)
    w = ((q.float() - z.float().repeat_interleave(g, 0)) * s.repeat_interleave(g, 0)).t()  # [N,K]
    order = Q.AWQ_REVERSE_ORDER

    def pack(t):
        R, C = t.shape
        v = t.view(R, C // 8, 8).to(torch.int64)
        out = torch.zeros(R, C // 8, dtype=torch.int64)
        for c in range(8):
            out |= v[:, :, c] << (4 * order[c])
        return _to_i32(out)

    layer = ColumnParallelLinear(K, N, dtype=torch.float32, device="cpu",
                                 quant_method=Q.WNA16LinearMethod("awq", 4, g))
    layer.load_weight("qweight", pack(q))
    layer.load_weight("qzeros", pack(z))
    layer.load_weight("scales", s)
    layer.finalize()
    x = torch.randn(5, K)
    assert torch.allclose(layer(x), x @ w.t(), atol=1e-4, rtol=1e-4)


def test_gptq_linear_4_and_8_bit():
    torch.manual_seed(1)
    for bits in (4, 8):
        K, N, g = 128, 64, 32
        per = 32 // bits
        q = torch.randint(0, 2 ** bits, (K, N), dtype=torch.int64)
        zp = torch.randint(1, 2 ** bits, (K // g, N), dtype=torch.int64)
        s = torch.rand(K // g, N) * 0.02 + 0.01
        w = ((q.float() - zp.float().repeat_interleave(g, 0)) * s.repeat_interleave(g, 0)).t()
        qw = torch.zeros(K // per, N, dtype=torch.int64)
        for i in range(per):
            qw |= q[i::per] << (bits * i)
        qz = torch.zeros(K // g, N // per, dtype=torch.int64)
        for i in range(per):
            qz |= (zp[:, i::per] - 1) << (bits * i)
        layer = RowParallelLinear(K, N, dtype=torch.float32, device="cpu",
                                  quant_method=Q.WNA16LinearMethod("gptq", bits, g))
        layer.load_weight("qweight", _to_i32(qw))
        layer.load_weight("qzeros", _to_i32(qz))
        layer.load_weight("scales", s)
        layer.load_weight("g_idx", torch.arange(K, dtype=torch.int32) // g)
        layer.finalize()
        x = torch.randn(3, K)
        assert torch.allclose(layer(x), x @ w.t(), atol=1e-4, rtol=1e-4)


def test_fp8_per_channel_and_block():
    torch.manual_seed(2)
    K, N = 256, 384
    w = torch.randn(N, K) * 0.05
    x = torch.randn(7, K)
    # per channel, dynamic per-token activations
    qw, sw = ref.dynamic_per_token_fp8_quant(w)
    layer = ColumnParallelLinear(K, N, dtype=torch.float32, device="cpu",
                                 quant_method=Q.Fp8LinearMethod(None, False))
    layer.load_weight("weight", qw)
    layer.load_weight("weight_scale", sw.flatten())
    y = layer(x)
    assert (y - x @ w.t()).abs().max() < 0.15
    # 128x128 block scales + 1x128 activation scales
    wb = w.view(N // 128, 128, K // 128, 128)
    sb = wb.abs().amax(dim=(1, 3)) / 448.0
    qb = (wb / sb[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(N, K)
    layer2 = MergedColumnParallelLinear(K, [256, 128], dtype=torch.float32, device="cpu",
                                        quant_method=Q.Fp8LinearMethod([128, 128], False))
    layer2.load_weight("weight", qb[:256], 0)
    layer2.load_weight("weight", qb[256:], 1)
    layer2.load_weight("weight_scale_inv", sb[:2], 0)
    layer2.load_weight("weight_scale_inv", sb[2:], 1)
    y2 = layer2(x)
    assert (y2 - x @ w.t()).abs().max() < 0.15


def test_int8_w8a8():
    torch.manual_seed(3)
    K, N = 128, 96
    w = torch.randn(N, K) * 0.05
    ws = w.abs().amax(1) / 127
    qw = torch.round(w / ws[:, None]).clamp(-128, 127).to(torch.int8)
    x = torch.randn(4, K)
    layer = ColumnParallelLinear(K, N, bias=True, dtype=torch.float32, device="cpu",
                                 quant_method=Q.Int8LinearMethod(False))
    layer.load_weight("weight", qw)
    layer.load_weight("out_scales", ws)
    layer.load_weight("bias", torch.ones(N))
    assert (layer(x) - (x @ w.t() + 1)).abs().max() < 0.05


def _awq_pack(t):
    R, C = t.shape
    v = t.view(R, C // 8, 8).to(torch.int64)
    out = torch.zeros(R, C // 8, dtype=torch.int64)
    for c in range(8):
        out |= v[:, :, c] << (4 * Q.AWQ_REVERSE_ORDER[c])
    return _to_i32(out)


def test_moe_checkpoints_awq_fp8_block_and_int8_load_into_the_expert_tensors():
    """Quantised expert tensors (AWQ ``moe_wna16``, fp8 128x128 block, int8 per-channel) are
    de-quantised at load into the grouped-GEMM expert weights; the model then matches one
    loaded from the de-quantised bf16 checkpoint."""
    import dataclasses

    from vllm_gcu_b200.config import preset
    from vllm_gcu_b200.models import build_model
    torch.manual_seed(3)
    base_cfg = dataclasses.replace(preset("tiny-qwen3-moe"), dtype=torch.float32)
    ref_model = build_model(base_cfg, "cpu")
    ref_model.init_random(0)
    E, I, H = base_cfg.num_experts, base_cfg.moe_intermediate_size, base_cfg.hidden_size
    L = base_cfg.num_hidden_layers
    g = 32
    for kind in ("awq", "fp8", "w8a8"):
        qcfg = {"awq": {"quant_method": "awq", "bits": 4, "group_size": g,
                        "modules_to_not_convert": ["self_attn", "gate", "lm_head"]},
                "fp8": {"quant_method": "fp8", "weight_block_size": [128, 128],
                        "ignored_layers": ["self_attn", "mlp.gate", "lm_head"]},
                "w8a8": {"ignored_layers": ["self_attn", "mlp.gate", "lm_head"]}}[kind]
        name = {"awq": "moe_wna16_gcu", "fp8": "fp8", "w8a8": "w8a8"}[kind]
        cfg = dataclasses.replace(base_cfg, quantization=name, quant_config=qcfg)
        sd_q, sd_ref = {}, {}
        for k, v in ref_model.state_dict().items():
            if ".mlp.experts." not in k:
                sd_q["model." + k if not k.startswith(("model.", "lm_head")) else k] = v
        # rebuild per-expert HF tensors from the stacked parameters of the reference model
        for li in range(L):
            moe = ref_model.layers[str(li)].mlp.experts
            for e in range(E):
                mats = {"gate_proj": moe.w13.data[e, :I], "up_proj": moe.w13.data[e, I:],
                        "down_proj": moe.w2.data[e]}
                for proj, w in mats.items():
                    pre = f"model.layers.{li}.mlp.experts.{e}.{proj}."
                    N_, K_ = w.shape
                    if kind == "awq":
                        q = torch.randint(0, 16, (K_, N_), dtype=torch.uint8)
                        z = torch.randint(0, 16, (K_ // g, N_), dtype=torch.uint8)
                        s = torch.rand(K_ // g, N_) * 0.02 + 0.01
                        deq = ((q.float() - z.float().repeat_interleave(g, 0))
                               * s.repeat_interleave(g, 0)).t().contiguous()
                        sd_q[pre + "qweight"] = _awq_pack(q)
                        sd_q[pre + "qzeros"] = _awq_pack(z)
                        sd_q[pre + "scales"] = s
                    elif kind == "fp8":
                        q = (w * 8).to(torch.float8_e4m3fn)
                        s = torch.rand(-(-N_ // 128), -(-K_ // 128)) * 0.1 + 0.05
                        deq = q.float() * s.repeat_interleave(128, 0)[:N_].repeat_interleave(
                            128, 1)[:, :K_]
                        sd_q[pre + "weight"] = q
                        sd_q[pre + "weight_scale_inv"] = s
                    else:
                        q = torch.randint(-127, 128, (N_, K_), dtype=torch.int8)
                        s = torch.rand(N_) * 0.002 + 0.001
                        deq = q.float() * s[:, None]
                        sd_q[pre + "weight"] = q
                        sd_q[pre + "weight_scale"] = s
                    sd_ref[pre + "weight"] = deq
        # the un-quantised parts are shared; names follow the HF layout of the checkpoint
        hf_common = {k: v for k, v in sd_q.items() if ".experts." not in k}
        m_ref = build_model(base_cfg, "cpu")
        m_ref.load_weights(list(hf_common.items()) + list(sd_ref.items()))
        m_q = build_model(cfg, "cpu")
        m_q.load_weights(list(sd_q.items()))
        for li in range(L):
            a, b = m_ref.layers[str(li)].mlp.experts, m_q.layers[str(li)].mlp.experts
            assert torch.allclose(a.w13.data, b.w13.data, atol=1e-5), kind
            assert torch.allclose(a.w2.data, b.w2.data, atol=1e-5), kind


def test_expert_storage_by_checkpoint_format():
    """Which quantised expert formats stay quantised on a GPU (layers/quant/moe.py)."""
    from vllm_gcu_b200.layers.quant.moe import expert_storage
    assert expert_storage("fp8", {"quant_method": "fp8", "weight_block_size": [128, 128]}) == "fp8_block"
    assert expert_storage("fp8_gcu", {"weight_block_size": [64, 64]}) is None
    assert expert_storage("fp8", {"quant_method": "fp8"}) == "fp8"
    assert expert_storage("w8a8_gcu", {}) == "int8"
    assert expert_storage("compressed-tensors", {"quant_method": "compressed-tensors"}) == "int8"
    assert expert_storage("moe_wna16_gcu", {"quant_method": "awq", "bits": 4}) == "wna16"
    assert expert_storage(None, None) is None


def test_packed_wna16_experts_equal_dequantised_experts():
    """AWQ / GPTQ experts kept packed (integers + per-group scales, the layout of the grouped
    de-quantising GEMM) give the output of the experts de-quantised at load."""
    from vllm_gcu_b200.layers.moe import FusedMoE
    from vllm_gcu_b200.layers.quant.moe import dequant_wna16, expert_storage, unpack_wna16
    assert expert_storage("moe_wna16_gcu", {"quant_method": "awq", "bits": 4}) == "wna16"
    assert expert_storage("gptq", {"quant_method": "gptq", "bits": 8}) == "wna16"
    assert expert_storage("gptq", {"quant_method": "gptq", "bits": 4, "desc_act": True}) is None
    assert expert_storage("gptq", {"quant_method": "gptq", "bits": 3}) is None
    torch.manual_seed(5)
    E, I, H, g = 4, 128, 64, 32
    for kind, bits in (("awq", 4), ("gptq", 4), ("gptq", 8)):
        packed = FusedMoE(E, H, I, torch.float32, "cpu", False)
        plain = FusedMoE(E, H, I, torch.float32, "cpu", False)
        assert packed.enable_wna16(bits, g, any_device=True)
        assert not FusedMoE(E, H, 96, torch.float32, "cpu", False).enable_wna16(bits, g, True)
        for e in range(E):
            for which, (N_, K_) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
                top = 1 << bits
                q = torch.randint(0, top, (K_, N_), dtype=torch.int64)
                z = torch.randint(0, top, (K_ // g, N_), dtype=torch.int64)
                s = torch.rand(K_ // g, N_) * 0.02 + 0.01
                if kind == "awq":
                    qw, qz = _awq_pack(q), _awq_pack(z)
                else:
                    per = 32 // bits
                    qw = torch.zeros(K_ // per, N_, dtype=torch.int64)
                    for i in range(per):
                        qw |= q[i::per] << (bits * i)
                    qz = torch.zeros(K_ // g, N_ // per, dtype=torch.int64)
                    for i in range(per):
                        qz |= (z[:, i::per] - 1) << (bits * i)   # GPTQ stores zero - 1
                    qw, qz = _to_i32(qw), _to_i32(qz)
                want = dequant_wna16(kind, bits, g, qw, qz, s, torch.float32)
                qi, sc, zs = unpack_wna16(kind, bits, qw, qz, s)
                assert qi.dtype == torch.uint8 and qi.shape == (N_, K_)
                got = qi.float() * sc.repeat_interleave(g, 1) - zs.repeat_interleave(g, 1)
                assert torch.allclose(got, want, atol=1e-6)
                assert packed.load_expert_weight_wna16(e, which, qi, sc, zs)
                plain.load_expert_weight(e, which, want)
        x = torch.randn(9, H)
        ids = torch.randint(0, E, (9, 2), dtype=torch.int32)
        w = torch.rand(9, 2)
        assert packed.w13.numel() == 0 and packed.w13_q.shape == (E, 2 * I, H // (2 if bits == 4 else 1))
        a, b = packed(x, w, ids), plain(x, w, ids)
        assert (a - b).abs().max() <= 1e-5 * b.abs().max(), (kind, bits, (a - b).abs().max())
