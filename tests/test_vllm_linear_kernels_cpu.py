"""The fp8 / int8 linear-kernel classes offered to vLLM: registration at the head of vLLM's
priority lists, the configurations they accept, and the weight-scale layouts they take
(CPU: the GEMM itself is covered by the GPU plugin test)."""
import pytest
import torch

pytest.importorskip("vllm")


def test_registration_and_configs(monkeypatch):
    from vllm_gcu_b200.runtime import vllm_linear_kernels as LK
    try:
        import vllm.model_executor.kernels.linear as vk
        from vllm.model_executor.kernels.linear.scaled_mm.ScaledMMLinearKernel import (
            FP8ScaledMMLinearLayerConfig, Int8ScaledMMLinearLayerConfig)
        from vllm.model_executor.layers.quantization.utils.quant_utils import (
            kFp8Dynamic128Sym, kFp8DynamicTokenSym, kFp8StaticTensorSym)
        from vllm.platforms import PlatformEnum
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"this vLLM has no linear kernel lists: {e}")
    assert LK.register_linear_kernels() and LK.register_linear_kernels()
    fp8_list = vk._POSSIBLE_FP8_KERNELS[PlatformEnum.CUDA]
    int8_list = vk._POSSIBLE_INT8_KERNELS[PlatformEnum.CUDA]
    assert fp8_list[0] is LK.B200FP8ScaledMMLinearKernel
    assert int8_list[0] is LK.B200Int8ScaledMMLinearKernel
    assert sum(k.__name__ == "B200FP8ScaledMMLinearKernel" for k in fp8_list) == 1
    # only offered when the B200 platform is the active one
    assert LK.B200FP8ScaledMMLinearKernel.is_supported()[0] is False
    monkeypatch.setattr(LK, "_on_b200_platform", lambda: True)
    assert LK.B200FP8ScaledMMLinearKernel.is_supported()[0]

    def cfg(act, n=256, k=128, out=torch.bfloat16):
        return FP8ScaledMMLinearLayerConfig(weight_quant_key=kFp8StaticTensorSym,
                                            activation_quant_key=act, weight_shape=(n, k),
                                            input_dtype=torch.bfloat16, out_dtype=out)
    F = LK.B200FP8ScaledMMLinearKernel
    assert F.can_implement(cfg(kFp8DynamicTokenSym))[0]
    assert F.can_implement(cfg(kFp8StaticTensorSym))[0]
    assert not F.can_implement(cfg(kFp8Dynamic128Sym))[0]
    assert not F.can_implement(cfg(kFp8DynamicTokenSym, out=torch.float16))[0]
    assert not F.can_implement(cfg(kFp8DynamicTokenSym, n=250))[0]
    I = LK.B200Int8ScaledMMLinearKernel
    assert I.can_implement(Int8ScaledMMLinearLayerConfig(True, False, True))[0]
    assert not I.can_implement(Int8ScaledMMLinearLayerConfig(True, False, False))[0]

    # weight layouts: the fp8 class receives the [K, N] transpose and one scale per fused shard
    # (an instance needs a vLLM engine config: the methods are called on a stand-in here)
    import types
    k8 = types.SimpleNamespace(
        layer_param_names=["weight", "weight_scale", "input_scale", "input_scale_ub"],
        fp8_dtype=torch.float8_e4m3fn)
    layer = torch.nn.Module()
    w = (torch.randn(256, 128) * 0.1).to(torch.float8_e4m3fn)
    layer.weight = torch.nn.Parameter(w.t(), requires_grad=False)
    layer.weight_scale = torch.nn.Parameter(torch.tensor([0.5, 2.0]), requires_grad=False)
    layer.logical_widths = [64, 192]
    F.process_weights_after_loading(k8, layer)
    assert layer._b200_w.shape == (256, 128) and layer._b200_w.is_contiguous()
    assert layer._b200_w.data_ptr() == w.data_ptr()                 # no copy
    assert layer._b200_ws.tolist() == [0.5] * 64 + [2.0] * 192
    x = torch.randn(3, 128)
    y = F._fallback(k8, layer, x, None)
    want = x @ (w.float() * layer._b200_ws[:, None]).t()
    assert torch.allclose(y, want, atol=1e-4)
