"""Platform policy, environment flags, utilities and the plugin entry points."""
import os

import torch

import vllm_gcu_b200
from vllm_gcu_b200 import envs
from vllm_gcu_b200.platform import PolicyInput, apply_platform_policy


def test_entry_points_and_lazy_exports():
    assert vllm_gcu_b200.register_platform_plugins() == "vllm_gcu_b200.platform.B200Platform"
    vllm_gcu_b200.register_custom_models()          # must not raise with or without vLLM
    assert vllm_gcu_b200.LLM.__name__ == "LLM"
    assert vllm_gcu_b200.SamplingParams(max_tokens=3).max_tokens == 3


def test_policy_async_exclusions_and_dp_ep_rules():
    d = apply_platform_policy(PolicyInput(additional_config={"async_scheduling": True}))
    assert d.async_scheduling and d.executor_cls is None
    d = apply_platform_policy(PolicyInput(additional_config={"async_scheduling": True,
                                                             "async_executing": True}))
    assert d.async_executing and d.executor_cls.endswith("AsyncMultiprocExecutor")
    d = apply_platform_policy(PolicyInput(pipeline_parallel_size=2,
                                          additional_config={"async_scheduling": True}))
    assert not d.async_scheduling and any("pipeline" in n for n in d.notes)
    d = apply_platform_policy(PolicyInput(num_scheduler_steps=4,
                                          additional_config={"async_scheduling": True}))
    assert not d.async_scheduling
    d = apply_platform_policy(PolicyInput(data_parallel_size=2, enable_expert_parallel=True,
                                          cuda_graph_sizes=[1, 2, 4],
                                          scheduling_policy="priority",
                                          additional_config={"num_redundant_experts": 8,
                                                             "enable_eplb": True}))
    assert d.cuda_graph_sizes[0] == 0 and d.dp_padding is False
    assert d.scheduler_cls.endswith(":priority")
    assert d.enable_eplb and d.num_redundant_experts == 8
    d = apply_platform_policy(PolicyInput(additional_config={"num_redundant_experts": 8}))
    assert d.num_redundant_experts == 0 and d.notes


def test_env_flags_accept_both_prefixes(monkeypatch):
    monkeypatch.delenv("VLLM_B200_ORACLE", raising=False)
    assert envs.ORACLE is None and envs.NVTX is False
    monkeypatch.setenv("VLLM_GCU_ENABLE_SEQUENCE_PARALLEL", "1")      # the reference's spelling
    assert envs.ENABLE_SEQUENCE_PARALLEL is True
    monkeypatch.setenv("VLLM_B200_ORACLE", "gemm_bf16,paged_decode")
    assert envs.ORACLE == ["gemm_bf16", "paged_decode"]
    monkeypatch.setenv("VLLM_B200_HOOKS", "a,b")
    assert envs.HOOKS == ["a", "b"]


def test_utilities():
    from vllm_gcu_b200.utils import bind_cpu_affinity, ep_alltoall_threshold
    from vllm_gcu_b200.utils.sleep_mode import CuMemAllocator
    import pytest
    before = os.sched_getaffinity(0)
    try:
        mine = bind_cpu_affinity(0, 2)
        assert mine and set(mine) <= set(before)
    finally:
        os.sched_setaffinity(0, before)
    assert ep_alltoall_threshold(256, 256, 8) >= 256
    with pytest.raises(NotImplementedError):
        CuMemAllocator.get_instance().sleep()
    from vllm_gcu_b200.layers.quant import SUPPORTED_QUANTIZATION
    for name in ("fp8_gcu", "awq_gcu", "gptq_gcu", "w8a8_gcu", "moe_wna16_gcu", "w4a8_gcu"):
        assert name in SUPPORTED_QUANTIZATION
    assert torch.float8_e4m3fn is not None


def test_host_sanitizer_build_options():
    """``csrc/build.py --sanitize``: flags, separate object directory and library name."""
    import pytest
    from vllm_gcu_b200.csrc import build as B
    assert B.sanitize_flags(None) == []
    fl = B.sanitize_flags("address")
    assert fl[0] == "-Xcompiler" and "-fsanitize=address" in fl[1]
    assert B.lib_path_for(None).name == "_b200.so"
    assert B.lib_path_for("thread").name == "_b200.thread.so"
    with pytest.raises(ValueError):
        B.sanitize_flags("memory")


def test_vllm_model_registry_gets_the_extra_architectures():
    """The general-plugin hook registers the reference's extra architecture names with vLLM's
    ``ModelRegistry`` (lazily, by string), and the DeepSeek-VL2 class reads both spellings of
    the separator parameter."""
    import pytest
    pytest.importorskip("vllm")
    from vllm import ModelRegistry
    from vllm_gcu_b200.runtime import vllm_models
    done = vllm_models.register_models()
    archs = set(ModelRegistry.get_supported_archs())
    assert set(done) <= archs and "QuantMixtralForCausalLM" in archs
    for arch, target in vllm_models.ALIASES.items():
        ent = ModelRegistry.models[arch]
        assert f"{ent.module_name}:{ent.class_name}" == target
    import importlib
    for target in vllm_models.ALIASES.values():       # every target resolves to a class
        mod, _, cls = target.partition(":")
        assert isinstance(getattr(importlib.import_module(mod), cls), type)
    from vllm_gcu_b200.runtime.vllm_deepseek_vl2 import _OTHER, _OWN, DeepseekVLV2ForCausalLMB200
    names = [(_OTHER, None), (_OWN, None), ("language.model.embed_tokens.weight", None),
             ("vision.blocks.0.attn.qkv.weight", None)]
    got = [n for n, _ in DeepseekVLV2ForCausalLMB200.hf_to_vllm_mapper.apply(names)]
    assert got == [_OWN, _OWN, "language_model.model.embed_tokens.weight",
                   "vision.blocks.0.attn.qkv.weight"]


def test_vllm_worker_step_hooks(monkeypatch):
    """The vLLM worker subclass wraps every step: the status word is read every n-th step and
    an error recorded by a kernel surfaces as an exception of the step."""
    import pytest
    pytest.importorskip("vllm")
    try:
        from vllm_gcu_b200.runtime.vllm_worker import B200Worker
    except Exception as e:  # noqa: BLE001 - vLLM's GPU worker does not import on this machine
        pytest.skip(f"vLLM's GPU worker cannot be imported here: {e}")
    from vllm_gcu_b200.ops import _native
    w = object.__new__(B200Worker)
    calls = []
    checks = []
    monkeypatch.setattr(_native, "check_status", lambda: checks.append(len(calls)))
    monkeypatch.setenv("VLLM_B200_CHECK_STATUS_EVERY", "2")

    def inner(a, b=0):
        calls.append((a, b))
        return a + b
    assert [w._step(inner, i, b=1) for i in range(5)] == [1, 2, 3, 4, 5]
    assert calls == [(i, 1) for i in range(5)] and checks == [2, 4]

    def failing():
        raise KeyError("boom")
    with pytest.raises(KeyError):
        w._step(failing)
    monkeypatch.setenv("VLLM_B200_CHECK_STATUS_EVERY", "0")
    w._step(inner, 1)
    assert checks == [2, 4]
