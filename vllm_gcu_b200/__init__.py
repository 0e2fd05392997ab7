"""vllm_gcu_b200 – Blackwell-native counterpart of the vllm-gcu platform plugin.

Two ways in:

* the built-in engine: ``from vllm_gcu_b200.engine.llm import LLM`` (one process per GPU,
  hand-written sm_100a kernels, fused tensor-parallel collectives);
* the vLLM platform plugin: entry points ``vllm.platform_plugins`` ->
  :func:`register_platform_plugins` and ``vllm.general_plugins`` ->
  :func:`register_custom_models` (see ``setup.py``), as in vllm_gcu/__init__.py:22-23 and
  vllm_gcu/models/__init__.py:20-40.
"""
from __future__ import annotations

__version__ = "0.1.0"


def register_platform_plugins() -> str:
    return "vllm_gcu_b200.platform.B200Platform"


def register_custom_models() -> None:
    """General plugin hook (runs in every vLLM process): registers this package's attention
    backend under ``AttentionBackendEnum.CUSTOM``, its layer kernels (RMSNorm, SiLU-and-mul,
    unquantised GEMM, fp8 / int8 scaled GEMMs), its quantisation configs and the architecture
    names upstream lacks (``runtime/vllm_models.py``) with vLLM.  The model classes of the
    built-in engine use their own registry (``vllm_gcu_b200.models``); under vLLM the upstream
    model definitions run on these kernels."""
    try:
        from .runtime import vllm_quant
        vllm_quant.register_all()
    except Exception:   # vLLM absent or too old: the built-in engine is unaffected
        pass
    try:
        from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend
        register_backend(AttentionBackendEnum.CUSTOM,
                         "vllm_gcu_b200.runtime.vllm_attention.B200AttentionBackend")
    except Exception:
        pass
    try:
        from .runtime import vllm_models
        vllm_models.register_models()
    except Exception:
        pass
    try:
        import os
        if os.environ.get("VLLM_B200_VLLM_NATIVE_OPS", "1") != "0":
            from .runtime import vllm_ops
            vllm_ops.register_ops()
            from .runtime import vllm_linear_kernels
            vllm_linear_kernels.register_linear_kernels()
    except Exception:
        pass


def __getattr__(name: str):
    # lazy: importing the package must stay cheap for the vLLM plugin loader
    if name in ("LLM", "LLMEngine"):
        from .engine import llm as _llm
        return getattr(_llm, name)
    if name in ("SamplingParams", "RequestOutput", "CompletionOutput"):
        from .engine import request as _req
        return getattr(_req, name)
    raise AttributeError(name)
