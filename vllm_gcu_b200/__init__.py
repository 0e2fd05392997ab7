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
    """Registers the quantisation configs of this package with vLLM (the model classes of the
    built-in engine use their own registry, ``vllm_gcu_b200.models``)."""
    try:
        from .runtime import vllm_quant
        vllm_quant.register_all()
    except Exception:   # vLLM absent or too old: the built-in engine is unaffected
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
