"""Registers this package's quantisation names with vLLM so ``--quantization awq_gcu`` etc.
resolve when the plugin is active.  The ``*_gcu`` names of the reference are aliases of the
upstream schemes with the same checkpoint format
(vllm_gcu/kernels/quantization/utils.py:10-13)."""
from __future__ import annotations

ALIASES = {"awq_gcu": "awq", "gptq_gcu": "gptq", "fp8_gcu": "fp8", "w8a8_gcu": "compressed-tensors",
           "moe_wna16_gcu": "moe_wna16"}


def register_all() -> list[str]:
    from vllm.model_executor.layers.quantization import (get_quantization_config,
                                                         register_quantization_config)
    done = []
    for alias, target in ALIASES.items():
        try:
            base = get_quantization_config(target)
        except Exception:
            continue
        try:
            cls = type(f"{base.__name__}Alias_{alias}", (base,), {
                "get_name": classmethod(lambda c, _a=alias: _a)})
            register_quantization_config(alias)(cls)
            done.append(alias)
        except Exception:
            continue
    return done
