"""Model registration with vLLM's ``ModelRegistry`` (the plugin's counterpart of
vllm_gcu/models/__init__.py:20-40).

Under vLLM the upstream model definitions run on this package's kernels (platform, attention
backend, layer kernels, communicator), so what is registered here is what upstream lacks:

* the architecture names the reference adds for its quantised and customer checkpoints
  (``QuantMixtralForCausalLM``, ``QuantDeepseekForCausalLM``, ``CustomerLlaMAForCausalLM``),
  mapped to the upstream classes of the same mathematics: per-expert quantised linears are
  what vLLM's fused-MoE quantisation methods already load;
* a DeepSeek-VL2 class that accepts both spellings of the view-separator parameter
  (vllm_gcu/models/deepseek_vl2/deepseek_vl2.py:11-20 re-aliases them after construction;
  here the checkpoint name is mapped at load time).

Every entry is registered lazily by ``"module:Class"`` string, so nothing heavy is imported
until vLLM resolves that architecture.
"""
from __future__ import annotations

ALIASES = {
    "QuantMixtralForCausalLM": "vllm.model_executor.models.mixtral:MixtralForCausalLM",
    "QuantDeepseekForCausalLM": "vllm.model_executor.models.deepseek_v2:DeepseekForCausalLM",
    "CustomerLlaMAForCausalLM": "vllm.model_executor.models.llama:LlamaForCausalLM",
    "DeepseekVLV2ForCausalLM":
        "vllm_gcu_b200.runtime.vllm_deepseek_vl2:DeepseekVLV2ForCausalLMB200",
}


def register_models() -> list[str]:
    """Registers :data:`ALIASES`; returns the architecture names that were registered."""
    from vllm import ModelRegistry
    done = []
    for arch, target in ALIASES.items():
        ModelRegistry.register_model(arch, target)
        done.append(arch)
    return done
