"""DeepSeek-VL2 under vLLM with both spellings of the view-separator parameter: checkpoints
name it ``view_seperator`` (the original spelling, also the attribute of vLLM's class) or
``view_separator`` (re-saved after the spelling fix).  The reference patches the attribute after
construction (vllm_gcu/models/deepseek_vl2/deepseek_vl2.py:11-20); here the checkpoint name is
mapped while loading, so one class reads either kind."""
from __future__ import annotations

from vllm.model_executor.models.deepseek_vl2 import (DeepseekVL2DummyInputsBuilder,
                                                     DeepseekVL2MultiModalProcessor,
                                                     DeepseekVL2ProcessingInfo,
                                                     DeepseekVLV2ForCausalLM)
from vllm.model_executor.models.utils import WeightsMapper
from vllm.multimodal import MULTIMODAL_REGISTRY


def _separator_attribute() -> str:
    """The spelling vLLM's class uses for the parameter in this vLLM version."""
    import inspect
    src = inspect.getsource(DeepseekVLV2ForCausalLM.__init__)
    return "view_seperator" if "self.view_seperator" in src else "view_separator"


_OWN = _separator_attribute()
_OTHER = "view_separator" if _OWN == "view_seperator" else "view_seperator"


@MULTIMODAL_REGISTRY.register_processor(DeepseekVL2MultiModalProcessor,
                                        info=DeepseekVL2ProcessingInfo,
                                        dummy_inputs=DeepseekVL2DummyInputsBuilder)
class DeepseekVLV2ForCausalLMB200(DeepseekVLV2ForCausalLM):
    hf_to_vllm_mapper = WeightsMapper(
        orig_to_new_prefix={**DeepseekVLV2ForCausalLM.hf_to_vllm_mapper.orig_to_new_prefix,
                            _OTHER: _OWN})
