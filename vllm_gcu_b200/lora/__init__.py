"""Multi-LoRA serving: batched gather kernels, adapter manager and the punica-style wrapper
(vllm_gcu/lora/punica_gcu.py:22-366, vllm_gcu/lora/lora_ops.py)."""
from .manager import LoRAManager, LoRARequest  # noqa: F401
from .ops import bgmv_expand, bgmv_expand_slice, bgmv_shrink, sgmv_expand, sgmv_shrink  # noqa: F401
from .punica import PunicaWrapperB200  # noqa: F401
