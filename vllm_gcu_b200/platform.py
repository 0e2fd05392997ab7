"""vLLM out-of-tree platform for B200.

``register_platform_plugins`` (``vllm.platform_plugins`` entry point, see ``setup.py``)
returns ``"vllm_gcu_b200.platform.B200Platform"``.  The class mirrors the reference's
``GCUPlatform`` (vllm_gcu/gcu.py:45-509): device naming, supported quantisation list,
attention backend selection, communicator / punica hooks and the configuration policy of
``check_and_update_config``.

The policy itself lives in :func:`apply_platform_policy`, a function over duck-typed config
objects, so it is unit-tested without importing vLLM; ``B200Platform`` adapts vLLM's
``VllmConfig`` to it.  The class is created on first access (importing vLLM is optional).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from .layers.quant import SUPPORTED_QUANTIZATION

DEVICE_NAME = "B200"
DEVICE_TYPE = "cuda"
DEFAULT_BLOCK_SIZE = 16


@dataclass
class PolicyInput:
    """The configuration facts the policy looks at."""
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    enable_expert_parallel: bool = False
    scheduling_policy: str = "fcfs"
    block_size: Optional[int] = None
    cache_dtype: str = "auto"
    enforce_eager: bool = False
    speculative: bool = False
    num_scheduler_steps: int = 1
    cuda_graph_sizes: list[int] = field(default_factory=list)
    is_deepseek_mla: bool = False
    additional_config: dict = field(default_factory=dict)


@dataclass
class PolicyDecision:
    worker_cls: str = "auto"
    executor_cls: Optional[str] = None
    scheduler_cls: Optional[str] = None
    multiproc_method: str = "spawn"
    block_size: int = DEFAULT_BLOCK_SIZE
    disable_custom_all_reduce: bool = True      # replaced by the fused symmetric-memory paths
    cuda_graph_sizes: list[int] = field(default_factory=list)
    async_scheduling: bool = False
    async_executing: bool = False
    enable_eplb: bool = False
    num_redundant_experts: int = 0
    mla_fusion: bool = False
    dp_padding: bool = True
    notes: list[str] = field(default_factory=list)


def apply_platform_policy(p: PolicyInput) -> PolicyDecision:
    """Decisions of ``check_and_update_config`` (vllm_gcu/gcu.py:184-354), minus the parts
    that only existed to work around the GCU software stack."""
    d = PolicyDecision()
    ac = p.additional_config or {}
    d.block_size = p.block_size or DEFAULT_BLOCK_SIZE
    d.cuda_graph_sizes = sorted(set(p.cuda_graph_sizes))
    # DP + EP: every rank must enter the expert collectives each step, also with no work:
    # capture a graph for batch size 0 and do not pad token counts across DP ranks
    if p.data_parallel_size > 1 and not p.enforce_eager and 0 not in d.cuda_graph_sizes:
        d.cuda_graph_sizes = [0] + d.cuda_graph_sizes
    if p.enable_expert_parallel:
        d.dp_padding = False
    # priority scheduling under DP + EP keeps prefill and decode phases apart
    if (p.data_parallel_size > 1 and p.enable_expert_parallel
            and p.scheduling_policy == "priority"):
        d.scheduler_cls = "vllm_gcu_b200.engine.scheduler.Scheduler:priority"
    # expert load balancing
    d.enable_eplb = bool(ac.get("enable_eplb", False))
    d.num_redundant_experts = int(ac.get("num_redundant_experts", 0))
    if d.num_redundant_experts and not p.enable_expert_parallel:
        d.notes.append("num_redundant_experts ignored without expert parallelism")
        d.num_redundant_experts = 0
    d.mla_fusion = p.is_deepseek_mla
    # asynchronous scheduling / executing and their exclusions
    want_async = bool(ac.get("async_scheduling", False))
    want_exec = bool(ac.get("async_executing", False))
    if want_async or want_exec:
        if p.pipeline_parallel_size > 1:
            d.notes.append("async scheduling disabled: pipeline parallelism")
        elif p.num_scheduler_steps > 1:
            d.notes.append("async scheduling disabled: multi-step scheduling")
        else:
            d.async_scheduling = True
            d.async_executing = want_exec
            d.executor_cls = "vllm_gcu_b200.engine.executor.AsyncMultiprocExecutor" \
                if want_exec else None
            if p.speculative:
                d.notes.append("async scheduling with speculative decoding: draft tokens are "
                               "scheduled as placeholders")
    return d


def register() -> str:
    return "vllm_gcu_b200.platform.B200Platform"


_PLATFORM_CLS = None


def _make_platform_class():
    """Builds ``B200Platform`` on first use (importing vLLM is slow and optional).

    The class extends vLLM's CUDA platform, so upstream code that asks ``is_cuda()`` keeps
    working, and overrides what this package provides: the configuration policy, the list of
    quantisation names, the device communicator and the punica wrapper.  Attention backends
    (``get_attn_backend_cls`` returns ``runtime.vllm_attention.B200AttentionBackend`` for the
    configurations it covers), the worker class, the layer kernels (``runtime.vllm_ops``)."""
    global _PLATFORM_CLS
    if _PLATFORM_CLS is not None:
        return _PLATFORM_CLS
    from vllm.platforms.cuda import CudaPlatform

    class B200Platform(CudaPlatform):  # type: ignore[misc, valid-type]
        device_name: str = DEVICE_NAME
        supported_quantization: list[str] = sorted(
            set(getattr(CudaPlatform, "supported_quantization", [])) | set(SUPPORTED_QUANTIZATION))

        @classmethod
        def pre_register_and_update(cls, parser=None) -> None:
            import os
            os.environ.setdefault("VLLM_WORKER_MULTIPROC_METHOD", "spawn")

        @classmethod
        def import_kernels(cls) -> None:
            try:
                super().import_kernels()
            finally:
                from .ops import _native
                _native.lib()

        @classmethod
        def is_sleep_mode_available(cls) -> bool:
            return False

        @classmethod
        def use_custom_allreduce(cls) -> bool:
            return False

        @classmethod
        def get_device_communicator_cls(cls) -> str:
            return "vllm_gcu_b200.runtime.vllm_communicator.B200Communicator"

        @classmethod
        def get_punica_wrapper(cls) -> str:
            return "vllm_gcu_b200.runtime.vllm_punica.PunicaWrapperB200"

        # vLLM's NIXL connector asks the platform which KV buffer devices it can register.
        # The reference has to allocate its KV cache as host-accessible device memory for
        # this (vllm_gcu/worker/worker_v1.py:191-221); B200 device memory registers with
        # NIXL / UCX as it is (GPUDirect), so the stock allocation is kept.
        @classmethod
        def get_nixl_supported_devices(cls) -> dict:
            return {"cuda": ("cuda", "cpu")}

        @classmethod
        def get_nixl_memory_type(cls):
            return "VRAM"

        @classmethod
        def get_attn_backend_cls(cls, selected_backend, attn_selector_config, num_heads=None
                                 ) -> str:
            """This package's paged attention backend for what it covers (decoder attention,
            head size 64 / 128, 16-bit KV cache); everything else, and an explicitly selected
            upstream backend, goes to the CUDA platform's choice (vllm_gcu/gcu.py:70-104)."""
            import os
            from .runtime import vllm_attention as va
            explicit = selected_backend is not None and \
                getattr(selected_backend, "name", "") != "CUSTOM"
            if (not explicit and os.environ.get("VLLM_B200_ATTENTION", "1") != "0"
                    and va.accepts(attn_selector_config)):
                return va.BACKEND_PATH
            return super().get_attn_backend_cls(selected_backend, attn_selector_config, num_heads)

        @classmethod
        def verify_quantization(cls, quant: str) -> None:
            if quant not in cls.supported_quantization:
                raise ValueError(f"{quant} quantization is not supported on {DEVICE_NAME}")

        @classmethod
        def check_and_update_config(cls, vllm_config: Any) -> None:
            super().check_and_update_config(vllm_config)
            pc = vllm_config.parallel_config
            sc = vllm_config.scheduler_config
            cc = vllm_config.cache_config
            mc = vllm_config.model_config
            cg = getattr(vllm_config, "compilation_config", None)
            inp = PolicyInput(
                tensor_parallel_size=pc.tensor_parallel_size,
                pipeline_parallel_size=pc.pipeline_parallel_size,
                data_parallel_size=getattr(pc, "data_parallel_size", 1),
                enable_expert_parallel=getattr(pc, "enable_expert_parallel", False),
                scheduling_policy=getattr(sc, "policy", "fcfs"),
                block_size=getattr(cc, "block_size", None),
                cache_dtype=getattr(cc, "cache_dtype", "auto"),
                enforce_eager=bool(getattr(mc, "enforce_eager", False)) if mc else False,
                speculative=getattr(vllm_config, "speculative_config", None) is not None,
                cuda_graph_sizes=list(getattr(cg, "cudagraph_capture_sizes", None) or []),
                is_deepseek_mla=bool(getattr(mc, "use_mla", False)) if mc else False,
                additional_config=dict(getattr(vllm_config, "additional_config", None) or {}),
            )
            d = apply_platform_policy(inp)
            import os
            if pc.worker_cls in ("auto", "vllm.v1.worker.gpu_worker.Worker"):
                pc.worker_cls = "vllm_gcu_b200.runtime.vllm_worker.B200Worker"
            if os.environ.get("VLLM_B200_VLLM_NATIVE_OPS", "1") != "0" and cg is not None:
                # the layer kernels of this package are eager launches: no tracing compiler in
                # front of them (CUDA graphs of decode batches stay available)
                try:
                    from vllm.config.compilation import CompilationMode
                    cg.mode = CompilationMode.NONE
                except Exception:  # noqa: BLE001
                    pass
            if cc is not None and getattr(cc, "block_size", None) is None:
                cc.block_size = d.block_size
            if hasattr(pc, "disable_custom_all_reduce"):
                pc.disable_custom_all_reduce = d.disable_custom_all_reduce
            if d.async_scheduling and hasattr(sc, "async_scheduling"):
                sc.async_scheduling = True
            if cg is not None and d.cuda_graph_sizes and hasattr(cg, "cudagraph_capture_sizes") \
                    and 0 in d.cuda_graph_sizes:
                cg.cudagraph_capture_sizes = d.cuda_graph_sizes

    _PLATFORM_CLS = B200Platform
    return B200Platform


def __getattr__(name: str):
    if name == "B200Platform":
        return _make_platform_class()
    raise AttributeError(name)
