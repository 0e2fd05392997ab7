"""Device communicator for vLLM's tensor-parallel groups on B200.

``Platform.get_device_communicator_cls`` points here.  All-reduce goes through the
symmetric-memory kernel of this package when the message fits its workspace and falls back
to vLLM's CUDA communicator (NCCL) otherwise; the variable-size collectives used by
sequence parallelism are added on top (role of ``GCUCommunicator``,
vllm_gcu/distributed/gcu_communicator.py:40-126).  Defined lazily because it subclasses a
vLLM class.
"""
from __future__ import annotations

from typing import Optional

import torch


def _base():
    from vllm.distributed.device_communicators.cuda_communicator import CudaCommunicator
    return CudaCommunicator


def __getattr__(name: str):
    if name != "B200Communicator":
        raise AttributeError(name)
    Base = _base()

    class B200Communicator(Base):  # type: ignore[misc, valid-type]
        def __init__(self, *args, **kwargs):
            super().__init__(*args, **kwargs)
            self._fused = None
            self._fused_tried = False

        def _get_fused(self, x: torch.Tensor):
            if self._fused_tried:
                return self._fused
            self._fused_tried = True
            try:
                from ..parallel.symm import SymmetricBuffer  # noqa: F401
                from ..parallel.vllm_bridge import fused_for_group
                self._fused = fused_for_group(self.device_group, x.device)
            except Exception:
                self._fused = None
            return self._fused

        def all_reduce(self, input_: torch.Tensor) -> torch.Tensor:
            if self.world_size > 1 and input_.dtype == torch.bfloat16 and input_.is_contiguous():
                fused = self._get_fused(input_)
                if fused is not None:
                    out = fused.all_reduce(input_)
                    if out is not None:
                        return out.clone()
            return super().all_reduce(input_)

        def all_gather_v(self, x: torch.Tensor, sizes: Optional[list[int]] = None) -> torch.Tensor:
            import torch.distributed as dist
            if self.world_size == 1:
                return x
            if sizes is None:
                sizes = [x.shape[0]] * self.world_size
            outs = [torch.empty((s,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
                    for s in sizes]
            dist.all_gather(outs, x.contiguous(), group=self.device_group)
            return torch.cat(outs, dim=0)

        def reduce_scatter_v(self, x: torch.Tensor, sizes: list[int]) -> torch.Tensor:
            import torch.distributed as dist
            if self.world_size == 1:
                return x
            chunks = list(torch.split(x.contiguous(), sizes, dim=0))
            out = torch.empty_like(chunks[self.rank_in_group])
            dist.reduce_scatter(out, chunks, group=self.device_group)
            return out

    globals()["B200Communicator"] = B200Communicator
    return B200Communicator
