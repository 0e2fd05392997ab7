"""Rejection sampler: verifies draft tokens against the target model's distribution.

GPU: one native kernel per step (``csrc/spec.cu``); elsewhere the torch oracle of
``ops.ref``.  With ``REJECT_SAMPLER_CHECK`` set, the GPU result is cross-checked against the
oracle at run time, as the reference does with ``VLLM_GCU_REJECT_SAMPLER_CHECK``
(vllm_gcu/patch/patch_0_9_2/rejection_sampler.py:214-226).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import envs, ops
from ..ops import ref
from ..ops._native import call, ptr, stream_ptr


@dataclass
class SpecMetrics:
    """Running acceptance statistics (vllm_gcu/worker/spec_decode/metrics.py:8-62)."""
    num_drafts: int = 0
    num_draft_tokens: int = 0
    num_accepted_tokens: int = 0
    num_emitted_tokens: int = 0

    def update(self, num_draft: int, num_emitted: int) -> None:
        self.num_drafts += 1
        self.num_draft_tokens += num_draft
        self.num_accepted_tokens += max(0, min(num_draft, num_emitted - 1))
        self.num_emitted_tokens += num_emitted

    @property
    def acceptance_rate(self) -> float:
        return self.num_accepted_tokens / max(1, self.num_draft_tokens)

    @property
    def mean_acceptance_length(self) -> float:
        return self.num_emitted_tokens / max(1, self.num_drafts)


class RejectionSampler:
    def greedy(self, draft_ids: torch.Tensor, target_argmax: torch.Tensor,
               num_draft: torch.Tensor) -> torch.Tensor:
        """draft_ids int32 ``[B, S]``, target_argmax int64 ``[B, S + 1]`` (the last valid column
        of each row is the bonus position), num_draft int32 ``[B]`` -> int32 ``[B, S + 1]``."""
        B, S = draft_ids.shape
        if ops.use_native(draft_ids):
            out = torch.empty((B, S + 1), dtype=torch.int32, device=draft_ids.device)
            call("b200_rejection_greedy", ptr(out), ptr(draft_ids.contiguous()),
                 ptr(target_argmax.contiguous()), None, ptr(num_draft), B, S, stream_ptr())
            if envs.REJECT_SAMPLER_CHECK:
                want = self._greedy_ref(draft_ids, target_argmax, num_draft)
                assert torch.equal(out.cpu(), want.cpu()), "rejection_greedy mismatch"
            return out
        return self._greedy_ref(draft_ids, target_argmax, num_draft)

    @staticmethod
    def _greedy_ref(draft_ids, target_argmax, num_draft):
        B, S = draft_ids.shape
        idx = num_draft.long().clamp(max=S)
        bonus = target_argmax.gather(1, idx[:, None]).squeeze(1)
        return ref.rejection_greedy_sample(draft_ids, target_argmax[:, :S], bonus, num_draft)

    def random(self, draft_ids: torch.Tensor, draft_probs: Optional[torch.Tensor],
               target_probs: torch.Tensor, bonus_ids: torch.Tensor, num_draft: torch.Tensor,
               generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """target_probs ``[B, S, V]`` fp32; returns int32 ``[B, S + 1]``."""
        B, S = draft_ids.shape
        V = target_probs.shape[-1]
        dev = draft_ids.device
        uniform = torch.rand((B, S), device=dev, generator=generator)
        noise = torch.empty((B, S, V), device=dev).exponential_(generator=generator)
        if ops.use_native(draft_ids):
            recovered = torch.empty((B, S), dtype=torch.int32, device=dev)
            call("b200_sample_recovered_tokens", ptr(recovered), ptr(draft_ids.contiguous()),
                 ptr(draft_probs.contiguous() if draft_probs is not None else None),
                 ptr(target_probs.contiguous()), ptr(noise), B, S, V, stream_ptr())
            if envs.REJECT_SAMPLER_CHECK:
                want = ref.sample_recovered_tokens(draft_ids, draft_probs, target_probs, noise)
                assert torch.equal(recovered.cpu(), want.cpu()), "recovered tokens mismatch"
        else:
            recovered = ref.sample_recovered_tokens(draft_ids, draft_probs, target_probs, noise)
        if ops.use_native(draft_ids):
            out = torch.empty((B, S + 1), dtype=torch.int32, device=dev)
            call("b200_rejection_random", ptr(out), ptr(draft_ids.contiguous()),
                 ptr(draft_probs.contiguous() if draft_probs is not None else None),
                 ptr(target_probs.contiguous()), ptr(bonus_ids.contiguous()),
                 ptr(recovered.contiguous()), ptr(uniform), ptr(num_draft), B, S, V, stream_ptr())
            if envs.REJECT_SAMPLER_CHECK:
                want = ref.rejection_random_sample(draft_ids, draft_probs, target_probs, bonus_ids,
                                                   recovered, uniform, num_draft)
                assert torch.equal(out.cpu(), want.cpu()), "rejection_random mismatch"
            return out
        return ref.rejection_random_sample(draft_ids, draft_probs, target_probs, bonus_ids,
                                           recovered, uniform, num_draft)
