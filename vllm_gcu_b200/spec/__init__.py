"""Speculative decoding: proposers (n-gram prompt lookup, DeepSeek MTP, EAGLE head, Medusa
heads, MLP speculator) and the rejection sampler that verifies their drafts.

The reference wires vLLM's spec-decode worker with n-gram / MLPSpeculator / Medusa /
multi-step proposers and MTP (vllm_gcu/worker/spec_decode/spec_decode_worker.py:41-212) and
replaces the v1 rejection-sampler kernels with native ops
(vllm_gcu/patch/patch_0_9_2/rejection_sampler.py:174-466).  Here the proposer runs inside the
model runner right after the target step and the verification is one kernel per step.
"""
from .eagle import EagleDrafter  # noqa: F401
from .heads import MedusaProposer, MLPSpeculatorProposer  # noqa: F401
from .ngram import NgramProposer  # noqa: F401
from .rejection import RejectionSampler, SpecMetrics  # noqa: F401
