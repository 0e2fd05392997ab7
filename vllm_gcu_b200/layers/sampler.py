"""Token sampler: penalties, temperature, top-k / top-p, Gumbel-max, log-probabilities.

GPU path: one fused kernel per step (``ops.cuda.sample``), radix selection instead of a
vocabulary sort.  The reference's samplers are ``GCUTopKTopPSampler`` (fused mask +
exponential-noise sampling, vllm_gcu/kernels/sampler.py:102-129), tensorised penalties
(:74-100) and ``DPParallelSampler`` (each TP rank samples a slice of the batch and the ids
are all-gathered, :13-71), implemented here by ``Sampler`` / ``apply_penalties`` /
``RowParallelSampler``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import cuda as C
from ..ops import ref
from ..parallel.communicator import get_comm, scatter_sizes


@dataclass
class SamplingTensors:
    temperature: torch.Tensor            # [B] fp32, <= 0 means greedy
    top_k: Optional[torch.Tensor]        # [B] int32, <= 0 means off
    top_p: Optional[torch.Tensor]        # [B] fp32, >= 1 means off
    seeds: Optional[torch.Tensor]        # [B] int64


def apply_penalties(logits: torch.Tensor, prompt_mask: torch.Tensor, output_counts: torch.Tensor,
                    presence: torch.Tensor, frequency: torch.Tensor, repetition: torch.Tensor
                    ) -> torch.Tensor:
    """In-place penalties.  ``prompt_mask`` bool ``[B, V]`` marks prompt tokens,
    ``output_counts`` int ``[B, V]`` counts generated tokens."""
    seen = prompt_mask | (output_counts > 0)
    rep = torch.where(seen, repetition[:, None], torch.ones_like(logits, dtype=repetition.dtype))
    lg = logits.float()
    lg = torch.where(lg > 0, lg / rep, lg * rep)
    lg = lg - frequency[:, None] * output_counts.float()
    lg = lg - presence[:, None] * (output_counts > 0).float()
    logits.copy_(lg.to(logits.dtype))
    return logits


class Sampler(nn.Module):
    def __init__(self, vocab_size: int):
        super().__init__()
        self.vocab_size = vocab_size

    def forward(self, logits: torch.Tensor, st: Optional[SamplingTensors],
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Returns int64 token ids ``[B]`` (written into ``out`` when given)."""
        from .. import envs
        if envs.SAMPLER_ON_CPU and logits.is_cuda:
            # debugging aid: the torch reference on the host (VLLM_GCU_SAMPLER_ON_CPU)
            cpu_st = None
            if st is not None:
                cpu_st = SamplingTensors(st.temperature.cpu(),
                                         None if st.top_k is None else st.top_k.cpu(),
                                         None if st.top_p is None else st.top_p.cpu(),
                                         None if st.seeds is None else st.seeds.cpu())
            ids = self.forward(logits.float().cpu(), cpu_st).to(logits.device)
            if out is not None:
                out.copy_(ids)
                return out
            return ids
        if ops.use_native(logits):
            if not logits.is_contiguous():
                logits = logits.contiguous()
            if st is None:
                return C.sample(logits, out=out)
            return C.sample(logits, st.temperature, st.top_k, st.top_p, seeds=st.seeds, out=out)
        if st is None:
            ids = logits.float().argmax(-1)
        else:
            noise = None
            if st.seeds is not None and st.seeds.numel() > 0:
                # one generator per row, as in the kernel: a request's draw depends on its own
                # seed only, not on which other requests share the step
                noise = torch.empty(logits.shape, dtype=torch.float32, device=logits.device)
                g = torch.Generator(device=logits.device)
                for r, sd in enumerate(st.seeds.tolist()):
                    g.manual_seed(int(sd) & 0x7FFFFFFFFFFFFFFF)
                    noise[r].exponential_(generator=g)
            ids = ref.sample(logits, st.temperature, st.top_k, st.top_p, noise=noise)
        if out is not None:
            out.copy_(ids)
            return out
        return ids

    @staticmethod
    def logprobs(logits: torch.Tensor, token_ids: torch.Tensor, k: int
                 ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(logprob of the sampled token [B], top-k logprobs [B, k], top-k ids [B, k])."""
        lp = torch.log_softmax(logits.float(), dim=-1)
        chosen = lp.gather(-1, token_ids[:, None]).squeeze(-1)
        if k > 0:
            tv, ti = lp.topk(k, dim=-1)
        else:
            tv = lp.new_zeros((lp.shape[0], 0))
            ti = token_ids.new_zeros((lp.shape[0], 0))
        return chosen, tv, ti


class RowParallelSampler(Sampler):
    """Splits the batch rows over the TP ranks, samples locally and all-gathers the ids,
    so the full-vocabulary passes run on B/tp rows per rank."""

    def forward(self, logits, st, out=None):
        comm = get_comm("tp")
        tp, r = comm.world_size, comm.rank
        B = logits.shape[0]
        if tp == 1 or B < tp:
            return super().forward(logits, st, out)
        sizes = scatter_sizes(B, tp)
        lo = sum(sizes[:r])
        hi = lo + sizes[r]
        sub = None
        if st is not None:
            sub = SamplingTensors(st.temperature[lo:hi],
                                  None if st.top_k is None else st.top_k[lo:hi],
                                  None if st.top_p is None else st.top_p[lo:hi],
                                  None if st.seeds is None else st.seeds[lo:hi])
        ids = super().forward(logits[lo:hi], sub)
        full = comm.all_gather_v(ids, sizes)
        if out is not None:
            out.copy_(full)
            return out
        return full
