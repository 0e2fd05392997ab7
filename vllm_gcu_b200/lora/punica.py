"""Punica-style wrapper: maps the tokens of a batch to adapter slots and applies LoRA to
linear, embedding and logits layers (``PunicaWrapperGCU``,
vllm_gcu/lora/punica_gcu.py:22-366)."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import ops as L


class PunicaWrapperB200:
    def __init__(self, max_num_batched_tokens: int, max_batches: int, device, **kwargs):
        self.device = torch.device(device)
        self.max_tokens = max_num_batched_tokens
        self.token_lora_indices = torch.full((max_num_batched_tokens,), -1, dtype=torch.int32,
                                             device=self.device)
        self.sampler_indices = torch.full((max_batches,), -1, dtype=torch.int32,
                                          device=self.device)
        self.num_tokens = 0
        self.num_samples = 0
        self.no_lora = True

    # -- metadata ------------------------------------------------------------------
    def update_metadata(self, token_lora_ids: Sequence[int],
                        sampler_lora_ids: Optional[Sequence[int]] = None) -> None:
        """``token_lora_ids[t]`` is the adapter slot of token t (-1: no adapter)."""
        n = len(token_lora_ids)
        self.num_tokens = n
        self.no_lora = all(i < 0 for i in token_lora_ids)
        if n:
            self.token_lora_indices[:n].copy_(
                torch.as_tensor(list(token_lora_ids), dtype=torch.int32), non_blocking=True)
        if sampler_lora_ids is not None:
            m = len(sampler_lora_ids)
            self.num_samples = m
            if m:
                self.sampler_indices[:m].copy_(
                    torch.as_tensor(list(sampler_lora_ids), dtype=torch.int32), non_blocking=True)

    @property
    def token_indices(self) -> torch.Tensor:
        return self.token_lora_indices[: self.num_tokens]

    # -- linear layers ----------------------------------------------------------------
    def add_shrink(self, y: Sequence[torch.Tensor], x: torch.Tensor,
                   lora_a_stacked: Sequence[torch.Tensor], scale: float) -> None:
        """``y[i] = scale * A_i[idx] @ x`` for every slice i (q/k/v or gate/up)."""
        x2 = x.reshape(-1, x.shape[-1])
        for yi, a in zip(y, lora_a_stacked):
            L.bgmv_shrink(x2, a, yi, self.token_indices, scale)

    def add_expand(self, y: torch.Tensor, x: Sequence[torch.Tensor],
                   lora_b_stacked: Sequence[torch.Tensor], output_slices: Sequence[int],
                   offset_start: int = 0, add_inputs: bool = True) -> None:
        y2 = y.reshape(-1, y.shape[-1])
        off = offset_start
        for xi, b, n in zip(x, lora_b_stacked, output_slices):
            L.bgmv_expand_slice(xi, b, y2, self.token_indices, off, n, add_inputs)
            off += n

    def add_lora_linear(self, y: torch.Tensor, x: torch.Tensor,
                        lora_a_stacked: Sequence[torch.Tensor],
                        lora_b_stacked: Sequence[torch.Tensor], scale: float,
                        output_slices: Sequence[int]) -> torch.Tensor:
        """``y[:, slice_i] += B_i[idx] @ (scale * A_i[idx] @ x)``."""
        if self.no_lora:
            return y
        T = x.reshape(-1, x.shape[-1]).shape[0]
        bufs = []
        for a in lora_a_stacked:
            r = (a[:, 0] if a.dim() == 4 else a).shape[1]
            bufs.append(torch.zeros((T, r), dtype=torch.float32 if x.is_cuda else x.dtype,
                                    device=x.device))
        self.add_shrink(bufs, x, lora_a_stacked, scale)
        bufs = [b.to(x.dtype) for b in bufs]
        self.add_expand(y, bufs, lora_b_stacked, output_slices)
        return y

    def add_lora_embedding(self, y: torch.Tensor, x: torch.Tensor, lora_b_stacked: torch.Tensor,
                           add_inputs: bool = True) -> torch.Tensor:
        """``x`` already holds the gathered rows of the embedding-LoRA A matrix."""
        if self.no_lora:
            return y
        L.bgmv_expand(x, lora_b_stacked, y, self.token_indices, add_inputs)
        return y

    def add_lora_logits(self, y: torch.Tensor, x: torch.Tensor, lora_a_stacked: torch.Tensor,
                        lora_b_stacked: torch.Tensor, scale: float) -> torch.Tensor:
        if self.no_lora:
            return y
        idx = self.sampler_indices[: self.num_samples]
        r = (lora_a_stacked[:, 0] if lora_a_stacked.dim() == 4 else lora_a_stacked).shape[1]
        buf = torch.zeros((x.shape[0], r), dtype=torch.float32 if x.is_cuda else x.dtype,
                          device=x.device)
        L.bgmv_shrink(x, lora_a_stacked, buf, idx, scale)
        L.bgmv_expand(buf.to(x.dtype), lora_b_stacked, y, idx, True)
        return y
