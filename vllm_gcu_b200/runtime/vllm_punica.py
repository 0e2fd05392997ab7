"""``PunicaWrapperBase`` subclass for vLLM's multi-LoRA layers on this package's ``b200_bgmv``
kernel (the reference's ``PunicaWrapperGCU``, vllm_gcu/lora/punica_gcu.py:22-366, returned by
``Platform.get_punica_wrapper``, vllm_gcu/gcu.py:384-389).  Shrink / expand are evaluated per
token with the adapter index of every token (``token_lora_indices``), for prefill and decode
alike."""
from __future__ import annotations

import torch

from vllm.lora.punica_wrapper.punica_base import PunicaWrapperBase

from ..lora import ops as L


class PunicaWrapperB200(PunicaWrapperBase):
    def __init__(self, max_num_batched_tokens: int, max_batches: int, device, **kwargs):
        super().__init__(max_num_batched_tokens, max_batches, device)

    def add_shrink(self, y, x, lora_a_stacked, scale: float, **kwargs):
        """``y[i] += scale * A_i[idx] @ x`` for every slice i."""
        x2 = x.reshape(-1, x.shape[-1])
        idx = self.token_lora_indices
        for i, a in enumerate(lora_a_stacked):
            yi = y[i]
            tmp = torch.zeros_like(yi)
            L.bgmv_shrink(x2, a, tmp, idx, scale)
            yi += tmp

    def add_expand(self, y, x, lora_b_stacked, output_slices, offset_start: int = 0,
                   add_inputs: bool = True, **kwargs):
        y2 = y.reshape(-1, y.shape[-1])
        idx = self.token_lora_indices
        off = offset_start
        for i, (b, n) in enumerate(zip(lora_b_stacked, output_slices)):
            L.bgmv_expand_slice(x[i], b, y2, idx, off, n, add_inputs)
            off += n

    def add_lora_embedding(self, y, x, lora_b_stacked, add_inputs: bool = True, **kwargs):
        L.bgmv_expand(x, lora_b_stacked, y, self.token_lora_indices, add_inputs)

    def add_lora_linear(self, y, x, lora_a_stacked, lora_b_stacked, scale: float, output_slices,
                        *, buffer=None, **kwargs):
        """``y[:, slice_i] += B_i[idx] @ (scale * A_i[idx] @ x)``."""
        x2 = x.reshape(-1, x.shape[-1])
        T = x2.shape[0]
        bufs = []
        for a in lora_a_stacked:
            r = (a[:, 0] if a.dim() == 4 else a).shape[1]
            bufs.append(torch.zeros((T, r), dtype=torch.float32, device=x.device))
        idx = self.token_lora_indices
        for buf, a in zip(bufs, lora_a_stacked):
            L.bgmv_shrink(x2, a, buf, idx, scale)
        self.add_expand(y, [b.to(x.dtype) for b in bufs], lora_b_stacked, output_slices,
                        add_inputs=True)

    def add_lora_logits(self, y, x, lora_a_stacked, lora_b_stacked, scale, *, buffer=None,
                        **kwargs):
        y2 = y.reshape(-1, y.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        idx = self.sampler_indices
        r = (lora_a_stacked[:, 0] if lora_a_stacked.dim() == 4 else lora_a_stacked).shape[1]
        buf = torch.zeros((x2.shape[0], r), dtype=torch.float32, device=x.device)
        L.bgmv_shrink(x2, lora_a_stacked, buf, idx, scale)
        L.bgmv_expand(buf.to(x.dtype), lora_b_stacked, y2, idx, True)
