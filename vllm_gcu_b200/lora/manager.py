"""Adapter manager: loads PEFT-format LoRA checkpoints into stacked per-layer slots and
attaches LoRA to the linear layers of a model."""
from __future__ import annotations

import json
import re
from collections import OrderedDict
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

import torch
import torch.nn as nn

from ..layers.linear import (LinearBase, MergedColumnParallelLinear, QKVParallelLinear,
                             RowParallelLinear)
from ..parallel.state import tp_rank, tp_size
from .punica import PunicaWrapperB200


@dataclass
class LoRARequest:
    lora_name: str
    lora_int_id: int
    lora_path: str


_TARGETS = {"q_proj": ("qkv_proj", 0), "k_proj": ("qkv_proj", 1), "v_proj": ("qkv_proj", 2),
            "o_proj": ("o_proj", 0), "gate_proj": ("gate_up_proj", 0),
            "up_proj": ("gate_up_proj", 1), "down_proj": ("down_proj", 0)}


class LoRALinear(nn.Module):
    """Wraps a linear layer: ``y = base(x) + B[idx] (scale * A[idx] x)`` per output slice."""

    def __init__(self, base: LinearBase, max_loras: int, max_rank: int, punica: PunicaWrapperB200):
        super().__init__()
        self.base = base
        self.punica = punica
        dev, dt = base.weight.device if hasattr(base, "weight") else base.device, base.dtype
        if isinstance(base, QKVParallelLinear):
            self.slices = [base.q_size, base.kv_size, base.kv_size]
        elif isinstance(base, MergedColumnParallelLinear):
            tp = tp_size()
            self.slices = [s // tp for s in base.output_sizes]
        else:
            self.slices = [base.out_per_rank]
        self.lora_a = nn.ParameterList([nn.Parameter(torch.zeros(
            max_loras, max_rank, base.in_per_rank, dtype=dt, device=dev), requires_grad=False)
            for _ in self.slices])
        self.lora_b = nn.ParameterList([nn.Parameter(torch.zeros(
            max_loras, n, max_rank, dtype=dt, device=dev), requires_grad=False)
            for n in self.slices])
        self.scaling = torch.ones(max_loras)
        for attr in ("fuse_silu", "_interleaved", "num_heads", "num_kv_heads", "head_dim",
                     "q_size", "kv_size", "output_sizes"):
            if hasattr(base, attr):
                object.__setattr__(self, attr, getattr(base, attr))

    def set_lora(self, slot: int, sub: int, a: torch.Tensor, b: torch.Tensor, scaling: float
                 ) -> None:
        """a ``[r, in_full]``, b ``[out_full, r]`` (full, unsharded adapter tensors)."""
        base = self.base
        r = a.shape[0]
        tp, rk = tp_size(), tp_rank()
        if isinstance(base, RowParallelLinear):
            n = base.in_per_rank
            a = a[:, rk * n:(rk + 1) * n]
        else:
            n = self.slices[sub]
            if isinstance(base, QKVParallelLinear) and sub > 0:
                kv_rank = rk // base.kv_replicas
                b = b[kv_rank * n:(kv_rank + 1) * n]
            elif tp > 1:
                b = b[rk * n:(rk + 1) * n]
        self.lora_a[sub].data[slot].zero_()
        self.lora_b[sub].data[slot].zero_()
        self.lora_a[sub].data[slot, :r].copy_(a)
        # fold the adapter scaling into B so one scale serves the whole batch
        self.lora_b[sub].data[slot, :, :r].copy_(b * scaling)

    def clear_lora(self, slot: int) -> None:
        for p in list(self.lora_a) + list(self.lora_b):
            p.data[slot].zero_()

    def forward(self, x: torch.Tensor, **kw) -> torch.Tensor:
        base = self.base
        if self.punica.no_lora:
            return base(x, **kw)
        fused_silu = getattr(base, "fuse_silu", False)
        if fused_silu:
            # the LoRA delta must be added before the activation: run the plain GEMM
            from ..layers.activation import act_and_mul
            w = base.weight
            if getattr(base, "_interleaved", False):
                from ..ops import ref as _ref
                w = _ref.deinterleave_gate_up(w)
            y = torch.nn.functional.linear(x, w, base.bias)
            self.punica.add_lora_linear(y, x, list(self.lora_a), list(self.lora_b), 1.0,
                                        self.slices)
            return act_and_mul(y, "silu")
        if isinstance(base, RowParallelLinear) and tp_size() > 1:
            # the delta is a partial sum over the sharded input like the base output
            y = base.quant_method.apply(base, x, skip_bias=True)
            self.punica.add_lora_linear(y, x, list(self.lora_a), list(self.lora_b), 1.0,
                                        self.slices)
            from ..parallel.communicator import get_comm
            y = get_comm("tp").all_reduce(y)
            return y if base.bias is None else y + base.bias
        y = base(x, **kw)
        if not y.is_contiguous():
            y = y.contiguous()
        self.punica.add_lora_linear(y, x, list(self.lora_a), list(self.lora_b), 1.0, self.slices)
        return y

    # weight loading of the base layer passes through
    def load_weight(self, name, full, shard_id=None):
        self.base.load_weight(name, full, shard_id)

    def finalize(self):
        self.base.finalize()

    @property
    def weight(self):
        return self.base.weight


class LoRAManager:
    def __init__(self, model: nn.Module, max_loras: int, max_rank: int, max_tokens: int,
                 max_seqs: int, device):
        self.model = model
        self.max_loras, self.max_rank = max_loras, max_rank
        self.punica = PunicaWrapperB200(max_tokens, max_seqs, device)
        self.slots: "OrderedDict[int, int]" = OrderedDict()      # lora_int_id -> slot (LRU)
        self.layers: dict[str, LoRALinear] = {}
        self._wrap(model)

    def _wrap(self, module: nn.Module, prefix: str = "") -> None:
        for name, child in list(module.named_children()):
            path = f"{prefix}.{name}" if prefix else name
            if isinstance(child, LinearBase) and name in ("qkv_proj", "o_proj", "gate_up_proj",
                                                          "down_proj"):
                wrapped = LoRALinear(child, self.max_loras, self.max_rank, self.punica)
                setattr(module, name, wrapped)
                self.layers[path] = wrapped
            else:
                self._wrap(child, path)

    # -- adapters --------------------------------------------------------------------
    def slot_of(self, lora_int_id: int) -> int:
        if lora_int_id in self.slots:
            self.slots.move_to_end(lora_int_id)
            return self.slots[lora_int_id]
        return -1

    def add_adapter(self, req: LoRARequest, tensors: Optional[dict] = None,
                    config: Optional[dict] = None) -> int:
        """Loads an adapter (PEFT layout: ``adapter_config.json`` +
        ``adapter_model.safetensors``) into a free slot, evicting the least recently used."""
        if req.lora_int_id in self.slots:
            return self.slot_of(req.lora_int_id)
        if len(self.slots) >= self.max_loras:
            _, slot = self.slots.popitem(last=False)
            for l in self.layers.values():
                l.clear_lora(slot)
        else:
            used = set(self.slots.values())
            slot = next(i for i in range(self.max_loras) if i not in used)
        if tensors is None:
            from ..utils.weights import read_safetensors
            p = Path(req.lora_path)
            config = json.loads((p / "adapter_config.json").read_text())
            tensors = dict(read_safetensors(str(p / "adapter_model.safetensors")))
        config = config or {}
        r = int(config.get("r", 8))
        alpha = float(config.get("lora_alpha", r))
        scaling = alpha / r
        if r > self.max_rank:
            raise ValueError(f"adapter rank {r} exceeds max_lora_rank {self.max_rank}")
        pat = re.compile(r"layers\.(\d+)\.(self_attn|mlp)\.(\w+)\.lora_A(?:\.\w+)?\.weight$")
        for name, a in tensors.items():
            m = pat.search(name)
            if m is None:
                continue
            b = tensors[name.replace("lora_A", "lora_B")]
            tgt = _TARGETS.get(m.group(3))
            if tgt is None:
                continue
            path = f"layers.{m.group(1)}.{m.group(2)}.{tgt[0]}"
            layer = self.layers.get(path)
            if layer is not None:
                dt = layer.lora_a[0].dtype
                layer.set_lora(slot, tgt[1], a.to(dt), b.to(dt), scaling)
        self.slots[req.lora_int_id] = slot
        return slot

    def remove_adapter(self, lora_int_id: int) -> None:
        slot = self.slots.pop(lora_int_id, None)
        if slot is not None:
            for l in self.layers.values():
                l.clear_lora(slot)

    def set_batch(self, token_lora_ids: list[int], sampler_lora_ids: Optional[list[int]] = None
                  ) -> None:
        """Per-token adapter ids (``lora_int_id`` or -1) of the step that is about to run."""
        tok = [self.slot_of(i) if i >= 0 else -1 for i in token_lora_ids]
        smp = None if sampler_lora_ids is None else \
            [self.slot_of(i) if i >= 0 else -1 for i in sampler_lora_ids]
        self.punica.update_metadata(tok, smp)
