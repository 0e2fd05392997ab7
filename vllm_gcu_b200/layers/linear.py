"""Linear layers with tensor-parallel sharding and pluggable quantisation.

Weights keep the ``[out_features, in_features]`` checkpoint layout, which is the
K-major "B" operand of the tcgen05 GEMM, so loading is a slice-and-copy.

Parallel flavours (names follow the checkpoint conventions the reference loads,
vllm_gcu/models/deepseek_v3/deepseek_v3.py:1037-1173):

* ``ColumnParallelLinear``        – output sharded over TP
* ``MergedColumnParallelLinear``  – several column-parallel matrices stacked
  (``gate_up_proj``); with ``fuse_silu`` the gate/up rows are interleaved in blocks
  of 128 at load time and SiLU(gate)*up runs in the GEMM epilogue
* ``QKVParallelLinear``           – fused q/k/v with GQA-aware sharding
* ``RowParallelLinear``           – input sharded, output all-reduced (or left partial /
  reduce-scattered for sequence parallelism)
* ``ReplicatedLinear`` / ``MergedReplicatedLinear`` – unsharded (router gate, MLA
  ``q_a_proj`` + ``kv_a_proj_with_mqa`` fused as in vllm_gcu/kernels/linear.py:21-149)
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import cuda as C
from ..ops import ref
from ..parallel.communicator import get_comm
from ..parallel.state import tp_rank, tp_size


class LinearMethod:
    """Strategy object: creates the parameters of a layer and applies it."""

    def create_weights(self, layer: "LinearBase") -> None:
        raise NotImplementedError

    def apply(self, layer: "LinearBase", x: torch.Tensor, **kw) -> torch.Tensor:
        raise NotImplementedError

    def process_weights_after_loading(self, layer: "LinearBase") -> None:
        pass

    def input_quant(self, layer: "LinearBase"):
        """``(mode, static scale or None)`` when ``apply`` quantises its input and also accepts
        it already quantised (``x`` 8-bit plus ``x_scale=``), so that the producing norm /
        activation kernel can emit the quantised rows itself; None otherwise."""
        return None


class UnquantizedLinearMethod(LinearMethod):
    def create_weights(self, layer: "LinearBase") -> None:
        layer.weight = nn.Parameter(torch.empty(layer.out_per_rank, layer.in_per_rank,
                                                dtype=layer.dtype, device=layer.device),
                                    requires_grad=False)

    def process_weights_after_loading(self, layer: "LinearBase") -> None:
        if getattr(layer, "fuse_silu", False) and not getattr(layer, "_interleaved", False):
            w = layer.weight.data
            half = w.shape[0] // 2
            if half % ref.GATE_UP_BLOCK == 0 and w.dtype == torch.bfloat16:
                layer.weight.data = ref.interleave_gate_up(w[:half], w[half:]).contiguous()
                layer._interleaved = True

    def apply(self, layer: "LinearBase", x: torch.Tensor, residual=None, skip_bias=False,
              **kw) -> torch.Tensor:
        w = layer.weight
        bias = None if skip_bias else layer.bias
        if ops.use_native(x) and x.dtype == torch.bfloat16:
            shape = x.shape
            x2 = x.reshape(-1, shape[-1])
            if getattr(layer, "_interleaved", False):
                y = C.gemm_bf16(x2, w, epilogue=C.EPI_SILU_MUL)
            else:
                if bias is not None and residual is not None:
                    y = C.gemm_bf16(x2, w, bias=bias)
                    y += residual
                else:
                    y = C.gemm_bf16(x2, w, bias=bias, residual=residual)
                if getattr(layer, "fuse_silu", False):
                    y = C.activation(y, "silu")
            return y.view(*shape[:-1], y.shape[-1])
        y = F.linear(x, w, bias)
        if residual is not None:
            y = y + residual
        if getattr(layer, "fuse_silu", False):
            y = ref.silu_and_mul(y)
        return y


class LinearBase(nn.Module):
    def __init__(self, in_features: int, out_features: int, in_per_rank: int, out_per_rank: int,
                 bias: bool, dtype: torch.dtype, device, quant_method: Optional[LinearMethod],
                 prefix: str = ""):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.in_per_rank, self.out_per_rank = in_per_rank, out_per_rank
        self.dtype, self.device, self.prefix = dtype, device, prefix
        self.quant_method = quant_method or UnquantizedLinearMethod()
        self.quant_method.create_weights(self)
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_per_rank, dtype=dtype, device=device),
                                     requires_grad=False)
        else:
            self.bias = None

    def forward(self, x: torch.Tensor, **kw) -> torch.Tensor:
        return self.quant_method.apply(self, x, **kw)

    # -- loading -----------------------------------------------------------
    def shard_spec(self, shard_id=None):
        """Which part of a full (unsharded) checkpoint tensor belongs to this rank:
        ``(out_segments, in_range)`` in feature units.  ``out_segments`` is a list of
        ``(src_offset, size, dst_offset)`` along the output dimension (None = everything),
        ``in_range`` is ``(src_offset, size)`` along the input dimension (None = everything)."""
        return None, None

    def copy_sharded(self, dst: torch.Tensor, full: torch.Tensor, shard_id, out_dim: int,
                     in_dim: int, out_pack: int = 1, in_pack: int = 1) -> None:
        """Copies this rank's part of ``full`` into ``dst``.  ``out_dim`` / ``in_dim`` name the
        tensor dimensions that run along output / input features (-1: absent) and
        ``*_pack`` how many features one element of that dimension holds."""
        segs, rng = self.shard_spec(shard_id)
        src = full
        if rng is not None and in_dim >= 0:
            src = src.narrow(in_dim, rng[0] // in_pack, rng[1] // in_pack)
        if segs is None or out_dim < 0:
            assert dst.shape == src.shape, \
                f"{self.prefix}: {tuple(dst.shape)} vs {tuple(src.shape)}"
            dst.copy_(src)
            return
        for so, n, do in segs:
            dst.narrow(out_dim, do // out_pack, n // out_pack).copy_(
                src.narrow(out_dim, so // out_pack, n // out_pack))

    def load_weight(self, name: str, full: torch.Tensor, shard_id=None) -> None:
        """Copies the part of checkpoint tensor ``full`` (parameter ``name``: 'weight',
        'bias', or a quantisation tensor) that belongs to this rank."""
        loader = getattr(self.quant_method, "load_weight", None)
        if loader is not None and loader(self, name, full, shard_id):
            return
        param = getattr(self, name)
        if full.dim() == 1:
            self.copy_sharded(param.data, full, shard_id, 0, -1)
        else:
            self.copy_sharded(param.data, full, shard_id, 0, 1)

    def finalize(self) -> None:
        self.quant_method.process_weights_after_loading(self)


class ReplicatedLinear(LinearBase):
    def __init__(self, in_features, out_features, bias=False, dtype=torch.bfloat16,
                 device=None, quant_method=None, prefix=""):
        super().__init__(in_features, out_features, in_features, out_features, bias, dtype,
                         device, quant_method, prefix)


class MergedReplicatedLinear(ReplicatedLinear):
    """Several replicated projections of the same input stacked along the output dim."""

    def __init__(self, in_features, output_sizes: Sequence[int], **kw):
        self.output_sizes = list(output_sizes)
        super().__init__(in_features, sum(output_sizes), **kw)

    def shard_spec(self, shard_id=None):
        if shard_id is None:
            return None, None
        off = sum(self.output_sizes[:shard_id])
        return [(0, self.output_sizes[shard_id], off)], None


class ColumnParallelLinear(LinearBase):
    def __init__(self, in_features, out_features, bias=False, gather_output=False,
                 dtype=torch.bfloat16, device=None, quant_method=None, prefix=""):
        tp = tp_size()
        assert out_features % tp == 0
        self.gather_output = gather_output
        super().__init__(in_features, out_features, in_features, out_features // tp, bias, dtype,
                         device, quant_method, prefix)

    def shard_spec(self, shard_id=None):
        n = self.out_per_rank
        return [(tp_rank() * n, n, 0)], None

    def forward(self, x, **kw):
        y = super().forward(x, **kw)
        if self.gather_output and tp_size() > 1:
            y = get_comm("tp").all_gather(y, dim=-1)
        return y


class MergedColumnParallelLinear(LinearBase):
    def __init__(self, in_features, output_sizes: Sequence[int], bias=False, fuse_silu=False,
                 dtype=torch.bfloat16, device=None, quant_method=None, prefix=""):
        tp = tp_size()
        self.output_sizes = list(output_sizes)
        assert all(s % tp == 0 for s in output_sizes)
        self.fuse_silu = fuse_silu
        self._interleaved = False
        super().__init__(in_features, sum(output_sizes), in_features, sum(output_sizes) // tp,
                         bias, dtype, device, quant_method, prefix)

    def shard_spec(self, shard_id=None):
        tp, r = tp_size(), tp_rank()
        ids = range(len(self.output_sizes)) if shard_id is None else [shard_id]
        segs = []
        for i in ids:
            n = self.output_sizes[i] // tp
            dst = sum(s // tp for s in self.output_sizes[:i])
            base = sum(self.output_sizes[:i]) if shard_id is None else 0
            segs.append((base + r * n, n, dst))
        return segs, None


class QKVParallelLinear(LinearBase):
    def __init__(self, hidden_size, head_dim, num_heads, num_kv_heads, bias=False,
                 dtype=torch.bfloat16, device=None, quant_method=None, prefix=""):
        tp = tp_size()
        assert num_heads % tp == 0
        self.head_dim = head_dim
        self.num_heads = num_heads // tp
        if num_kv_heads >= tp:
            assert num_kv_heads % tp == 0
            self.num_kv_heads, self.kv_replicas = num_kv_heads // tp, 1
        else:
            assert tp % num_kv_heads == 0
            self.num_kv_heads, self.kv_replicas = 1, tp // num_kv_heads
        self.total_kv_heads = num_kv_heads
        out_pr = (self.num_heads + 2 * self.num_kv_heads) * head_dim
        super().__init__(hidden_size, (num_heads + 2 * num_kv_heads) * head_dim, hidden_size,
                         out_pr, bias, dtype, device, quant_method, prefix)

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def shard_spec(self, shard_id=None):
        r = tp_rank()
        tq = self.num_heads * tp_size() * self.head_dim
        tkv = self.total_kv_heads * self.head_dim
        kv_rank = r // self.kv_replicas
        spec = {"q": (r * self.q_size, self.q_size, 0, 0),
                "k": (kv_rank * self.kv_size, self.kv_size, self.q_size, tq),
                "v": (kv_rank * self.kv_size, self.kv_size, self.q_size + self.kv_size, tq + tkv)}
        ids = ["q", "k", "v"] if shard_id is None else [shard_id]
        segs = []
        for i in ids:
            so, n, do, base = spec[i]
            segs.append(((base if shard_id is None else 0) + so, n, do))
        return segs, None


class RowParallelLinear(LinearBase):
    def __init__(self, in_features, out_features, bias=False, reduce_results=True,
                 dtype=torch.bfloat16, device=None, quant_method=None, prefix=""):
        tp = tp_size()
        assert in_features % tp == 0
        self.reduce_results = reduce_results
        super().__init__(in_features, out_features, in_features // tp, out_features, bias, dtype,
                         device, quant_method, prefix)

    def shard_spec(self, shard_id=None):
        n = self.in_per_rank
        return None, (tp_rank() * n, n)

    def forward(self, x, **kw):
        if tp_size() == 1 or not self.reduce_results:
            return super().forward(x, **kw)
        comm = get_comm("tp")
        fused = getattr(comm, "fused", None)
        if fused is not None and isinstance(self.quant_method, UnquantizedLinearMethod) \
                and self.bias is None:
            y = fused.gemm_all_reduce(x, self.weight)
            if y is not None:
                return y
        y = self.quant_method.apply(self, x, skip_bias=True, **kw)
        y = comm.all_reduce(y)
        if self.bias is not None:   # added once, after the reduction
            y = y + self.bias
        return y
