"""Mixture-of-experts layers.

``FusedMoE`` holds the stacked expert weights of this rank (``w13 [E_local, 2I, H]``,
``w2 [E_local, H, I]``) and runs routed tokens through them: on the GPU with the native
pipeline (align -> permute -> grouped tcgen05 GEMM with SiLU-mul epilogue -> grouped GEMM
scaled by the routing weight -> un-permute + sum), elsewhere with the torch reference.

Parallel layouts (vllm_gcu/kernels/prepare_finalize.py:19-610, patch_0_9_2/moe_layer.py):

* no EP: the intermediate dimension of every expert is sharded over TP; partial sums are
  all-reduced by the caller (``MoEPrepareAndFinalizeNoEP``);
* EP with replicated tokens (attention is tensor parallel, so every rank holds the same
  hidden states): each rank owns ``E / ep`` contiguous experts, computes their contribution
  for all tokens and the partial sums are all-reduced – no dispatch is needed;
* EP with data-parallel attention (every rank holds different tokens): tokens travel to the
  ranks that own their experts and back, see ``layers/moe_ep.py``;
* "ETP" – data-parallel attention without EP (vllm_gcu/distributed/gcu_communicator.py:65-83,
  113-126): the intermediate dimension of every expert is sharded over all ``dp * tp`` ranks,
  the hidden states and router logits of every replica are gathered (all-gather-v over the
  DP group), each rank computes its slice for all tokens, and a reduce-scatter-v over DP
  followed by the TP all-reduce brings every replica the full sum for its own rows.

``SparseMoeBlock`` = router gate + ``FusedMoE`` (+ shared experts whose output seeds the
result, vllm_gcu/kernels/modular_kernel.py:288-295).
"""
from __future__ import annotations

import re

from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..config import ModelConfig
from ..ops import cuda as C
from ..ops import ref
from ..parallel.communicator import get_comm
from ..parallel.state import (ep_rank, ep_size, exchange_dp_rows, get_state, tp_rank,
                              tp_size)
from .linear import ReplicatedLinear


def select_experts(router_logits: torch.Tensor, cfg: ModelConfig,
                   bias: Optional[torch.Tensor] = None, eplb=None
                   ) -> tuple[torch.Tensor, torch.Tensor]:
    """Routing weights fp32 ``[T, k]`` and expert ids int32 ``[T, k]``."""
    k = cfg.num_experts_per_tok
    from .. import envs
    if envs.FORCE_EP_BALANCE:
        # synthetic round-robin routing with uniform weights: every expert (hence every
        # expert-parallel rank) gets the same load, for benchmarking the dispatch path
        # (VLLM_GCU_FORCE_EP_BALANCE, vllm_gcu/kernels/modular_kernel.py:99-128)
        T = router_logits.shape[0]
        E = router_logits.shape[1] if eplb is None else eplb.num_physical
        base = torch.arange(T, device=router_logits.device)[:, None] * k
        ids = ((base + torch.arange(k, device=router_logits.device)[None, :]) % E).to(torch.int32)
        w = torch.full((T, k), 1.0 / k, dtype=torch.float32, device=router_logits.device)
        return w, ids
    grouped = cfg.n_group > 1 or cfg.scoring_func == "sigmoid" or bias is not None
    scale = cfg.routed_scaling_factor if grouped else 1.0
    # plain softmax top-k with a scaling factor (DeepSeek-V2 "greedy" routing): the router
    # paths below fold the factor in only for the grouped form
    post = float(cfg.routed_scaling_factor) if not grouped else 1.0
    if ops.use_native(router_logits):
        w, ids = C.moe_topk(router_logits, k, cfg.norm_topk_prob, cfg.n_group, cfg.topk_group,
                            bias, cfg.scoring_func == "sigmoid", scale,
                            log2phy=eplb.log2phy if eplb is not None else None,
                            replica_count=eplb.replica_count if eplb is not None else None,
                            load=eplb.load if eplb is not None else None)
        return (w * post if post != 1.0 else w), ids
    if grouped:
        w, ids = ref.grouped_topk(router_logits, k, cfg.norm_topk_prob, max(cfg.n_group, 1),
                                  max(cfg.topk_group, 1), bias, cfg.scoring_func, scale)
    else:
        w, ids = ref.topk_softmax(router_logits, k, cfg.norm_topk_prob)
    if eplb is not None:
        ids = ref.eplb_map_to_physical(ids, eplb.log2phy, eplb.replica_count, eplb.load)
    return (w * post if post != 1.0 else w), ids


class FusedMoE(nn.Module):
    def __init__(self, num_experts: int, hidden: int, inter: int, dtype, device,
                 use_ep: bool, prefix: str = "", num_redundant: int = 0, etp: bool = False):
        super().__init__()
        self.global_experts = num_experts + num_redundant
        self.hidden, self.inter_full = hidden, inter
        self.use_ep = use_ep and ep_size() > 1
        if self.use_ep:
            ep, r = ep_size(), ep_rank()
            assert self.global_experts % ep == 0
            self.local_experts = self.global_experts // ep
            self.expert_start = r * self.local_experts
            self.inter = inter
            self.shard_index = 0
            emap = torch.full((self.global_experts,), -1, dtype=torch.int32)
            emap[self.expert_start:self.expert_start + self.local_experts] = torch.arange(
                self.local_experts, dtype=torch.int32)
            self.register_buffer("expert_map", emap.to(device), persistent=False)
        else:
            # the intermediate dimension is cut into `shards` slices: over TP, or over all
            # dp * tp ranks in ETP mode (slice index = dp_rank * tp + tp_rank)
            shards, self.shard_index = tp_size(), tp_rank()
            if etp:
                dpg = get_state().dp
                shards, self.shard_index = dpg.world_size * tp_size(), \
                    dpg.rank_in_group * tp_size() + tp_rank()
            assert inter % shards == 0
            self.local_experts, self.expert_start = self.global_experts, 0
            self.inter = inter // shards
            self.expert_map = None
        E, I, H = self.local_experts, self.inter, hidden
        self.w13 = nn.Parameter(torch.empty(E, 2 * I, H, dtype=dtype, device=device),
                                requires_grad=False)
        self.w2 = nn.Parameter(torch.empty(E, H, I, dtype=dtype, device=device),
                               requires_grad=False)
        self.prefix = prefix
        self._interleaved = False
        self.fp8_block = False
        self.q8_channel = False
        self.wna16 = None           # (bits, group) when the experts stay packed

    def enable_wna16(self, bits: int, group: int, any_device: bool = False) -> bool:
        """Keeps the experts as packed 4 / 8-bit integers with per-group scales (AWQ / GPTQ /
        ``moe_wna16`` checkpoints, vllm_gcu/kernels/quantization/moe_wna16.py:26-643) instead
        of de-quantising them at load: a quarter (an eighth of fp32) of the bf16 footprint; the
        grouped GEMM de-quantises on the fly.  Layout per expert as for the dense layers: ``q``
        uint8 ``[N, K/2]`` (low nibble = even k) or ``[N, K]``, ``s`` and ``z = zero * scale``
        bf16 ``[N, K/g]``.  Returns False when the shapes or the device do not allow it
        (``any_device``: also off the GPU, where the forward de-quantises per call)."""
        E, I, H = self.local_experts, self.inter, self.hidden
        g = int(group)
        if bits not in (4, 8) or g < 32 or g & (g - 1) or H % 64 or I % 64 or H % g or I % g:
            return False
        if not any_device and (not self.w13.is_cuda or self.w13.dtype != torch.bfloat16):
            return False
        dev = self.w13.device
        self._wna16_dtype = self.w13.dtype
        pk = 2 if bits == 4 else 1

        def buf(*shape, dtype):
            return nn.Parameter(torch.zeros(*shape, dtype=dtype, device=dev), requires_grad=False)
        self.w13_q = buf(E, 2 * I, H // pk, dtype=torch.uint8)
        sdt = self._wna16_dtype
        self.w13_s = buf(E, 2 * I, H // g, dtype=sdt)
        self.w13_z = buf(E, 2 * I, H // g, dtype=sdt)
        self.w2_q = buf(E, H, I // pk, dtype=torch.uint8)
        self.w2_s = buf(E, H, I // g, dtype=sdt)
        self.w2_z = buf(E, H, I // g, dtype=sdt)
        self.w13 = nn.Parameter(torch.empty(0, dtype=sdt, device=dev), requires_grad=False)
        self.w2 = nn.Parameter(torch.empty(0, dtype=sdt, device=dev), requires_grad=False)
        self.wna16 = (int(bits), g)
        return True

    def load_expert_weight_wna16(self, expert_id: int, which: str, q: torch.Tensor,
                                 scale: torch.Tensor, zs: torch.Tensor) -> bool:
        """Unpacked integers ``q [N, K]`` (uint8), ``scale`` and ``zs = zero * scale``
        ``[N, K/g]`` of one projection of a logical expert."""
        return any([self._load_one_wna16(p_, which, q, scale, zs) for p_ in self._slots(expert_id)])

    def _load_one_wna16(self, expert_id: int, which: str, q: torch.Tensor, scale: torch.Tensor,
                        zs: torch.Tensor) -> bool:
        le = expert_id - self.expert_start
        if le < 0 or le >= self.local_experts:
            return False
        bits, g = self.wna16
        I = self.inter
        lo = self.shard_index * I

        def pack(t):
            t = t.to(torch.uint8)
            return (t[:, 0::2] | (t[:, 1::2] << 4)).contiguous() if bits == 4 else t
        if which in ("gate", "up"):
            r0 = 0 if which == "gate" else I
            self.w13_q.data[le, r0:r0 + I].copy_(pack(q[lo:lo + I]))
            self.w13_s.data[le, r0:r0 + I].copy_(scale[lo:lo + I])
            self.w13_z.data[le, r0:r0 + I].copy_(zs[lo:lo + I])
        elif which == "down":
            self.w2_q.data[le].copy_(pack(q[:, lo:lo + I]))
            self.w2_s.data[le].copy_(scale[:, lo // g:(lo + I) // g])
            self.w2_z.data[le].copy_(zs[:, lo // g:(lo + I) // g])
        else:
            raise ValueError(which)
        return True

    def enable_fp8_block(self) -> bool:
        """Keeps the experts as fp8 e4m3 with 128 x 128 block scales (the layout of DeepSeek-V3
        checkpoints, vllm_gcu/kernels/quantization/fp8.py:248-420 serves them through
        ``fused_moe_quant_kernel``) instead of de-quantising them at load: half the memory of
        bf16 and fp8 tensor-core GEMMs.  Returns False when the shapes do not allow it."""
        E, I, H = self.local_experts, self.inter, self.hidden
        if I % 128 != 0 or H % 128 != 0 or not self.w13.is_cuda:
            return False
        dev = self.w13.device
        f8 = torch.float8_e4m3fn
        self.w13 = nn.Parameter(torch.zeros(E, 2 * I, H, dtype=f8, device=dev), requires_grad=False)
        self.w2 = nn.Parameter(torch.zeros(E, H, I, dtype=f8, device=dev), requires_grad=False)
        self.w13_scale = nn.Parameter(torch.ones(E, 2 * I // 128, H // 128, dtype=torch.float32,
                                                 device=dev), requires_grad=False)
        self.w2_scale = nn.Parameter(torch.ones(E, H // 128, I // 128, dtype=torch.float32,
                                                device=dev), requires_grad=False)
        self.fp8_block = True
        return True

    def enable_q8_channel(self, dtype: torch.dtype) -> bool:
        """Keeps the experts as int8 or fp8 with one scale per output channel (w8a8
        checkpoints, vllm_gcu/kernels/quantization/w8a8.py:174-342); activations are
        quantised per token in front of each grouped GEMM."""
        E, I, H = self.local_experts, self.inter, self.hidden
        if I % 16 != 0 or H % 16 != 0 or not self.w13.is_cuda:
            return False
        dev = self.w13.device
        self.w13 = nn.Parameter(torch.zeros(E, 2 * I, H, dtype=dtype, device=dev),
                                requires_grad=False)
        self.w2 = nn.Parameter(torch.zeros(E, H, I, dtype=dtype, device=dev), requires_grad=False)
        self.w13_scale = nn.Parameter(torch.ones(E, 2 * I, dtype=torch.float32, device=dev),
                                      requires_grad=False)
        self.w2_scale = nn.Parameter(torch.ones(E, H, dtype=torch.float32, device=dev),
                                     requires_grad=False)
        self.q8_channel = True
        return True

    def _load_one_q8(self, expert_id: int, which: str, weight: torch.Tensor,
                     scale: Optional[torch.Tensor]) -> bool:
        """8-bit ``weight [N, K]`` with a per-tensor or per-channel ``scale`` (None: 1)."""
        le = expert_id - self.expert_start
        if le < 0 or le >= self.local_experts:
            return False
        I = self.inter
        lo = self.shard_index * I
        N = weight.shape[0]
        sc = torch.ones(N, dtype=torch.float32, device=weight.device) if scale is None else \
            scale.to(torch.float32).reshape(-1)
        if sc.numel() == 1:
            sc = sc.expand(N)
        if which == "gate":
            self.w13.data[le, :I].copy_(weight[lo:lo + I])
            self.w13_scale.data[le, :I].copy_(sc[lo:lo + I])
        elif which == "up":
            self.w13.data[le, I:].copy_(weight[lo:lo + I])
            self.w13_scale.data[le, I:].copy_(sc[lo:lo + I])
        elif which == "down":
            self.w2.data[le].copy_(weight[:, lo:lo + I])
            self.w2_scale.data[le].copy_(sc)
        else:
            raise ValueError(which)
        return True

    def _load_one_fp8(self, expert_id: int, which: str, weight: torch.Tensor,
                      scale: torch.Tensor) -> bool:
        """fp8 ``weight [N, K]`` with its ``scale [N/128, K/128]`` (``weight_scale_inv``)."""
        le = expert_id - self.expert_start
        if le < 0 or le >= self.local_experts:
            return False
        I = self.inter
        lo = self.shard_index * I
        b0, nb = lo // 128, I // 128
        if which == "gate":
            self.w13.data[le, :I].copy_(weight[lo:lo + I])
            self.w13_scale.data[le, :nb].copy_(scale[b0:b0 + nb])
        elif which == "up":
            self.w13.data[le, I:].copy_(weight[lo:lo + I])
            self.w13_scale.data[le, nb:].copy_(scale[b0:b0 + nb])
        elif which == "down":
            self.w2.data[le].copy_(weight[:, lo:lo + I])
            self.w2_scale.data[le].copy_(scale[:, b0:b0 + nb])
        else:
            raise ValueError(which)
        return True

    # -- weights -------------------------------------------------------------------
    def set_placement(self, phy2log) -> None:
        """Physical slot -> logical expert (redundant experts): checkpoint tensors of a logical
        expert are loaded into every physical slot that holds a replica of it."""
        self.replicas: dict[int, list[int]] = {}
        for p_, l_ in enumerate(phy2log.tolist() if hasattr(phy2log, "tolist") else phy2log):
            self.replicas.setdefault(int(l_), []).append(p_)

    def _slots(self, expert_id: int) -> list:
        rp = getattr(self, "replicas", None)
        return rp.get(expert_id, []) if rp else [expert_id]

    def load_expert_weight(self, expert_id: int, which: str, full: torch.Tensor) -> bool:
        """Logical expert id (checkpoint numbering); True when a slot of this rank took it."""
        return any([self._load_one(p_, which, full) for p_ in self._slots(expert_id)])

    def load_expert_weight_q8(self, expert_id: int, which: str, weight: torch.Tensor,
                              scale: Optional[torch.Tensor]) -> bool:
        return any([self._load_one_q8(p_, which, weight, scale) for p_ in self._slots(expert_id)])

    def load_expert_weight_fp8(self, expert_id: int, which: str, weight: torch.Tensor,
                               scale: torch.Tensor) -> bool:
        return any([self._load_one_fp8(p_, which, weight, scale) for p_ in self._slots(expert_id)])

    def _load_one(self, expert_id: int, which: str, full: torch.Tensor) -> bool:
        """``which`` in {gate, up, down} (HF ``gate_proj`` / ``up_proj`` / ``down_proj`` or
        Mixtral ``w1`` / ``w3`` / ``w2``).  Returns False when the expert lives elsewhere."""
        le = expert_id - self.expert_start
        if le < 0 or le >= self.local_experts:
            return False
        I = self.inter
        lo = self.shard_index * I
        if which == "gate":
            self.w13.data[le, :I].copy_(full[lo:lo + I])
        elif which == "up":
            self.w13.data[le, I:].copy_(full[lo:lo + I])
        elif which == "down":
            self.w2.data[le].copy_(full[:, lo:lo + I])
        else:
            raise ValueError(which)
        return True

    def finalize(self) -> None:
        """GPU layout: gate / up rows of every expert interleaved in blocks of
        ``ref.GATE_UP_BLOCK`` rows so the grouped GEMM applies SiLU(gate) * up in its epilogue
        (its tiles are 256 columns wide: 2 * I must be a multiple of 256)."""
        if self.wna16 or self._interleaved or not self.w13.is_cuda \
                or self.w13.dtype != torch.bfloat16:
            return
        I = self.inter
        if I % 128 != 0 or self.hidden % 64 != 0:
            return
        w = self.w13.data
        E = w.shape[0]
        B = ref.GATE_UP_BLOCK
        g = w[:, :I].reshape(E, I // B, B, -1)
        u = w[:, I:].reshape(E, I // B, B, -1)
        self.w13.data = torch.stack([g, u], dim=2).reshape(E, 2 * I, -1).contiguous()
        self._interleaved = True

    # -- compute -------------------------------------------------------------------
    def forward(self, x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor,
                add: Optional[torch.Tensor] = None, alpha: float = 1.0,
                valid_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Contribution of this rank's experts (partial sum over TP / EP ranks) plus ``add``.
        ``valid_tokens`` (device int32 scalar) bounds the rows of ``x`` that are in use; rows
        past it produce unspecified output."""
        if x.shape[0] == 0:
            return x if add is None else add
        from .. import envs
        chunk = envs.FUSED_MOE_CHUNK_SIZE
        if chunk > 0 and x.shape[0] > chunk:
            # chunks of token rows, each with its own clamp of the valid-row count
            outs = []
            for lo in range(0, x.shape[0], chunk):
                hi = min(lo + chunk, x.shape[0])
                vt = None if valid_tokens is None else (valid_tokens - lo).clamp(0, hi - lo).to(
                    valid_tokens.dtype)
                outs.append(self.forward(x[lo:hi], topk_w[lo:hi], topk_ids[lo:hi],
                                         None if add is None else add[lo:hi], alpha, vt))
            return torch.cat(outs, dim=0)
        if self.fp8_block:
            return C.fused_experts_fp8(x, self.w13, self.w13_scale, self.w2, self.w2_scale,
                                       topk_w, topk_ids, self.expert_map, add=add, alpha=alpha,
                                       valid_tokens=valid_tokens)
        if self.q8_channel:
            return C.fused_experts_q8(x, self.w13, self.w13_scale, self.w2, self.w2_scale,
                                      topk_w, topk_ids, self.expert_map, add=add, alpha=alpha,
                                      valid_tokens=valid_tokens)
        if self.wna16 and not (ops.use_native(x) and x.dtype == torch.bfloat16):
            # reference path: de-quantise this call's experts (w = q * scale - zs)
            bits, g = self.wna16

            def deq(q, s_, z_):
                if bits == 4:
                    q = torch.stack([q & 0xF, q >> 4], dim=-1).flatten(-2)
                return (q.float() * s_.float().repeat_interleave(g, -1)
                        - z_.float().repeat_interleave(g, -1)).to(x.dtype)
            y = ref.fused_experts(x, deq(self.w13_q, self.w13_s, self.w13_z),
                                  deq(self.w2_q, self.w2_s, self.w2_z), topk_w, topk_ids,
                                  self.expert_map)
            if alpha != 1.0:
                y = (y.float() * alpha).to(x.dtype)
            return y if add is None else y + add
        if self.wna16:
            return C.fused_experts_wna16(x, self.w13_q, self.w13_s, self.w13_z, self.w2_q,
                                         self.w2_s, self.w2_z, self.wna16[1], self.wna16[0],
                                         topk_w, topk_ids, self.expert_map, add=add, alpha=alpha,
                                         valid_tokens=valid_tokens)
        if self._interleaved and ops.use_native(x):
            return C.fused_experts(x, self.w13, self.w2, topk_w, topk_ids, self.expert_map,
                                   add=add, alpha=alpha, valid_tokens=valid_tokens)
        w13 = self.w13
        if self._interleaved:    # undo the GPU layout for the reference path
            w13 = ref.deinterleave_gate_up(w13)
        y = ref.fused_experts(x, w13, self.w2, topk_w, topk_ids, self.expert_map)
        if alpha != 1.0:
            y = (y.float() * alpha).to(x.dtype)
        return y if add is None else y + add


class EplbState:
    """Logical -> physical expert mapping with redundant replicas and a load histogram
    (``enable_eplb`` / ``num_redundant_experts`` of the reference's ``additional_config``,
    vllm_gcu/gcu.py:302-308; static placement from ``expert_map_path``,
    vllm_gcu/models/deepseek_v3/deepseek_v3.py:880-913)."""

    def __init__(self, num_logical: int, num_redundant: int, device,
                 phy2log: Optional[torch.Tensor] = None):
        num_phys = num_logical + num_redundant
        if phy2log is None:
            phy2log = torch.cat([torch.arange(num_logical),
                                 torch.arange(num_redundant) % max(num_logical, 1)])
        self.phy2log = phy2log.to(torch.int32)
        reps: list[list[int]] = [[] for _ in range(num_logical)]
        for p, l in enumerate(self.phy2log.tolist()):
            reps[l].append(p)
        R = max(len(r) for r in reps)
        l2p = torch.zeros(num_logical, R, dtype=torch.int32)
        cnt = torch.zeros(num_logical, dtype=torch.int32)
        for l, r in enumerate(reps):
            cnt[l] = len(r)
            for j in range(R):
                l2p[l, j] = r[j % len(r)]
        self.log2phy = l2p.to(device)
        self.replica_count = cnt.to(device)
        self.load = torch.zeros(num_phys, dtype=torch.int32, device=device)
        self.num_physical = num_phys

    def rebalance(self) -> torch.Tensor:
        """Greedy re-placement of the redundant slots onto the most loaded logical experts.
        Returns the new ``phy2log`` (weights must be re-homed by the caller)."""
        num_logical = self.log2phy.shape[0]
        load_l = torch.zeros(num_logical, dtype=torch.float64)
        load_l.index_add_(0, self.phy2log.long(), self.load.double().cpu())
        num_red = self.num_physical - num_logical
        cnt = torch.ones(num_logical, dtype=torch.float64)
        extra = []
        for _ in range(num_red):
            j = int(torch.argmax(load_l / cnt))
            extra.append(j)
            cnt[j] += 1
        return torch.cat([torch.arange(num_logical), torch.tensor(extra, dtype=torch.long)]).to(
            torch.int32)


class SparseMoeBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, device, prefix: str):
        super().__init__()
        self.cfg = cfg
        st = get_state()
        self.use_ep = st.ep.world_size > 1
        self.gate = ReplicatedLinear(cfg.hidden_size, cfg.num_experts, bias=False,
                                     dtype=cfg.dtype, device=device, prefix=prefix + ".gate")
        if cfg.topk_method == "noaux_tc":
            self.e_score_correction_bias = nn.Parameter(
                torch.zeros(cfg.num_experts, dtype=torch.float32, device=device),
                requires_grad=False)
        else:
            self.e_score_correction_bias = None
        num_red = int(cfg.extra.get("num_redundant_experts", 0))
        self.dp_attention = bool(cfg.extra.get("dp_attention", False))
        # data-parallel attention without EP: experts sharded over dp * tp
        # (gcu_communicator.py:65-68 turns this on under the same condition)
        self.use_etp = (self.dp_attention and not self.use_ep and st.dp.world_size > 1
                        and bool(cfg.extra.get("etp", True)))
        self.experts = FusedMoE(cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size,
                                cfg.dtype, device, self.use_ep, prefix + ".experts", num_red,
                                etp=self.use_etp)
        if cfg.quantization and cfg.dtype == torch.bfloat16 and cfg.extra.get("q8_experts", True):
            from .quant.moe import expert_storage
            kind = expert_storage(cfg.quantization, cfg.quant_config)
            if kind == "fp8_block":
                self.experts.enable_fp8_block()
            elif kind == "int8":
                self.experts.enable_q8_channel(torch.int8)
            elif kind == "fp8":
                self.experts.enable_q8_channel(torch.float8_e4m3fn)
            elif kind == "wna16":
                qc = cfg.quant_config or {}
                self.experts.enable_wna16(int(qc.get("bits", qc.get("w_bit", 4))),
                                          int(qc.get("group_size", qc.get("q_group_size", 128))))
        phy2log = None
        map_path = cfg.extra.get("expert_map_path")
        if map_path:
            # static placement file of the reference: (phy2log [moe layers, devices, experts per
            # device], log2phy), vllm_gcu/models/deepseek_v3/deepseek_v3.py:880-913
            loaded = torch.load(map_path, map_location="cpu")
            table = loaded[0] if isinstance(loaded, (tuple, list)) else loaded
            m_ = re.search(r"layers\.(\d+)\.", prefix + ".")
            li = (int(m_.group(1)) if m_ else 0) - int(cfg.first_k_dense_replace or 0)
            phy2log = table[max(li, 0)].reshape(-1).to(torch.int32)
            assert phy2log.numel() == cfg.num_experts + num_red, \
                "expert_map_path does not match num_experts + num_redundant_experts"
        self.eplb = EplbState(cfg.num_experts, num_red, device, phy2log) \
            if (num_red > 0 or phy2log is not None) else None
        if self.eplb is not None:
            self.experts.set_placement(self.eplb.phy2log)
        if cfg.num_shared_experts > 0:
            from ..models.decoder import DenseMLP
            self.shared_experts = DenseMLP(cfg, cfg.hidden_size,
                                           cfg.moe_intermediate_size * cfg.num_shared_experts,
                                           device, prefix + ".shared_experts",
                                           reduce_results=False)
        else:
            self.shared_experts = None
        self.dispatcher = None
        if self.use_ep and self.dp_attention:
            from .moe_ep import AllToAllDispatcher, FusedEPDispatcher
            fused_ok = (torch.device(device).type == "cuda" and st.ep.world_size <= 8
                        and cfg.dtype == torch.bfloat16
                        and cfg.extra.get("ep_backend", "fused") == "fused")
            if fused_ok:
                self.dispatcher = FusedEPDispatcher(
                    self.experts, cfg, int(cfg.extra.get("ep_max_tokens", 8192)),
                    torch.device(device))
            else:
                self.dispatcher = AllToAllDispatcher(self.experts, cfg)

    def load_weight(self, name: str, full: torch.Tensor, shard_id=None) -> None:
        if name == "e_score_correction_bias":
            self.e_score_correction_bias.data.copy_(full)
        else:
            raise KeyError(name)

    def _forward_etp(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        """Gather every replica's rows, run this rank's slice of all experts over them, and
        scatter the sums back (dispatch / combine of gcu_communicator.py:113-126 with the
        all-gather-v manager of :22-31)."""
        st = get_state()
        dp = get_comm("dp")
        # the model publishes the row counts once per forward; a block used on its own asks
        # for them itself (every rank takes the same branch)
        sizes = st.dp_rows if st.dp_rows is not None else exchange_dp_rows(x.shape[0])
        xg = dp.all_gather_v(x, sizes)
        lg = dp.all_gather_v(logits, sizes)
        shared = self.shared_experts(x) if self.shared_experts is not None else None
        if xg.shape[0]:
            topk_w, topk_ids = select_experts(lg, self.cfg, self.e_score_correction_bias, None)
            yg = self.experts(xg, topk_w, topk_ids)
        else:
            yg = xg
        out = dp.reduce_scatter_v(yg, sizes)
        if shared is not None:
            out = out + shared
        return get_comm("tp").all_reduce(out) if tp_size() > 1 else out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x = x.reshape(-1, shape[-1])
        logits = self.gate(x)
        if self.use_etp:
            return self._forward_etp(x, logits).view(shape)
        topk_w, topk_ids = select_experts(logits, self.cfg, self.e_score_correction_bias,
                                          self.eplb)
        from .. import envs
        # Tensor-parallel ranks of one replica hold the same rows after attention.  Each of
        # them dispatches only its own slice of the rows (uneven split, as sequence
        # parallelism uses), so a token visits its experts once per replica instead of once
        # per tensor-parallel rank; the slices are put together again below.
        tp = tp_size()
        sliced = self.dispatcher is not None and tp > 1 and envs.EP_TP_SLICE
        xd, wd, idd = x, topk_w, topk_ids
        if sliced:
            from ..parallel.sp import scatter
            sizes = scatter(x.shape[0], tp)
            lo = sum(sizes[:tp_rank()])
            hi = lo + sizes[tp_rank()]
            xd, wd, idd = x[lo:hi], topk_w[lo:hi], topk_ids[lo:hi]

        def merge(routed: torch.Tensor, shared_) -> torch.Tensor:
            """Sliced mode: routed rows of this rank + TP-partial shared-expert output of all
            rows -> full output on every rank."""
            if shared_ is None:
                return get_comm("tp").all_gather_v(routed, sizes)
            shared_[lo:hi] += routed.to(shared_.dtype)      # a fresh tensor of this call
            return get_comm("tp").all_reduce(shared_)

        def unsliced(out_: torch.Tensor, shared_) -> torch.Tensor:
            """Every rank dispatched all rows: the routed sum is whole on every rank, only the
            shared experts' output is a partial sum over the tensor-parallel ranks."""
            if tp > 1 and shared_ is not None:
                out_ = out_ - shared_ + get_comm("tp").all_reduce(shared_.clone())
            return out_

        side = None
        if (self.shared_experts is not None and self.dispatcher is not None and x.is_cuda
                and envs.ENABLE_PARALLEL_COMPUTE and not torch.cuda.is_current_stream_capturing()):
            # shared experts on a side stream, overlapped with the dispatch kernels
            # (VLLM_GCU_ENABLE_PARALLEL_COMPUTE, vllm_gcu/kernels/prepare_finalize.py:326-336)
            if not hasattr(self, "_side_stream"):
                self._side_stream = torch.cuda.Stream()
            side = self._side_stream
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                shared = self.shared_experts(x)
        else:
            shared = self.shared_experts(x) if self.shared_experts is not None else None
        if side is not None:
            # the dispatcher adds `shared` in its combine step: join before that
            xr = self.dispatcher.ws.dispatch(xd, wd.float(), idd.to(torch.int32),
                                             get_state().dp_max_tokens) \
                if hasattr(self.dispatcher, "ws") else None
            torch.cuda.current_stream().wait_stream(side)
            if xr is not None:
                rx, rw, rids, total = xr
                yr = self.experts(rx, rw, rids, valid_tokens=total)
                if sliced:
                    return merge(self.dispatcher.ws.combine(yr, xd.shape[0], None),
                                 shared).view(shape)
                out = self.dispatcher.ws.combine(yr, x.shape[0], shared)
                return unsliced(out, shared).view(shape)
        if self.dispatcher is not None:
            # tokens differ per rank: all-to-all dispatch / combine, seeded with the shared
            # experts' output (a replica without tensor parallelism holds them whole)
            if sliced:
                routed = self.dispatcher(xd, wd, idd, None, get_state().dp_max_tokens)
                return merge(routed, shared).view(shape)
            out = self.dispatcher(x, topk_w, topk_ids, shared, get_state().dp_max_tokens)
            return unsliced(out, shared).view(shape)
        # For plain top-k routing the scaling factor is applied on the combined output;
        # the grouped router already folded it into the weights.
        out = self.experts(x, topk_w, topk_ids, add=shared)
        if self.use_ep:
            out = get_comm("ep").all_reduce(out)
        elif tp_size() > 1:
            out = get_comm("tp").all_reduce(out)
        return out.view(shape)
