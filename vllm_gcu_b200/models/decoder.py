"""Generic pre-norm decoder-only transformer.

One implementation, configured by :class:`ModelConfig`, serves the dense families the
reference supports through its own or upstream model code (Llama 2/3, Qwen 2/2.5/3,
GLM-4-0414 with sandwich norms and partial GPT-J rotary, Mistral/Yi/InternLM-style
checkpoints) and hosts the MoE and MLA blocks of the Qwen3-MoE / Mixtral / DeepSeek
models.  The layer structure follows vllm_gcu/models/qwen3/qwen3.py:437 and
vllm_gcu/models/glm4/glm4.py:173-231; checkpoint names are the HuggingFace ones.
"""
from __future__ import annotations

import zlib
from typing import Iterable, Optional

import torch
import torch.nn as nn

from ..config import ModelConfig
from ..layers.attention import AttentionMetadata, PagedAttention
from ..layers.basic import ParallelLMHead, RMSNorm, RotaryEmbedding, VocabParallelEmbedding
from ..layers.linear import (MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear)
from ..ops import cuda as C
from ..parallel.state import get_state, tp_rank, tp_size


def get_linear_method(cfg: ModelConfig, prefix: str):
    """Quantised linear method for the layer called ``prefix`` (None = unquantised)."""
    if not cfg.quantization:
        return None
    from ..layers.quant import get_quant_config
    return get_quant_config(cfg).get_linear_method(prefix)


def fused_input_quant(linear, x: torch.Tensor, width: Optional[int] = None):
    """``(mode, static scale)`` when the kernel that produces ``linear``'s input (a norm or a
    gated activation of ``width`` output columns) should emit it quantised: the layer runs on
    8-bit activations, the tensors are on the GPU in a 16-bit type, and the width suits the
    mode.  The reference gets the same effect from its compile-time fusion pass
    (vllm_gcu/compilation/fusion.py:889-1023)."""
    from .. import envs, ops
    if not (ops.use_native(x) and x.dtype in (torch.bfloat16, torch.float16)):
        return None
    if not type(linear).__module__.endswith("layers.linear"):
        return None            # wrapped layers (LoRA) need the 16-bit rows as well
    iq = linear.quant_method.input_quant(linear)
    if iq is None or not envs.FUSE_ACT_QUANT:
        return None
    width = x.shape[-1] if width is None else width
    if width % 8 != 0 or (iq[0] == "fp8_group128" and width % 128 != 0):
        return None
    return iq


class DenseMLP(nn.Module):
    def __init__(self, cfg: ModelConfig, hidden: int, inter: int, device, prefix: str,
                 reduce_results: bool = True):
        super().__init__()
        self.gate_up_proj = MergedColumnParallelLinear(
            hidden, [inter, inter], bias=cfg.mlp_bias, fuse_silu=(cfg.hidden_act == "silu"),
            dtype=cfg.dtype, device=device,
            quant_method=get_linear_method(cfg, prefix + ".gate_up_proj"),
            prefix=prefix + ".gate_up_proj")
        self.down_proj = RowParallelLinear(
            inter, hidden, bias=cfg.mlp_bias, reduce_results=reduce_results, dtype=cfg.dtype,
            device=device, quant_method=get_linear_method(cfg, prefix + ".down_proj"),
            prefix=prefix + ".down_proj")
        self.act = cfg.hidden_act
        from ..layers.linear import UnquantizedLinearMethod
        if not isinstance(self.gate_up_proj.quant_method, UnquantizedLinearMethod):
            self.gate_up_proj.fuse_silu = False   # quantised GEMMs have no SiLU epilogue yet

    def before_down_proj(self, x: torch.Tensor) -> torch.Tensor:
        h = self.gate_up_proj(x)
        if not self.gate_up_proj.fuse_silu:
            from ..layers.activation import act_and_mul
            h = act_and_mul(h, self.act)
        return h

    def _act_quant(self, h: torch.Tensor):
        """Gated activation, fused with the quantisation of down_proj's input when that layer
        runs on 8-bit activations in a mode the activation kernel can emit (128-wide fp8 groups
        or a static scale).  Returns ``(tensor, kwargs for down_proj)``."""
        from ..layers.activation import act_and_mul
        iq = fused_input_quant(self.down_proj, h, h.shape[-1] // 2)
        if iq is not None and iq[0] in C.ACT_QUANT and self.act in C.ACT_CODES:
            out = C.activation(h, self.act, "act_mul", quant=iq[0], scale=iq[1])
            if isinstance(out, tuple):
                return out[0], {"x_scale": out[1]}
            return out, {"x_scale": iq[1].reshape(1).expand(out.shape[0]).contiguous()}
        return act_and_mul(h, self.act), {}

    def forward(self, x: torch.Tensor, sp_sizes: Optional[list] = None,
                x_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``sp_sizes`` (sequence parallelism): ``x`` holds this rank's rows; the rows are
        gathered for the column-parallel projection and the row-parallel output is
        reduce-scattered back to rows.  ``x_scale``: ``x`` is already quantised for
        gate_up_proj (see ``fused_input_quant``)."""
        kw = {}
        if sp_sizes is not None:
            from ..parallel import sp
            h = sp.sp_gather_linear(self.gate_up_proj, x, sp_sizes)
        else:
            h = self.gate_up_proj(x) if x_scale is None else self.gate_up_proj(x, x_scale=x_scale)
        if not self.gate_up_proj.fuse_silu:
            if sp_sizes is None:
                h, kw = self._act_quant(h)
            else:
                from ..layers.activation import act_and_mul
                h = act_and_mul(h, self.act)
        if sp_sizes is not None:
            from ..parallel import sp
            keep, self.down_proj.reduce_results = self.down_proj.reduce_results, False
            try:
                y = self.down_proj(h)
            finally:
                self.down_proj.reduce_results = keep
            return sp.reduce_scatter_rows(y, sp_sizes)
        return self.down_proj(h, **kw)


_QKV_BIAS_ONLY = frozenset({
    "Qwen2ForCausalLM", "Qwen2Model", "Qwen2EmbeddingModel", "Qwen2VLForConditionalGeneration",
    "Qwen2_5_VLForConditionalGeneration", "Glm4ForCausalLM", "Glm4vForConditionalGeneration",
    "ChatGLMModel", "ChatGLMForConditionalGeneration", "GotOcr2ForConditionalGeneration",
    "GOTQwenForCausalLM", "InternVLChatModel", "InternVLForConditionalGeneration"})


class GQAAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device, prefix: str):
        super().__init__()
        D = cfg.head_dim
        self.qkv_proj = QKVParallelLinear(
            cfg.hidden_size, D, cfg.num_attention_heads, cfg.num_key_value_heads,
            bias=cfg.attention_bias, dtype=cfg.dtype, device=device,
            quant_method=get_linear_method(cfg, prefix + ".qkv_proj"), prefix=prefix + ".qkv_proj")
        # ``attention_bias`` of Llama / Qwen3 / Gemma / InternLM2 configs covers the output
        # projection too; Qwen2 and the GLM families have biases on q / k / v only
        o_bias = cfg.extra.get("o_proj_bias")
        if o_bias is None:
            o_bias = bool(cfg.attention_bias) and cfg.architecture not in _QKV_BIAS_ONLY
        self.o_proj = RowParallelLinear(
            cfg.num_attention_heads * D, cfg.hidden_size, bias=bool(o_bias), dtype=cfg.dtype,
            device=device, quant_method=get_linear_method(cfg, prefix + ".o_proj"),
            prefix=prefix + ".o_proj")
        alibi = None
        if str(cfg.extra.get("position_embedding", "ROPE")).upper() == "ALIBI":
            # linear position biases instead of rotary embeddings; heads are sharded over TP
            from ..layers.attention import alibi_slopes
            nh = self.qkv_proj.num_heads
            alibi = alibi_slopes(cfg.num_attention_heads)[tp_rank() * nh:(tp_rank() + 1) * nh] \
                .contiguous().to(device)
            rotary = None
        else:
            rotary = RotaryEmbedding(D, cfg.rotary_dim, cfg.max_position_embeddings,
                                     cfg.rope_theta, cfg.rope_is_neox, cfg.rope_scaling,
                                     cfg.dtype, device)
        qn = kn = None
        if cfg.qk_norm:
            qn = RMSNorm(D, cfg.rms_norm_eps, cfg.dtype, device)
            kn = RMSNorm(D, cfg.rms_norm_eps, cfg.dtype, device)
        self.q_norm, self.k_norm = qn, kn
        self.attn = PagedAttention(self.qkv_proj.num_heads, self.qkv_proj.num_kv_heads, D,
                                   D ** -0.5, rotary, qn, kn, cfg.window_for_layer(layer_idx),
                                   alibi)

    def before_o_proj(self, x: torch.Tensor, kv_cache: torch.Tensor, md: AttentionMetadata,
                      x_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Attention output of this rank's heads (the input of the row-parallel o_proj)."""
        qkv = self.qkv_proj(x) if x_scale is None else self.qkv_proj(x, x_scale=x_scale)
        return self.attn(qkv, kv_cache, md)

    def forward(self, x: torch.Tensor, kv_cache: torch.Tensor, md: AttentionMetadata,
                sp_sizes: Optional[list] = None, x_scale: Optional[torch.Tensor] = None
                ) -> torch.Tensor:
        if sp_sizes is None:
            return self.o_proj(self.before_o_proj(x, kv_cache, md, x_scale))
        # sequence parallelism: rows in, rows out (vllm_gcu/models/deepseek_v3/
        # deepseek_v3.py:611-612,747-748: sp_to_tp before the projections, tp_to_sp after o_proj)
        from ..parallel import sp
        qkv = sp.sp_gather_linear(self.qkv_proj, x, sp_sizes)
        keep, self.o_proj.reduce_results = self.o_proj.reduce_results, False
        try:
            y = self.o_proj(self.attn(qkv, kv_cache, md))
        finally:
            self.o_proj.reduce_results = keep
        return sp.reduce_scatter_rows(y, sp_sizes)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device, prefix: str):
        super().__init__()
        self.layer_idx = layer_idx
        H = cfg.hidden_size
        if cfg.is_mla:
            from .deepseek import MLAAttention
            self.self_attn = MLAAttention(cfg, layer_idx, device, prefix + ".self_attn")
        else:
            self.self_attn = GQAAttention(cfg, layer_idx, device, prefix + ".self_attn")
        if cfg.is_moe_layer(layer_idx):
            from ..layers.moe import SparseMoeBlock
            self.mlp = SparseMoeBlock(cfg, device, prefix + ".mlp")
        else:
            self.mlp = DenseMLP(cfg, H, cfg.intermediate_size, device, prefix + ".mlp")
        self.input_layernorm = RMSNorm(H, cfg.rms_norm_eps, cfg.dtype, device)
        self.post_attention_layernorm = RMSNorm(H, cfg.rms_norm_eps, cfg.dtype, device)
        self.sandwich = cfg.sandwich_norm
        if self.sandwich:
            self.post_self_attn_layernorm = RMSNorm(H, cfg.rms_norm_eps, cfg.dtype, device)
            self.post_mlp_layernorm = RMSNorm(H, cfg.rms_norm_eps, cfg.dtype, device)

    # -- tensor parallel with the reductions fused into the GEMMs --------------------------
    def fusable(self) -> tuple[bool, bool]:
        """(attention block, MLP block) can use ``FusedTP.gemm_ar_norm``: plain bf16
        row-parallel projections without bias / LoRA wrapper and plain RMSNorms around them."""
        from ..layers.linear import UnquantizedLinearMethod

        def row_ok(m) -> bool:
            return (type(m) is RowParallelLinear and m.bias is None and m.reduce_results
                    and isinstance(m.quant_method, UnquantizedLinearMethod)
                    and m.weight.dtype == torch.bfloat16)

        norms_ok = (not self.sandwich and type(self.input_layernorm) is RMSNorm
                    and type(self.post_attention_layernorm) is RMSNorm)
        attn_ok = norms_ok and isinstance(self.self_attn, GQAAttention) \
            and row_ok(self.self_attn.o_proj)
        mlp_ok = attn_ok and isinstance(self.mlp, DenseMLP) and row_ok(self.mlp.down_proj)
        return attn_ok, mlp_ok

    def forward_fused_tp(self, x: torch.Tensor, residual: Optional[torch.Tensor],
                         kv_cache: torch.Tensor, md: AttentionMetadata, fused,
                         x_is_normed: bool, next_norm: Optional[RMSNorm]):
        """Layer forward where o_proj and down_proj run as one kernel each with their
        all-reduce, the residual add and the RMSNorm that follows them.  ``x_is_normed``: ``x``
        already went through this layer's input norm (the previous layer's down_proj did it).
        Returns ``(x, residual, x_is_normed)`` for the next layer; ``next_norm`` is the norm
        that follows this layer (the next layer's input norm, or the final norm)."""
        _, mlp_ok = self.fusable()
        if x_is_normed:
            h = x
        elif residual is None:
            residual = x
            h = self.input_layernorm(x)
        else:
            h, residual = self.input_layernorm(x, residual)
        a = self.self_attn.before_o_proj(h, kv_cache, md)
        pn = self.post_attention_layernorm
        # the new residual is needed on every rank only if a plain norm reads it next
        fuse_mlp = mlp_ok and next_norm is not None
        h, residual = fused.gemm_ar_norm(a, self.self_attn.o_proj.weight, residual, pn.weight,
                                         pn.eps, bcast_residual=not fuse_mlp)
        if not fuse_mlp:
            h = self.mlp(h)
            return h, residual, False
        h = self.mlp.before_down_proj(h)
        h, residual = fused.gemm_ar_norm(h, self.mlp.down_proj.weight, residual,
                                         next_norm.weight, next_norm.eps, bcast_residual=False)
        return h, residual, True

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor], kv_cache: torch.Tensor,
                md: AttentionMetadata, sp_sizes: Optional[list] = None):
        # 8-bit qkv / gate_up projections take their input quantised by the norm kernel
        iq_attn = iq_mlp = None
        if sp_sizes is None and x.shape[0] > 0 and type(self.input_layernorm) is RMSNorm:
            if isinstance(self.self_attn, GQAAttention):
                iq_attn = fused_input_quant(self.self_attn.qkv_proj, x)
            if isinstance(self.mlp, DenseMLP) and type(self.post_attention_layernorm) is RMSNorm:
                iq_mlp = fused_input_quant(self.mlp.gate_up_proj, x)
        if iq_attn is not None:
            if residual is None:
                residual = x
                h, xs, _ = self.input_layernorm.forward_quant(x, None, *iq_attn)
            else:
                h, xs, residual = self.input_layernorm.forward_quant(x, residual, *iq_attn)
            h = self.self_attn(h, kv_cache, md, x_scale=xs)
        else:
            if residual is None:
                residual = x
                h = self.input_layernorm(x)
            else:
                h, residual = self.input_layernorm(x, residual)
            if sp_sizes is not None and isinstance(self.self_attn, GQAAttention):
                h = self.self_attn(h, kv_cache, md, sp_sizes)
            elif sp_sizes is not None:
                from ..parallel import sp
                full = self.self_attn(sp.sp_to_tp(h, sum(sp_sizes)), kv_cache, md)
                h = sp.slice_tensor_sp(full)
            else:
                h = self.self_attn(h, kv_cache, md)
        if self.sandwich:
            h = self.post_self_attn_layernorm(h)
        if iq_mlp is not None:
            h, xs, residual = self.post_attention_layernorm.forward_quant(h, residual, *iq_mlp)
            h = self.mlp(h, x_scale=xs)
            if self.sandwich:
                h = self.post_mlp_layernorm(h)
            return h, residual
        h, residual = self.post_attention_layernorm(h, residual)
        if sp_sizes is not None and isinstance(self.mlp, DenseMLP):
            h = self.mlp(h, sp_sizes)
        elif sp_sizes is not None:
            # MoE blocks reduce over their own group: run them on all rows, keep ours
            from ..parallel import sp
            h = sp.slice_tensor_sp(self.mlp(sp.sp_to_tp(h, sum(sp_sizes))))
        else:
            h = self.mlp(h)
        if self.sandwich:
            h = self.post_mlp_layernorm(h)
        return h, residual


class DecoderLM(nn.Module):
    """Embedding -> N decoder layers -> final norm -> vocab-parallel LM head."""

    # checkpoint-name fragments that are stacked into one parameter: (param, ckpt, shard id)
    stacked_params = [
        ("qkv_proj", "q_proj", "q"), ("qkv_proj", "k_proj", "k"), ("qkv_proj", "v_proj", "v"),
        ("gate_up_proj", "gate_proj", 0), ("gate_up_proj", "up_proj", 1),
    ]

    def __init__(self, cfg: ModelConfig, device="cpu"):
        super().__init__()
        self.cfg = cfg
        self.device = torch.device(device)
        st = get_state()
        pp, pp_rank = st.pp.world_size, st.pp.rank_in_group
        L = cfg.num_hidden_layers
        per = -(-L // pp)
        self.start_layer, self.end_layer = min(L, pp_rank * per), min(L, (pp_rank + 1) * per)
        self.is_first_stage, self.is_last_stage = pp_rank == 0, pp_rank == pp - 1
        from .. import envs
        self.sequence_parallel = bool(cfg.extra.get("sequence_parallel")
                                      or envs.ENABLE_SEQUENCE_PARALLEL)
        if self.is_first_stage or (cfg.tie_word_embeddings and self.is_last_stage):
            # a tied embedding also serves as the output projection
            emb_cls = ParallelLMHead if cfg.tie_word_embeddings else VocabParallelEmbedding
            self.embed_tokens = emb_cls(cfg.vocab_size, cfg.hidden_size, cfg.dtype, device)
        self.layers = nn.ModuleDict({
            str(i): DecoderLayer(cfg, i, device, f"model.layers.{i}")
            for i in range(self.start_layer, self.end_layer)})
        if self.is_last_stage:
            self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)
            if cfg.tie_word_embeddings:
                self.lm_head = None
            else:
                self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype, device)

    # -- execution ---------------------------------------------------------------
    @property
    def num_local_layers(self) -> int:
        return self.end_layer - self.start_layer

    def kv_cache_spec(self) -> dict:
        """Shape information the runner needs to allocate this model's KV cache."""
        cfg = self.cfg
        if cfg.is_mla:
            return {"type": "mla", "layers": self.num_local_layers,
                    "width": cfg.kv_lora_rank + cfg.qk_rope_head_dim}
        kvh = max(1, cfg.num_key_value_heads // tp_size())
        return {"type": "gqa", "layers": self.num_local_layers, "kv_heads": kvh,
                "head_dim": cfg.head_dim}

    def forward(self, input_ids: Optional[torch.Tensor], md: AttentionMetadata,
                kv_caches: list[torch.Tensor],
                intermediate: Optional[tuple[torch.Tensor, torch.Tensor]] = None,
                inputs_embeds: Optional[torch.Tensor] = None):
        """Returns final hidden states ``[T, H]`` on the last pipeline stage, otherwise the
        ``(hidden, residual)`` pair handed to the next stage."""
        if self.is_first_stage:
            x = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
            scale = getattr(self, "embed_scale", None)
            if scale is not None and inputs_embeds is None:
                x = x * scale
            residual = None
        else:
            x, residual = intermediate
        sp_sizes = None
        if self.sequence_parallel and tp_size() > 1 and x.shape[0] > 0 \
                and get_state().pp.world_size == 1:
            # the residual stream is sharded by rows between the attention / MLP blocks
            from ..parallel import sp
            total = x.shape[0]
            sp_sizes = sp.scatter(total, tp_size())
            x = sp.slice_tensor_sp(x)
        fused = self._fused_tp(x) if sp_sizes is None else None
        normed = False
        ids = list(range(self.start_layer, self.end_layer))
        if getattr(self, "_etp", None) is None:
            self._etp = any(getattr(m, "use_etp", False) for m in self.modules())
        if self._etp and sp_sizes is None:
            # ETP experts gather / scatter rows over the DP group: one host exchange of the
            # row counts per forward instead of one per layer
            from ..parallel.state import exchange_dp_rows
            get_state().dp_rows = exchange_dp_rows(x.shape[0])
        for j, i in enumerate(ids):
            layer = self.layers[str(i)]
            if fused is not None and layer.fusable()[0]:
                if j + 1 < len(ids):
                    nxt = self.layers[str(ids[j + 1])]
                    next_norm = nxt.input_layernorm if nxt.fusable()[0] else None
                else:
                    next_norm = self.norm if self.is_last_stage and type(self.norm) is RMSNorm \
                        else None
                x, residual, normed = layer.forward_fused_tp(x, residual, kv_caches[j], md, fused,
                                                             normed, next_norm)
            else:
                assert not normed
                x, residual = layer(x, residual, kv_caches[j], md, sp_sizes)
        if self._etp:
            get_state().dp_rows = None
        if not self.is_last_stage:
            return x, residual
        if normed:
            pass                        # the last down_proj applied the final norm
        elif residual is None:
            x = self.norm(x)
        else:
            x, _ = self.norm(x, residual)
        if sp_sizes is not None:
            from ..parallel import sp
            x = sp.sp_to_tp(x, sum(sp_sizes))
        return x

    def _fused_tp(self, x: torch.Tensor):
        """The tensor-parallel workspace when this step can run the fused
        GEMM + all-reduce + norm kernels (GPU, TP > 1, ``comm_backend="fused"``, the token
        count fits the workspace); None otherwise."""
        if tp_size() <= 1 or not x.is_cuda or x.dtype != torch.bfloat16 or x.shape[0] == 0:
            return None
        from ..parallel.communicator import get_comm
        fused = getattr(get_comm("tp"), "fused", None)
        if fused is None or not getattr(fused, "fuse_norm", True):
            return None
        if x.shape[0] > fused.max_tokens or x.shape[1] > min(fused.max_n, 8192):
            return None
        return fused

    def _head(self) -> ParallelLMHead:
        return self.lm_head if self.lm_head is not None else self.embed_tokens  # type: ignore

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        head = self._head()
        if isinstance(head, ParallelLMHead):
            return head.logits(hidden)
        return ParallelLMHead.logits(head, hidden)  # tied embedding

    def greedy_tokens(self, hidden: torch.Tensor) -> torch.Tensor:
        head = self._head()
        return ParallelLMHead.greedy(head, hidden)

    # -- weights --------------------------------------------------------------------
    def named_loadables(self) -> dict[str, nn.Module]:
        """Maps parameter-owner module paths (``model.layers.0.self_attn.qkv_proj``) to
        modules that implement ``load_weight``."""
        out: dict[str, nn.Module] = {}
        for name, mod in self.named_modules():
            if hasattr(mod, "load_weight"):
                out[self._ckpt_prefix(name)] = mod
        return out

    @staticmethod
    def _ckpt_prefix(module_path: str) -> str:
        # self.layers is a ModuleDict keyed by layer index
        if module_path.startswith("layers."):
            return "model." + module_path
        if module_path in ("embed_tokens", "norm"):
            return "model." + module_path
        return module_path

    def map_weight_name(self, name: str) -> Optional[tuple[str, str, object]]:
        """checkpoint tensor name -> (owner module path, parameter name, shard id)."""
        if "rotary_emb.inv_freq" in name:
            return None
        owner, _, pname = name.rpartition(".")
        for stacked, ckpt, sid in self.stacked_params:
            if owner.endswith("." + ckpt):
                return owner[: -len(ckpt)] + stacked, pname, sid
        if owner.endswith(".q_norm") or owner.endswith(".k_norm"):
            return owner, pname, None
        return owner, pname, None

    def load_special(self, name: str, tensor: torch.Tensor, owners: dict) -> bool:
        """Hook for tensors that do not map 1:1 onto a ``load_weight`` owner (stacked
        experts, renamed modules).  Returns True when the tensor was consumed."""
        return False

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        owners = self.named_loadables()
        loaded: set[str] = set()
        for name, tensor in weights:
            if self._load_kv_scale(name, tensor):
                loaded.add(name)
                continue
            if self.load_special(name, tensor, owners):
                loaded.add(name)
                continue
            m = self.map_weight_name(name)
            if m is None:
                continue
            owner, pname, sid = m
            mod = owners.get(owner)
            if mod is None:
                continue        # another pipeline stage / unused tensor
            mod.load_weight(pname, tensor, sid)
            loaded.add(name)
        fin = getattr(self, "finish_loading", None)
        if fin is not None:
            fin()
        self.finalize_weights()
        return loaded

    def _load_kv_scale(self, name: str, tensor: torch.Tensor) -> bool:
        """Per-tensor scales of an 8-bit KV cache stored in the checkpoint
        (``...self_attn.k_scale`` / ``v_scale``, or one ``kv_scale`` for both; also under
        ``...self_attn.attn.``): value = stored * scale."""
        for suf in ("k_scale", "v_scale", "kv_scale"):
            for mid in (".self_attn.", ".self_attn.attn."):
                if name.endswith(mid + suf) and name.startswith("model.layers."):
                    layer = self.layers[name.split(".")[2]] if name.split(".")[2] in self.layers \
                        else None
                    attn = getattr(getattr(layer, "self_attn", None), "attn", None)
                    if attn is not None and hasattr(attn, "k_scale"):
                        v = float(tensor.float().reshape(-1)[0])
                        if suf in ("k_scale", "kv_scale"):
                            attn.k_scale = v
                        if suf in ("v_scale", "kv_scale"):
                            attn.v_scale = v
                        attn._scale_t = None
                    return True
        return False

    def load_kv_cache_scales(self, path: str) -> int:
        """Scales of an 8-bit KV cache from a quantisation-parameter file
        (``--quantization-param-path`` of the reference's launch lines, e.g.
        vllm_gcu/models/glm/glm.md ``int8_kv_cache.json``; schema of
        ``load_kv_cache_scales`` that vllm_gcu/models/deepseek_moe_quant/deepseek_moe_quant.py:
        487-489 calls): ``{"kv_cache": {"dtype": ..., "scaling_factor": {tp_rank: {layer: s}}}}``
        where ``s`` is one number for keys and values, a ``[k, v]`` pair or
        ``{"k_scale": .., "v_scale": ..}``.  Returns the number of layers that got scales."""
        import json
        from ..parallel.state import tp_rank as _tp_rank
        with open(path) as f:
            doc = json.load(f)
        table = (doc.get("kv_cache") or {}).get("scaling_factor") or {}
        per_layer = table.get(str(_tp_rank()), table.get("0", {}))
        n = 0
        for idx, val in per_layer.items():
            layer = self.layers[str(idx)] if str(idx) in self.layers else None
            attn = getattr(getattr(layer, "self_attn", None), "attn", None)
            if attn is None or not hasattr(attn, "k_scale"):
                continue
            if isinstance(val, dict):
                k, v = val.get("k_scale", val.get("k", 1.0)), val.get("v_scale", val.get("v", 1.0))
            elif isinstance(val, (list, tuple)):
                k, v = val[0], val[-1]
            else:
                k = v = val
            attn.k_scale, attn.v_scale, attn._scale_t = float(k), float(v), None
            n += 1
        return n

    def finalize_weights(self) -> None:
        for mod in self.modules():
            fin = getattr(mod, "finalize", None)
            if fin is not None and mod is not self:
                fin()

    @torch.no_grad()
    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        """Random initialisation N(0, std) of this rank's shards ("dummy" load format of
        the benchmarks); norm weights are one, biases zero."""
        gen_dev = self.device
        for name, p in sorted(self.named_parameters()):
            g = torch.Generator(device=gen_dev)
            g.manual_seed(zlib.crc32(name.encode()) ^ seed)
            if p.dtype == torch.float8_e4m3fn:       # fp8 experts: unit-variance codes ...
                chunk = torch.empty(p.shape, dtype=torch.float32, device=gen_dev)
                chunk.normal_(0.0, 1.0, generator=g)
                p.data.copy_(chunk.to(p.dtype))
                continue
            if name.endswith("_scale") and p.dtype == torch.float32:
                p.data.fill_(std)                    # ... times a block scale of std
                continue
            if p.dtype not in (torch.float32, torch.bfloat16, torch.float16):
                continue
            if name.endswith("norm.weight") or ".q_norm." in name or ".k_norm." in name \
                    or name.endswith("layernorm.weight") \
                    or (".ln_" in name and name.endswith(".weight")):
                p.data.fill_(1.0)
            elif name.endswith(".bias") or "e_score_correction_bias" in name:
                p.data.zero_()
            else:
                chunk = torch.empty(p.shape, dtype=torch.float32, device=gen_dev)
                chunk.normal_(0.0, std, generator=g)
                p.data.copy_(chunk)
        self.finalize_weights()
