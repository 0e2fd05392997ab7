"""Typed configuration of the engine.

``ModelConfig`` is built from a HuggingFace-style ``config.json`` dict (or one of
the named architecture presets used by the benchmarks), the remaining classes
mirror the knobs the reference exposes through vLLM's ``EngineArgs`` and its
``additional_config`` dictionary (vllm_gcu/gcu.py:184-354).
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional

import torch

_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32,
           "bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32,
           "half": torch.float16, "float": torch.float32}


def to_dtype(x: Any) -> torch.dtype:
    if isinstance(x, torch.dtype):
        return x
    return _DTYPES[str(x).replace("torch.", "")]


@dataclass
class ModelConfig:
    architecture: str = "LlamaForCausalLM"
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    head_dim: int = 0                      # 0 -> hidden_size // num_attention_heads
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: Optional[dict] = None
    partial_rotary_factor: float = 1.0
    rope_is_neox: bool = True
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    mlp_bias: bool = False
    hidden_act: str = "silu"
    qk_norm: bool = False                  # per-head RMSNorm on q and k (Qwen3)
    sandwich_norm: bool = False            # GLM-4-0414: extra post-attn / post-mlp norms
    sliding_window: int = 0
    dtype: torch.dtype = torch.bfloat16
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    num_shared_experts: int = 0
    first_k_dense_replace: int = 0
    moe_layer_freq: int = 1
    norm_topk_prob: bool = True
    scoring_func: str = "softmax"
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    topk_method: str = "greedy"            # "noaux_tc" adds e_score_correction_bias
    # MLA
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # MTP
    num_nextn_predict_layers: int = 0
    # quantisation (HF quantization_config / quantize_config.json, see layers/quant)
    quantization: Optional[str] = None
    quant_config: Optional[dict] = None
    kv_cache_dtype: str = "auto"
    extra: dict = field(default_factory=dict)

    def __post_init__(self) -> None:
        self.dtype = to_dtype(self.dtype)
        if self.head_dim <= 0:
            self.head_dim = self.hidden_size // self.num_attention_heads

    # -- derived ---------------------------------------------------------
    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def rotary_dim(self) -> int:
        d = self.qk_rope_head_dim if self.is_mla else self.head_dim
        return int(d * self.partial_rotary_factor)

    def is_moe_layer(self, layer_idx: int) -> bool:
        if not self.is_moe or layer_idx < self.first_k_dense_replace \
                or layer_idx % self.moe_layer_freq != 0:
            return False
        # Qwen MoE configs: dense layers listed by index, experts on every n-th layer
        if layer_idx in (self.extra.get("mlp_only_layers") or ()):
            return False
        step = int(self.extra.get("decoder_sparse_step") or 1)
        return (layer_idx + 1) % step == 0

    def kv_bytes_per_token(self, tp_size: int = 1) -> int:
        es = 1 if self.kv_cache_dtype.startswith("fp8") or self.kv_cache_dtype == "int8" else \
            torch.empty((), dtype=self.dtype).element_size()
        if self.is_mla:
            return self.num_hidden_layers * (self.kv_lora_rank + self.qk_rope_head_dim) * es
        kvh = max(1, self.num_key_value_heads // tp_size)
        return self.num_hidden_layers * 2 * kvh * self.head_dim * es

    def window_for_layer(self, layer_idx: int) -> int:
        """Sliding-window length of one layer (0 = full attention).  Checkpoints name the
        layers that use the window by ``layer_types``, or by ``use_sliding_window`` with
        ``max_window_layers`` (Qwen2: the layers from that index on); a ``sliding_window`` value
        next to ``use_sliding_window: false`` is not in force."""
        w = int(self.sliding_window or 0)
        if w <= 0:
            return 0
        types = self.extra.get("layer_types")
        if isinstance(types, (list, tuple)) and layer_idx < len(types):
            return w if "sliding" in str(types[layer_idx]) else 0
        use = self.extra.get("use_sliding_window")
        if use is False:
            return 0
        if use is True and self.extra.get("max_window_layers") is not None:
            return w if layer_idx >= int(self.extra["max_window_layers"]) else 0
        return w

    @property
    def eos_token_ids(self) -> tuple[int, ...]:
        """End-of-sequence ids of the checkpoint (``eos_token_id`` of ``config.json``, an int or
        a list, plus those of ``generation_config.json``); empty for architecture presets."""
        out: list[int] = []
        for src in (self.extra.get("eos_token_id"), self.extra.get("generation_eos_token_id")):
            for t in (src if isinstance(src, (list, tuple)) else [src]):
                if isinstance(t, int) and t >= 0 and t not in out:
                    out.append(t)
        return tuple(out)

    @property
    def eos_token_id(self) -> Optional[int]:
        ids = self.eos_token_ids
        return ids[0] if ids else None

    # -- construction ----------------------------------------------------
    @classmethod
    def from_hf_dict(cls, d: dict, **overrides) -> "ModelConfig":
        archs = d.get("architectures") or ["LlamaForCausalLM"]
        for nested in ("text_config", "language_config", "llm_config"):
            if isinstance(d.get(nested), dict):
                # multimodal configs nest the language model's fields; vision_config, token
                # ids and everything else stay reachable through ``extra``
                inner_arch = (d[nested].get("architectures") or [None])[0]
                d = {**{k: v for k, v in d.items() if k != nested},
                     "llm_architecture": inner_arch, "llm_model_type": d[nested].get("model_type"),
                     **{k: v for k, v in d[nested].items()
                        if k not in ("architectures", "model_type")}}
        if archs[0] == "GPTBigCodeForCausalLM":
            # GPT-2 style field names; multi-query attention = one key / value head
            d = dict(d)
            heads = d["n_head"]
            d.setdefault("hidden_size", d["n_embd"])
            d.setdefault("num_hidden_layers", d["n_layer"])
            d.setdefault("num_attention_heads", heads)
            d.setdefault("num_key_value_heads", 1 if d.get("multi_query", True) else heads)
            d.setdefault("intermediate_size", d.get("n_inner") or 4 * d["n_embd"])
            d.setdefault("max_position_embeddings", d.get("n_positions", 8192))
            d.setdefault("rms_norm_eps", d.get("layer_norm_epsilon", 1e-5))
            d.setdefault("hidden_act", d.get("activation_function", "gelu_pytorch_tanh"))
            d.setdefault("head_dim", d["n_embd"] // heads)
            d["tie_word_embeddings"] = True
            d["attention_bias"] = True
        if archs[0] in ("ChatGLMModel", "ChatGLMForConditionalGeneration"):
            # ChatGLM2 / 3 / GLM-4-9B configs use their own field names
            d = dict(d)
            heads = d["num_attention_heads"]
            d.setdefault("num_hidden_layers", d.get("num_layers"))
            d.setdefault("intermediate_size", d.get("ffn_hidden_size"))
            d.setdefault("num_key_value_heads",
                         d.get("multi_query_group_num", heads) if d.get("multi_query_attention")
                         else heads)
            d.setdefault("head_dim", d.get("kv_channels", d["hidden_size"] // heads))
            d.setdefault("rms_norm_eps", d.get("layernorm_epsilon", 1e-5))
            d.setdefault("vocab_size", d.get("padded_vocab_size"))
            d.setdefault("max_position_embeddings", d.get("seq_length", 8192))
            d.setdefault("attention_bias", bool(d.get("add_qkv_bias", False)))
            d.setdefault("rope_theta", 10000.0 * float(d.get("rope_ratio", 1.0)))
            d.setdefault("tie_word_embeddings", False)
        names = {f.name for f in dataclasses.fields(cls)}
        kw: dict[str, Any] = {"architecture": archs[0]}
        alias = {"n_routed_experts": "num_experts", "num_local_experts": "num_experts",
                 "n_shared_experts": "num_shared_experts", "torch_dtype": "dtype"}
        extra = {}
        for k, v in d.items():
            k2 = alias.get(k, k)
            if k2 in names and v is not None:
                kw[k2] = v
            else:
                extra[k] = v
        arch = archs[0]
        if "Qwen3" in arch:
            kw.setdefault("qk_norm", True)
        if arch.startswith("Glm4"):
            kw.setdefault("sandwich_norm", True)
            kw.setdefault("rope_is_neox", False)
            kw.setdefault("partial_rotary_factor", d.get("partial_rotary_factor", 0.5))
        if "Deepseek" in arch:
            kw.setdefault("rope_is_neox", False)
        if arch in ("DeepseekV3ForCausalLM", "DeepSeekMTPModel") or \
                d.get("model_type") == "deepseek_v3":
            # configs written by newer libraries leave the V3 routing to the model type:
            # sigmoid scores, group-limited top-k with a learnt selection bias
            kw.setdefault("scoring_func", "sigmoid")
            kw.setdefault("topk_method", "noaux_tc")
        if arch.startswith("ChatGLM"):
            kw.setdefault("rope_is_neox", False)
            kw.setdefault("partial_rotary_factor", 0.5)
        if "rope_parameters" in d and isinstance(d["rope_parameters"], dict):
            rp = d["rope_parameters"]
            kw.setdefault("rope_theta", rp.get("rope_theta", kw.get("rope_theta", 10000.0)))
            if kw.get("rope_scaling") is None and (rp.get("mrope_section") or
                                                   rp.get("rope_type", "default") != "default"):
                kw["rope_scaling"] = rp
        qc = d.get("quantization_config")
        if qc:
            kw["quant_config"] = qc
            kw["quantization"] = qc.get("quant_method")
        kw["extra"] = extra
        kw.update(overrides)
        return cls(**kw)

    @classmethod
    def from_pretrained(cls, path: str, **overrides) -> "ModelConfig":
        p = Path(path)
        d = json.loads((p / "config.json").read_text())
        cfg = cls.from_hf_dict(d, **overrides)
        gpath = p / "generation_config.json"
        if gpath.exists():
            try:
                gen = json.loads(gpath.read_text())
                cfg.extra["generation_eos_token_id"] = gen.get("eos_token_id")
                # sampling defaults the checkpoint recommends; the server applies them to
                # requests that leave the field out
                cfg.extra["generation_defaults"] = {
                    k: gen[k] for k in ("temperature", "top_p", "top_k", "repetition_penalty")
                    if gen.get(k) is not None and gen.get("do_sample", True)}
            except (OSError, ValueError):
                pass
        qpath = p / "quantize_config.json"
        if cfg.quant_config is None and qpath.exists():
            cfg.quant_config = json.loads(qpath.read_text())
            cfg.quantization = cfg.quantization or cfg.quant_config.get("quant_method")
        return cfg


def preset(name: str, **overrides) -> ModelConfig:
    """Architecture presets of the benchmark configurations (random-init weights)."""
    presets: dict[str, dict] = {
        "tiny-llama": dict(vocab_size=32000, hidden_size=256, intermediate_size=688,
                           num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                           head_dim=64, rms_norm_eps=1e-6, rope_theta=10000.0,
                           max_position_embeddings=2048, dtype="float32"),
        "llama-3-8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                           num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                           head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0,
                           max_position_embeddings=8192, dtype="bfloat16"),
        "llama-3-70b": dict(vocab_size=128256, hidden_size=8192, intermediate_size=28672,
                            num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8,
                            head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0,
                            max_position_embeddings=8192, dtype="bfloat16"),
        "qwen3-30b-a3b": dict(architecture="Qwen3MoeForCausalLM", vocab_size=151936,
                              hidden_size=2048, intermediate_size=6144, num_hidden_layers=48,
                              num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                              qk_norm=True, num_experts=128, num_experts_per_tok=8,
                              moe_intermediate_size=768, norm_topk_prob=True,
                              rms_norm_eps=1e-6, rope_theta=1000000.0,
                              max_position_embeddings=40960, dtype="bfloat16"),
        "deepseek-v3": dict(architecture="DeepseekV3ForCausalLM", vocab_size=129280,
                            hidden_size=7168, intermediate_size=18432, num_hidden_layers=61,
                            num_attention_heads=128, num_key_value_heads=128,
                            q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
                            qk_rope_head_dim=64, v_head_dim=128, head_dim=192,
                            num_experts=256, num_experts_per_tok=8, moe_intermediate_size=2048,
                            num_shared_experts=1, first_k_dense_replace=3, n_group=8,
                            topk_group=4, scoring_func="sigmoid", topk_method="noaux_tc",
                            routed_scaling_factor=2.5, norm_topk_prob=True,
                            num_nextn_predict_layers=1, rope_is_neox=False,
                            rms_norm_eps=1e-6, rope_theta=10000.0,
                            max_position_embeddings=163840, dtype="bfloat16"),
        "tiny-qwen3-moe": dict(architecture="Qwen3MoeForCausalLM", vocab_size=1024,
                               hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                               num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                               qk_norm=True, num_experts=8, num_experts_per_tok=2,
                               moe_intermediate_size=64, dtype="float32"),
        "tiny-deepseek": dict(architecture="DeepseekV3ForCausalLM", vocab_size=1024,
                              hidden_size=128, intermediate_size=256, num_hidden_layers=3,
                              num_attention_heads=4, num_key_value_heads=4, q_lora_rank=48,
                              kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8,
                              v_head_dim=16, head_dim=24, num_experts=8, num_experts_per_tok=2,
                              moe_intermediate_size=32, num_shared_experts=1,
                              first_k_dense_replace=1, n_group=2, topk_group=1,
                              scoring_func="sigmoid", topk_method="noaux_tc",
                              routed_scaling_factor=2.5, num_nextn_predict_layers=1,
                              rope_is_neox=False, dtype="float32"),
    }
    kw = dict(presets[name])
    kw.update(overrides)
    return ModelConfig(**kw)


@dataclass
class CacheConfig:
    block_size: int = 16
    gpu_memory_utilization: float = 0.90
    num_gpu_blocks: Optional[int] = None   # override of the profiled value
    num_cpu_blocks: int = 0                # swap space
    enable_prefix_caching: bool = True
    cache_dtype: str = "auto"


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    max_model_len: int = 8192
    enable_chunked_prefill: bool = True
    policy: str = "fcfs"                   # or "priority"
    async_scheduling: bool = False
    num_scheduler_steps: int = 1           # multi-step decode (device-side advance)
    long_prefill_token_threshold: int = 0


@dataclass
class ParallelConfig:
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    enable_expert_parallel: bool = False
    enable_sequence_parallel: bool = False
    comm_backend: str = "fused"            # "fused" (symmetric-memory kernels) | "nccl"
    num_redundant_experts: int = 0
    enable_eplb: bool = False

    @property
    def world_size(self) -> int:
        return self.tensor_parallel_size * self.pipeline_parallel_size * self.data_parallel_size


@dataclass
class SpeculativeConfig:
    method: Optional[str] = None           # "ngram" | "mtp" | "draft_model"
    num_speculative_tokens: int = 0
    prompt_lookup_max: int = 4
    prompt_lookup_min: int = 1
    draft_model: Optional[str] = None


@dataclass
class EngineConfig:
    model: ModelConfig
    cache: CacheConfig = field(default_factory=CacheConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    speculative: SpeculativeConfig = field(default_factory=SpeculativeConfig)
    device: str = "auto"
    seed: int = 0
    enforce_eager: bool = False
    cuda_graph_sizes: Optional[list[int]] = None
    load_format: str = "dummy"             # "dummy" (random init) | "safetensors"
    model_path: Optional[str] = None
    quantization_param_path: Optional[str] = None   # JSON with the scales of an 8-bit KV cache
    additional_config: dict = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.device == "auto":
            self.device = "cuda" if torch.cuda.is_available() else "cpu"
        self.scheduler.max_model_len = min(self.scheduler.max_model_len,
                                           self.model.max_position_embeddings)
        if not self.scheduler.enable_chunked_prefill:
            self.scheduler.max_num_batched_tokens = max(self.scheduler.max_num_batched_tokens,
                                                        self.scheduler.max_model_len)
