"""Dense decoder families on the generic :class:`DecoderLM`.

``LlamaForCausalLM`` covers Llama 2/3/3.1, Mistral, Yi and InternLM2-style
checkpoints; ``Qwen2ForCausalLM`` adds q/k/v biases; ``Qwen3ForCausalLM`` adds
per-head QK RMSNorm (vllm_gcu/models/qwen3/qwen3.py:437); ``Glm4ForCausalLM`` is the
GLM-4-0414 variant with four norms per layer, GPT-J rotary on half of the head and a
fused ``gate_up_proj`` checkpoint tensor (vllm_gcu/models/glm4/glm4.py:82-231).
"""
from __future__ import annotations

import dataclasses

import torch

from ..config import ModelConfig
from .decoder import DecoderLM


class LlamaForCausalLM(DecoderLM):
    pass


class Qwen2ForCausalLM(DecoderLM):
    def __init__(self, cfg: ModelConfig, device="cpu"):
        if not cfg.attention_bias:
            cfg = dataclasses.replace(cfg, attention_bias=True)
        super().__init__(cfg, device)


class Qwen2EmbeddingModel(Qwen2ForCausalLM):
    """Qwen2 checkpoints published as embedding models (gte-Qwen2: listed in
    docs/source/user_guide/support_matrix/supported_models.md:22).  The mathematics is the
    Qwen2 decoder; the vector of a text is the final-norm hidden state of its last token
    (``LLMEngine.embed``).  Checkpoints saved from the bare ``Qwen2Model`` carry tensor names
    without the ``model.`` prefix and no LM head."""

    def load_weights(self, weights):
        def named():
            for name, t in weights:
                if not name.startswith(("model.", "lm_head.")):
                    name = "model." + name
                yield name, t
        return super().load_weights(named())


class Qwen3ForCausalLM(DecoderLM):
    def __init__(self, cfg: ModelConfig, device="cpu"):
        if not cfg.qk_norm:
            cfg = dataclasses.replace(cfg, qk_norm=True)
        super().__init__(cfg, device)


class Glm4ForCausalLM(DecoderLM):
    def __init__(self, cfg: ModelConfig, device="cpu"):
        cfg = dataclasses.replace(cfg, sandwich_norm=True, rope_is_neox=False,
                                  partial_rotary_factor=cfg.partial_rotary_factor
                                  if cfg.partial_rotary_factor < 1.0 else 0.5)
        super().__init__(cfg, device)


class InternLM2ForCausalLM(DecoderLM):
    """InternLM2 / 2.5 checkpoints: Llama mathematics under other tensor names, with q / k / v
    fused per KV group in ``attention.wqkv`` (rows ``[kv_head][q_0 .. q_{g-1}, k, v][head_dim]``).
    The reference lists InternLM2 in every precision column
    (docs/source/user_guide/support_matrix/supported_models.md:7-24)."""

    _RENAME = (("model.tok_embeddings.", "model.embed_tokens."), ("output.", "lm_head."),
               (".attention.wo.", ".self_attn.o_proj."), (".attention_norm.", ".input_layernorm."),
               (".ffn_norm.", ".post_attention_layernorm."), (".feed_forward.w1.", ".mlp.gate_proj."),
               (".feed_forward.w3.", ".mlp.up_proj."), (".feed_forward.w2.", ".mlp.down_proj."))

    def load_special(self, name, tensor, owners) -> bool:
        if ".attention.wqkv." in name:
            owner = name.split(".attention.wqkv.")[0] + ".self_attn.qkv_proj"
            mod = owners.get(owner)
            if mod is None:
                return True
            pname = name.rsplit(".", 1)[1]
            cfg = self.cfg
            kvh, g, d = cfg.num_key_value_heads, cfg.num_attention_heads // cfg.num_key_value_heads, \
                cfg.head_dim
            w = tensor.reshape(kvh, g + 2, d, *tensor.shape[1:])
            mod.load_weight(pname, w[:, :g].reshape(kvh * g * d, *tensor.shape[1:]), "q")
            mod.load_weight(pname, w[:, g].reshape(kvh * d, *tensor.shape[1:]), "k")
            mod.load_weight(pname, w[:, g + 1].reshape(kvh * d, *tensor.shape[1:]), "v")
            return True
        new = name
        for a, b in self._RENAME:
            if new.startswith(a) or (a.startswith(".") and a in new):
                new = new.replace(a, b, 1)
        if new == name:
            return False
        m = self.map_weight_name(new)
        if m is not None and m[0] in owners:
            owners[m[0]].load_weight(m[1], tensor, m[2])
        return True


class BaichuanForCausalLM(DecoderLM):
    """Baichuan / Baichuan2: q, k, v packed in ``W_pack``; Baichuan2 normalises the rows of the
    LM head (its ``NormHead``), which is done once at load.  The 7B models use rotary
    positions; the 13B models (architecture ``BaichuanForCausalLM`` with a hidden size other
    than 4096) use ALiBi position biases, which the attention kernels take as per-head slopes."""

    def __init__(self, cfg: ModelConfig, device="cpu"):
        if "position_embedding" not in cfg.extra:
            alibi = cfg.architecture == "BaichuanForCausalLM" and cfg.hidden_size != 4096
            cfg = dataclasses.replace(cfg, extra={**cfg.extra, "position_embedding":
                                                  "ALIBI" if alibi else "ROPE"})
        super().__init__(cfg, device)

    def load_special(self, name, tensor, owners) -> bool:
        if ".self_attn.W_pack." in name:
            owner = name.split(".self_attn.W_pack.")[0] + ".self_attn.qkv_proj"
            mod = owners.get(owner)
            if mod is not None:
                pname = name.rsplit(".", 1)[1]
                for part, sid in zip(tensor.chunk(3, dim=0), ("q", "k", "v")):
                    mod.load_weight(pname, part, sid)
            return True
        if name == "lm_head.weight" and self.cfg.vocab_size == 125696 and "lm_head" in owners:
            import torch.nn.functional as F
            owners["lm_head"].load_weight("weight", F.normalize(tensor.float()).to(tensor.dtype),
                                          None)
            return True
        return False


class GemmaForCausalLM(DecoderLM):
    """Gemma / CodeGemma: GeGLU MLP, RMSNorm with ``(1 + weight)``, embeddings scaled by
    ``sqrt(hidden_size)``, tied LM head.  The norm offset is folded into the weights at load."""

    def __init__(self, cfg: ModelConfig, device="cpu"):
        act = {"gelu": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh"}.get(cfg.hidden_act,
                                                                           cfg.hidden_act)
        cfg = dataclasses.replace(cfg, hidden_act=act, tie_word_embeddings=True)
        super().__init__(cfg, device)
        # rounded to the model dtype first, as the reference implementation multiplies by a
        # tensor of that dtype
        self.embed_scale = float(torch.tensor(float(cfg.hidden_size) ** 0.5, dtype=cfg.dtype))

    def load_special(self, name, tensor, owners) -> bool:
        if name.endswith("norm.weight"):
            m = self.map_weight_name(name)
            if m is not None and m[0] in owners:
                owners[m[0]].load_weight(m[1], (tensor.float() + 1.0).to(tensor.dtype), m[2])
            return True
        return name == "lm_head.weight"              # tied to the embedding


class ChatGLMForCausalLM(DecoderLM):
    """ChatGLM2 / ChatGLM3 / GLM-4-9B in their original checkpoint layout
    (``transformer.encoder.layers.N.self_attention.query_key_value`` ...): grouped-query
    attention with q / k / v biases fused in one tensor, interleaved (GPT-J) rotary embedding
    on the first half of every head, fused ``dense_h_to_4h`` = [gate | up] with SwiGLU."""

    _RENAME = ((".self_attention.dense.", ".self_attn.o_proj."),
               (".mlp.dense_4h_to_h.", ".mlp.down_proj."))

    def load_special(self, name, tensor, owners) -> bool:
        if not name.startswith("transformer."):
            return False
        if "rotary_pos_emb" in name:
            return True
        new = name[len("transformer."):]
        new = new.replace("encoder.layers.", "model.layers.")
        if new.startswith("embedding.word_embeddings."):
            new = "model.embed_tokens." + new.rsplit(".", 1)[1]
        elif new.startswith("encoder.final_layernorm."):
            new = "model.norm." + new.rsplit(".", 1)[1]
        elif new.startswith("output_layer."):
            new = "lm_head." + new.rsplit(".", 1)[1]
        pname = new.rsplit(".", 1)[1]
        cfg = self.cfg
        if ".self_attention.query_key_value." in new:
            mod = owners.get(new.split(".self_attention.")[0] + ".self_attn.qkv_proj")
            if mod is not None:
                nq = cfg.num_attention_heads * cfg.head_dim
                nkv = cfg.num_key_value_heads * cfg.head_dim
                for part, sid in zip(tensor.split([nq, nkv, nkv], dim=0), ("q", "k", "v")):
                    mod.load_weight(pname, part, sid)
            return True
        if ".mlp.dense_h_to_4h." in new:
            mod = owners.get(new.split(".mlp.")[0] + ".mlp.gate_up_proj")
            if mod is not None:
                for sid, part in enumerate(tensor.chunk(2, dim=0)):
                    mod.load_weight(pname, part, sid)
            return True
        for a, b in self._RENAME:
            new = new.replace(a, b)
        m = self.map_weight_name(new)
        if m is not None and m[0] in owners:
            owners[m[0]].load_weight(m[1], tensor, m[2])
        return True
