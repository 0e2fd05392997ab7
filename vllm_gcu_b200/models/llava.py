"""LLaVA-1.5 and LLaVA-NeXT style models: CLIP vision transformer + two-layer MLP projector + a Llama language
model.  The reference lists LLaVA in its support matrix and serves it through vLLM's upstream
class (docs/source/user_guide/support_matrix/supported_models.md).

Vision side: patches of ``patch_size`` pixels plus a class token, learnt position embeddings,
``pre_layrnorm``, pre-norm blocks (LayerNorm, attention with biases, quick-GELU MLP).  The
features are the hidden states after layer ``vision_feature_layer`` (default: the second to
last), without the class token for the ``"default"`` selection strategy; the projector maps
them to the language model's width.  The prompt carries one placeholder token per feature row.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Iterable, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelConfig
from .llama import LlamaForCausalLM


@dataclass
class ClipVisionConfig:
    hidden_size: int = 1024
    intermediate_size: int = 4096
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    image_size: int = 336
    patch_size: int = 14
    hidden_act: str = "quick_gelu"
    layer_norm_eps: float = 1e-5

    @classmethod
    def from_hf_dict(cls, d: dict) -> "ClipVisionConfig":
        return cls(**{f: d[f] for f in cls.__dataclass_fields__ if f in d})


def _act(name: str, x: torch.Tensor) -> torch.Tensor:
    if name == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    if name in ("gelu_pytorch_tanh", "gelu_tanh", "gelu_new"):
        return F.gelu(x, approximate="tanh")
    return F.gelu(x)


class ClipEncoderLayer(nn.Module):
    def __init__(self, c: ClipVisionConfig, dtype, device):
        super().__init__()
        H = c.hidden_size
        kw = dict(dtype=dtype, device=device)
        self.layer_norm1 = nn.LayerNorm(H, eps=c.layer_norm_eps, **kw)
        self.layer_norm2 = nn.LayerNorm(H, eps=c.layer_norm_eps, **kw)
        self.self_attn = nn.ModuleDict({n: nn.Linear(H, H, **kw)
                                        for n in ("q_proj", "k_proj", "v_proj", "out_proj")})
        self.mlp = nn.ModuleDict({"fc1": nn.Linear(H, c.intermediate_size, **kw),
                                  "fc2": nn.Linear(c.intermediate_size, H, **kw)})
        self.heads, self.act = c.num_attention_heads, c.hidden_act

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, N, H = x.shape
        h = self.layer_norm1(x)
        q, k, v = (self.self_attn[n](h).view(B, N, self.heads, H // self.heads).transpose(1, 2)
                   for n in ("q_proj", "k_proj", "v_proj"))
        a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, N, H)
        x = x + self.self_attn["out_proj"](a)
        return x + self.mlp["fc2"](_act(self.act, self.mlp["fc1"](self.layer_norm2(x))))


class ClipVisionTower(nn.Module):
    """Parameter names follow the checkpoints below ``vision_model.``."""

    def __init__(self, c: ClipVisionConfig, feature_layer: int = -2, dtype=torch.bfloat16,
                 device="cpu"):
        super().__init__()
        self.cfg = c
        kw = dict(dtype=dtype, device=device)
        n = (c.image_size // c.patch_size) ** 2
        self.embeddings = nn.ModuleDict({
            "patch_embedding": nn.Conv2d(3, c.hidden_size, c.patch_size, c.patch_size,
                                         bias=False, **kw),
            "position_embedding": nn.Embedding(n + 1, c.hidden_size, **kw)})
        self.class_embedding = nn.Parameter(torch.zeros(c.hidden_size, **kw), requires_grad=False)
        self.pre_layrnorm = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps, **kw)
        # hidden_states[k] of the original model = output after k layers; a negative index
        # counts from the end of that list (length num_hidden_layers + 1)
        L = c.num_hidden_layers
        self.num_run = feature_layer if feature_layer >= 0 else L + 1 + feature_layer
        self.layers = nn.ModuleList([ClipEncoderLayer(c, dtype, device)
                                     for _ in range(self.num_run)])

    @torch.inference_mode()
    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """``[images, 3, S, S]`` -> ``[images, 1 + patches, hidden]`` (class token first)."""
        w = self.embeddings["patch_embedding"].weight
        x = self.embeddings["patch_embedding"](pixel_values.to(device=w.device, dtype=w.dtype))
        x = x.flatten(2).transpose(1, 2)
        cls = self.class_embedding.expand(x.shape[0], 1, -1)
        x = torch.cat([cls, x], dim=1) + self.embeddings["position_embedding"].weight[None]
        x = self.pre_layrnorm(x)
        for layer in self.layers:
            x = layer(x)
        return x

    def load_weight(self, name: str, t: torch.Tensor) -> bool:
        """``name`` below ``vision_model.``; layers past the feature layer and the final norm
        are not part of this model."""
        if name == "embeddings.class_embedding":
            self.class_embedding.data.copy_(t)
            return True
        if name.startswith("post_layernorm.") or name == "embeddings.position_ids":
            return True
        if name.startswith("encoder.layers."):
            idx = int(name.split(".")[2])
            if idx >= self.num_run:
                return True
            name = "layers." + name[len("encoder.layers."):]
        params = dict(self.named_parameters())
        if name in params:
            params[name].data.copy_(t.reshape(params[name].shape))
            return True
        return False


class LlavaForConditionalGeneration(LlamaForCausalLM):
    def __init__(self, cfg: ModelConfig, device="cpu"):
        super().__init__(cfg, device)
        vc = cfg.extra.get("vision_config") or {}
        self.vision_cfg = ClipVisionConfig.from_hf_dict(vc if isinstance(vc, dict) else {})
        self.image_token_id = int(cfg.extra.get("image_token_index",
                                                cfg.extra.get("image_token_id", 32000)))
        self.select = cfg.extra.get("vision_feature_select_strategy", "default")
        layer = cfg.extra.get("vision_feature_layer", -2)
        if not isinstance(layer, int):
            raise ValueError("a list of vision feature layers is not supported")
        act = cfg.extra.get("projector_hidden_act", "gelu")
        bias = bool(cfg.extra.get("multimodal_projector_bias", True))
        if self.is_first_stage:
            kw = dict(dtype=cfg.dtype, device=device)
            self.vision_tower = ClipVisionTower(self.vision_cfg, layer, cfg.dtype, device)
            self.projector = nn.ModuleDict({
                "linear_1": nn.Linear(self.vision_cfg.hidden_size, cfg.hidden_size, bias=bias, **kw),
                "linear_2": nn.Linear(cfg.hidden_size, cfg.hidden_size, bias=bias, **kw)})
            self.projector_act = act
        else:
            self.vision_tower = self.projector = None

    @property
    def tokens_per_image(self) -> int:
        n = (self.vision_cfg.image_size // self.vision_cfg.patch_size) ** 2
        return n if self.select == "default" else n + 1

    def encode_images(self, pixel_values: torch.Tensor) -> torch.Tensor:
        feats = self.vision_tower(pixel_values)
        if self.select == "default":
            feats = feats[:, 1:]
        with torch.inference_mode():
            h = self.projector["linear_2"](_act(self.projector_act,
                                                self.projector["linear_1"](feats)))
        return h.flatten(0, 1)

    def prepare_request(self, prompt_token_ids: Sequence[int], pixel_values: torch.Tensor,
                        image_grid_thw=None) -> dict:
        emb = self.encode_images(pixel_values)
        positions = [i for i, t in enumerate(prompt_token_ids) if t == self.image_token_id]
        assert len(positions) == emb.shape[0], \
            f"{len(positions)} placeholder tokens for {emb.shape[0]} image feature rows"
        salt = hash(pixel_values.detach().float().cpu().numpy().tobytes())
        return {"mm_embeds": emb, "mm_positions": positions, "cache_salt": salt}

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        lm, loaded = [], set()
        for name, t in weights:
            n = name[len("model."):] if name.startswith("model.") and not \
                name.startswith("model.layers.") and not name.startswith(
                    ("model.embed_tokens.", "model.norm.")) else name
            if n.startswith("vision_tower.vision_model."):
                if self.vision_tower is None or self.vision_tower.load_weight(
                        n[len("vision_tower.vision_model."):], t):
                    loaded.add(name)
                continue
            if n.startswith("multi_modal_projector."):
                if self.projector is not None:
                    sub = n[len("multi_modal_projector."):]
                    params = dict(self.projector.named_parameters())
                    if sub in params:
                        params[sub].data.copy_(t)
                        loaded.add(name)
                continue
            if n.startswith("language_model.model."):
                n = "model." + n[len("language_model.model."):]
            elif n.startswith("language_model.lm_head."):
                n = n[len("language_model."):]
            elif n.startswith("language_model."):
                n = "model." + n[len("language_model."):]
            lm.append((n, t))
        return loaded | super().load_weights(lm)


def anyres_grid(image_size: Sequence[int], pinpoints: Sequence[Sequence[int]], tile: int
                ) -> tuple[int, int]:
    """(tile rows, tile columns) of the high-resolution view of an image of ``(height, width)``
    pixels: the ``(height, width)`` candidate that keeps the most of the image's resolution,
    in tiles of ``tile`` pixels."""
    from .deepseek_vl2 import select_best_resolution
    h, w = int(image_size[0]), int(image_size[1])
    bw, bh = select_best_resolution((w, h), [(int(pw), int(ph)) for ph, pw in pinpoints])
    return bh // tile, bw // tile


def crop_to_aspect(grid: torch.Tensor, image_size: Sequence[int]) -> torch.Tensor:
    """``grid [rows, cols, C]`` covers an image of ``(height, width)`` pixels that was scaled to
    fit and centred; the rows (or columns) that only saw padding are cut off."""
    oh, ow = int(image_size[0]), int(image_size[1])
    rows, cols = grid.shape[0], grid.shape[1]
    if ow / oh > cols / rows:
        keep = int(round(oh * (cols / ow), 7))
        pad = (rows - keep) // 2
        return grid[pad:rows - pad]
    keep = int(round(ow * (rows / oh), 7))
    pad = (cols - keep) // 2
    return grid[:, pad:cols - pad]


class LlavaNextForConditionalGeneration(LlavaForConditionalGeneration):
    """LLaVA-NeXT (LLaVA-1.6): every image is seen as one down-scaled base view plus a grid of
    full-resolution tiles chosen from ``image_grid_pinpoints``.  The tile features are laid
    out as one 2-D map, rows or columns that only saw padding are dropped, a learnt
    ``image_newline`` row ends every row of the map, and the result follows the base view's
    features.  ``multi_modal_data``: ``pixel_values [views, 3, S, S]`` (base view first; a
    list of such tensors for several images) and ``image_sizes [[height, width], ...]``."""

    def __init__(self, cfg: ModelConfig, device="cpu"):
        super().__init__(cfg, device)
        self.pinpoints = [list(p) for p in cfg.extra.get(
            "image_grid_pinpoints", [[336, 672], [672, 336], [672, 672], [1008, 336], [336, 1008]])]
        if self.is_first_stage:
            self.image_newline = nn.Parameter(torch.zeros(cfg.hidden_size, dtype=cfg.dtype,
                                                          device=device), requires_grad=False)

    def num_image_tokens(self, image_size: Sequence[int], views: int) -> int:
        side = self.vision_cfg.image_size // self.vision_cfg.patch_size
        base = side * side + (0 if self.select == "default" else 1)
        if views == 1:
            return base + 1
        gh, gw = anyres_grid(image_size, self.pinpoints, self.vision_cfg.image_size)
        probe = torch.empty(gh * side, gw * side, 0)
        kept = crop_to_aspect(probe, image_size)
        return base + kept.shape[0] * (kept.shape[1] + 1)

    def pack_views(self, feats: torch.Tensor, image_size: Sequence[int]) -> torch.Tensor:
        """``feats [views, tokens, C]`` of one image -> ``[rows, C]`` in prompt order."""
        nl = self.image_newline.to(feats.dtype)
        if feats.shape[0] == 1:
            return torch.cat([feats[0], nl[None]], dim=0)
        side = self.vision_cfg.image_size // self.vision_cfg.patch_size
        gh, gw = anyres_grid(image_size, self.pinpoints, self.vision_cfg.image_size)
        C = feats.shape[-1]
        tiles = feats[1:]
        if tiles.shape[0] != gh * gw or tiles.shape[1] != side * side:
            raise ValueError(f"{tiles.shape[0]} tiles of {tiles.shape[1]} rows do not form a "
                             f"{gh} x {gw} grid of {side} x {side} patches")
        grid = tiles.reshape(gh, gw, side, side, C).permute(0, 2, 1, 3, 4) \
            .reshape(gh * side, gw * side, C)
        grid = crop_to_aspect(grid, image_size)
        grid = torch.cat([grid, nl.expand(grid.shape[0], 1, C)], dim=1)
        return torch.cat([feats[0], grid.reshape(-1, C)], dim=0)

    def encode_images(self, pixel_values, image_sizes=None) -> torch.Tensor:
        images = list(pixel_values) if isinstance(pixel_values, (list, tuple)) or \
            pixel_values.dim() == 5 else [pixel_values]
        if image_sizes is None:
            raise ValueError("LLaVA-NeXT needs image_sizes with its pixel_values")
        sizes = torch.as_tensor(image_sizes).reshape(-1, 2).tolist()
        out = []
        for views, size in zip(images, sizes):
            feats = self.vision_tower(views)
            if self.select == "default":
                feats = feats[:, 1:]
            with torch.inference_mode():
                h = self.projector["linear_2"](_act(self.projector_act,
                                                    self.projector["linear_1"](feats)))
                out.append(self.pack_views(h, size))
        return torch.cat(out, dim=0)

    def prepare_request(self, prompt_token_ids: Sequence[int], pixel_values,
                        image_grid_thw=None) -> dict:
        emb = self.encode_images(pixel_values, image_grid_thw)
        positions = [i for i, t in enumerate(prompt_token_ids) if t == self.image_token_id]
        assert len(positions) == emb.shape[0], \
            f"{len(positions)} placeholder tokens for {emb.shape[0]} image feature rows"
        first = pixel_values[0] if isinstance(pixel_values, (list, tuple)) else pixel_values
        salt = hash((first.detach().float().cpu().numpy().tobytes(),
                     tuple(torch.as_tensor(image_grid_thw).reshape(-1).tolist())))
        return {"mm_embeds": emb, "mm_positions": positions, "cache_salt": salt}

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        rest, loaded = [], set()
        for name, t in weights:
            if name in ("image_newline", "model.image_newline"):
                if self.is_first_stage:
                    self.image_newline.data.copy_(t)
                loaded.add(name)
            else:
                rest.append((name, t))
        return loaded | super().load_weights(rest)
