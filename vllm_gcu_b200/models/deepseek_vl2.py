"""DeepSeek-VL2: SigLIP vision transformer + down-sampling MLP projector + a DeepSeek language
model (MoE with plain multi-head attention for the "tiny" model, latent attention for the
larger ones).

The reference serves this family through the upstream class and only re-aliases one
mis-spelt parameter of it (vllm_gcu/models/deepseek_vl2/deepseek_vl2.py:11-20:
``view_seperator`` is the spelling of the checkpoints); here the whole model is built.

Image layout ("2D" tile tag): the processor cuts every image into one global view and
``num_w x num_h`` local tiles of ``image_size`` pixels.  Each view gives ``h x w`` projected
tokens; a learnt ``image_newline`` vector closes every row of the global view and of the
re-assembled local grid, and a learnt ``view_seperator`` vector sits between the two.  The
prompt carries one placeholder token per resulting row of the embedding matrix.
"""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass
from typing import Iterable, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelConfig


@dataclass
class SiglipConfig:
    image_size: int = 384
    patch_size: int = 14
    width: int = 1152
    layers: int = 27
    heads: int = 16
    mlp_ratio: float = 3.7362
    hidden_act: str = "gelu_tanh"
    eps: float = 1e-6

    @classmethod
    def from_hf_dict(cls, d: dict) -> "SiglipConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})


@dataclass
class ProjectorConfig:
    projector_type: str = "downsample_mlp_gelu"
    input_dim: int = 1152
    n_embed: int = 2048
    depth: int = 2
    mlp_ratio: int = 1
    downsample_ratio: int = 2

    @classmethod
    def from_hf_dict(cls, d: dict) -> "ProjectorConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})


class SiglipBlock(nn.Module):
    def __init__(self, c: SiglipConfig, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        hidden = int(c.width * c.mlp_ratio)
        self.heads = c.heads
        self.norm1 = nn.LayerNorm(c.width, eps=c.eps, **kw)
        self.attn = nn.ModuleDict({"qkv": nn.Linear(c.width, 3 * c.width, **kw),
                                   "proj": nn.Linear(c.width, c.width, **kw)})
        self.norm2 = nn.LayerNorm(c.width, eps=c.eps, **kw)
        self.mlp = nn.ModuleDict({"fc1": nn.Linear(c.width, hidden, **kw),
                                  "fc2": nn.Linear(hidden, c.width, **kw)})
        self.act_tanh = c.hidden_act in ("gelu_tanh", "gelu_pytorch_tanh")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, N, C = x.shape
        qkv = self.attn["qkv"](self.norm1(x)).view(B, N, 3, self.heads, C // self.heads)
        q, k, v = qkv.permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, N, C)
        x = x + self.attn["proj"](a)
        h = F.gelu(self.mlp["fc1"](self.norm2(x)), approximate="tanh" if self.act_tanh else "none")
        return x + self.mlp["fc2"](h)


class SiglipVisionTransformer(nn.Module):
    """Pre-norm ViT without a class token; parameter names follow the checkpoints
    (``patch_embed.proj``, ``pos_embed``, ``blocks.N.*``, ``norm``).  The attention-pooling
    head of the original encoder is not used by the language model and is not built."""

    def __init__(self, c: SiglipConfig, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.cfg = c
        kw = dict(dtype=dtype, device=device)
        self.grid = c.image_size // c.patch_size
        self.patch_embed = nn.ModuleDict({"proj": nn.Conv2d(3, c.width, c.patch_size,
                                                            c.patch_size, **kw)})
        self.pos_embed = nn.Parameter(torch.zeros(1, self.grid * self.grid, c.width, **kw),
                                      requires_grad=False)
        self.blocks = nn.ModuleList([SiglipBlock(c, dtype, device) for _ in range(c.layers)])
        self.norm = nn.LayerNorm(c.width, eps=c.eps, **kw)

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """``pixels [tiles, 3, S, S]`` -> ``[tiles, (S / patch)^2, width]``."""
        x = self.patch_embed["proj"](pixels.to(self.pos_embed.dtype)).flatten(2).transpose(1, 2)
        x = x + self.pos_embed
        for blk in self.blocks:
            x = blk(x)
        return self.norm(x)


class MlpProjector(nn.Module):
    """``downsample_mlp_gelu``: ``r x r`` neighbouring vision tokens are concatenated
    (zero padding on the right / bottom edge when the grid is not a multiple of r), then an MLP
    maps them to the language model's width.  ``layers.{0, 2, ...}`` are the linear layers."""

    def __init__(self, c: ProjectorConfig, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        if c.projector_type != "downsample_mlp_gelu":
            raise ValueError(f"projector type {c.projector_type!r} is not supported")
        self.cfg = c
        kw = dict(dtype=dtype, device=device)
        r = c.downsample_ratio
        mods: list[nn.Module] = [nn.Linear(c.input_dim * r * r, c.n_embed * c.mlp_ratio, **kw)]
        for _ in range(1, c.depth - 1):
            mods += [nn.GELU(), nn.Linear(c.n_embed * c.mlp_ratio, c.n_embed * c.mlp_ratio, **kw)]
        mods += [nn.GELU(), nn.Linear(c.n_embed * c.mlp_ratio, c.n_embed, **kw)]
        self.layers = nn.Sequential(*mods)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, hw, C = x.shape
        h = w = int(math.isqrt(hw))
        r = self.cfg.downsample_ratio
        pad = (r - h % r) % r
        x = x.reshape(B, h, w, C)
        if pad:
            x = F.pad(x, (0, 0, 0, pad, 0, pad))
        H2, W2 = (h + pad) // r, (w + pad) // r
        # channel-major order inside a window, as an unfold over [B, C, H, W] gives it
        x = x.view(B, H2, r, W2, r, C).permute(0, 1, 3, 5, 2, 4).reshape(B, H2 * W2, C * r * r)
        return self.layers(x)


def tile_embeddings(feats: torch.Tensor, crops: Sequence[Sequence[int]], newline: torch.Tensor,
                    separator: torch.Tensor, global_first: bool = True) -> torch.Tensor:
    """Rows of the placeholder embeddings for all images of a request.  ``feats [tiles, h*w, D]``
    holds, per image, the global view followed by its ``num_w * num_h`` local tiles (row-major);
    ``crops[i] = (num_w, num_h)``."""
    _, hw, D = feats.shape
    h = w = int(math.isqrt(hw))
    out, t = [], 0
    for num_w, num_h in crops:
        num_w, num_h = int(num_w), int(num_h)
        n = num_w * num_h
        g = feats[t].view(h, w, D)
        g = torch.cat([g, newline.expand(h, 1, D)], dim=1).reshape(-1, D)
        parts = [g, separator[None, :]]
        if n > 0:
            loc = feats[t + 1:t + 1 + n].view(num_h, num_w, h, w, D).permute(0, 2, 1, 3, 4) \
                .reshape(num_h * h, num_w * w, D)
            loc = torch.cat([loc, newline.expand(num_h * h, 1, D)], dim=1).reshape(-1, D)
            parts = [g, separator[None, :], loc] if global_first else \
                [loc, separator[None, :], g]
        out.append(torch.cat(parts, dim=0))
        t += n + 1
    return torch.cat(out, dim=0)


def select_best_resolution(image_size: Sequence[int], candidates: Sequence[Sequence[int]]
                           ) -> tuple[int, int]:
    """The candidate ``(width, height)`` that keeps the most of the image's resolution when the
    image is scaled to fit inside it, ties broken by the least unused area (the rule of the
    DeepSeek-VL2 processor)."""
    ow, oh = int(image_size[0]), int(image_size[1])
    best, best_fit, min_waste = None, -1, float("inf")
    for w, h in candidates:
        scale = min(w / ow, h / oh)
        dw, dh = int(ow * scale), int(oh * scale)
        eff = min(dw * dh, ow * oh)
        waste = w * h - eff
        if eff > best_fit or (eff == best_fit and waste < min_waste):
            best, best_fit, min_waste = (int(w), int(h)), eff, waste
    return best


def _fit_and_pad(img: torch.Tensor, width: int, height: int, fill: float) -> torch.Tensor:
    """``img [3, H, W]`` scaled (aspect ratio kept, bicubic) to fit ``width x height`` and
    centred on a canvas of that size filled with ``fill``."""
    _, h, w = img.shape
    scale = min(width / w, height / h)
    nw, nh = max(1, min(width, round(w * scale))), max(1, min(height, round(h * scale)))
    r = F.interpolate(img[None], size=(nh, nw), mode="bicubic", align_corners=False,
                      antialias=True)[0].clamp(0.0, 1.0)
    out = torch.full((3, height, width), fill, dtype=img.dtype)
    y0, x0 = (height - nh) // 2, (width - nw) // 2
    out[:, y0:y0 + nh, x0:x0 + nw] = r
    return out


def process_images(images: Sequence[torch.Tensor], candidate_resolutions: Sequence[Sequence[int]],
                   image_size: int = 384, mean: float = 0.5, std: float = 0.5):
    """Tiles images the way the model expects them: per image one global view (the whole image
    fitted into ``image_size x image_size``) followed by the local tiles of the image fitted
    into the best candidate resolution, row by row.  ``images``: float ``[3, H, W]`` in
    [0, 1].  Returns ``(pixel_values [tiles, 3, S, S]`` normalised with ``mean`` / ``std``,
    ``images_spatial_crop [(num_w, num_h), ...])``."""
    tiles, crops = [], []
    S = int(image_size)
    for img in images:
        img = img.float()
        bw, bh = select_best_resolution((img.shape[2], img.shape[1]), candidate_resolutions)
        tiles.append(_fit_and_pad(img, S, S, mean))
        local = _fit_and_pad(img, bw, bh, mean)
        for y in range(0, bh, S):
            for x in range(0, bw, S):
                tiles.append(local[:, y:y + S, x:x + S])
        crops.append((bw // S, bh // S))
    px = (torch.stack(tiles) - mean) / std
    return px, crops


class _VL2Mixin:
    """Vision side of DeepSeek-VL2 on top of one of the DeepSeek language models."""

    def _init_vision(self, cfg: ModelConfig, device) -> None:
        vc, pc = cfg.extra.get("vision_config") or {}, cfg.extra.get("projector_config") or {}
        self.vision_cfg = SiglipConfig.from_hf_dict(vc)
        self.projector_cfg = ProjectorConfig.from_hf_dict(pc)
        if not pc:
            self.projector_cfg = dataclasses.replace(self.projector_cfg,
                                                     input_dim=self.vision_cfg.width,
                                                     n_embed=cfg.hidden_size)
        if self.projector_cfg.n_embed != cfg.hidden_size:
            raise ValueError("projector_config.n_embed must equal the language model's width")
        self.tile_tag = cfg.extra.get("tile_tag", "2D")
        if self.tile_tag != "2D":
            raise ValueError(f"tile tag {self.tile_tag!r} is not supported")
        self.global_first = cfg.extra.get("global_view_pos", "head") == "head"
        self.image_token_id = int(cfg.extra.get("image_token_id",
                                                cfg.extra.get("image_token_index", 128815)))
        if self.is_first_stage:
            self.vision = SiglipVisionTransformer(self.vision_cfg, cfg.dtype, device)
            self.projector = MlpProjector(self.projector_cfg, cfg.dtype, device)
            std = 1.0 / math.sqrt(cfg.hidden_size)
            kw = dict(dtype=cfg.dtype, device=device)
            self.image_newline = nn.Parameter(torch.randn(cfg.hidden_size, **kw) * std,
                                              requires_grad=False)
            self.view_seperator = nn.Parameter(torch.randn(cfg.hidden_size, **kw) * std,
                                               requires_grad=False)
        else:
            self.vision = self.projector = None

    def num_image_tokens(self, crop: Sequence[int]) -> int:
        """Placeholder tokens one image takes for ``crop = (num_w, num_h)`` local tiles."""
        r = self.projector_cfg.downsample_ratio
        g = self.vision_cfg.image_size // self.vision_cfg.patch_size
        h = (g + r - 1) // r
        num_w, num_h = int(crop[0]), int(crop[1])
        local = (num_h * h) * (num_w * h + 1) if num_w * num_h > 0 else 0
        return h * (h + 1) + 1 + local

    def prepare_images(self, images: Sequence[torch.Tensor], prompt_token_ids: Sequence[int]):
        """From raw images to engine inputs: tiles the images and expands every single image
        placeholder of the prompt to as many placeholders as that image has embedding rows.
        Returns ``(prompt_token_ids, multi_modal_data)`` for ``LLM.generate``."""
        cands = self.cfg.extra.get("candidate_resolutions") or [[self.vision_cfg.image_size] * 2]
        px, crops = process_images(images, cands, self.vision_cfg.image_size)
        out, k = [], 0
        for t in prompt_token_ids:
            if t == self.image_token_id and k < len(crops):
                out.extend([self.image_token_id] * self.num_image_tokens(crops[k]))
                k += 1
            else:
                out.append(int(t))
        assert k == len(crops), "one image placeholder per image is expected in the prompt"
        return out, {"pixel_values": px, "images_spatial_crop": crops}

    def encode_images(self, pixel_values: torch.Tensor, images_spatial_crop) -> torch.Tensor:
        feats = self.projector(self.vision(pixel_values))
        return tile_embeddings(feats, images_spatial_crop, self.image_newline,
                               self.view_seperator, self.global_first)

    def prepare_request(self, prompt_token_ids: Sequence[int], pixel_values: torch.Tensor,
                        images_spatial_crop) -> dict:
        crops = [tuple(int(v) for v in c) for c in images_spatial_crop]
        with torch.inference_mode():
            emb = self.encode_images(pixel_values, crops)
        positions = [i for i, t in enumerate(prompt_token_ids) if t == self.image_token_id]
        assert len(positions) == emb.shape[0], \
            f"{len(positions)} placeholder tokens for {emb.shape[0]} image embedding rows"
        salt = hash(pixel_values.detach().float().cpu().numpy().tobytes())
        return {"mm_embeds": emb, "mm_positions": positions, "cache_salt": salt}

    def _load_vision_weight(self, name: str, t: torch.Tensor) -> bool:
        if self.vision is None:
            return True
        if name in ("image_newline", "view_seperator", "view_separator"):
            getattr(self, "image_newline" if name == "image_newline" else "view_seperator") \
                .data.copy_(t)
            return True
        for pre, mod in (("vision.", self.vision), ("projector.", self.projector)):
            if name.startswith(pre):
                sub = name[len(pre):]
                if sub.startswith("attn_pool."):
                    return True                      # pooling head: not part of this model
                params = dict(mod.named_parameters())
                if sub not in params:
                    return False
                params[sub].data.copy_(t.reshape(params[sub].shape))
                return True
        return False

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        lm, loaded = [], set()
        for name, t in weights:
            if name.startswith(("vision.", "projector.")) or name in (
                    "image_newline", "view_seperator", "view_separator"):
                if self._load_vision_weight(name, t):
                    loaded.add(name)
                continue
            n = name[len("language."):] if name.startswith("language.") else name
            lm.append((n, t))
        return loaded | super().load_weights(lm)


_CLASSES: dict = {}


def DeepseekVLV2ForCausalLM(cfg: ModelConfig, device="cpu"):
    """Builds the model on the language model its ``language_config`` names: latent attention
    (``kv_lora_rank`` set) gives the DeepSeek-V2 / V3 class, otherwise the DeepSeek-MoE class
    with plain attention (the "tiny" checkpoints)."""
    if cfg.is_mla:
        from .deepseek import DeepseekV3ForCausalLM as base
    else:
        from .moe_models import DeepseekMoeForCausalLM as base
    cls = _CLASSES.get(base)
    if cls is None:
        def __init__(self, cfg_, device_="cpu"):
            base.__init__(self, cfg_, device_)
            self._init_vision(cfg_, device_)
        cls = _CLASSES[base] = type("DeepseekVLV2ForCausalLM", (_VL2Mixin, base),
                                    {"__init__": __init__, "__doc__": __doc__})
    return cls(cfg, device)
