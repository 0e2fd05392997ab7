"""InternVL2 / InternVL2.5: InternViT vision transformer + pixel-shuffle down-sampling + MLP
projector in front of an InternLM2, Qwen2 or Llama language model.  The reference lists both
generations in its multimodal table and serves them through vLLM's upstream class
(docs/source/user_guide/support_matrix/supported_models.md:32-33).

Vision side: patches + class token with learnt positions; pre-norm blocks (LayerNorm or RMSNorm
by ``norm_type``) whose attention and MLP outputs are scaled per channel (``ls1`` / ``ls2``)
before the residual add; the 6B tower also RMS-normalises q and k over the full width.  The
patch rows of the selected layer form an ``s x s`` map; each 2 x 2 neighbourhood is folded into
the channel axis (``downsample_ratio`` 0.5), then LayerNorm -> Linear -> GELU -> Linear maps to
the language model's width.  Every 448-pixel tile therefore gives 256 rows.

Two checkpoint layouts load: the original one (``vision_model.`` with fused ``attn.qkv``,
``mlp1.{0,1,3}``, ``language_model.``) and the transformers one (``model.vision_tower.`` with
separate projections, ``model.multi_modal_projector.``, ``model.language_model.``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Iterable, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelConfig


@dataclass
class InternViTConfig:
    hidden_size: int = 1024
    intermediate_size: int = 4096
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    image_size: int = 448
    patch_size: int = 14
    norm_type: str = "layer_norm"
    layer_norm_eps: float = 1e-6
    qkv_bias: bool = True
    qk_normalization: bool = False
    hidden_act: str = "gelu"

    @classmethod
    def from_hf_dict(cls, d: dict) -> "InternViTConfig":
        d = dict(d)
        if "attention_bias" in d:                 # field names of the transformers layout
            d.setdefault("qkv_bias", d["attention_bias"])
        if "use_qk_norm" in d:
            d.setdefault("qk_normalization", d["use_qk_norm"])
        for k in ("image_size", "patch_size"):
            if isinstance(d.get(k), (list, tuple)):
                d[k] = int(d[k][0])
        return cls(**{f: d[f] for f in cls.__dataclass_fields__ if f in d})


class _RMS(nn.Module):
    def __init__(self, n: int, eps: float, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(n, dtype=dtype, device=device), requires_grad=False)
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        f = x.float()
        f = f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + self.eps)
        return self.weight * f.to(x.dtype)


def _norm(c: InternViTConfig, dtype, device) -> nn.Module:
    if c.norm_type == "rms_norm":
        return _RMS(c.hidden_size, c.layer_norm_eps, dtype, device)
    return nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps, dtype=dtype, device=device)


class InternViTBlock(nn.Module):
    def __init__(self, c: InternViTConfig, dtype, device):
        super().__init__()
        H, kw = c.hidden_size, dict(dtype=dtype, device=device)
        self.norm1, self.norm2 = _norm(c, dtype, device), _norm(c, dtype, device)
        self.q, self.k, self.v = (nn.Linear(H, H, bias=c.qkv_bias, **kw) for _ in range(3))
        self.proj = nn.Linear(H, H, **kw)
        if c.qk_normalization:
            self.q_norm = _RMS(H, c.layer_norm_eps, dtype, device)
            self.k_norm = _RMS(H, c.layer_norm_eps, dtype, device)
        else:
            self.q_norm = self.k_norm = None
        self.fc1 = nn.Linear(H, c.intermediate_size, **kw)
        self.fc2 = nn.Linear(c.intermediate_size, H, **kw)
        self.ls1 = nn.Parameter(torch.ones(H, **kw), requires_grad=False)
        self.ls2 = nn.Parameter(torch.ones(H, **kw), requires_grad=False)
        self.heads = c.num_attention_heads
        self.act = c.hidden_act

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, N, H = x.shape
        h = self.norm1(x)
        q, k, v = self.q(h), self.k(h), self.v(h)
        if self.q_norm is not None:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k, v = (t.view(B, N, self.heads, H // self.heads).transpose(1, 2) for t in (q, k, v))
        a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, N, H)
        x = x + self.ls1 * self.proj(a)
        h = self.fc1(self.norm2(x))
        h = F.gelu(h) if self.act == "gelu" else F.gelu(h, approximate="tanh")
        return x + self.ls2 * self.fc2(h)


class InternViT(nn.Module):
    def __init__(self, c: InternViTConfig, select_layer: int = -1, dtype=torch.bfloat16,
                 device="cpu"):
        super().__init__()
        self.cfg = c
        kw = dict(dtype=dtype, device=device)
        n = (c.image_size // c.patch_size) ** 2
        self.patch_embedding = nn.Conv2d(3, c.hidden_size, c.patch_size, c.patch_size, **kw)
        self.class_embedding = nn.Parameter(torch.zeros(1, 1, c.hidden_size, **kw),
                                            requires_grad=False)
        self.position_embedding = nn.Parameter(torch.zeros(1, n + 1, c.hidden_size, **kw),
                                               requires_grad=False)
        L = c.num_hidden_layers
        # index into the list [embeddings, after layer 1, ..., after layer L]
        self.num_run = select_layer if select_layer >= 0 else L + 1 + select_layer
        self.layers = nn.ModuleList([InternViTBlock(c, dtype, device)
                                     for _ in range(self.num_run)])

    @torch.inference_mode()
    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """``[tiles, 3, S, S]`` -> ``[tiles, 1 + patches, hidden]``."""
        w = self.patch_embedding.weight
        x = self.patch_embedding(pixel_values.to(device=w.device, dtype=w.dtype))
        x = x.flatten(2).transpose(1, 2)
        x = torch.cat([self.class_embedding.expand(x.shape[0], 1, -1), x], dim=1)
        x = x + self.position_embedding
        for blk in self.layers:
            x = blk(x)
        return x

    # checkpoint tensor (below ``vision_model.`` / ``vision_tower.``) -> parameter of this module
    _HF_ATTN = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "projection_layer": "proj",
                "q_norm": "q_norm", "k_norm": "k_norm"}

    def load_weight(self, name: str, t: torch.Tensor) -> bool:
        params = dict(self.named_parameters())

        def put(pname: str, value: torch.Tensor) -> bool:
            if pname not in params:
                return False
            params[pname].data.copy_(value.reshape(params[pname].shape))
            return True

        top = {"embeddings.class_embedding": "class_embedding",
               "embeddings.cls_token": "class_embedding",
               "embeddings.position_embedding": "position_embedding",
               "embeddings.position_embeddings": "position_embedding",
               "embeddings.patch_embedding.weight": "patch_embedding.weight",
               "embeddings.patch_embedding.bias": "patch_embedding.bias",
               "embeddings.patch_embeddings.projection.weight": "patch_embedding.weight",
               "embeddings.patch_embeddings.projection.bias": "patch_embedding.bias"}
        if name in top:
            return put(top[name], t)
        for prefix in ("encoder.layers.", "encoder.layer."):
            if name.startswith(prefix):
                idx, _, rest = name[len(prefix):].partition(".")
                if int(idx) >= self.num_run:
                    return True               # past the selected layer: not part of this model
                base = f"layers.{idx}."
                if rest.startswith("attn.qkv."):
                    kind = rest.rsplit(".", 1)[1]
                    parts = t.chunk(3, dim=0)
                    return all(put(f"{base}{n}.{kind}", p) for n, p in zip("qkv", parts))
                rest = rest.replace("attn.proj.", "proj.").replace("attn.q_norm.", "q_norm.") \
                    .replace("attn.k_norm.", "k_norm.").replace("mlp.fc", "fc")
                if rest.startswith("attention."):
                    _, mod, kind = rest.split(".", 2)
                    rest = f"{self._HF_ATTN.get(mod, mod)}.{kind}"
                rest = {"layernorm_before.weight": "norm1.weight",
                        "layernorm_before.bias": "norm1.bias",
                        "layernorm_after.weight": "norm2.weight",
                        "layernorm_after.bias": "norm2.bias",
                        "lambda_1": "ls1", "lambda_2": "ls2"}.get(rest, rest)
                return put(base + rest, t)
        return False


def fold_neighbourhoods(x: torch.Tensor, r: int, transposed: bool = True) -> torch.Tensor:
    """``x [B, s, s, C]`` -> ``[B, s/r, s/r, r*r*C]``: the channels of every ``r x r`` block of
    positions side by side (first-axis offset major).  ``transposed=False`` gives the layout of
    the first InternVL release (``ps_version`` v1), whose output map has its axes swapped."""
    B, s0, s1, C = x.shape
    y = x.reshape(B, s0 // r, r, s1 // r, r, C).permute(0, 1, 3, 2, 4, 5) \
        .reshape(B, s0 // r, s1 // r, r * r * C)
    return y if transposed else y.transpose(1, 2)


def tile_grid(width: int, height: int, min_tiles: int, max_tiles: int, tile: int = 448
              ) -> tuple[int, int]:
    """(columns, rows) of the tile grid for an image: among all grids with between
    ``min_tiles`` and ``max_tiles`` tiles (smaller grids first), the one whose aspect ratio is
    closest to the image's; a later grid of the same distance replaces the choice when the
    image has more than half of that grid's pixels."""
    grids = sorted({(i, j) for i in range(1, max_tiles + 1) for j in range(1, max_tiles + 1)
                    if min_tiles <= i * j <= max_tiles}, key=lambda p: p[0] * p[1])
    aspect, best, best_diff = width / height, (1, 1), float("inf")
    for i, j in grids:
        diff = abs(aspect - i / j)
        if diff < best_diff:
            best, best_diff = (i, j), diff
        elif diff == best_diff and width * height > 0.5 * tile * tile * i * j:
            best = (i, j)
    return best


def dynamic_tiles(img: torch.Tensor, tile: int = 448, min_tiles: int = 1, max_tiles: int = 12,
                  thumbnail: bool = True) -> torch.Tensor:
    """``img [3, H, W]`` in [0, 1] -> ``[tiles, 3, tile, tile]``: the image stretched onto its
    tile grid and cut row by row, followed by a whole-image thumbnail when there is more than
    one tile."""
    _, h, w = img.shape
    cols, rows = tile_grid(w, h, min_tiles, max_tiles, tile)
    big = F.interpolate(img[None], size=(rows * tile, cols * tile), mode="bicubic",
                        align_corners=False, antialias=True)[0].clamp(0.0, 1.0)
    out = [big[:, r * tile:(r + 1) * tile, c * tile:(c + 1) * tile]
           for r in range(rows) for c in range(cols)]
    if thumbnail and len(out) > 1:
        out.append(F.interpolate(img[None], size=(tile, tile), mode="bicubic",
                                 align_corners=False, antialias=True)[0].clamp(0.0, 1.0))
    return torch.stack(out)


_MEAN = torch.tensor([0.485, 0.456, 0.406]).view(1, 3, 1, 1)
_STD = torch.tensor([0.229, 0.224, 0.225]).view(1, 3, 1, 1)


class _InternVLMixin:
    def _init_vision(self, cfg: ModelConfig, device) -> None:
        vc = cfg.extra.get("vision_config") or {}
        self.vision_cfg = InternViTConfig.from_hf_dict(vc if isinstance(vc, dict) else {})
        self.downsample = int(round(1.0 / float(cfg.extra.get("downsample_ratio", 0.5))))
        self.ps_v2 = cfg.extra.get("ps_version", "v2") != "v1"
        layer = cfg.extra.get("select_layer", cfg.extra.get("vision_feature_layer", -1))
        self.image_token_id = int(cfg.extra.get("img_context_token_id",
                                                cfg.extra.get("image_token_id", 151667)))
        if self.is_first_stage:
            kw = dict(dtype=cfg.dtype, device=device)
            self.vision_model = InternViT(self.vision_cfg, int(layer), cfg.dtype, device)
            width = self.vision_cfg.hidden_size * self.downsample ** 2
            self.mlp1 = nn.ModuleDict({"norm": nn.LayerNorm(width, **kw),
                                       "fc1": nn.Linear(width, cfg.hidden_size, **kw),
                                       "fc2": nn.Linear(cfg.hidden_size, cfg.hidden_size, **kw)})
        else:
            self.vision_model = self.mlp1 = None

    @property
    def tokens_per_tile(self) -> int:
        s = self.vision_cfg.image_size // self.vision_cfg.patch_size
        return (s // self.downsample) ** 2

    def encode_images(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """``[tiles, 3, S, S]`` -> ``[tiles * tokens_per_tile, hidden]``."""
        feats = self.vision_model(pixel_values)[:, 1:]
        B, n, C = feats.shape
        s = int(math.isqrt(n))
        with torch.inference_mode():
            x = fold_neighbourhoods(feats.reshape(B, s, s, C), self.downsample, self.ps_v2)
            x = x.reshape(B, -1, x.shape[-1])
            x = self.mlp1["fc2"](F.gelu(self.mlp1["fc1"](self.mlp1["norm"](x))))
        return x.flatten(0, 1)

    def prepare_images(self, images: Sequence[torch.Tensor], prompt_token_ids: Sequence[int]):
        """Raw images (``[3, H, W]`` in [0, 1]) -> tiles, and one placeholder of the prompt per
        image expanded to that image's row count.  Returns ``(prompt_token_ids,
        multi_modal_data)`` for ``LLM.generate``."""
        ex = self.cfg.extra
        tile = self.vision_cfg.image_size
        dyn = bool(ex.get("dynamic_image_size", True))
        tiles = [((dynamic_tiles(im.float(), tile, int(ex.get("min_dynamic_patch", 1)),
                                 int(ex.get("max_dynamic_patch", 12)),
                                 bool(ex.get("use_thumbnail", True))) if dyn else
                   F.interpolate(im.float()[None], size=(tile, tile), mode="bicubic",
                                 align_corners=False, antialias=True).clamp(0.0, 1.0))
                  - _MEAN) / _STD for im in images]
        out, k = [], 0
        for t in prompt_token_ids:
            if t == self.image_token_id and k < len(tiles):
                out.extend([self.image_token_id] * (tiles[k].shape[0] * self.tokens_per_tile))
                k += 1
            else:
                out.append(int(t))
        assert k == len(tiles), "one image placeholder per image is expected in the prompt"
        return out, {"pixel_values": torch.cat(tiles, dim=0)}

    def prepare_request(self, prompt_token_ids: Sequence[int], pixel_values: torch.Tensor,
                        image_grid_thw=None) -> dict:
        emb = self.encode_images(pixel_values)
        positions = [i for i, t in enumerate(prompt_token_ids) if t == self.image_token_id]
        assert len(positions) == emb.shape[0], \
            f"{len(positions)} placeholder tokens for {emb.shape[0]} image feature rows"
        salt = hash(pixel_values.detach().float().cpu().numpy().tobytes())
        return {"mm_embeds": emb, "mm_positions": positions, "cache_salt": salt}

    _PROJ = {"0.": "norm.", "1.": "fc1.", "3.": "fc2.", "layer_norm.": "norm.",
             "linear_1.": "fc1.", "linear_2.": "fc2."}

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        lm, loaded, back = [], set(), {}
        for name, t in weights:
            n = name
            if n.startswith("model.") and n.startswith(("model.vision_tower.",
                                                        "model.multi_modal_projector.",
                                                        "model.language_model.")):
                n = n[len("model."):]
            for pre in ("vision_model.", "vision_tower."):
                if n.startswith(pre):
                    if self.vision_model is None or self.vision_model.load_weight(
                            n[len(pre):], t):
                        loaded.add(name)
                    break
            else:
                for pre in ("mlp1.", "multi_modal_projector."):
                    if n.startswith(pre):
                        if self.mlp1 is not None:
                            sub = n[len(pre):]
                            for a, b in self._PROJ.items():
                                if sub.startswith(a):
                                    sub = b + sub[len(a):]
                                    break
                            params = dict(self.mlp1.named_parameters())
                            if sub in params:
                                params[sub].data.copy_(t)
                                loaded.add(name)
                        break
                else:
                    if n.startswith("language_model."):
                        n = n[len("language_model."):]
                        # the transformers layout stores the decoder without its "model." level
                        if not n.startswith(("model.", "lm_head.", "output.")):
                            n = "model." + n
                    back[n] = name
                    lm.append((n, t))
        return loaded | {back.get(n, n) for n in super().load_weights(lm)}


_CLASSES: dict = {}


def _language_class(cfg: ModelConfig):
    from . import llama
    arch = str(cfg.extra.get("llm_architecture") or "")
    mtype = str(cfg.extra.get("llm_model_type") or "")
    if "InternLM2" in arch or mtype == "internlm2":
        return llama.InternLM2ForCausalLM
    if "Qwen2" in arch or mtype == "qwen2":
        return llama.Qwen2ForCausalLM
    if "Qwen3" in arch or mtype == "qwen3":
        return llama.Qwen3ForCausalLM
    return llama.LlamaForCausalLM


def InternVLChatModel(cfg: ModelConfig, device="cpu"):
    """Builds the model on the language model its ``llm_config`` / ``text_config`` names
    (InternLM2 for InternVL2-2B / 8B / 26B, Qwen2 for InternVL2-1B and most of InternVL2.5,
    Llama otherwise)."""
    base = _language_class(cfg)
    cls = _CLASSES.get(base)
    if cls is None:
        def __init__(self, cfg_, device_="cpu"):
            base.__init__(self, cfg_, device_)
            self._init_vision(cfg_, device_)
        cls = _CLASSES[base] = type("InternVLChatModel", (_InternVLMixin, base),
                                    {"__init__": __init__, "__doc__": __doc__})
    return cls(cfg, device)
