"""GLM-4.1V (``Glm4vForConditionalGeneration``): vision transformer + GLM-4-0414 language model
with multimodal rotary positions.  The reference lists GLM-4V in its multimodal table and
serves it through vLLM's upstream class
(docs/source/user_guide/support_matrix/supported_models.md:30).

Vision tower: patches of ``temporal_patch_size x patch x patch`` pixels go through a 3-D
convolution (a linear map of the flattened patch) and an RMSNorm; a learnt position table of
``(image_size / patch)^2`` rows is sampled bicubically at every patch's relative place in its
image, so any grid size works; pre-norm blocks (RMSNorm, attention with a 2-D rotary embedding
over the patch's row and column, SwiGLU MLP without biases) attend within one frame; after a
final RMSNorm every ``merge x merge`` neighbourhood is folded by a strided convolution to the
language model's width, and a merger (linear, LayerNorm, GELU, SwiGLU) finishes the rows.

Language side: the GLM-4-0414 decoder (four norms per layer, interleaved rotary pairs on half of
the head) with its rotary frequencies split into (t, h, w) sections; image tokens take their
grid coordinates (``get_rope_index`` of the Qwen2-VL family, without temporal scaling).
Parameter names follow the checkpoint below ``model.visual.``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelConfig
from ..ops import ref
from .llama import Glm4ForCausalLM
from .qwen2_5_vl import _RMSNorm, get_rope_index


@dataclass
class Glm4vVisionConfig:
    depth: int = 24
    hidden_size: int = 1536
    intermediate_size: int = 13696
    num_heads: int = 12
    in_channels: int = 3
    image_size: int = 336
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    out_hidden_size: int = 4096
    rms_norm_eps: float = 1e-5
    attention_bias: bool = False
    hidden_act: str = "silu"

    @classmethod
    def from_hf_dict(cls, d: dict) -> "Glm4vVisionConfig":
        return cls(**{f: d[f] for f in cls.__dataclass_fields__ if f in d})


def _act(name: str, x: torch.Tensor) -> torch.Tensor:
    return F.silu(x) if name == "silu" else F.gelu(x)


class _Attn(nn.Module):
    def __init__(self, c: Glm4vVisionConfig, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.qkv = nn.Linear(c.hidden_size, 3 * c.hidden_size, bias=c.attention_bias, **kw)
        self.proj = nn.Linear(c.hidden_size, c.hidden_size, bias=False, **kw)


class _Mlp(nn.Module):
    def __init__(self, hidden: int, inter: int, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device, bias=False)
        self.gate_proj = nn.Linear(hidden, inter, **kw)
        self.up_proj = nn.Linear(hidden, inter, **kw)
        self.down_proj = nn.Linear(inter, hidden, **kw)


class Glm4vVisionBlock(nn.Module):
    def __init__(self, c: Glm4vVisionConfig, dtype, device):
        super().__init__()
        self.norm1 = _RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, device)
        self.norm2 = _RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, device)
        self.attn = _Attn(c, dtype, device)
        self.mlp = _Mlp(c.hidden_size, c.out_hidden_size, dtype, device)
        self.heads, self.act = c.num_heads, c.hidden_act

    def forward(self, x: torch.Tensor, cu: Sequence[int], cos_sin: torch.Tensor) -> torch.Tensor:
        n, H = x.shape
        D = H // self.heads
        q, k, v = self.attn.qkv(self.norm1(x)).split(H, dim=-1)
        pos = torch.arange(n, device=x.device)
        q, k = ref.rotary_embedding(pos, q.contiguous(), k.contiguous(), D, cos_sin, True)
        q, k, v = (t.reshape(n, self.heads, D).transpose(0, 1) for t in (q, k, v))
        a = torch.cat([F.scaled_dot_product_attention(q[:, s:e], k[:, s:e], v[:, s:e])
                       for s, e in zip(cu[:-1], cu[1:])], dim=1)
        x = x + self.attn.proj(a.transpose(0, 1).reshape(n, H))
        h = self.norm2(x)
        return x + self.mlp.down_proj(_act(self.act, self.mlp.gate_proj(h)) * self.mlp.up_proj(h))


class _Merger(nn.Module):
    def __init__(self, dim: int, inter: int, act: str, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.proj = nn.Linear(dim, dim, bias=False, **kw)
        self.post_projection_norm = nn.LayerNorm(dim, **kw)
        self.gate_proj = nn.Linear(dim, inter, bias=False, **kw)
        self.up_proj = nn.Linear(dim, inter, bias=False, **kw)
        self.down_proj = nn.Linear(inter, dim, bias=False, **kw)
        self.act = act

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = F.gelu(self.post_projection_norm(self.proj(x)))
        return self.down_proj(_act(self.act, self.gate_proj(x)) * self.up_proj(x))


class Glm4vVisionModel(nn.Module):
    def __init__(self, c: Glm4vVisionConfig, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.cfg = c
        kw = dict(dtype=dtype, device=device)
        self.patch_embed = nn.ModuleDict({"proj": nn.Conv3d(
            c.in_channels, c.hidden_size, (c.temporal_patch_size, c.patch_size, c.patch_size),
            (c.temporal_patch_size, c.patch_size, c.patch_size), **kw)})
        self.embeddings = nn.ModuleDict({"position_embedding": nn.Embedding(
            (c.image_size // c.patch_size) ** 2, c.hidden_size, **kw)})
        self.post_conv_layernorm = _RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, device)
        self.blocks = nn.ModuleList([Glm4vVisionBlock(c, dtype, device) for _ in range(c.depth)])
        self.post_layernorm = _RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, device)
        self.downsample = nn.Conv2d(c.hidden_size, c.out_hidden_size, c.spatial_merge_size,
                                    c.spatial_merge_size, **kw)
        self.merger = _Merger(c.out_hidden_size, c.intermediate_size, c.hidden_act, dtype, device)
        self.head_dim = c.hidden_size // c.num_heads

    def _patch_coords(self, grid_thw: Sequence[Sequence[int]]) -> torch.Tensor:
        """(row, column) of every patch in the processor's order: merge-sized neighbourhoods
        are contiguous."""
        m = self.cfg.spatial_merge_size
        out = []
        for t, h, w in grid_thw:
            rows = torch.arange(h)[:, None].expand(h, w)
            cols = torch.arange(w)[None, :].expand(h, w)
            rows = rows.reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            cols = cols.reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            out.append(torch.stack([rows, cols], dim=-1).repeat(t, 1))
        return torch.cat(out, dim=0)

    def _position_rows(self, coords: torch.Tensor, grid_thw: Sequence[Sequence[int]]
                       ) -> torch.Tensor:
        """The learnt position table sampled (bicubic, border padding) at the centre of every
        patch, measured relative to its own image's grid."""
        table = self.embeddings["position_embedding"].weight
        side = int(round(table.shape[0] ** 0.5))
        plane = table.float().view(side, side, -1).permute(2, 0, 1)[None]
        hs = torch.cat([torch.full((t * h * w,), float(h)) for t, h, w in grid_thw])
        ws = torch.cat([torch.full((t * h * w,), float(w)) for t, h, w in grid_thw])
        y = (coords[:, 0].float() + 0.5) / hs * 2 - 1
        x = (coords[:, 1].float() + 0.5) / ws * 2 - 1
        grid = torch.stack([x, y], dim=-1)[None, :, None, :].to(plane.device)
        rows = F.grid_sample(plane, grid, mode="bicubic", align_corners=False,
                             padding_mode="border")
        return rows[0, :, :, 0].t().to(table.dtype)

    @torch.inference_mode()
    def forward(self, pixel_patches: torch.Tensor, grid_thw: Sequence[Sequence[int]]
                ) -> torch.Tensor:
        """``pixel_patches [n_patches, C * Tp * P * P]``, one (t, h, w) patch grid per image
        -> ``[n_patches / merge^2, out_hidden_size]``."""
        c = self.cfg
        w = self.patch_embed["proj"].weight
        x = F.linear(pixel_patches.to(device=w.device, dtype=w.dtype), w.flatten(1),
                     self.patch_embed["proj"].bias)
        x = self.post_conv_layernorm(x)
        coords = self._patch_coords(grid_thw)
        dim = self.head_dim // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        freqs = torch.outer(torch.arange(max(max(h, w_) for _, h, w_ in grid_thw),
                                         dtype=torch.float32), inv)
        rot = freqs[coords].flatten(1)                                  # [n, head_dim / 2]
        cos_sin = torch.cat([rot.cos(), rot.sin()], dim=-1).to(x.device)
        x = x + self._position_rows(coords, grid_thw).to(x.device)
        cu = [0]
        for t, h, w_ in grid_thw:
            for _ in range(t):
                cu.append(cu[-1] + h * w_)
        for blk in self.blocks:
            x = blk(x, cu, cos_sin)
        x = self.post_layernorm(x)
        m = c.spatial_merge_size
        x = x.view(-1, m, m, x.shape[-1]).permute(0, 3, 1, 2)
        x = self.downsample(x).view(-1, c.out_hidden_size)
        return self.merger(x)

    def load_weight(self, name: str, tensor: torch.Tensor) -> bool:
        params = dict(self.named_parameters())
        if name in params:
            params[name].data.copy_(tensor.reshape(params[name].shape))
            return True
        return False


class Glm4vForConditionalGeneration(Glm4ForCausalLM):
    def __init__(self, cfg: ModelConfig, device="cpu"):
        super().__init__(cfg, device)
        vc = cfg.extra.get("vision_config") or {}
        self.vision_cfg = Glm4vVisionConfig.from_hf_dict(vc if isinstance(vc, dict) else {})
        self.visual = Glm4vVisionModel(self.vision_cfg, cfg.dtype, device) \
            if self.is_first_stage else None
        self.image_token_id = int(cfg.extra.get("image_token_id", 151343))
        section = (cfg.rope_scaling or {}).get("mrope_section")
        if section:
            for layer in self.layers.values():
                layer.self_attn.attn.mrope_section = list(section)

    def encode_images(self, pixel_patches: torch.Tensor, grid_thw) -> torch.Tensor:
        return self.visual(pixel_patches, [tuple(int(v) for v in g) for g in grid_thw])

    def prepare_request(self, prompt_token_ids: Sequence[int], pixel_patches: torch.Tensor,
                        grid_thw) -> dict:
        grids = [tuple(int(v) for v in g) for g in grid_thw]
        if any(t != 1 for t, _, _ in grids):
            raise ValueError("video inputs are not supported: one frame per grid")
        emb = self.encode_images(pixel_patches, grids)
        positions = [i for i, t in enumerate(prompt_token_ids) if t == self.image_token_id]
        assert len(positions) == emb.shape[0], "placeholder count must match the vision output"
        mpos, delta = get_rope_index(prompt_token_ids, grids, self.image_token_id,
                                     self.vision_cfg.spatial_merge_size)
        salt = hash(pixel_patches.detach().float().cpu().numpy().tobytes())
        return {"mm_embeds": emb, "mm_positions": positions, "mrope_positions": mpos,
                "mrope_delta": delta, "cache_salt": salt}

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        lm, loaded, back = [], set(), {}
        for name, t in weights:
            n = name
            for pre in ("model.visual.", "visual."):
                if n.startswith(pre):
                    if self.visual is None or self.visual.load_weight(n[len(pre):], t):
                        loaded.add(name)
                    n = None
                    break
            if n is None:
                continue
            if n.startswith("model.language_model."):
                n = "model." + n[len("model.language_model."):]
            back[n] = name
            lm.append((n, t))
        return loaded | {back.get(n, n) for n in super().load_weights(lm)}
