"""Qwen2.5-VL: vision transformer + Qwen2 language model with multimodal rotary embedding.

Vision tower (vllm_gcu/models/qwen2_5_vl/qwen2_5_vl.py:235-401, 784): patches of
``temporal_patch_size x patch x patch`` pixels are embedded by a linear map, blocks of
RMSNorm -> attention -> RMSNorm -> SwiGLU run over the patch sequence with a 2-D rotary
embedding (row / column position of the patch); most blocks attend inside windows of
``window_size`` pixels, the blocks listed in ``fullatt_block_indexes`` attend over a whole
frame; a merger concatenates each ``spatial_merge_size``^2 neighbourhood and projects it to
the language model's width.  The rotary embedding goes through the same rotary kernel as
the language model (positions 0..n-1 over a pre-gathered cos/sin table), attention is
block-diagonal over the windows / frames.

Language side: ``get_rope_index`` gives every prompt token a (t, h, w) position; image
tokens take their grid coordinates, text tokens a running index; the engine passes these as
``mrope_positions`` and offsets later tokens by ``mrope_delta``.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Iterable, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config import ModelConfig
from ..ops import ref
from .llama import Qwen2ForCausalLM


@dataclass
class VisionConfig:
    depth: int = 32
    hidden_size: int = 1280
    intermediate_size: int = 3420
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    window_size: int = 112
    out_hidden_size: int = 3584
    fullatt_block_indexes: list = field(default_factory=lambda: [7, 15, 23, 31])
    tokens_per_second: int = 2
    rms_norm_eps: float = 1e-6

    @classmethod
    def from_hf_dict(cls, d: dict) -> "VisionConfig":
        return cls(**{f: d[f] for f in cls.__dataclass_fields__ if f in d})


class _RMSNorm(nn.Module):
    def __init__(self, dim, eps, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device),
                                   requires_grad=False)
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
                * self.weight.float()).to(x.dtype)


class VisionBlock(nn.Module):
    def __init__(self, c: VisionConfig, dtype, device):
        super().__init__()
        H, I = c.hidden_size, c.intermediate_size
        kw = dict(dtype=dtype, device=device)
        self.norm1 = _RMSNorm(H, c.rms_norm_eps, dtype, device)
        self.norm2 = _RMSNorm(H, c.rms_norm_eps, dtype, device)
        self.qkv = nn.Linear(H, 3 * H, bias=True, **kw)
        self.proj = nn.Linear(H, H, bias=True, **kw)
        self.gate_proj = nn.Linear(H, I, bias=True, **kw)
        self.up_proj = nn.Linear(H, I, bias=True, **kw)
        self.down_proj = nn.Linear(I, H, bias=True, **kw)
        self.heads = c.num_heads

    def forward(self, x: torch.Tensor, cu: Sequence[int], cos_sin: torch.Tensor) -> torch.Tensor:
        n, H = x.shape
        D = H // self.heads
        qkv = self.qkv(self.norm1(x))
        q, k, v = qkv.split(H, dim=-1)
        pos = torch.arange(n, device=x.device)
        if ops.use_native(q) and q.dtype in (torch.bfloat16, torch.float16):
            from ..ops import cuda as C
            q, k = q.contiguous(), k.contiguous()
            C.rope_cache_flash(q, k, None, pos, cos_sin, True, D)
        else:
            q, k = ref.rotary_embedding(pos, q, k, D, cos_sin, True)
        q, k, v = (t.reshape(n, self.heads, D).transpose(0, 1) for t in (q, k, v))
        outs = []
        for s, e in zip(cu[:-1], cu[1:]):           # block-diagonal (window / frame) attention
            outs.append(F.scaled_dot_product_attention(q[:, s:e], k[:, s:e], v[:, s:e]))
        a = torch.cat(outs, dim=1).transpose(0, 1).reshape(n, H)
        x = x + self.proj(a)
        h = self.norm2(x)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


class VisionTransformer(nn.Module):
    def __init__(self, c: VisionConfig, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.cfg = c
        kw = dict(dtype=dtype, device=device)
        self.patch_dim = c.in_channels * c.temporal_patch_size * c.patch_size * c.patch_size
        self.patch_embed = nn.Linear(self.patch_dim, c.hidden_size, bias=False, **kw)
        self.blocks = nn.ModuleList([VisionBlock(c, dtype, device) for _ in range(c.depth)])
        self.ln_q = _RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, device)
        m2 = c.spatial_merge_size ** 2
        self.merger_fc1 = nn.Linear(c.hidden_size * m2, c.hidden_size * m2, **kw)
        self.merger_fc2 = nn.Linear(c.hidden_size * m2, c.out_hidden_size, **kw)
        self.head_dim = c.hidden_size // c.num_heads

    # -- position helpers ------------------------------------------------------------
    def _rot_pos_ids(self, grid_thw: Sequence[Sequence[int]]) -> torch.Tensor:
        m = self.cfg.spatial_merge_size
        out = []
        for t, h, w in grid_thw:
            hp = torch.arange(h)[:, None].expand(h, w)
            wp = torch.arange(w)[None, :].expand(h, w)
            hp = hp.reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            wp = wp.reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            out.append(torch.stack([hp, wp], dim=-1).repeat(t, 1))
        return torch.cat(out, dim=0)

    def _window_index(self, grid_thw: Sequence[Sequence[int]]):
        c = self.cfg
        m = c.spatial_merge_size
        win = c.window_size // m // c.patch_size
        unit = m * m
        index, cu, base = [], [0], 0
        for t, h, w in grid_thw:
            gh, gw = h // m, w // m
            idx = torch.arange(t * gh * gw).reshape(t, gh, gw)
            ph, pw = (win - gh % win) % win, (win - gw % win) % win
            nh, nw = (gh + ph) // win, (gw + pw) // win
            pad = F.pad(idx, (0, pw, 0, ph), value=-100)
            pad = pad.reshape(t, nh, win, nw, win).permute(0, 1, 3, 2, 4).reshape(
                t, nh * nw, win, win)
            lens = (pad != -100).sum(dim=(2, 3)).reshape(-1)
            flat = pad.reshape(-1)
            index.append(flat[flat != -100] + base)
            cu += (lens.cumsum(0) * unit + cu[-1]).tolist()
            base += t * gh * gw
        dedup = [cu[0]]
        for v in cu[1:]:
            if v != dedup[-1]:
                dedup.append(v)
        return torch.cat(index), dedup

    @torch.inference_mode()
    def forward(self, pixel_patches: torch.Tensor, grid_thw: Sequence[Sequence[int]]
                ) -> torch.Tensor:
        """``pixel_patches [n_patches, C * Tp * P * P]`` (the processor's flattened patches),
        ``grid_thw`` one (t, h, w) patch grid per image -> ``[n_patches / merge^2, out]``."""
        c = self.cfg
        dev = self.patch_embed.weight.device
        x = self.patch_embed(pixel_patches.to(device=dev, dtype=self.patch_embed.weight.dtype))
        n = x.shape[0]
        unit = c.spatial_merge_size ** 2
        pos_ids = self._rot_pos_ids(grid_thw)                         # [n, 2]
        dim = self.head_dim // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        max_grid = max(max(h, w) for _, h, w in grid_thw)
        freqs = torch.outer(torch.arange(max_grid, dtype=torch.float32), inv)
        rot = freqs[pos_ids].flatten(1)                               # [n, head_dim / 2]
        win_idx, cu_win = self._window_index(grid_thw)
        x = x.reshape(n // unit, unit, -1)[win_idx.to(dev)].reshape(n, -1)
        rot = rot.reshape(n // unit, unit, -1)[win_idx].reshape(n, -1)
        cos_sin = torch.cat([rot.cos(), rot.sin()], dim=-1).to(dev)   # [n, head_dim] = cos | sin
        cu_full = [0]
        for t, h, w in grid_thw:
            for _ in range(t):
                cu_full.append(cu_full[-1] + h * w)
        for i, blk in enumerate(self.blocks):
            x = blk(x, cu_full if i in c.fullatt_block_indexes else cu_win, cos_sin)
        x = self.ln_q(x).reshape(n // unit, -1)
        x = self.merger_fc2(F.gelu(self.merger_fc1(x)))
        return x[torch.argsort(win_idx).to(dev)]

    _NAME_MAP = {"merger.ln_q.": "ln_q.", "merger.mlp.0.": "merger_fc1.",
                 "merger.mlp.2.": "merger_fc2.", ".attn.qkv.": ".qkv.", ".attn.proj.": ".proj.",
                 ".mlp.gate_proj.": ".gate_proj.", ".mlp.up_proj.": ".up_proj.",
                 ".mlp.down_proj.": ".down_proj."}

    def load_weight(self, name: str, tensor: torch.Tensor) -> bool:
        """``name`` without the ``visual.`` prefix (HuggingFace layout)."""
        if name == "patch_embed.proj.weight":
            self.patch_embed.weight.data.copy_(tensor.reshape(tensor.shape[0], -1))
            return True
        for a, b in self._NAME_MAP.items():
            name = name.replace(a, b)
        params = dict(self.named_parameters())
        if name in params:
            params[name].data.copy_(tensor)
            return True
        return False


def get_rope_index(input_ids: Sequence[int], grids: Sequence[Sequence[int]],
                   image_token_id: int, spatial_merge_size: int,
                   second_per_grid: Optional[Sequence[float]] = None,
                   tokens_per_second: float = 2.0) -> tuple[torch.Tensor, int]:
    """(t, h, w) positions ``[3, len(input_ids)]`` and the offset of later tokens.  Runs of
    ``image_token_id`` take the coordinates of the merged patch grid of the next entry of
    ``grids``; the temporal index of a video frame is scaled by its duration."""
    ids = list(input_ids)
    pos = torch.zeros(3, len(ids), dtype=torch.long)
    nxt, i, g = 0, 0, 0
    while i < len(ids):
        if ids[i] == image_token_id and g < len(grids):
            t, h, w = grids[g]
            gh, gw = h // spatial_merge_size, w // spatial_merge_size
            n = t * gh * gw
            spg = float(second_per_grid[g]) if second_per_grid else 0.0
            ti = (torch.arange(t).float() * spg * tokens_per_second).long()
            tt = ti[:, None, None].expand(t, gh, gw).reshape(-1)
            hh = torch.arange(gh)[None, :, None].expand(t, gh, gw).reshape(-1)
            ww = torch.arange(gw)[None, None, :].expand(t, gh, gw).reshape(-1)
            pos[:, i:i + n] = torch.stack([tt, hh, ww]) + nxt
            nxt = int(pos[:, i:i + n].max()) + 1
            i += n
            g += 1
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    return pos, nxt - len(ids)


class Qwen2_5_VLForConditionalGeneration(Qwen2ForCausalLM):
    """Language model + vision tower.  ``encode_images`` turns processor outputs into the
    embeddings of the image placeholder tokens; ``prepare_request`` computes what the engine
    needs per request (placeholder positions, M-RoPE positions and offset, cache salt)."""

    def __init__(self, cfg: ModelConfig, device="cpu"):
        super().__init__(cfg, device)
        vc = cfg.extra.get("vision_config") or {}
        self.vision_cfg = VisionConfig.from_hf_dict(vc) if isinstance(vc, dict) else vc
        if self.vision_cfg.out_hidden_size != cfg.hidden_size and not vc:
            self.vision_cfg = dataclasses.replace(self.vision_cfg, out_hidden_size=cfg.hidden_size)
        self.visual = VisionTransformer(self.vision_cfg, cfg.dtype, device) \
            if self.is_first_stage else None
        self.image_token_id = int(cfg.extra.get("image_token_id", 151655))
        self.video_token_id = int(cfg.extra.get("video_token_id", 151656))
        section = (cfg.rope_scaling or {}).get("mrope_section")
        if section:
            for layer in self.layers.values():
                layer.self_attn.attn.mrope_section = list(section)

    def encode_images(self, pixel_patches: torch.Tensor, grid_thw) -> torch.Tensor:
        return self.visual(pixel_patches, [tuple(int(v) for v in g) for g in grid_thw])

    def prepare_request(self, prompt_token_ids: Sequence[int], pixel_patches: torch.Tensor,
                        grid_thw) -> dict:
        grids = [tuple(int(v) for v in g) for g in grid_thw]
        emb = self.encode_images(pixel_patches, grids)
        positions = [i for i, t in enumerate(prompt_token_ids) if t == self.image_token_id]
        assert len(positions) == emb.shape[0], "placeholder count must match the vision output"
        mpos, delta = get_rope_index(prompt_token_ids, grids, self.image_token_id,
                                     self.vision_cfg.spatial_merge_size)
        salt = hash(pixel_patches.detach().float().cpu().numpy().tobytes())
        return {"mm_embeds": emb, "mm_positions": positions, "mrope_positions": mpos,
                "mrope_delta": delta, "cache_salt": salt}

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        lm, loaded = [], set()
        for name, t in weights:
            n = name
            for pre in ("model.visual.", "visual."):
                if n.startswith(pre):
                    if self.visual is not None and self.visual.load_weight(n[len(pre):], t):
                        loaded.add(name)
                    n = None
                    break
            if n is None:
                continue
            if n.startswith("model.language_model."):
                n = "model." + n[len("model.language_model."):]
            elif n.startswith("language_model.model."):
                n = "model." + n[len("language_model.model."):]
            elif n.startswith("language_model.lm_head."):
                n = n[len("language_model."):]
            lm.append((n, t))
        return loaded | super().load_weights(lm)
