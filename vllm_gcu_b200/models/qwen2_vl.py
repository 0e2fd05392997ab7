"""Qwen2-VL (also the architecture of QVQ-72B-preview): the vision transformer of the first
Qwen2 vision-language generation in front of the Qwen2 language model with multimodal rotary
embedding.  The reference lists both in its support matrix and serves them through vLLM's
upstream classes (docs/source/user_guide/support_matrix/supported_models.md).

Against Qwen2.5-VL (``models/qwen2_5_vl.py``, whose patch ordering, M-RoPE index and engine
hooks are reused): LayerNorm with bias instead of RMSNorm, a two-layer MLP with the quick-GELU
activation instead of SwiGLU, and every block attends over a whole frame (no windows).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config import ModelConfig
from ..ops import ref
from .qwen2_5_vl import Qwen2_5_VLForConditionalGeneration, get_rope_index


@dataclass
class Qwen2VLVisionConfig:
    depth: int = 32
    embed_dim: int = 1280
    hidden_size: int = 3584          # output width = the language model's hidden size
    mlp_ratio: float = 4.0
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    hidden_act: str = "quick_gelu"

    @classmethod
    def from_hf_dict(cls, d: dict) -> "Qwen2VLVisionConfig":
        return cls(**{f: d[f] for f in cls.__dataclass_fields__ if f in d})


def _act(name: str, x: torch.Tensor) -> torch.Tensor:
    if name == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    if name in ("gelu_pytorch_tanh", "gelu_tanh"):
        return F.gelu(x, approximate="tanh")
    return F.gelu(x)


class Qwen2VLVisionBlock(nn.Module):
    def __init__(self, c: Qwen2VLVisionConfig, dtype, device):
        super().__init__()
        H = c.embed_dim
        I = int(H * c.mlp_ratio)
        kw = dict(dtype=dtype, device=device)
        self.norm1 = nn.LayerNorm(H, eps=1e-6, **kw)
        self.norm2 = nn.LayerNorm(H, eps=1e-6, **kw)
        self.qkv = nn.Linear(H, 3 * H, bias=True, **kw)
        self.proj = nn.Linear(H, H, bias=True, **kw)
        self.fc1 = nn.Linear(H, I, **kw)
        self.fc2 = nn.Linear(I, H, **kw)
        self.heads, self.act = c.num_heads, c.hidden_act

    def forward(self, x: torch.Tensor, cu: Sequence[int], cos_sin: torch.Tensor) -> torch.Tensor:
        n, H = x.shape
        D = H // self.heads
        q, k, v = self.qkv(self.norm1(x)).split(H, dim=-1)
        pos = torch.arange(n, device=x.device)
        if ops.use_native(q) and q.dtype in (torch.bfloat16, torch.float16):
            from ..ops import cuda as C
            q, k = q.contiguous(), k.contiguous()
            C.rope_cache_flash(q, k, None, pos, cos_sin, True, D)
        else:
            q, k = ref.rotary_embedding(pos, q, k, D, cos_sin, True)
        q, k, v = (t.reshape(n, self.heads, D).transpose(0, 1) for t in (q, k, v))
        outs = [F.scaled_dot_product_attention(q[:, s:e], k[:, s:e], v[:, s:e])
                for s, e in zip(cu[:-1], cu[1:])]                  # one frame at a time
        a = torch.cat(outs, dim=1).transpose(0, 1).reshape(n, H)
        x = x + self.proj(a)
        return x + self.fc2(_act(self.act, self.fc1(self.norm2(x))))


class Qwen2VLVisionTransformer(nn.Module):
    def __init__(self, c: Qwen2VLVisionConfig, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.cfg = c
        kw = dict(dtype=dtype, device=device)
        self.patch_dim = c.in_channels * c.temporal_patch_size * c.patch_size * c.patch_size
        self.patch_embed = nn.Linear(self.patch_dim, c.embed_dim, bias=False, **kw)
        self.blocks = nn.ModuleList([Qwen2VLVisionBlock(c, dtype, device)
                                     for _ in range(c.depth)])
        m2 = c.spatial_merge_size ** 2
        self.ln_q = nn.LayerNorm(c.embed_dim, eps=1e-6, **kw)
        self.merger_fc1 = nn.Linear(c.embed_dim * m2, c.embed_dim * m2, **kw)
        self.merger_fc2 = nn.Linear(c.embed_dim * m2, c.hidden_size, **kw)
        self.head_dim = c.embed_dim // c.num_heads

    def _rot_pos_ids(self, grid_thw) -> torch.Tensor:
        m = self.cfg.spatial_merge_size
        out = []
        for t, h, w in grid_thw:
            hp = torch.arange(h)[:, None].expand(h, w)
            wp = torch.arange(w)[None, :].expand(h, w)
            hp = hp.reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            wp = wp.reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            out.append(torch.stack([hp, wp], dim=-1).repeat(t, 1))
        return torch.cat(out, dim=0)

    @torch.inference_mode()
    def forward(self, pixel_patches: torch.Tensor, grid_thw) -> torch.Tensor:
        """``pixel_patches [n_patches, C * Tp * P * P]``, ``grid_thw`` one (t, h, w) patch grid
        per image -> ``[n_patches / merge^2, hidden_size]``."""
        c = self.cfg
        dev = self.patch_embed.weight.device
        x = self.patch_embed(pixel_patches.to(device=dev, dtype=self.patch_embed.weight.dtype))
        n = x.shape[0]
        pos_ids = self._rot_pos_ids(grid_thw)
        dim = self.head_dim // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        max_grid = max(max(h, w) for _, h, w in grid_thw)
        rot = torch.outer(torch.arange(max_grid, dtype=torch.float32), inv)[pos_ids].flatten(1)
        cos_sin = torch.cat([rot.cos(), rot.sin()], dim=-1).to(dev)
        cu = [0]
        for t, h, w in grid_thw:
            for _ in range(t):
                cu.append(cu[-1] + h * w)
        for blk in self.blocks:
            x = blk(x, cu, cos_sin)
        x = self.ln_q(x).reshape(n // c.spatial_merge_size ** 2, -1)
        return self.merger_fc2(F.gelu(self.merger_fc1(x)))

    _NAME_MAP = {"merger.ln_q.": "ln_q.", "merger.mlp.0.": "merger_fc1.",
                 "merger.mlp.2.": "merger_fc2.", ".attn.qkv.": ".qkv.", ".attn.proj.": ".proj.",
                 ".mlp.fc1.": ".fc1.", ".mlp.fc2.": ".fc2."}

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


class Qwen2VLForConditionalGeneration(Qwen2_5_VLForConditionalGeneration):
    """Same engine hooks as Qwen2.5-VL; the temporal rotary index of a video counts frames
    (no seconds-per-grid scaling)."""

    def __init__(self, cfg: ModelConfig, device="cpu"):
        vc = cfg.extra.get("vision_config") or {}
        # build the language model (and a throw-away default tower config) through the parent
        nn.Module.__init__(self)
        from .llama import Qwen2ForCausalLM
        Qwen2ForCausalLM.__init__(self, cfg, device)
        self.vision_cfg = Qwen2VLVisionConfig.from_hf_dict(vc if isinstance(vc, dict) else {})
        if not vc:
            self.vision_cfg = dataclasses.replace(self.vision_cfg, hidden_size=cfg.hidden_size)
        self.visual = Qwen2VLVisionTransformer(self.vision_cfg, cfg.dtype, device) \
            if self.is_first_stage else None
        self.image_token_id = int(cfg.extra.get("image_token_id", 151655))
        self.video_token_id = int(cfg.extra.get("video_token_id", 151656))
        section = (cfg.rope_scaling or {}).get("mrope_section")
        if section:
            for layer in self.layers.values():
                layer.self_attn.attn.mrope_section = list(section)

    def prepare_request(self, prompt_token_ids, pixel_patches: torch.Tensor, grid_thw) -> dict:
        grids = [tuple(int(v) for v in g) for g in grid_thw]
        emb = self.encode_images(pixel_patches, grids)
        positions = [i for i, t in enumerate(prompt_token_ids) if t == self.image_token_id]
        assert len(positions) == emb.shape[0], "placeholder count must match the vision output"
        mpos, delta = get_rope_index(prompt_token_ids, grids, self.image_token_id,
                                     self.vision_cfg.spatial_merge_size,
                                     second_per_grid=[1.0] * len(grids), tokens_per_second=1.0)
        salt = hash(pixel_patches.detach().float().cpu().numpy().tobytes())
        return {"mm_embeds": emb, "mm_positions": positions, "mrope_positions": mpos,
                "mrope_delta": delta, "cache_salt": salt}
