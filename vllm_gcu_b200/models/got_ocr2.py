"""GOT-OCR-2.0: SAM-style ViT-Det image encoder + convolutional projector + Qwen2 decoder.

Image encoder (vllm_gcu/models/got_ocr2/got_ocr2.py:98-447): 16x16 patch embedding with a
learned absolute position grid, transformer blocks whose attention adds a decomposed
relative position bias (separate row / column tables, interpolated when the table length
differs from the window), most blocks windowed (partition into ``window_size`` squares with
padding, un-partition after attention) and the blocks of ``global_attn_indexes`` global; a
neck of 1x1 and 3x3 convolutions with channel-wise LayerNorm.  Two stride-2 convolutions and a
linear layer (:544-562) map the 64x64x256 feature map to 256 tokens of the language model's
width, which replace the image placeholder tokens of the prompt.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelConfig
from .llama import Qwen2ForCausalLM


@dataclass
class GotVisionConfig:
    hidden_size: int = 768
    output_channels: int = 256
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    image_size: int = 1024
    patch_size: int = 16
    window_size: int = 14
    global_attn_indexes: list = field(default_factory=lambda: [2, 5, 8, 11])
    mlp_dim: int = 3072
    layer_norm_eps: float = 1e-6
    use_rel_pos: bool = True
    use_abs_pos: bool = True
    qkv_bias: bool = True

    @classmethod
    def from_hf_dict(cls, d: dict) -> "GotVisionConfig":
        return cls(**{f: d[f] for f in cls.__dataclass_fields__ if f in d})


def get_rel_pos(q_size: int, k_size: int, rel_pos: torch.Tensor) -> torch.Tensor:
    """Relative position rows for every (query, key) coordinate pair; the table is linearly
    interpolated when its length is not ``2 * max(q, k) - 1``."""
    max_rel = 2 * max(q_size, k_size) - 1
    if rel_pos.shape[0] != max_rel:
        r = F.interpolate(rel_pos.float().reshape(1, rel_pos.shape[0], -1).permute(0, 2, 1),
                          size=max_rel, mode="linear")
        rel_pos = r.reshape(-1, max_rel).permute(1, 0).to(rel_pos.dtype)
    q = torch.arange(q_size)[:, None] * max(k_size / q_size, 1.0)
    k = torch.arange(k_size)[None, :] * max(q_size / k_size, 1.0)
    idx = (q - k) + (k_size - 1) * max(q_size / k_size, 1.0)
    return rel_pos[idx.long()]


class GotAttention(nn.Module):
    def __init__(self, c: GotVisionConfig, window: int, dtype, device):
        super().__init__()
        H = c.hidden_size
        self.heads = c.num_attention_heads
        self.qkv = nn.Linear(H, 3 * H, bias=c.qkv_bias, dtype=dtype, device=device)
        self.proj = nn.Linear(H, H, dtype=dtype, device=device)
        side = window if window > 0 else c.image_size // c.patch_size
        D = H // self.heads
        self.use_rel_pos = c.use_rel_pos
        if c.use_rel_pos:
            self.rel_pos_h = nn.Parameter(torch.zeros(2 * side - 1, D, dtype=dtype, device=device),
                                          requires_grad=False)
            self.rel_pos_w = nn.Parameter(torch.zeros(2 * side - 1, D, dtype=dtype, device=device),
                                          requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, Hh, Ww, C = x.shape
        D = C // self.heads
        qkv = self.qkv(x).reshape(B, Hh * Ww, 3, self.heads, D).permute(2, 0, 3, 1, 4)
        q, k, v = qkv.reshape(3, B * self.heads, Hh * Ww, D).unbind(0)
        bias = None
        if self.use_rel_pos:
            rh = get_rel_pos(Hh, Hh, self.rel_pos_h).to(q.device)
            rw = get_rel_pos(Ww, Ww, self.rel_pos_w).to(q.device)
            rq = q.reshape(B * self.heads, Hh, Ww, D)
            bh = torch.einsum("bhwc,hkc->bhwk", rq, rh)
            bw = torch.einsum("bhwc,wkc->bhwk", rq, rw)
            bias = (bh[:, :, :, :, None] + bw[:, :, :, None, :]).reshape(
                B * self.heads, Hh * Ww, Hh * Ww)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=bias)
        o = o.reshape(B, self.heads, Hh, Ww, D).permute(0, 2, 3, 1, 4).reshape(B, Hh, Ww, C)
        return self.proj(o)


def window_partition(x: torch.Tensor, w: int):
    B, H, W, C = x.shape
    ph, pw = (w - H % w) % w, (w - W % w) % w
    x = F.pad(x, (0, 0, 0, pw, 0, ph))
    Hp, Wp = H + ph, W + pw
    x = x.reshape(B, Hp // w, w, Wp // w, w, C).permute(0, 1, 3, 2, 4, 5).reshape(-1, w, w, C)
    return x, (Hp, Wp)


def window_unpartition(x: torch.Tensor, w: int, pad_hw, hw):
    Hp, Wp = pad_hw
    H, W = hw
    B = x.shape[0] // (Hp * Wp // w // w)
    x = x.reshape(B, Hp // w, Wp // w, w, w, -1).permute(0, 1, 3, 2, 4, 5).reshape(B, Hp, Wp, -1)
    return x[:, :H, :W].contiguous()


class GotBlock(nn.Module):
    def __init__(self, c: GotVisionConfig, window: int, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        self.layer_norm1 = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps, **kw)
        self.attn = GotAttention(c, window, dtype, device)
        self.layer_norm2 = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps, **kw)
        self.lin1 = nn.Linear(c.hidden_size, c.mlp_dim, **kw)
        self.lin2 = nn.Linear(c.mlp_dim, c.hidden_size, **kw)
        self.window = window

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        res = x
        x = self.layer_norm1(x)
        if self.window > 0:
            hw = (x.shape[1], x.shape[2])
            x, pad_hw = window_partition(x, self.window)
        x = self.attn(x)
        if self.window > 0:
            x = window_unpartition(x, self.window, pad_hw, hw)
        x = res + x
        return x + self.lin2(F.gelu(self.lin1(self.layer_norm2(x))))


class _LayerNorm2d(nn.Module):
    def __init__(self, ch, eps, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(ch, dtype=dtype, device=device), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(ch, dtype=dtype, device=device), requires_grad=False)
        self.eps = eps

    def forward(self, x):      # [B, C, H, W], normalised over C
        return F.layer_norm(x.permute(0, 2, 3, 1), (x.shape[1],), self.weight, self.bias,
                            self.eps).permute(0, 3, 1, 2)


class GotVisionEncoder(nn.Module):
    def __init__(self, c: GotVisionConfig, lm_hidden: int, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.cfg = c
        kw = dict(dtype=dtype, device=device)
        side = c.image_size // c.patch_size
        self.patch_embed = nn.Conv2d(3, c.hidden_size, c.patch_size, c.patch_size, **kw)
        self.pos_embed = nn.Parameter(torch.zeros(1, side, side, c.hidden_size, **kw),
                                      requires_grad=False) if c.use_abs_pos else None
        self.layers = nn.ModuleList([
            GotBlock(c, 0 if i in c.global_attn_indexes else c.window_size, dtype, device)
            for i in range(c.num_hidden_layers)])
        oc = c.output_channels
        self.neck_conv1 = nn.Conv2d(c.hidden_size, oc, 1, bias=False, **kw)
        self.neck_norm1 = _LayerNorm2d(oc, 1e-6, dtype, device)
        self.neck_conv2 = nn.Conv2d(oc, oc, 3, padding=1, bias=False, **kw)
        self.neck_norm2 = _LayerNorm2d(oc, 1e-6, dtype, device)
        self.up1 = nn.Conv2d(oc, oc * 2, 3, stride=2, padding=1, bias=False, **kw)
        self.up2 = nn.Conv2d(oc * 2, lm_hidden, 3, stride=2, padding=1, bias=False, **kw)
        self.proj = nn.Linear(lm_hidden, lm_hidden, **kw)

    @torch.inference_mode()
    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """``[B, 3, S, S]`` -> ``[B, (S / 64)^2, lm_hidden]`` image tokens."""
        w = self.patch_embed.weight
        x = self.patch_embed(pixel_values.to(device=w.device, dtype=w.dtype)).permute(0, 2, 3, 1)
        if self.pos_embed is not None:
            x = x + self.pos_embed
        for blk in self.layers:
            x = blk(x)
        x = x.permute(0, 3, 1, 2)
        x = self.neck_norm2(self.neck_conv2(self.neck_norm1(self.neck_conv1(x))))
        x = self.up2(self.up1(x))
        return self.proj(x.flatten(2).permute(0, 2, 1))

    _MAP = {"patch_embed.projection.": "patch_embed.", "neck.conv1.": "neck_conv1.",
            "neck.layer_norm1.": "neck_norm1.", "neck.conv2.": "neck_conv2.",
            "neck.layer_norm2.": "neck_norm2.", ".mlp.lin1.": ".lin1.", ".mlp.lin2.": ".lin2.",
            # original GOT checkpoint names (vision_tower_high / mm_projector_vary)
            "patch_embed.proj.": "patch_embed.", "blocks.": "layers.", ".norm1.": ".layer_norm1.",
            ".norm2.": ".layer_norm2.", "neck.0.": "neck_conv1.", "neck.1.": "neck_norm1.",
            "neck.2.": "neck_conv2.", "neck.3.": "neck_norm2.", "net_2.": "up1.", "net_3.": "up2."}

    def load_weight(self, name: str, tensor: torch.Tensor) -> bool:
        for a, b in self._MAP.items():
            name = name.replace(a, b)
        name = (name.replace("conv_upsampler1.", "up1.").replace("conv_upsampler2.", "up2.")
                .replace("multimodal_projector.", "proj."))
        params = dict(self.named_parameters())
        if name in params:
            params[name].data.copy_(tensor.reshape(params[name].shape))
            return True
        return False


class GotOcr2ForConditionalGeneration(Qwen2ForCausalLM):
    def __init__(self, cfg: ModelConfig, device="cpu"):
        super().__init__(cfg, device)
        vc = cfg.extra.get("vision_config") or {}
        self.vision_cfg = GotVisionConfig.from_hf_dict(vc if isinstance(vc, dict) else {})
        self.vision_tower = GotVisionEncoder(self.vision_cfg, cfg.hidden_size, cfg.dtype, device) \
            if self.is_first_stage else None
        self.image_token_id = int(cfg.extra.get("image_token_index",
                                                cfg.extra.get("image_token_id", 151859)))

    def encode_images(self, pixel_values: torch.Tensor) -> torch.Tensor:
        return self.vision_tower(pixel_values).flatten(0, 1)

    def prepare_request(self, prompt_token_ids: Sequence[int], pixel_values: torch.Tensor,
                        image_grid_thw=None) -> dict:
        emb = self.encode_images(pixel_values)
        positions = [i for i, t in enumerate(prompt_token_ids) if t == self.image_token_id]
        assert len(positions) == emb.shape[0], "placeholder count must match the vision output"
        salt = hash(pixel_values.detach().float().cpu().numpy().tobytes())
        return {"mm_embeds": emb, "mm_positions": positions, "cache_salt": salt}

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        lm, loaded = [], set()
        vis_prefixes = ("model.vision_tower.", "model.multi_modal_projector.",
                        "model.vision_tower_high.", "model.mm_projector_vary.")
        for name, t in weights:
            hit = False
            for pre in vis_prefixes:
                if name.startswith(pre):
                    sub = name[len(pre):]
                    if pre == "model.mm_projector_vary.":
                        sub = "proj." + sub
                    if self.vision_tower is not None and self.vision_tower.load_weight(sub, t):
                        loaded.add(name)
                    hit = True
                    break
            if hit:
                continue
            n = name
            if n.startswith("model.language_model."):
                n = "model." + n[len("model.language_model."):]
            lm.append((n, t))
        return loaded | super().load_weights(lm)
