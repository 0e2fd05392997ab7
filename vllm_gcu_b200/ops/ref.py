"""Plain PyTorch reference implementation of every op in this package.

These functions define the semantics.  They run on any device in fp32
internally, serve as the oracle of the kernel tests, and are the execution
path on machines without a GPU (the tiny-Llama CPU configuration).
The contracts are those of the reference plugin's custom ops
(``vllm_gcu/kernels/_custom_ops.py``) unless a docstring says otherwise.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

FP8_MAX = 448.0
FP8_DTYPE = torch.float8_e4m3fn


# ---------------------------------------------------------------------------
# normalisation
# ---------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * w`` (csrc/src/rms_norm.cpp:38)."""
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return (xf * torch.rsqrt(var + eps) * weight.float()).to(x.dtype)


def fused_add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                       eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    """``residual <- x + residual; out <- rms_norm(residual)``; returns
    (out, residual) (csrc/src/fused_add_rms_norm.cpp:40)."""
    new_res = (x.float() + residual.float()).to(x.dtype)
    return rms_norm(new_res, weight, eps), new_res


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
               eps: float) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(),
                        None if bias is None else bias.float(), eps).to(x.dtype)


# ---------------------------------------------------------------------------
# quantisation
# ---------------------------------------------------------------------------
def _to_fp8(x: torch.Tensor) -> torch.Tensor:
    return x.clamp(-FP8_MAX, FP8_MAX).to(FP8_DTYPE)


def static_scaled_fp8_quant(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """``q = clamp(x / scale)`` (csrc/src/static_scaled_fp8_quant.cpp:37)."""
    return _to_fp8(x.float() / scale.float())


def dynamic_per_token_fp8_quant(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per row ``s = max|x| / 448`` (floored at 1e-10/448), ``q = x / s``
    (csrc/src/dynamic_per_token_scaled_fp8_quant.cpp:33)."""
    xf = x.float()
    s = xf.abs().amax(-1, keepdim=True).clamp_min(1e-10) / FP8_MAX
    return _to_fp8(xf / s), s


def dynamic_per_tensor_fp8_quant(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    xf = x.float()
    s = (xf.abs().amax().clamp_min(1e-10) / FP8_MAX).reshape(1)
    return _to_fp8(xf / s), s


def per_token_group_fp8_quant(x: torch.Tensor, group: int = 128,
                              valid_rows: Optional[int] = None
                              ) -> tuple[torch.Tensor, torch.Tensor]:
    """1 x ``group`` dynamic fp8 quantisation; scales are ``[T, K / group]`` fp32
    (vllm_gcu/kernels/_custom_ops.py:465-486)."""
    T, K = x.shape
    xf = x.float().reshape(T, K // group, group)
    s = xf.abs().amax(-1, keepdim=True).clamp_min(1e-10) / FP8_MAX
    q = _to_fp8(xf / s).reshape(T, K)
    s = s.reshape(T, K // group)
    if valid_rows is not None:
        q = q.clone()
        q.view(torch.uint8)[valid_rows:] = 0
        s = s.clone()
        s[valid_rows:] = 0
    return q, s


def static_scaled_int8_quant(x: torch.Tensor, scale: torch.Tensor,
                             azp: Optional[torch.Tensor] = None) -> torch.Tensor:
    q = torch.round(x.float() / scale.float())
    if azp is not None:
        q = q + azp.float()
    return q.clamp(-128, 127).to(torch.int8)


def dynamic_scaled_int8_quant(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    xf = x.float()
    s = xf.abs().amax(-1, keepdim=True).clamp_min(1e-10) / 127.0
    return torch.round(xf / s).clamp(-128, 127).to(torch.int8), s


def static_scaled_int8_dequant(q: torch.Tensor, scale: torch.Tensor,
                               azp: Optional[torch.Tensor] = None,
                               dtype: torch.dtype = torch.float32) -> torch.Tensor:
    x = q.float()
    if azp is not None:
        x = x - azp.float()
    return (x * scale.float()).to(dtype)


def rms_norm_quant(x: torch.Tensor, weight: torch.Tensor, eps: float, mode: str,
                   residual: Optional[torch.Tensor] = None,
                   scale: Optional[torch.Tensor] = None):
    """RMSNorm (optionally with residual add) followed by quantisation.
    mode: fp8_static | fp8_token | fp8_group128 | int8_static | int8_token.
    Returns (q, scale_or_None, new_residual_or_None)
    (vllm_gcu/compilation/fusion.py:185-1137 lists the fused patterns)."""
    new_res = None
    if residual is not None:
        y, new_res = fused_add_rms_norm(x, residual, weight, eps)
    else:
        y = rms_norm(x, weight, eps)
    if mode == "fp8_static":
        return static_scaled_fp8_quant(y, scale), None, new_res
    if mode == "fp8_token":
        q, s = dynamic_per_token_fp8_quant(y)
        return q, s, new_res
    if mode == "fp8_group128":
        q, s = per_token_group_fp8_quant(y, 128)
        return q, s, new_res
    if mode == "int8_static":
        return static_scaled_int8_quant(y, scale), None, new_res
    if mode == "int8_token":
        q, s = dynamic_scaled_int8_quant(y)
        return q, s, new_res
    raise ValueError(mode)


# ---------------------------------------------------------------------------
# activations
# ---------------------------------------------------------------------------
def _act(name: str, x: torch.Tensor, threshold: float = 0.0) -> torch.Tensor:
    if name == "silu":
        return F.silu(x)
    if name == "gelu":
        return F.gelu(x)
    if name in ("gelu_tanh", "gelu_new"):
        return F.gelu(x, approximate="tanh")
    if name == "gelu_fast":
        return 0.5 * x * (1.0 + torch.tanh(x * 0.79788456 * (1.0 + 0.044715 * x * x)))
    if name == "gelu_quick":
        return x * torch.sigmoid(1.702 * x)
    if name == "fatrelu":
        return torch.where(x > threshold, x, torch.zeros_like(x))
    if name == "identity":
        return x
    raise ValueError(name)


def act_and_mul(x: torch.Tensor, act: str = "silu", threshold: float = 0.0) -> torch.Tensor:
    """``act(x[..., :d]) * x[..., d:]`` (csrc/src/silu_and_mul.cpp:44 and siblings)."""
    d = x.shape[-1] // 2
    xf = x.float()
    return (_act(act, xf[..., :d], threshold) * xf[..., d:]).to(x.dtype)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    return act_and_mul(x, "silu")


def mul_and_silu(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    xf = x.float()
    return (xf[..., :d] * F.silu(xf[..., d:])).to(x.dtype)


def activation(x: torch.Tensor, act: str) -> torch.Tensor:
    return _act(act, x.float()).to(x.dtype)


# ---------------------------------------------------------------------------
# rotary embedding
# ---------------------------------------------------------------------------
def make_cos_sin_cache(rot_dim: int, max_pos: int, base: float = 10000.0,
                       dtype: torch.dtype = torch.float32,
                       scaling_factor: float = 1.0) -> torch.Tensor:
    inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    t = torch.arange(max_pos, dtype=torch.float32) / scaling_factor
    freqs = torch.outer(t, inv_freq)
    return torch.cat([freqs.cos(), freqs.sin()], dim=-1).to(dtype)


def rotary_embedding(positions: torch.Tensor, q: torch.Tensor, k: Optional[torch.Tensor],
                     head_size: int, cos_sin_cache: torch.Tensor, is_neox: bool
                     ) -> tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Out-of-place reference of the in-place op (csrc/src/rotary_embedding.cpp:38):
    q ``[T, H*D]``, k ``[T, Hkv*D]``, cache ``[max_pos, rot]`` = ``[cos | sin]``."""
    rot = cos_sin_cache.shape[-1]
    cs = cos_sin_cache.float()[positions.long()]
    cos, sin = cs[:, : rot // 2], cs[:, rot // 2:]

    def apply(x: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if x is None:
            return None
        T = x.shape[0]
        xf = x.float().reshape(T, -1, head_size)
        xr, xp = xf[..., :rot], xf[..., rot:]
        c, s = cos[:, None, :], sin[:, None, :]
        if is_neox:
            x1, x2 = xr[..., : rot // 2], xr[..., rot // 2:]
            out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
        else:
            x1, x2 = xr[..., 0::2], xr[..., 1::2]
            out = torch.stack([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).flatten(-2)
        return torch.cat([out, xp], dim=-1).reshape(x.shape).to(x.dtype)

    return apply(q), apply(k)


# ---------------------------------------------------------------------------
# KV cache
# ---------------------------------------------------------------------------
def reshape_and_cache_flash(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor,
                            v_cache: torch.Tensor, slot_mapping: torch.Tensor,
                            k_scale: Optional[torch.Tensor] = None,
                            v_scale: Optional[torch.Tensor] = None) -> None:
    """Caches are ``[blocks, block_size, Hkv, D]``; slots < 0 are skipped
    (csrc/src/reshape_and_cache_flash.cpp:23)."""
    nb, bs, H, D = k_cache.shape
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    kc = k_cache.view(nb * bs, H, D)
    vc = v_cache.view(nb * bs, H, D)
    k = key.reshape(-1, H, D)[valid]
    v = value.reshape(-1, H, D)[valid]
    if k_cache.dtype == FP8_DTYPE:
        kc[slots] = _to_fp8(k.float() / k_scale.float())
        vc[slots] = _to_fp8(v.float() / v_scale.float())
    else:
        kc[slots] = k.to(k_cache.dtype)
        vc[slots] = v.to(v_cache.dtype)


def reshape_and_cache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, slot_mapping: torch.Tensor,
                      k_scale: float = 1.0, v_scale: float = 1.0, k_zp: float = 0.0,
                      v_zp: float = 0.0) -> None:
    """x-packed layout: K ``[blocks, Hkv, D/x, bs, x]``, V ``[blocks, Hkv, D, bs]``;
    int8 caches store ``round(v / scale) + zero`` (csrc/src/reshape_and_cache.cpp:34,
    vllm_gcu/attention/ops/paged_attn.py:27-65)."""
    nb, H, Dx, bs, x = k_cache.shape
    D = Dx * x
    T = key.shape[0]
    k = key.reshape(T, H, D).float()
    v = value.reshape(T, H, D).float()
    for t in range(T):
        slot = int(slot_mapping[t])
        if slot < 0:
            continue
        b, off = divmod(slot, bs)
        kq, vq = k[t], v[t]
        if k_cache.dtype == torch.int8:
            kq = (torch.round(kq / k_scale) + k_zp).clamp(-128, 127)
            vq = (torch.round(vq / v_scale) + v_zp).clamp(-128, 127)
        elif k_cache.dtype == FP8_DTYPE:
            kq = (kq / k_scale).clamp(-FP8_MAX, FP8_MAX)
            vq = (vq / v_scale).clamp(-FP8_MAX, FP8_MAX)
        k_cache[b, :, :, off, :] = kq.reshape(H, Dx, x).to(k_cache.dtype)
        v_cache[b, :, :, off] = vq.to(v_cache.dtype)


def concat_and_cache_mla(kv_c: torch.Tensor, k_pe: torch.Tensor, kv_cache: torch.Tensor,
                         slot_mapping: torch.Tensor, scale: Optional[torch.Tensor] = None
                         ) -> None:
    """``kv_cache[slot] = [kv_c | k_pe]``, cache ``[blocks, bs, L+R]``
    (csrc/src/concat_and_cache_mla.cpp:35)."""
    W = kv_cache.shape[-1]
    flat = kv_cache.view(-1, W)
    valid = slot_mapping >= 0
    row = torch.cat([kv_c, k_pe.reshape(kv_c.shape[0], -1)], dim=-1)[valid]
    if kv_cache.dtype == FP8_DTYPE:
        flat[slot_mapping[valid].long()] = _to_fp8(row.float() / scale.float())
    else:
        flat[slot_mapping[valid].long()] = row.to(kv_cache.dtype)


def mla_rope_cache(q_pe: torch.Tensor, kv: torch.Tensor, positions: torch.Tensor,
                   cos_sin: torch.Tensor, weight: torch.Tensor, eps: float,
                   kv_cache: Optional[torch.Tensor], slot_mapping: Optional[torch.Tensor],
                   kv_lora_rank: int, is_neox: bool = False,
                   scale: Optional[torch.Tensor] = None):
    """Fused MLA cache update: split latent, RMSNorm(kv_c), RoPE(q_pe, k_pe), write
    ``[kv_c | k_pe]`` at the slots.  Returns (q_pe_rot, k_pe_rot, kv_c_normed)
    (native fallback vllm_gcu/attention/backends/mla_fusion.py:73-106)."""
    L = kv_lora_rank
    R = kv.shape[-1] - L
    kv_c = rms_norm(kv[:, :L].contiguous(), weight, eps)
    k_pe = kv[:, L:].contiguous()
    T, H = q_pe.shape[0], q_pe.shape[1]
    q_rot, k_rot = rotary_embedding(positions, q_pe.reshape(T, H * R), k_pe, R, cos_sin, is_neox)
    q_rot = q_rot.reshape(T, H, R)
    if kv_cache is not None and slot_mapping is not None:
        concat_and_cache_mla(kv_c, k_rot, kv_cache, slot_mapping, scale)
    return q_rot, k_rot, kv_c


def gather_cache(src_cache: torch.Tensor, block_table: torch.Tensor, cu_seq_lens: torch.Tensor,
                 seq_starts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Copies ``len_b`` tokens of every sequence, starting at ``seq_starts[b]``, from the
    pages into one contiguous ``[total, W]`` tensor (csrc/src/gather_cache.cpp:18)."""
    nb, bs = src_cache.shape[0], src_cache.shape[1]
    W = src_cache.shape[2:].numel()
    flat = src_cache.reshape(nb * bs, W)
    rows = []
    B = block_table.shape[0]
    for b in range(B):
        n = int(cu_seq_lens[b + 1] - cu_seq_lens[b])
        st = 0 if seq_starts is None else int(seq_starts[b])
        pos = torch.arange(st, st + n, device=src_cache.device)
        blk = block_table[b, (pos // bs).long()].long()
        rows.append(flat[blk * bs + pos % bs])
    if not rows:
        return flat[:0]
    return torch.cat(rows, dim=0)


def copy_blocks(caches: Sequence[torch.Tensor], mapping: torch.Tensor) -> None:
    """For every cache tensor (block index = dim 0): ``cache[dst] = cache[src]`` for each
    ``(src, dst)`` row of ``mapping`` (csrc/src/cache_kernels.cpp:43-58)."""
    if mapping.numel() == 0:
        return
    src, dst = mapping[:, 0].long(), mapping[:, 1].long()
    for c in caches:
        c[dst] = c[src]


def swap_blocks(src: torch.Tensor, dst: torch.Tensor, mapping: torch.Tensor) -> None:
    """``dst[d] = src[s]`` for each ``(s, d)``; tensors may live on different devices
    (csrc/src/cache_kernels.cpp:10-41)."""
    for s, d in mapping.tolist():
        dst[d].copy_(src[s], non_blocking=True)


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------
def _gather_kv(k_cache: torch.Tensor, v_cache: torch.Tensor, block_table_row: torch.Tensor,
               n: int, k_scale=None, v_scale=None):
    nb, bs, H, D = k_cache.shape
    pos = torch.arange(n, device=k_cache.device)
    blk = block_table_row[(pos // bs).long()].long()
    slots = blk * bs + pos % bs
    k = k_cache.view(nb * bs, H, D)[slots].float()
    v = v_cache.view(nb * bs, H, D)[slots].float()
    if k_scale is not None:
        k = k * k_scale.float()
    if v_scale is not None:
        v = v * v_scale.float()
    return k, v


def paged_attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                           block_tables: torch.Tensor, seq_lens: torch.Tensor, scale: float,
                           k_scale=None, v_scale=None, alibi_slopes=None) -> torch.Tensor:
    """One query token per sequence; q ``[B, Hq, D]``; flash-layout caches
    (csrc/src/paged_attention_v1.cpp:68 semantics on the layout of
    csrc/src/reshape_and_cache_flash.cpp).  ``alibi_slopes`` fp32 ``[Hq]``: slope times
    (key position - query position) is added to the scores."""
    B, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    G = Hq // Hkv
    out = torch.zeros_like(q)
    for b in range(B):
        n = int(seq_lens[b])
        if n == 0:
            continue
        k, v = _gather_kv(k_cache, v_cache, block_tables[b], n, k_scale, v_scale)
        k = k.repeat_interleave(G, dim=1)
        v = v.repeat_interleave(G, dim=1)
        s = torch.einsum("hd,nhd->hn", q[b].float(), k) * scale
        if alibi_slopes is not None:
            rel = torch.arange(n, device=q.device, dtype=torch.float32) - (n - 1)
            s = s + alibi_slopes.float()[:, None] * rel[None, :]
        p = torch.softmax(s, dim=-1)
        out[b] = torch.einsum("hn,nhd->hd", p, v).to(q.dtype)
    return out


def varlen_prefill_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                             block_tables: torch.Tensor, cu_q: torch.Tensor,
                             seq_lens: torch.Tensor, scale: float, causal: bool = True,
                             window: int = 0, return_lse: bool = False, alibi_slopes=None):
    """Attention of the new tokens of each sequence (``cu_q`` offsets into q
    ``[T, Hq, D]``) over all ``seq_lens[b]`` cached tokens, causal with respect to
    absolute positions (csrc/src/context_attention_forward.cpp:49)."""
    T, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    G = Hq // Hkv
    out = torch.zeros_like(q)
    lse = torch.full((Hq, T), float("-inf"), dtype=torch.float32, device=q.device)
    for b in range(block_tables.shape[0]):
        q0, q1 = int(cu_q[b]), int(cu_q[b + 1])
        n = int(seq_lens[b])
        ql = q1 - q0
        if ql == 0 or n == 0:
            continue
        k, v = _gather_kv(k_cache, v_cache, block_tables[b], n)
        k = k.repeat_interleave(G, dim=1)
        v = v.repeat_interleave(G, dim=1)
        s = torch.einsum("qhd,nhd->hqn", q[q0:q1].float(), k) * scale
        qpos = torch.arange(n - ql, n, device=q.device)[:, None]
        kpos = torch.arange(n, device=q.device)[None, :]
        if alibi_slopes is not None:
            s = s + alibi_slopes.float()[:, None, None] * (kpos - qpos).float()[None]
        mask = torch.ones(ql, n, dtype=torch.bool, device=q.device)
        if causal:
            mask &= kpos <= qpos
        if window > 0:
            mask &= kpos > qpos - window
        s = s.masked_fill(~mask[None], float("-inf"))
        l = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - l[..., None])
        p = torch.nan_to_num(p, nan=0.0)
        out[q0:q1] = torch.einsum("hqn,nhd->qhd", p, v).to(q.dtype)
        lse[:, q0:q1] = l
    return (out, lse) if return_lse else out


def merge_attn_states(p_out: torch.Tensor, p_lse: torch.Tensor, s_out: torch.Tensor,
                      s_lse: torch.Tensor):
    """LSE-weighted merge; outs ``[T, H, D]``, lses ``[H, T]``
    (vllm_gcu/v1/attention/flash_attn.py:165-177)."""
    pl = torch.where(torch.isposinf(p_lse), torch.full_like(p_lse, float("-inf")), p_lse)
    sl = torch.where(torch.isposinf(s_lse), torch.full_like(s_lse, float("-inf")), s_lse)
    m = torch.maximum(pl, sl)
    ep = torch.exp(pl - m)
    es = torch.exp(sl - m)
    ep = torch.nan_to_num(ep, nan=0.0)
    es = torch.nan_to_num(es, nan=0.0)
    den = ep + es
    wp = torch.where(den > 0, ep / den, torch.zeros_like(den)).transpose(0, 1)[..., None]
    ws = torch.where(den > 0, es / den, torch.zeros_like(den)).transpose(0, 1)[..., None]
    out = (p_out.float() * wp + s_out.float() * ws).to(p_out.dtype)
    lse = torch.where(den > 0, m + torch.log(den), torch.full_like(m, float("-inf")))
    return out, lse


def dense_causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float
                           ) -> torch.Tensor:
    """No-cache oracle: q ``[S, Hq, D]``, k/v ``[S, Hkv, D]``, one sequence."""
    S, Hq, D = q.shape
    G = Hq // k.shape[1]
    kf = k.float().repeat_interleave(G, dim=1)
    vf = v.float().repeat_interleave(G, dim=1)
    s = torch.einsum("qhd,nhd->hqn", q.float(), kf) * scale
    mask = torch.tril(torch.ones(S, S, dtype=torch.bool, device=q.device))
    s = s.masked_fill(~mask[None], float("-inf"))
    return torch.einsum("hqn,nhd->qhd", torch.softmax(s, -1), vf).to(q.dtype)


# ---------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None
         ) -> torch.Tensor:
    """``a [M,K] @ b[N,K]^T`` with fp32 accumulation."""
    y = a.float() @ b.float().t()
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or a.dtype)


#: rows per block of the gate / up interleaving that the fused SiLU-mul GEMM epilogues expect:
#: 32 gate rows, the matching 32 up rows, and so on, so that every 64-column group of an output
#: tile holds matching halves whatever the tile width (64, 128 or 256)
GATE_UP_BLOCK = 32


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor, block: int = GATE_UP_BLOCK
                       ) -> torch.Tensor:
    """Weight layout of the fused SiLU-mul GEMM epilogue: alternating blocks of
    ``block`` gate rows and the matching ``block`` up rows."""
    I, K = w_gate.shape
    assert I % block == 0
    g = w_gate.reshape(I // block, block, K)
    u = w_up.reshape(I // block, block, K)
    return torch.stack([g, u], dim=1).reshape(2 * I, K)


def deinterleave_gate_up(w_inter: torch.Tensor, block: int = GATE_UP_BLOCK) -> torch.Tensor:
    """Inverse of :func:`interleave_gate_up` along dim -2: ``[..., 2 I, K]`` interleaved ->
    ``[..., 2 I, K]`` with all gate rows first."""
    *lead, N2, K = w_inter.shape
    w4 = w_inter.reshape(*lead, N2 // (2 * block), 2, block, K)
    g = w4[..., 0, :, :].reshape(*lead, N2 // 2, K)
    u = w4[..., 1, :, :].reshape(*lead, N2 // 2, K)
    return torch.cat([g, u], dim=-2)


def gemm_silu_mul_interleaved(a: torch.Tensor, w_inter: torch.Tensor,
                              block: int = GATE_UP_BLOCK) -> torch.Tensor:
    y = a.float() @ w_inter.float().t()
    M, N2 = y.shape
    y = y.reshape(M, N2 // (2 * block), 2, block)
    return (F.silu(y[:, :, 0]) * y[:, :, 1]).reshape(M, N2 // 2).to(a.dtype)


# ---------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------
def apply_top_k_top_p(logits: torch.Tensor, k: Optional[torch.Tensor],
                      p: Optional[torch.Tensor]) -> torch.Tensor:
    """Masks to -inf everything outside top-k and the nucleus-p
    (vllm_gcu/kernels/sampler.py:132-134; upstream semantics: ascending sort, drop the
    tail whose cumulative probability is <= 1 - p, always keep the best token)."""
    lg = logits.float().clone()
    V = lg.shape[-1]
    if k is not None:
        kk = k.long().clamp(min=1, max=V)
        kk = torch.where(k.long() <= 0, torch.full_like(kk, V), kk)
        srt = lg.sort(dim=-1, descending=True).values
        thr = srt.gather(-1, (kk - 1)[:, None])
        lg = lg.masked_fill(lg < thr, float("-inf"))
    if p is not None:
        srt, idx = lg.sort(dim=-1, descending=False)
        probs = srt.softmax(-1)
        cum = probs.cumsum(-1)
        mask = cum <= (1.0 - p.float())[:, None]
        mask[:, -1] = False
        srt = srt.masked_fill(mask, float("-inf"))
        lg = torch.empty_like(lg).scatter_(-1, idx, srt)
    return lg.to(logits.dtype)


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor],
           top_k: Optional[torch.Tensor], top_p: Optional[torch.Tensor],
           noise: Optional[torch.Tensor] = None,
           generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Greedy where temperature <= 0, else ``argmax(softmax(masked / T) / q)`` with
    ``q ~ Exp(1)`` (vllm_gcu/kernels/sampler.py:102-129)."""
    lg = logits.float()
    greedy = lg.argmax(-1)
    if temperature is None:
        return greedy
    t = temperature.float()
    safe_t = torch.where(t > 0, t, torch.ones_like(t))
    scaled = lg / safe_t[:, None]
    masked = apply_top_k_top_p(scaled, top_k, top_p).float()
    if noise is None:
        noise = torch.empty_like(masked).exponential_(generator=generator)
    probs = masked.softmax(-1)
    sampled = (probs / noise.float().clamp_min(1e-30)).argmax(-1)
    return torch.where(t > 0, sampled, greedy)


# ---------------------------------------------------------------------------
# step bookkeeping
# ---------------------------------------------------------------------------
def advance_step(num_seqs: int, num_queries: int, block_size: int, input_tokens: torch.Tensor,
                 sampled: torch.Tensor, positions: torch.Tensor, seq_lens: torch.Tensor,
                 slot_mapping: torch.Tensor, block_tables: torch.Tensor) -> None:
    """tests/kernels/test_advance_step.py:8-27 semantics, in place."""
    n = num_queries
    sl = seq_lens[:n].long()
    input_tokens[:n] = sampled.reshape(-1)[:n]
    positions[:n] = sl
    blk = block_tables[torch.arange(n, device=sl.device), (sl // block_size)].long()
    slot_mapping[:n] = blk * block_size + sl % block_size
    seq_lens[:n] = (sl + 1).to(seq_lens.dtype)
    if num_seqs > n:
        slot_mapping[n:num_seqs] = -1


# ---------------------------------------------------------------------------
# mixture of experts
# ---------------------------------------------------------------------------
def topk_softmax(gating: torch.Tensor, k: int, renormalize: bool
                 ) -> tuple[torch.Tensor, torch.Tensor]:
    """softmax over experts then top-k (csrc/src/topk_softmax.cpp:32).  Returns
    (weights fp32 ``[T, k]``, ids int32 ``[T, k]``)."""
    probs = torch.softmax(gating.float(), dim=-1)
    w, ids = probs.topk(k, dim=-1)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return w, ids.to(torch.int32)


def grouped_topk(gating: torch.Tensor, k: int, renormalize: bool, n_group: int, topk_group: int,
                 bias: Optional[torch.Tensor] = None, scoring: str = "softmax",
                 routed_scaling_factor: float = 1.0) -> tuple[torch.Tensor, torch.Tensor]:
    """DeepSeek grouped routing (csrc/src/fused_grouped_topk.cpp:35,
    vllm_gcu/kernels/fused_moe.py:234-267): score = sigmoid | softmax; selection uses
    ``score + bias``; group score = sum of the top-2 biased scores of the group (max without
    bias); keep ``topk_group`` groups, then top-k experts; the returned weights are the
    unbiased scores (optionally renormalised)."""
    g = gating.float()
    scores = torch.sigmoid(g) if scoring == "sigmoid" else torch.softmax(g, dim=-1)
    T, E = scores.shape
    sel = scores + bias.float()[None] if bias is not None else scores
    grp = sel.view(T, n_group, E // n_group)
    if bias is not None:
        gscore = grp.topk(2, dim=-1).values.sum(-1)
    else:
        gscore = grp.max(-1).values
    gidx = gscore.topk(topk_group, dim=-1).indices
    gmask = torch.zeros_like(gscore).scatter_(1, gidx, 1.0)
    mask = gmask[:, :, None].expand(T, n_group, E // n_group).reshape(T, E)
    masked = sel.masked_fill(mask == 0, float("-inf"))
    ids = masked.topk(k, dim=-1).indices
    w = scores.gather(1, ids)
    if renormalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * routed_scaling_factor, ids.to(torch.int32)


def moe_align_block_size(topk_ids: torch.Tensor, num_experts: int, block: int,
                         valid_tokens: Optional[int] = None,
                         expert_map: Optional[torch.Tensor] = None):
    """Stable counting sort of the flattened (token, slot) pairs by expert; every expert
    segment is padded to a multiple of ``block`` with the sentinel ``numel``.  Returns
    (sorted_ids, expert_ids per block, num_tokens_post_pad) like
    csrc/src/moe_align_block_size.cpp:37; ``valid_tokens`` limits the input to its first
    rows (``_pad`` variant) and ``expert_map`` maps global to local expert ids with -1 for
    experts that live elsewhere (``exts_`` variant), whose pairs are dropped."""
    flat = topk_ids.reshape(-1).long()
    numel = flat.numel()
    k = topk_ids.shape[1]
    if valid_tokens is not None:
        flat = flat[: valid_tokens * k]
    idx = torch.arange(flat.numel(), device=flat.device)
    if expert_map is not None:
        flat = expert_map.long()[flat]
        keep = flat >= 0
        flat, idx = flat[keep], idx[keep]
    sorted_ids, expert_ids = [], []
    for e in range(num_experts):
        sel = idx[flat == e]
        n = sel.numel()
        if n == 0:
            continue
        pad = (-n) % block
        sorted_ids.append(sel)
        if pad:
            sorted_ids.append(torch.full((pad,), numel, device=flat.device, dtype=idx.dtype))
        expert_ids += [e] * ((n + pad) // block)
    if sorted_ids:
        sid = torch.cat(sorted_ids)
    else:
        sid = idx[:0]
    return (sid.to(torch.int32),
            torch.tensor(expert_ids, dtype=torch.int32, device=flat.device),
            torch.tensor([sid.numel()], dtype=torch.int32, device=flat.device))


def fused_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_w: torch.Tensor,
                  topk_ids: torch.Tensor, expert_map: Optional[torch.Tensor] = None,
                  act: str = "silu") -> torch.Tensor:
    """``sum_k w_k * down_e(act(gate_e(x)) * up_e(x))`` with ``w13 [E, 2I, H]`` (gate rows
    first) and ``w2 [E, H, I]`` (csrc/src/fused_moe_kernel.cpp:43-63 +
    vllm_gcu/kernels/modular_experts.py:81-288).  With ``expert_map`` only local experts
    contribute (others add zero), which is what one EP rank computes."""
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    ids = topk_ids.long()
    if expert_map is not None:
        ids = expert_map.long()[ids]
    E = w13.shape[0]
    xf = x.float()
    for e in range(E):
        tok, slot = (ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = xf[tok] @ w13[e].float().t()
        h = act_and_mul(h.to(x.dtype), act).float()
        y = h @ w2[e].float().t()
        out.index_add_(0, tok, y * topk_w[tok, slot].float()[:, None])
    return out.to(x.dtype)


def moe_sum(x: torch.Tensor, valid_rows: Optional[int] = None) -> torch.Tensor:
    """``[M, topk, K] -> [M, K]`` (csrc/src/moe_sum.cpp:75)."""
    out = x.float().sum(1).to(x.dtype)
    if valid_rows is not None:
        out[valid_rows:] = 0
    return out


def get_ep_indices(topk_ids: torch.Tensor, experts_per_rank: int, ep: int):
    """Per destination rank: the tokens that have at least one selected expert there
    (a token is listed once per rank).  Returns (count ``[ep]``, token indices rank-major,
    total) as in tests/kernels/test_get_ep_indices.py:5-53."""
    T = topk_ids.shape[0]
    rank_of = (topk_ids.long() // experts_per_rank)
    counts, idxs = [], []
    for r in range(ep):
        hit = (rank_of == r).any(dim=1).nonzero(as_tuple=True)[0]
        counts.append(hit.numel())
        idxs.append(hit)
    idx = torch.cat(idxs) if idxs else torch.zeros(0, dtype=torch.long)
    return (torch.tensor(counts, dtype=torch.int32, device=topk_ids.device), idx.to(torch.int32),
            int(sum(counts)))


def eplb_map_to_physical(topk_ids: torch.Tensor, log2phy: torch.Tensor,
                         replica_count: torch.Tensor, load: Optional[torch.Tensor] = None
                         ) -> torch.Tensor:
    """Logical -> physical expert ids; the replica is chosen from the (token, slot)
    position modulo the replica count, and the per-physical-expert load histogram is
    updated (csrc/src/eplb_map_to_physical_and_record.cpp:36,
    vllm_gcu/kernels/quantization/utils.py:23-54)."""
    ids = topk_ids.long()
    T, k = ids.shape
    pos = torch.arange(T * k, device=ids.device).view(T, k)
    rep = pos % replica_count.long()[ids]
    phys = log2phy.long()[ids, rep]
    if load is not None:
        load.index_add_(0, phys.reshape(-1), torch.ones(T * k, dtype=load.dtype,
                                                        device=load.device))
    return phys.to(topk_ids.dtype)


# ---------------------------------------------------------------------------
# speculative decoding (vllm_gcu/patch/patch_0_9_2/rejection_sampler.py:11-120)
# ---------------------------------------------------------------------------
def rejection_greedy_sample(draft_ids: torch.Tensor, target_argmax: torch.Tensor,
                            bonus_ids: torch.Tensor, num_draft: torch.Tensor) -> torch.Tensor:
    """Greedy verification.  draft_ids ``[B, S]`` (padded), target_argmax ``[B, S]`` (argmax of
    the target at each draft position), bonus ``[B]``.  Output ``[B, S + 1]`` int32 filled
    with -1: accepted prefix, then the target's token at the first mismatch, or the bonus
    token when every draft token was accepted."""
    B, S = draft_ids.shape
    out = torch.full((B, S + 1), -1, dtype=torch.int32, device=draft_ids.device)
    for b in range(B):
        n = int(num_draft[b])
        rejected = False
        for i in range(n):
            out[b, i] = target_argmax[b, i]
            if int(draft_ids[b, i]) != int(target_argmax[b, i]):
                rejected = True
                break
        if not rejected:
            out[b, n] = bonus_ids[b]
    return out


def rejection_random_sample(draft_ids: torch.Tensor, draft_probs: Optional[torch.Tensor],
                            target_probs: torch.Tensor, bonus_ids: torch.Tensor,
                            recovered_ids: torch.Tensor, uniform: torch.Tensor,
                            num_draft: torch.Tensor) -> torch.Tensor:
    """Standard speculative rejection sampling: accept draft token x with probability
    ``min(1, p_target(x) / p_draft(x))`` (``p_draft = 1`` for draft-free proposers such as
    n-gram), otherwise emit the recovered token.  Shapes: probs ``[B, S, V]``,
    uniform ``[B, S]``."""
    B, S = draft_ids.shape
    out = torch.full((B, S + 1), -1, dtype=torch.int32, device=draft_ids.device)
    for b in range(B):
        n = int(num_draft[b])
        rejected = False
        for i in range(n):
            x = int(draft_ids[b, i])
            pt = float(target_probs[b, i, x])
            pd = 1.0 if draft_probs is None else float(draft_probs[b, i, x])
            if pd > 0 and pt / pd >= float(uniform[b, i]):
                out[b, i] = x
            else:
                out[b, i] = recovered_ids[b, i]
                rejected = True
                break
        if not rejected:
            out[b, n] = bonus_ids[b]
    return out


def sample_recovered_tokens(draft_ids: torch.Tensor, draft_probs: Optional[torch.Tensor],
                            target_probs: torch.Tensor, noise: torch.Tensor) -> torch.Tensor:
    """Recovered token at every draft position: argmax of ``max(0, p_t - p_d) / q`` with
    ``q ~ Exp(1)`` (for draft-free proposers the draft token itself is excluded)."""
    if draft_probs is None:
        adj = target_probs.clone()
        adj.scatter_(-1, draft_ids.long()[..., None], 0.0)
    else:
        adj = (target_probs - draft_probs).clamp_min(0.0)
    return (adj / noise.clamp_min(1e-30)).argmax(-1).to(torch.int32)


def expand_batch_to_tokens(x: torch.Tensor, cu_num_tokens: torch.Tensor,
                           replace_from: int = 0, replace_to: int = 0) -> torch.Tensor:
    """Repeats ``x[b]`` for each token of request b (``cu_num_tokens`` inclusive prefix
    sums), optionally replacing one value."""
    counts = torch.diff(cu_num_tokens, prepend=cu_num_tokens.new_zeros(1))
    y = torch.repeat_interleave(x, counts.long())
    if replace_from != replace_to:
        y = torch.where(y == replace_from, torch.full_like(y, replace_to), y)
    return y


# ---------------------------------------------------------------------------
# multi-LoRA (vllm_gcu/lora/lora_ops.py:10-139, csrc/src/dispatch_bgmv.cpp:19)
# ---------------------------------------------------------------------------
def bgmv(y: torch.Tensor, x: torch.Tensor, w: torch.Tensor, indices: torch.Tensor,
         scale: float = 1.0, y_offset: int = 0, y_slice: Optional[int] = None) -> torch.Tensor:
    """``y[t, off:off+n] += scale * w[idx[t]] @ x[t]`` for ``idx[t] >= 0``;
    ``w [L, h_out, h_in]`` (a leading singleton layer dim is accepted)."""
    if w.dim() == 4:
        w = w[:, 0]
    n = w.shape[1] if y_slice is None else y_slice
    valid = indices >= 0
    if valid.any():
        wi = w[indices[valid].long()].float()
        upd = torch.einsum("tnk,tk->tn", wi, x[valid].float()) * scale
        y[valid, y_offset:y_offset + n] += upd.to(y.dtype)
    return y
