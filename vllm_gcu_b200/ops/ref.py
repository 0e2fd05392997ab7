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
                           k_scale=None, v_scale=None) -> torch.Tensor:
    """One query token per sequence; q ``[B, Hq, D]``; flash-layout caches
    (csrc/src/paged_attention_v1.cpp:68 semantics on the layout of
    csrc/src/reshape_and_cache_flash.cpp)."""
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
        p = torch.softmax(s, dim=-1)
        out[b] = torch.einsum("hn,nhd->hd", p, v).to(q.dtype)
    return out


def varlen_prefill_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                             block_tables: torch.Tensor, cu_q: torch.Tensor,
                             seq_lens: torch.Tensor, scale: float, causal: bool = True,
                             window: int = 0, return_lse: bool = False):
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


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor, block: int = 128
                       ) -> torch.Tensor:
    """Weight layout of the fused SiLU-mul GEMM epilogue: alternating blocks of
    ``block`` gate rows and the matching ``block`` up rows."""
    I, K = w_gate.shape
    assert I % block == 0
    g = w_gate.reshape(I // block, block, K)
    u = w_up.reshape(I // block, block, K)
    return torch.stack([g, u], dim=1).reshape(2 * I, K)


def gemm_silu_mul_interleaved(a: torch.Tensor, w_inter: torch.Tensor, block: int = 128
                              ) -> torch.Tensor:
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
