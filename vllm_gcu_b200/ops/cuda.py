"""Thin wrappers that launch the sm_100a kernels of ``_b200.so`` on torch tensors.

All functions take CUDA tensors, launch on the current torch stream and never
synchronise.  Argument checking that would cost a device sync is left to the
kernels' own guards (status word, see ``_native.check_status``).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import _native as N
from ._native import DTYPE_CODE, call, ptr, stream_ptr

EPI_NONE, EPI_BIAS, EPI_SILU_MUL, EPI_RESIDUAL, EPI_FP32 = 0, 1, 2, 3, 4

NORM_QMODES = {None: 0, "fp8_static": 1, "fp8_token": 2, "fp8_group128": 3,
               "int8_static": 4, "int8_token": 5}
ACT_CODES = {"silu": 0, "gelu": 1, "gelu_tanh": 2, "fatrelu": 3, "gelu_new": 4,
             "gelu_fast": 5, "gelu_quick": 6, "identity": 7}
ACT_QUANT = {None: 0, "fp8_group128": 1, "fp8_static": 2, "int8_static": 3, "int8_asym": 4}
FP8 = torch.float8_e4m3fn
#: route head-dim-128 decode attention through the TMA-fed kernel (False: cp.async kernel)
USE_TMA_DECODE = True


def _rowmajor_2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        t = t.reshape(-1, t.shape[-1])
    if t.stride(-1) != 1:
        t = t.contiguous()
    return t


# ---------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------
# ---------------------------------------------------------------------------
# run-time oracle: selected ops are recomputed with the torch reference and compared
# ---------------------------------------------------------------------------
class OracleMismatch(AssertionError):
    """A native op disagreed with its torch reference (``VLLM_B200_ORACLE``)."""


def oracle_enabled(name: str) -> bool:
    """``VLLM_B200_ORACLE=all`` or a comma-separated list of op names switches the check on.
    The reference compiles the same idea into its extension as a debug layer: CPU
    re-implementations and ``*Check`` comparators wrapped around 22 ops
    (csrc/src/native_vllm.h:37-446)."""
    from .. import envs
    sel = envs.ORACLE
    return sel is not None and ("all" in sel or name in sel)


def oracle_compare(name: str, got: torch.Tensor, want: torch.Tensor, rtol: float = 3e-2,
                   atol: float = 3e-2) -> None:
    g, w = got.float(), want.float().to(got.device)
    bad = (g - w).abs() > atol + rtol * w.abs()
    if bool(bad.any()):
        idx = int(bad.flatten().nonzero()[0])
        raise OracleMismatch(
            f"{name}: {int(bad.sum())} of {bad.numel()} elements differ from the reference "
            f"(first at flat index {idx}: got {g.flatten()[idx].item():.6g}, "
            f"want {w.flatten()[idx].item():.6g})")


# Decode-sized activations (M <= 256) take the weight-streaming kernel of gemm_skinny.cu.
USE_PAIR_GEMM = True            # 256 x 256 tile per CTA pair, cta_group::2 (gemm_pair.cu)
USE_PAIR_SPLIT = False          # K split over pairs for few-tile decode GEMMs (gemm_pair.cu)
PAIR_MIN_M = 129                # below the large-M threshold the pair kernel runs when ...
PAIR_MIN_TILES = 48             # ... its tiles can occupy most of the 74 SM pairs
USE_WIDE2_GEMM = True           # persistent 256 x 256 tiles for large M (gemm_skinny.cu)
WIDE2_MIN_M = 1024
USE_SKINNY_GEMM = True
SKINNY_ALLOW_SPLIT = False      # K-split plans lose to the persistent-tile kernel (measured)
SKINNY_SPLIT2_MAX_M = 128       # up to this many rows a two-kernel K split is planned (o_proj /
                                # down_proj at M = 64: 15.7 -> 14.9 us, 43.2 -> 29.5 us)
SKINNY_MAX_M = 256
_SKINNY_WS: dict = {}


_SM_COUNT = 0


def _wide2_pays(M: int, Nn: int) -> bool:
    """256 x 256 tiles move a third less data per flop (measured +12 % on 8192 x 28672 x 4096)
    but leave a larger ragged last wave; take them unless that costs more than it gains."""
    global _SM_COUNT
    if _SM_COUNT == 0:
        _SM_COUNT = max(1, int(N.lib().b200_sm_count()))
    sms = _SM_COUNT
    t2 = -(-M // 256) * (Nn // 256)
    t1 = -(-M // 128) * (Nn // 256)
    eff2 = t2 / (-(-t2 // sms) * sms)
    eff1 = t1 / (-(-t1 // sms) * sms)
    return eff2 * 1.15 >= eff1


def _skinny_workspace(device: torch.device):
    """Per (device, stream) split-K workspace: fp32 partial sums + zeroed counters."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    w = _SKINNY_WS.get(key)
    if w is None:
        nbytes = ctypes.c_longlong()
        nctr = ctypes.c_int()
        N.lib().b200_gemm_skinny_workspace(1 << 20, ctypes.byref(nbytes), ctypes.byref(nctr))
        w = (torch.empty(nbytes.value // 4, dtype=torch.float32, device=device),
             torch.zeros(nctr.value, dtype=torch.int32, device=device))
        _SKINNY_WS[key] = w
    return w


_PAIR_SPLIT_WS: dict = {}


def _pair_split_workspace(device: torch.device):
    """Per (device, stream) workspace of the pair kernel's K split: fp32 partial sums and
    zeroed counters; None when the device cannot co-schedule clusters of two."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    w = _PAIR_SPLIT_WS.get(key, 0)
    if w == 0:
        nfl, nctr = ctypes.c_longlong(), ctypes.c_int()
        rc = N.lib().b200_gemm_pair_split_workspace(ctypes.byref(nfl), ctypes.byref(nctr))
        w = None if rc != 0 else (
            torch.empty(nfl.value, dtype=torch.float32, device=device),
            torch.zeros(nctr.value, dtype=torch.int32, device=device))
        _PAIR_SPLIT_WS[key] = w
    return w


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None,
              bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
              epilogue: int = EPI_NONE) -> torch.Tensor:
    res = _gemm_bf16(a, b, out, bias, residual, epilogue)
    if oracle_enabled("gemm_bf16") and not torch.cuda.is_current_stream_capturing():
        from . import ref
        a2 = a.reshape(-1, a.shape[-1])
        want = ref.gemm(a2, b, bias=bias, residual=residual, out_dtype=torch.float32)
        if bias is None and residual is None and epilogue == EPI_SILU_MUL:
            w4 = want.view(want.shape[0], -1, 2, ref.GATE_UP_BLOCK)
            want = (torch.nn.functional.silu(w4[:, :, 0]) * w4[:, :, 1]).reshape(want.shape[0], -1)
        oracle_compare("gemm_bf16", res, want, 3e-2, 3e-2 * max(1.0, float(want.abs().mean())))
    return res


def _gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None,
               bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
               epilogue: int = EPI_NONE) -> torch.Tensor:
    """``out[M,N] = a[M,K] @ b[N,K]^T`` on the tcgen05 path (bf16 in, fp32 accumulate).

    epilogue EPI_SILU_MUL expects ``b`` interleaved by ``ref.interleave_gate_up`` and
    yields ``[M, N/2]``; EPI_FP32 writes fp32."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    a = _rowmajor_2d(a)
    M, K = a.shape
    Nn = b.shape[0]
    assert b.shape[1] == K and b.stride(1) == 1
    if bias is not None:
        epilogue = EPI_BIAS
    if residual is not None:
        epilogue = EPI_RESIDUAL
    out_cols = Nn // 2 if epilogue == EPI_SILU_MUL else Nn
    if out is None:
        out = torch.empty((M, out_cols), device=a.device,
                          dtype=torch.float32 if epilogue == EPI_FP32 else torch.bfloat16)
    assert out.stride(-1) == 1 and out.shape[-1] == out_cols
    if (K % 8 or Nn % 8 or a.stride(0) % 8 or b.stride(0) % 8 or out.stride(0) % 8) \
            and epilogue != EPI_SILU_MUL:
        # rows that are not a multiple of 16 bytes cannot be described to TMA (a router over
        # four experts, an odd head count): the library GEMM takes these rare, tiny shapes
        y = torch.matmul(a.float() if epilogue == EPI_FP32 else a,
                         (b.float() if epilogue == EPI_FP32 else b).t())
        if bias is not None:
            y = y + bias
        if residual is not None:
            y = y + residual
        out.copy_(y)
        return out
    if (USE_PAIR_GEMM and PAIR_MIN_M <= M < WIDE2_MIN_M and Nn % 256 == 0 and K % 64 == 0
            and epilogue in (EPI_NONE, EPI_BIAS, EPI_SILU_MUL)
            and -(-M // 256) * (Nn // 256) >= PAIR_MIN_TILES):
        # enough 256 x 256 tiles to occupy the SM pairs (gate_up, LM head at decode batch sizes;
        # graph-replay timing at 256 rows: gate_up 62.5 -> 57.9 us, LM head 266 -> 228 us)
        rc = N.lib().b200_gemm_pair(ptr(a), a.stride(0), ptr(b), b.stride(0), ptr(out),
                                    out.stride(0), M, Nn, K, ptr(bias), epilogue, stream_ptr())
        N.launch_count += 1
        if rc == 0:
            return out
        if rc != -20:
            raise N.NativeError(f"b200_gemm_pair failed with code {rc}")
    if (USE_PAIR_SPLIT and PAIR_MIN_M <= M <= 512 and Nn % 256 == 0 and K % 64 == 0
            and epilogue in (EPI_NONE, EPI_BIAS, EPI_SILU_MUL)
            and -(-M // 256) * (Nn // 256) < PAIR_MIN_TILES):
        # few 256 x 256 tiles (qkv, o_proj, down_proj at decode batch sizes): K split over pairs
        wsp = _pair_split_workspace(a.device)
        if wsp is not None:
            rc = N.lib().b200_gemm_pair_split(ptr(a), a.stride(0), ptr(b), b.stride(0), ptr(out),
                                              out.stride(0), M, Nn, K, ptr(bias), epilogue,
                                              ptr(wsp[0]), ptr(wsp[1]), stream_ptr())
            N.launch_count += 1
            if rc == 0:
                return out
            if rc != -20:
                raise N.NativeError(f"b200_gemm_pair_split failed with code {rc}")
    silu_256 = epilogue != EPI_SILU_MUL or Nn % 256 == 0     # these two kernels: 256-wide tiles
    if M <= SKINNY_MAX_M and USE_SKINNY_GEMM and silu_256 \
            and epilogue in (EPI_NONE, EPI_BIAS, EPI_SILU_MUL):
        ws, ctr = _skinny_workspace(a.device)
        rc = N.lib().b200_gemm_skinny(
            ptr(a), a.stride(0), ptr(b), b.stride(0), ptr(out), out.stride(0), M, Nn, K,
            ptr(bias), epilogue, ptr(ws), ptr(ctr),
            2 if (M <= SKINNY_SPLIT2_MAX_M and not SKINNY_ALLOW_SPLIT) else int(SKINNY_ALLOW_SPLIT),
            stream_ptr())
        N.launch_count += 1
        if rc == 0:
            return out
        if rc != -20:
            raise N.NativeError(f"b200_gemm_skinny failed with code {rc}")
    if (USE_PAIR_GEMM and M >= WIDE2_MIN_M and Nn % 256 == 0 and K % 64 == 0
            and epilogue in (EPI_NONE, EPI_BIAS, EPI_SILU_MUL) and _wide2_pays(M, Nn)):
        # one 256 x 256 tile per pair of CTAs (gemm_pair.cu); -20 = shape or device not covered
        rc = N.lib().b200_gemm_pair(ptr(a), a.stride(0), ptr(b), b.stride(0), ptr(out),
                                    out.stride(0), M, Nn, K, ptr(bias), epilogue, stream_ptr())
        N.launch_count += 1
        if rc == 0:
            return out
        if rc != -20:
            raise N.NativeError(f"b200_gemm_pair failed with code {rc}")
    if (USE_WIDE2_GEMM and M >= WIDE2_MIN_M and Nn % 256 == 0
            and epilogue in (EPI_NONE, EPI_BIAS, EPI_SILU_MUL) and _wide2_pays(M, Nn)):
        rc = N.lib().b200_gemm_wide2(ptr(a), a.stride(0), ptr(b), b.stride(0), ptr(out),
                                     out.stride(0), M, Nn, K, ptr(bias), epilogue, stream_ptr())
        N.launch_count += 1
        if rc == 0:
            return out
        if rc != -20:
            raise N.NativeError(f"b200_gemm_wide2 failed with code {rc}")
    call("b200_gemm_bf16", ptr(a), a.stride(0), ptr(b), b.stride(0), ptr(out), out.stride(0),
         M, Nn, K, ptr(bias), ptr(residual), residual.stride(0) if residual is not None else 0,
         epilogue, stream_ptr())
    return out


# ---------------------------------------------------------------------------
# norm / activation
# ---------------------------------------------------------------------------
def norm(x: torch.Tensor, weight: torch.Tensor, eps: float,
         residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
         quant: Optional[str] = None, scale: Optional[torch.Tensor] = None,
         valid_rows: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
         layer_norm: bool = False):
    """RMSNorm / LayerNorm family.  With ``residual`` the residual tensor is updated in
    place.  Returns ``out`` or ``(out, scales)`` for the dynamic quant modes."""
    x2 = _rowmajor_2d(x)
    T, H = x2.shape
    qmode = NORM_QMODES[quant]
    scale_out = None
    if out is None:
        if qmode == 0:
            out = torch.empty_like(x2)
        elif qmode in (1, 2, 3):
            out = torch.empty((T, H), device=x.device, dtype=FP8)
        else:
            out = torch.empty((T, H), device=x.device, dtype=torch.int8)
    if qmode in (2, 5):
        scale_out = torch.empty((T, 1), device=x.device, dtype=torch.float32)
    elif qmode == 3:
        scale_out = torch.empty((T, H // 128), device=x.device, dtype=torch.float32)
    res2 = None
    if residual is not None:
        res2 = residual if residual.dim() == 2 else residual.view(-1, H)
    call("b200_norm", ptr(x2), x2.stride(0), ptr(res2), res2.stride(0) if res2 is not None else 0,
         ptr(weight), ptr(bias), ptr(out), out.stride(0) if out.dim() == 2 else H,
         ptr(scale_out), ptr(scale), ptr(valid_rows), T, H, float(eps), DTYPE_CODE[x.dtype],
         qmode, int(layer_norm), stream_ptr())
    out = out.view(x.shape) if out.shape != x.shape and out.numel() == x.numel() else out
    return (out, scale_out) if scale_out is not None else out


def activation(x: torch.Tensor, act: str = "silu", mode: str = "act_mul",
               out: Optional[torch.Tensor] = None, quant: Optional[str] = None,
               scale: Optional[torch.Tensor] = None, azp: Optional[torch.Tensor] = None,
               valid_rows: Optional[torch.Tensor] = None, threshold: float = 0.0):
    """Gated (``act_mul`` / ``mul_act``) or plain activation, optionally quantising."""
    x2 = _rowmajor_2d(x)
    T = x2.shape[0]
    m = {"act_mul": 0, "mul_act": 1, "plain": 2}[mode]
    d = x2.shape[1] if m == 2 else x2.shape[1] // 2
    q = ACT_QUANT[quant]
    scale_out = None
    if out is None:
        if q == 0:
            out = torch.empty((T, d), device=x.device, dtype=x.dtype)
        elif q in (1, 2):
            out = torch.empty((T, d), device=x.device, dtype=FP8)
        else:
            out = torch.empty((T, d), device=x.device, dtype=torch.int8)
    if q == 1:
        scale_out = torch.empty((T, d // 128), device=x.device, dtype=torch.float32)
    call("b200_activation", ptr(x2), x2.stride(0), ptr(out), out.stride(0), ptr(scale_out),
         ptr(scale), ptr(azp), ptr(valid_rows), T, d, ACT_CODES[act], m, q, float(threshold),
         DTYPE_CODE[x.dtype], stream_ptr())
    if x.dim() != 2:
        out = out.view(*x.shape[:-1], d)
    return (out, scale_out) if scale_out is not None else out


# ---------------------------------------------------------------------------
# rope / cache
# ---------------------------------------------------------------------------
def rope_cache_flash(q: Optional[torch.Tensor], k: Optional[torch.Tensor],
                     v: Optional[torch.Tensor], positions: Optional[torch.Tensor],
                     cos_sin: Optional[torch.Tensor], is_neox: bool, head_size: int,
                     slot_mapping: Optional[torch.Tensor] = None,
                     k_cache: Optional[torch.Tensor] = None,
                     v_cache: Optional[torch.Tensor] = None,
                     k_scale: Optional[torch.Tensor] = None,
                     v_scale: Optional[torch.Tensor] = None) -> None:
    """In-place RoPE on q ``[T, Hq*D]`` / k ``[T, Hkv*D]`` (views with a row stride are
    fine) and paged write of k, v into ``[blocks, bs, Hkv, D]`` caches."""
    ref_t = q if q is not None else k
    T = ref_t.shape[0]
    D = head_size
    Hq = q.shape[-1] // D if q is not None else 0
    kv_src = k if k is not None else v
    Hkv = kv_src.shape[-1] // D if kv_src is not None else 0
    for t in (q, k, v):
        assert t is None or t.stride(-1) == 1
    slot_stride = head_stride = num_slots = 0
    fp8 = 0
    if slot_mapping is not None:
        nb, bs = k_cache.shape[0], k_cache.shape[1]
        assert k_cache.stride(1) * bs == k_cache.stride(0), "slots must be evenly strided"
        slot_stride, head_stride, num_slots = k_cache.stride(1), k_cache.stride(2), nb * bs
        fp8 = 1 if k_cache.dtype == FP8 else (2 if k_cache.dtype == torch.int8 else 0)
    call("b200_rope_cache_flash", ptr(q), q.stride(0) if q is not None else 0, ptr(k),
         k.stride(0) if k is not None else 0, ptr(v), v.stride(0) if v is not None else 0,
         ptr(positions), ptr(cos_sin),
         int(cos_sin is not None and cos_sin.dtype == torch.float32),
         cos_sin.shape[-1] if cos_sin is not None else 0, int(is_neox), ptr(slot_mapping),
         ptr(k_cache), ptr(v_cache), slot_stride, head_stride, num_slots, fp8, ptr(k_scale),
         ptr(v_scale), T, Hq, Hkv, D, DTYPE_CODE[ref_t.dtype], stream_ptr())


def reshape_and_cache(key, value, k_cache, v_cache, slot_mapping, k_scale=1.0, v_scale=1.0,
                      k_zp=0.0, v_zp=0.0) -> None:
    nb, H, Dx, bs, x = k_cache.shape
    D = Dx * x
    T = key.shape[0]
    key = key.reshape(T, H * D)
    value = value.reshape(T, H * D)
    qmode = 1 if k_cache.dtype == torch.int8 else (2 if k_cache.dtype == FP8 else 0)
    call("b200_reshape_and_cache", ptr(key), key.stride(0), ptr(value), value.stride(0),
         ptr(k_cache), ptr(v_cache), ptr(slot_mapping), nb * bs, T, H, D, bs, x, qmode,
         float(k_scale), float(v_scale), float(k_zp), float(v_zp), DTYPE_CODE[key.dtype],
         stream_ptr())


def mla_rope_cache(q_pe: Optional[torch.Tensor], kv: torch.Tensor, positions: torch.Tensor,
                   cos_sin: torch.Tensor, weight: torch.Tensor, eps: float,
                   kv_cache: Optional[torch.Tensor], slot_mapping: Optional[torch.Tensor],
                   kv_lora_rank: int, is_neox: bool = False,
                   scale: Optional[torch.Tensor] = None, q_out: Optional[torch.Tensor] = None,
                   want_k_pe: bool = False, want_kv_c: bool = False):
    """Fused MLA cache update.  q_pe ``[T, H, R]`` is rotated in place unless ``q_out``
    (``[T, H, *]`` view whose last R columns receive the result) is given."""
    T = kv.shape[0]
    L = kv_lora_rank
    R = kv.shape[-1] - L
    assert cos_sin.dtype == torch.float32
    k_pe_out = torch.empty((T, R), device=kv.device, dtype=kv.dtype) if want_k_pe else None
    kv_c_out = torch.empty((T, L), device=kv.device, dtype=kv.dtype) if want_kv_c else None
    H = q_pe.shape[1] if q_pe is not None else 0
    slot_stride = num_slots = 0
    fp8 = 0
    if kv_cache is not None:
        W = kv_cache.shape[-1]
        flat = kv_cache.view(-1, W)
        slot_stride, num_slots = flat.stride(0), flat.shape[0]
        fp8 = int(kv_cache.dtype == FP8)
    call("b200_mla_rope_cache", ptr(q_pe), q_pe.stride(0) if q_pe is not None else 0,
         q_pe.stride(1) if q_pe is not None else 0, ptr(q_out),
         q_out.stride(0) if q_out is not None else 0,
         q_out.stride(1) if q_out is not None else 0, ptr(kv), kv.stride(0), None, None,
         ptr(kv_cache), slot_stride, num_slots, ptr(k_pe_out), ptr(kv_c_out), ptr(positions),
         ptr(cos_sin), ptr(weight), ptr(slot_mapping if kv_cache is not None else None),
         ptr(scale), T, H, L, R, float(eps), int(is_neox), fp8, DTYPE_CODE[kv.dtype],
         stream_ptr())
    return k_pe_out, kv_c_out


def concat_and_cache_mla(kv_c, k_pe, kv_cache, slot_mapping, scale=None) -> None:
    T, L = kv_c.shape
    k_pe = k_pe.reshape(T, -1).contiguous()
    kv_c = kv_c.contiguous()
    R = k_pe.shape[-1]
    W = kv_cache.shape[-1]
    flat = kv_cache.view(-1, W)
    call("b200_mla_rope_cache", None, 0, 0, None, 0, 0, None, 0, ptr(kv_c), ptr(k_pe),
         ptr(kv_cache), flat.stride(0), flat.shape[0], None, None, None, None, None,
         ptr(slot_mapping), ptr(scale), T, 0, L, R, 0.0, 0, int(kv_cache.dtype == FP8),
         DTYPE_CODE[kv_c.dtype], stream_ptr())


def gather_cache(src_cache, block_table, cu_seq_lens, total_tokens: int, seq_starts=None,
                 out=None) -> torch.Tensor:
    nb, bs = src_cache.shape[0], src_cache.shape[1]
    W = src_cache.shape[2:].numel()
    flat = src_cache.view(nb * bs, W)
    if out is None:
        out = torch.empty((total_tokens, W), device=src_cache.device, dtype=src_cache.dtype)
    es = src_cache.element_size()
    call("b200_gather_cache", ptr(flat), ptr(out), ptr(block_table), ptr(cu_seq_lens),
         ptr(seq_starts), block_table.shape[0], block_table.shape[1], bs, W * es,
         flat.stride(0) * es, nb * bs, total_tokens, stream_ptr())
    return out


def copy_blocks(caches: Sequence[torch.Tensor], mapping: torch.Tensor) -> None:
    if mapping.numel() == 0 or not caches:
        return
    ptrs = torch.tensor([c.data_ptr() for c in caches], dtype=torch.int64,
                        device=mapping.device)
    block_bytes = caches[0].stride(0) * caches[0].element_size()
    mapping = mapping.to(torch.int64).contiguous()
    call("b200_copy_blocks", ptr(ptrs), len(caches), ptr(mapping), mapping.shape[0],
         block_bytes, stream_ptr())


def swap_blocks(src: torch.Tensor, dst: torch.Tensor, mapping_cpu: torch.Tensor) -> None:
    """mapping_cpu: int64 ``[n, 2]`` on the host; src / dst: device or pinned host."""
    m = mapping_cpu.to(torch.int64).contiguous()
    block_bytes = src.stride(0) * src.element_size()
    call("b200_swap_blocks", ptr(src), ptr(dst), ptr(m), m.shape[0], block_bytes, stream_ptr())


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------
def decode_num_splits(B: int, Hkv: int, max_seq_len: int) -> int:
    return int(N.lib().b200_decode_num_splits(B, Hkv, max_seq_len))


def paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 block_tables: torch.Tensor, seq_lens: torch.Tensor, scale: float,
                 out: Optional[torch.Tensor] = None, num_splits: int = 0,
                 workspace: Optional[tuple[torch.Tensor, torch.Tensor]] = None,
                 max_seq_len: int = 0, kv_quant: Optional[tuple] = None,
                 alibi_slopes: Optional[torch.Tensor] = None) -> torch.Tensor:
    res = _paged_decode(q, k_cache, v_cache, block_tables, seq_lens, scale, out, num_splits,
                        workspace, max_seq_len, kv_quant, alibi_slopes)
    if (oracle_enabled("paged_decode") and k_cache.element_size() > 1 and alibi_slopes is None
            and not torch.cuda.is_current_stream_capturing()):
        from . import ref
        live = seq_lens > 0
        want = ref.paged_attention_decode(q, k_cache, v_cache, block_tables,
                                          seq_lens.clamp(min=1), scale)
        oracle_compare("paged_decode", res[live], want[live])
    return res


def _paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  block_tables: torch.Tensor, seq_lens: torch.Tensor, scale: float,
                  out: Optional[torch.Tensor] = None, num_splits: int = 0,
                  workspace: Optional[tuple[torch.Tensor, torch.Tensor]] = None,
                  max_seq_len: int = 0, kv_quant: Optional[tuple] = None,
                  alibi_slopes: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q ``[B, Hq, D]`` (row stride free), caches ``[blocks, bs, Hkv, D]``.  For fp8 / int8
    caches ``kv_quant = (k_scale, v_scale, k_zero_point, v_zero_point)`` (floats).
    ``alibi_slopes`` fp32 ``[Hq]`` adds slope * (key position - query position) to the scores
    (bf16 / fp16 caches)."""
    B, Hq, D = q.shape
    nb, bs, Hkv, _ = k_cache.shape
    assert q.stride(2) == 1 and q.stride(1) == D
    if out is None:
        out = torch.empty((B, Hq, D), device=q.device, dtype=q.dtype)
    if num_splits <= 0:
        num_splits = decode_num_splits(B, Hkv, max_seq_len or block_tables.shape[1] * bs)
    tmp_out = tmp_lse = None
    if num_splits > 1:
        if workspace is None:
            tmp_out = torch.empty((B, Hq, num_splits, D), device=q.device, dtype=torch.float32)
            tmp_lse = torch.empty((B, Hq, num_splits), device=q.device, dtype=torch.float32)
        else:
            tmp_out, tmp_lse = workspace
            assert tmp_out.numel() >= B * Hq * num_splits * D
            assert tmp_lse.numel() >= B * Hq * num_splits
    args = (ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_cache),
            ptr(v_cache), k_cache.stride(1), k_cache.stride(2), nb * bs, ptr(block_tables),
            block_tables.stride(0), bs, ptr(seq_lens), ptr(tmp_out), ptr(tmp_lse), num_splits,
            B, Hq, Hkv, D, float(scale), DTYPE_CODE[q.dtype], stream_ptr())
    if alibi_slopes is not None:
        if k_cache.element_size() == 1:
            raise NotImplementedError("ALiBi attention over an 8-bit KV cache")
        assert alibi_slopes.dtype == torch.float32 and alibi_slopes.numel() == Hq
        call("b200_paged_decode_alibi", *args[:-1], ptr(alibi_slopes), stream_ptr())
        return out
    if k_cache.element_size() == 1:
        ks, vs, kz, vz = kv_quant or (1.0, 1.0, 0.0, 0.0)
        call("b200_paged_decode_q8kv", *args[:-1], 1 if k_cache.dtype == FP8 else 2, float(ks),
             float(vs), float(kz), float(vz), stream_ptr())
        return out
    if USE_TMA_DECODE and D == 128 and bs % 16 == 0 and k_cache.stride(2) == 128 \
            and k_cache.stride(1) == Hkv * 128:
        rc = N.lib().b200_paged_decode_tma(*args)      # TMA-fed variant (attention_tma.cu)
        N.launch_count += 1
        if rc == 0:
            return out
        if rc != -20:
            raise N.NativeError(f"b200_paged_decode_tma failed with code {rc}")
    call("b200_paged_decode", *args)
    return out


USE_FMHA_PREFILL = True      # tcgen05 prefill attention for bf16 / head_dim 128


def varlen_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                   block_tables: torch.Tensor, cu_q: torch.Tensor, seq_lens: torch.Tensor,
                   scale: float, num_q_tiles: int, out: Optional[torch.Tensor] = None,
                   causal: bool = True, window: int = 0, return_lse: bool = False,
                   num_q_tiles_128: Optional[int] = None, kv_quant: Optional[tuple] = None,
                   alibi_slopes: Optional[torch.Tensor] = None):
    res = _varlen_prefill(q, k_cache, v_cache, block_tables, cu_q, seq_lens, scale, num_q_tiles,
                          out, causal, window, return_lse, num_q_tiles_128, kv_quant,
                          alibi_slopes)
    if (oracle_enabled("varlen_prefill") and k_cache.element_size() > 1 and causal
            and alibi_slopes is None):
        from . import ref
        want = ref.varlen_prefill_attention(q, k_cache, v_cache, block_tables, cu_q, seq_lens,
                                            scale, window=window)
        oracle_compare("varlen_prefill", res[0] if return_lse else res, want)
    return res


def _varlen_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    block_tables: torch.Tensor, cu_q: torch.Tensor, seq_lens: torch.Tensor,
                    scale: float, num_q_tiles: int, out: Optional[torch.Tensor] = None,
                    causal: bool = True, window: int = 0, return_lse: bool = False,
                    num_q_tiles_128: Optional[int] = None, kv_quant: Optional[tuple] = None,
                    alibi_slopes: Optional[torch.Tensor] = None):
    """q ``[T, Hq, D]``; ``num_q_tiles`` >= sum_b ceil(q_len_b / 64) (host-known);
    ``num_q_tiles_128`` the same for 128-row tiles (defaults to the 64-row bound).
    ``alibi_slopes``: see ``paged_decode``."""
    T, Hq, D = q.shape
    nb, bs, Hkv, _ = k_cache.shape
    assert q.stride(2) == 1 and q.stride(1) == D
    if out is None:
        out = torch.empty((T, Hq, D), device=q.device, dtype=q.dtype)
    lse = torch.empty((Hq, T), device=q.device, dtype=torch.float32) if return_lse else None
    if alibi_slopes is not None:
        if k_cache.element_size() == 1:
            raise NotImplementedError("ALiBi attention over an 8-bit KV cache")
        assert alibi_slopes.dtype == torch.float32 and alibi_slopes.numel() == Hq
        call("b200_varlen_prefill_alibi", ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(lse),
             ptr(cu_q), ptr(seq_lens), ptr(k_cache), ptr(v_cache), k_cache.stride(1),
             k_cache.stride(2), nb * bs, ptr(block_tables), block_tables.stride(0), bs,
             block_tables.shape[0], T, num_q_tiles, Hq, Hkv, D, float(scale), int(causal),
             int(window), DTYPE_CODE[q.dtype], ptr(alibi_slopes), stream_ptr())
        return (out, lse) if return_lse else out
    if k_cache.element_size() == 1:
        ks, vs, kz, vz = kv_quant or (1.0, 1.0, 0.0, 0.0)
        call("b200_varlen_prefill_q8kv", ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(lse),
             ptr(cu_q), ptr(seq_lens), ptr(k_cache), ptr(v_cache), k_cache.stride(1),
             k_cache.stride(2), nb * bs, ptr(block_tables), block_tables.stride(0), bs,
             block_tables.shape[0], T, num_q_tiles, Hq, Hkv, D, float(scale), int(causal),
             int(window), DTYPE_CODE[q.dtype], 1 if k_cache.dtype == FP8 else 2, float(ks),
             float(vs), float(kz), float(vz), stream_ptr())
        return (out, lse) if return_lse else out
    if USE_FMHA_PREFILL and q.dtype == torch.bfloat16 and D == 128:
        # tcgen05 kernel (attention_fmha.cu); -20 = layout outside what it covers
        rc = N.lib().b200_fmha_prefill(
            ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(lse), ptr(cu_q), ptr(seq_lens),
            ptr(k_cache), ptr(v_cache), k_cache.stride(1), k_cache.stride(2), nb * bs,
            ptr(block_tables), block_tables.stride(0), bs, block_tables.shape[0], T,
            num_q_tiles_128 if num_q_tiles_128 is not None else num_q_tiles,
            Hq, Hkv, D, float(scale), int(causal), int(window), DTYPE_CODE[q.dtype], stream_ptr())
        N.launch_count += 1
        if rc == 0:
            return (out, lse) if return_lse else out
        if rc != -20:
            raise N.NativeError(f"b200_fmha_prefill failed with code {rc}")
    call("b200_varlen_prefill", ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(lse), ptr(cu_q),
         ptr(seq_lens), ptr(k_cache), ptr(v_cache), k_cache.stride(1), k_cache.stride(2),
         nb * bs, ptr(block_tables), block_tables.stride(0), bs, block_tables.shape[0], T,
         num_q_tiles, Hq, Hkv, D, float(scale), int(causal), int(window),
         DTYPE_CODE[q.dtype], stream_ptr())
    return (out, lse) if return_lse else out


WNA16_FUSED_MAX_M = 256


def gemm_wna16(x: torch.Tensor, qw: torch.Tensor, scales: torch.Tensor, zs: torch.Tensor,
               group: int, bits: int, bias: Optional[torch.Tensor] = None
               ) -> Optional[torch.Tensor]:
    """Fused de-quantise + GEMM for decode-sized inputs (gemm_wna16.cu): ``x [M, K]`` bf16,
    ``qw [N, K/2]`` (4 bit) or ``[N, K]`` (8 bit) uint8, ``scales`` / ``zs`` ``[N, K/g]`` bf16.
    Returns None when the shape is outside what the kernel covers."""
    M, K = x.shape
    Nn = qw.shape[0]
    if (M > WNA16_FUSED_MAX_M or x.dtype != torch.bfloat16 or scales.dtype != torch.bfloat16
            or x.stride(1) != 1):
        return None
    out = torch.empty((M, Nn), dtype=x.dtype, device=x.device)
    nws = int(N.lib().b200_gemm_wna16_workspace(M, Nn, K))
    ws = torch.empty(nws, dtype=torch.float32, device=x.device) if nws > 0 else None
    rc = N.lib().b200_gemm_wna16(ptr(x), x.stride(0), ptr(qw), ptr(scales), ptr(zs), ptr(bias),
                                 ptr(out), out.stride(0), M, Nn, K, int(group), int(bits),
                                 ptr(ws), stream_ptr())
    N.launch_count += 1
    if rc == -20:
        return None
    if rc != 0:
        raise N.NativeError(f"b200_gemm_wna16 failed with code {rc}")
    return out


def mla_attention_supported(q: torch.Tensor, cache: torch.Tensor, L: int) -> bool:
    """Layouts the tcgen05 MLA kernel covers: bf16, 512 + 64 wide latent rows, a power-of-two
    number of heads up to 128, cache blocks that are a multiple of 16 tokens."""
    Nh = q.shape[1]
    return (q.is_cuda and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
            and L == 512 and q.shape[2] == 576 and cache.shape[-1] == 576
            and 0 < Nh <= 128 and (Nh & (Nh - 1)) == 0 and cache.shape[-2] % 16 == 0)


def mla_attention(q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor,
                  seq_lens: torch.Tensor, cu_q: Optional[torch.Tensor], num_tiles: int,
                  max_seq_len: int, scale: float, out: Optional[torch.Tensor] = None,
                  splits: Optional[int] = None) -> torch.Tensor:
    """Latent-absorbed multi-head latent attention (attention_mla.cu).  q ``[T, N, 576]``,
    cache ``[blocks, block_size, 576]``, returns ``[T, N, 512]``.  ``cu_q`` None: one query
    token per request (decode).  ``num_tiles`` >= sum over requests of
    ceil(q_len / (128 // N)).  Causal inside each request over absolute positions."""
    T, Nh, W = q.shape
    assert q.is_contiguous() and cache.is_contiguous()
    nb, bs, _ = cache.shape
    if out is None:
        out = torch.empty((T, Nh, 512), dtype=q.dtype, device=q.device)
    B = block_tables.shape[0]
    if splits is None:
        ctas = max(num_tiles, 1) * 2
        global _SM_COUNT
        if _SM_COUNT == 0:
            _SM_COUNT = max(1, int(N.lib().b200_sm_count()))
        splits = max(1, min(_SM_COUNT // ctas, (max_seq_len + 255) // 256, 16))
    ws = None
    if splits > 1:
        ws = torch.empty(splits * T * Nh * 513, dtype=torch.float32, device=q.device)
    rc = N.lib().b200_mla_attention(
        ptr(q), ptr(out), ptr(cache), nb * bs, ptr(cu_q), ptr(seq_lens), ptr(block_tables),
        block_tables.stride(0), bs, B, T, Nh, int(num_tiles), int(splits), ptr(ws), float(scale),
        stream_ptr())
    N.launch_count += 1
    if rc != 0:
        raise N.NativeError(f"b200_mla_attention failed with code {rc}")
    return out


def merge_attn_states(p_out, p_lse, s_out, s_lse, want_lse: bool = True):
    T, H, Dv = p_out.shape
    out = torch.empty_like(p_out)
    lse = torch.empty_like(p_lse) if want_lse else None
    call("b200_merge_attn_states", ptr(out), ptr(lse), ptr(p_out.contiguous()),
         ptr(p_lse.contiguous()), ptr(s_out.contiguous()), ptr(s_lse.contiguous()), T, H, Dv,
         DTYPE_CODE[p_out.dtype], stream_ptr())
    return out, lse


# ---------------------------------------------------------------------------
# sampling / step
# ---------------------------------------------------------------------------
def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           noise: Optional[torch.Tensor] = None, seeds: Optional[torch.Tensor] = None,
           step: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    B, V = logits.shape
    assert logits.stride(1) == 1
    if out is None:
        out = torch.empty((B,), device=logits.device, dtype=torch.int64)
    call("b200_sample", ptr(logits), logits.stride(0), B, V, DTYPE_CODE[logits.dtype],
         ptr(temperature), ptr(top_k), ptr(top_p), ptr(noise), ptr(seeds), int(step), ptr(out),
         stream_ptr())
    return out


def top_k_top_p_(logits: torch.Tensor, top_k: Optional[torch.Tensor],
                 top_p: Optional[torch.Tensor]) -> torch.Tensor:
    B, V = logits.shape
    call("b200_top_k_top_p", ptr(logits), logits.stride(0), B, V, DTYPE_CODE[logits.dtype],
         ptr(top_k), ptr(top_p), stream_ptr())
    return logits


def advance_step(num_seqs: int, num_queries: int, block_size: int, input_tokens, sampled,
                 positions, seq_lens, slot_mapping, block_tables, active_only: bool = False
                 ) -> None:
    call("b200_advance_step", num_seqs, num_queries, block_size, ptr(input_tokens), ptr(sampled),
         ptr(positions), ptr(seq_lens), ptr(slot_mapping), ptr(block_tables),
         block_tables.stride(0), int(active_only), stream_ptr())


def feed_tokens(input_ids, prev_sampled, dst_idx, src_idx, n: int) -> None:
    call("b200_feed_tokens", ptr(input_ids), ptr(prev_sampled), ptr(dst_idx), ptr(src_idx),
         n, stream_ptr())


# ---------------------------------------------------------------------------
# mixture of experts
# ---------------------------------------------------------------------------
def moe_topk(gating: torch.Tensor, k: int, renormalize: bool, n_group: int = 1,
             topk_group: int = 1, bias: Optional[torch.Tensor] = None, sigmoid: bool = False,
             scale: float = 1.0, log2phy: Optional[torch.Tensor] = None,
             replica_count: Optional[torch.Tensor] = None, load: Optional[torch.Tensor] = None
             ) -> tuple[torch.Tensor, torch.Tensor]:
    T, E = gating.shape
    w = torch.empty((T, k), device=gating.device, dtype=torch.float32)
    ids = torch.empty((T, k), device=gating.device, dtype=torch.int32)
    call("b200_moe_topk", ptr(gating), gating.stride(0), ptr(bias), ptr(w), ptr(ids), T, E, k,
         n_group, topk_group, int(sigmoid), int(renormalize), float(scale), ptr(log2phy),
         log2phy.shape[1] if log2phy is not None else 1, ptr(replica_count), ptr(load),
         DTYPE_CODE[gating.dtype], stream_ptr())
    return w, ids


def moe_align_cap(num_pairs: int, num_local_experts: int) -> int:
    return -(-(num_pairs + num_local_experts * 127) // 128) * 128


def moe_align(topk_ids: torch.Tensor, num_local_experts: int, cap: Optional[int] = None,
              expert_map: Optional[torch.Tensor] = None,
              valid_tokens: Optional[torch.Tensor] = None):
    """Returns (sorted_ids [cap], expert_ids [cap/128], num_post_pad [1], pos_of [T*k])."""
    T, k = topk_ids.shape
    numel = T * k
    cap = cap or moe_align_cap(numel, num_local_experts)
    dev = topk_ids.device
    sorted_ids = torch.empty(cap, device=dev, dtype=torch.int32)
    expert_ids = torch.empty(cap // 128, device=dev, dtype=torch.int32)
    npp = torch.empty(1, device=dev, dtype=torch.int32)
    pos_of = torch.empty(max(numel, 1), device=dev, dtype=torch.int32)
    call("b200_moe_align", ptr(topk_ids), ptr(expert_map), ptr(valid_tokens), ptr(sorted_ids),
         ptr(expert_ids), ptr(npp), ptr(pos_of), numel, k, num_local_experts, cap, stream_ptr())
    return sorted_ids, expert_ids, npp, pos_of


def gemm_bf16_grouped(a: torch.Tensor, w: torch.Tensor, expert_ids: torch.Tensor,
                      num_valid_rows: torch.Tensor, silu_mul: bool = False,
                      row_scale: Optional[torch.Tensor] = None,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a ``[M_cap, K]`` expert-sorted rows, w ``[E, N, K]``."""
    M_cap, K = a.shape
    E, Nn, _ = w.shape
    assert w.is_contiguous() and a.stride(1) == 1
    out_cols = Nn // 2 if silu_mul else Nn
    if out is None:
        out = torch.empty((M_cap, out_cols), device=a.device, dtype=torch.bfloat16)
    call("b200_gemm_bf16_grouped", ptr(a), a.stride(0), ptr(w), K, ptr(out), out.stride(0), M_cap,
         Nn, K, E, ptr(expert_ids), ptr(num_valid_rows), ptr(row_scale),
         EPI_SILU_MUL if silu_mul else EPI_NONE, stream_ptr())
    return out


def fused_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_w: torch.Tensor,
                  topk_ids: torch.Tensor, expert_map: Optional[torch.Tensor] = None,
                  add: Optional[torch.Tensor] = None, alpha: float = 1.0,
                  valid_tokens: Optional[torch.Tensor] = None,
                  w13_interleaved: bool = True) -> torch.Tensor:
    """Routed-expert MLP on the native path: align -> permute -> grouped GEMM1 with the
    SiLU-mul epilogue -> grouped GEMM2 scaled by the routing weight -> un-permute + sum
    (+ ``add``, e.g. the shared-expert output).  ``w13`` must hold gate/up interleaved in
    blocks of ``ref.GATE_UP_BLOCK`` rows per expert (``ref.interleave_gate_up``)."""
    T, H = x.shape
    k = topk_ids.shape[1]
    E = w13.shape[0]
    numel = T * k
    cap = moe_align_cap(numel, E)
    sorted_ids, expert_ids, npp, pos_of = moe_align(topk_ids, E, cap, expert_map, valid_tokens)
    a_sorted = torch.empty((cap, H), device=x.device, dtype=x.dtype)
    call("b200_moe_permute", ptr(x), x.stride(0), ptr(a_sorted), H, ptr(sorted_ids), ptr(npp),
         numel, k, H, cap, DTYPE_CODE[x.dtype], stream_ptr())
    row_w = torch.empty(cap, device=x.device, dtype=torch.float32)
    call("b200_moe_row_weights", ptr(sorted_ids), ptr(topk_w), ptr(npp), ptr(row_w), numel, cap,
         stream_ptr())
    h = gemm_bf16_grouped(a_sorted, w13, expert_ids, npp, silu_mul=True)
    y = gemm_bf16_grouped(h, w2, expert_ids, npp, row_scale=row_w)
    out = torch.empty((T, H), device=x.device, dtype=x.dtype)
    call("b200_moe_unpermute_sum", ptr(y), y.stride(0), ptr(pos_of), ptr(add),
         add.stride(0) if add is not None else 0, ptr(out), H, ptr(valid_tokens), T, k, H,
         float(alpha), DTYPE_CODE[x.dtype], stream_ptr())
    return out


def gemm_q8_grouped(a: torch.Tensor, a_scale: torch.Tensor, w: torch.Tensor,
                    w_scale: torch.Tensor, expert_ids: torch.Tensor, npp: torch.Tensor,
                    kind: int = 1, row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Grouped 8-bit GEMM: ``a [cap, K]`` rows sorted by expert in tiles of 128,
    ``w [E, N, K]``; scales as in :func:`gemm_q8` with a leading expert dimension on
    ``w_scale``.  Returns bf16 ``[cap, N]`` (rows of skipped tiles are not written)."""
    cap, K = a.shape
    E, Nn, _ = w.shape
    assert w.is_contiguous() and a.stride(1) == 1 and a.element_size() == 1
    out = torch.empty((cap, Nn), device=a.device, dtype=torch.bfloat16)
    a_scale = a_scale.contiguous()
    w_scale = w_scale.contiguous()
    lds_a = a_scale.stride(0) if kind == 1 else 1
    lds_b = w_scale.stride(-2) if kind == 1 else 1
    call("b200_gemm_q8_grouped", ptr(a), a.stride(0), ptr(w), K, ptr(out), out.stride(0), cap, Nn,
         K, E, ptr(a_scale), lds_a, ptr(w_scale), lds_b, ptr(expert_ids), ptr(npp),
         ptr(row_scale), kind, stream_ptr())
    return out


def fused_experts_fp8(x: torch.Tensor, w13: torch.Tensor, w13_scale: torch.Tensor,
                      w2: torch.Tensor, w2_scale: torch.Tensor, topk_w: torch.Tensor,
                      topk_ids: torch.Tensor, expert_map: Optional[torch.Tensor] = None,
                      add: Optional[torch.Tensor] = None, alpha: float = 1.0,
                      valid_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Routed-expert MLP with fp8 e4m3 expert weights and 128 x 128 block scales
    (DeepSeek-V3 checkpoints): align -> permute -> 1 x 128 activation quantisation ->
    grouped fp8 GEMM1 -> SiLU-mul + quantisation -> grouped fp8 GEMM2 scaled by the routing
    weight -> un-permute + sum.  ``w13 [E, 2I, H]`` gate rows first, ``w13_scale
    [E, 2I/128, H/128]``, ``w2 [E, H, I]``, ``w2_scale [E, H/128, I/128]``."""
    T, H = x.shape
    k = topk_ids.shape[1]
    E = w13.shape[0]
    numel = T * k
    cap = moe_align_cap(numel, E)
    sorted_ids, expert_ids, npp, pos_of = moe_align(topk_ids, E, cap, expert_map, valid_tokens)
    a_sorted = torch.empty((cap, H), device=x.device, dtype=x.dtype)
    call("b200_moe_permute", ptr(x), x.stride(0), ptr(a_sorted), H, ptr(sorted_ids), ptr(npp),
         numel, k, H, cap, DTYPE_CODE[x.dtype], stream_ptr())
    row_w = torch.empty(cap, device=x.device, dtype=torch.float32)
    call("b200_moe_row_weights", ptr(sorted_ids), ptr(topk_w), ptr(npp), ptr(row_w), numel, cap,
         stream_ptr())
    aq, a_s = activation(a_sorted, "identity", "plain", quant="fp8_group128", valid_rows=npp)
    h = gemm_q8_grouped(aq, a_s, w13, w13_scale, expert_ids, npp, kind=1)
    hq, h_s = activation(h, "silu", "act_mul", quant="fp8_group128", valid_rows=npp)
    y = gemm_q8_grouped(hq, h_s, w2, w2_scale, expert_ids, npp, kind=1, row_scale=row_w)
    out = torch.empty((T, H), device=x.device, dtype=x.dtype)
    call("b200_moe_unpermute_sum", ptr(y), y.stride(0), ptr(pos_of), ptr(add),
         add.stride(0) if add is not None else 0, ptr(out), H, ptr(valid_tokens), T, k, H,
         float(alpha), DTYPE_CODE[x.dtype], stream_ptr())
    return out


#: average rows per local expert up to which packed 4 / 8-bit experts run through the fused
#: de-quantising grouped GEMM; above it the layer's experts are de-quantised into a scratch
#: shared by all layers and the bf16 grouped GEMM runs (every row tile of the fused kernel
#: de-quantises its expert's weights again, which only pays while tiles per expert are few)
WNA16_GROUPED_MAX_ROWS_PER_EXPERT = 96
_WNA16_SCRATCH: dict = {}


def gemm_wna16_grouped(a: torch.Tensor, qw: torch.Tensor, scales: torch.Tensor, zs: torch.Tensor,
                       expert_ids: torch.Tensor, npp: torch.Tensor, group: int, bits: int,
                       row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Grouped de-quantising GEMM: ``a [cap, K]`` bf16 rows sorted by expert in tiles of 128,
    ``qw [E, N, K/2]`` (4 bit, low nibble = even k) or ``[E, N, K]`` (8 bit) uint8,
    ``scales`` / ``zs`` ``[E, N, K/g]`` bf16 (``w = q * scale - zs``).  Returns bf16
    ``[cap, N]`` (rows of tiles past ``npp`` are not written)."""
    cap, K = a.shape
    E, Nn = qw.shape[0], qw.shape[1]
    assert qw.is_contiguous() and scales.is_contiguous() and zs.is_contiguous()
    assert a.stride(1) == 1 and a.dtype == torch.bfloat16 and scales.dtype == torch.bfloat16
    out = torch.empty((cap, Nn), device=a.device, dtype=torch.bfloat16)
    call("b200_gemm_wna16_grouped", ptr(a), a.stride(0), ptr(qw), ptr(scales), ptr(zs), ptr(out),
         out.stride(0), cap, Nn, K, E, int(group), int(bits), ptr(expert_ids), ptr(npp),
         ptr(row_scale), stream_ptr())
    return out


def _wna16_scratch(name: str, shape, device) -> torch.Tensor:
    n = 1
    for d in shape:
        n *= d
    buf = _WNA16_SCRATCH.get((name, device))
    if buf is None or buf.numel() < n:
        buf = torch.empty(n, dtype=torch.bfloat16, device=device)
        _WNA16_SCRATCH[(name, device)] = buf
    return buf[:n].view(*shape)


def fused_experts_wna16(x: torch.Tensor, q13: torch.Tensor, s13: torch.Tensor, z13: torch.Tensor,
                        q2: torch.Tensor, s2: torch.Tensor, z2: torch.Tensor, group: int,
                        bits: int, topk_w: torch.Tensor, topk_ids: torch.Tensor,
                        expert_map: Optional[torch.Tensor] = None,
                        add: Optional[torch.Tensor] = None, alpha: float = 1.0,
                        valid_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Routed-expert MLP whose experts stay packed as 4 / 8-bit integers with per-group scales
    (AWQ / GPTQ / ``moe_wna16`` checkpoints; vllm_gcu/kernels/quantization/moe_wna16.py:487-572):
    align -> permute -> grouped de-quantising GEMM1 -> SiLU-mul -> grouped de-quantising GEMM2
    scaled by the routing weight -> un-permute + sum.  ``q13 [E, 2I, H/2]`` gate rows first,
    ``q2 [E, H, I/2]`` (``[.., K]`` for 8 bit)."""
    T, H = x.shape
    k = topk_ids.shape[1]
    E, N13 = q13.shape[0], q13.shape[1]
    numel = T * k
    cap = moe_align_cap(numel, E)
    sorted_ids, expert_ids, npp, pos_of = moe_align(topk_ids, E, cap, expert_map, valid_tokens)
    a_sorted = torch.empty((cap, H), device=x.device, dtype=x.dtype)
    call("b200_moe_permute", ptr(x), x.stride(0), ptr(a_sorted), H, ptr(sorted_ids), ptr(npp),
         numel, k, H, cap, DTYPE_CODE[x.dtype], stream_ptr())
    row_w = torch.empty(cap, device=x.device, dtype=torch.float32)
    call("b200_moe_row_weights", ptr(sorted_ids), ptr(topk_w), ptr(npp), ptr(row_w), numel, cap,
         stream_ptr())
    if numel <= WNA16_GROUPED_MAX_ROWS_PER_EXPERT * E:
        h = gemm_wna16_grouped(a_sorted, q13, s13, z13, expert_ids, npp, group, bits)
        hm = activation(h, "silu", "act_mul", valid_rows=npp)
        y = gemm_wna16_grouped(hm, q2, s2, z2, expert_ids, npp, group, bits, row_scale=row_w)
    else:
        I = N13 // 2
        w13 = _wna16_scratch("w13", (E, N13, H), x.device)
        w2 = _wna16_scratch("w2", (E, H, I), x.device)
        weight_dequant(q13.view(E * N13, -1), s13.view(E * N13, -1), z13.view(E * N13, -1),
                       w13.view(E * N13, H), group, bits)
        weight_dequant(q2.view(E * H, -1), s2.view(E * H, -1), z2.view(E * H, -1),
                       w2.view(E * H, I), group, bits)
        h = gemm_bf16_grouped(a_sorted, w13, expert_ids, npp)
        hm = activation(h, "silu", "act_mul", valid_rows=npp)
        y = gemm_bf16_grouped(hm, w2, expert_ids, npp, row_scale=row_w)
    out = torch.empty((T, H), device=x.device, dtype=x.dtype)
    call("b200_moe_unpermute_sum", ptr(y), y.stride(0), ptr(pos_of), ptr(add),
         add.stride(0) if add is not None else 0, ptr(out), H, ptr(valid_tokens), T, k, H,
         float(alpha), DTYPE_CODE[x.dtype], stream_ptr())
    return out


def fused_experts_q8(x: torch.Tensor, w13: torch.Tensor, w13_scale: torch.Tensor,
                     w2: torch.Tensor, w2_scale: torch.Tensor, topk_w: torch.Tensor,
                     topk_ids: torch.Tensor, expert_map: Optional[torch.Tensor] = None,
                     add: Optional[torch.Tensor] = None, alpha: float = 1.0,
                     valid_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Routed-expert MLP with int8 or fp8 expert weights and per-output-channel scales
    (w8a8 checkpoints): activations are quantised per token before each grouped GEMM.
    ``w13 [E, 2I, H]`` gate rows first, ``w13_scale [E, 2I]``, ``w2 [E, H, I]``,
    ``w2_scale [E, H]``; the weight dtype selects int8 (kind 2) or fp8 (kind 0)."""
    T, H = x.shape
    k = topk_ids.shape[1]
    E = w13.shape[0]
    numel = T * k
    kind = 2 if w13.dtype == torch.int8 else 0
    qname = "int8" if kind == 2 else "fp8"
    cap = moe_align_cap(numel, E)
    sorted_ids, expert_ids, npp, pos_of = moe_align(topk_ids, E, cap, expert_map, valid_tokens)
    a_sorted = torch.empty((cap, H), device=x.device, dtype=x.dtype)
    call("b200_moe_permute", ptr(x), x.stride(0), ptr(a_sorted), H, ptr(sorted_ids), ptr(npp),
         numel, k, H, cap, DTYPE_CODE[x.dtype], stream_ptr())
    row_w = torch.empty(cap, device=x.device, dtype=torch.float32)
    call("b200_moe_row_weights", ptr(sorted_ids), ptr(topk_w), ptr(npp), ptr(row_w), numel, cap,
         stream_ptr())
    aq, a_s = per_token_quant(a_sorted, qname, valid_rows=npp)
    h = gemm_q8_grouped(aq, a_s.view(-1), w13, w13_scale, expert_ids, npp, kind=kind)
    hm = activation(h, "silu", "act_mul", valid_rows=npp)
    hq, h_s = per_token_quant(hm, qname, valid_rows=npp)
    y = gemm_q8_grouped(hq, h_s.view(-1), w2, w2_scale, expert_ids, npp, kind=kind,
                        row_scale=row_w)
    out = torch.empty((T, H), device=x.device, dtype=x.dtype)
    call("b200_moe_unpermute_sum", ptr(y), y.stride(0), ptr(pos_of), ptr(add),
         add.stride(0) if add is not None else 0, ptr(out), H, ptr(valid_tokens), T, k, H,
         float(alpha), DTYPE_CODE[x.dtype], stream_ptr())
    return out


def get_ep_indices(topk_ids: torch.Tensor, experts_per_rank: int, ep: int):
    T, k = topk_ids.shape
    dev = topk_ids.device
    cnt = torch.empty(ep, device=dev, dtype=torch.int32)
    idx = torch.zeros(T * min(k, ep), device=dev, dtype=torch.int32)
    total = torch.empty(1, device=dev, dtype=torch.int32)
    call("b200_get_ep_indices", ptr(topk_ids), T, k, experts_per_rank, ep, ptr(cnt), ptr(idx),
         ptr(total), stream_ptr())
    return cnt, idx, total


# ---------------------------------------------------------------------------
# quantisation
# ---------------------------------------------------------------------------
def per_token_quant(x: torch.Tensor, kind: str = "fp8",
                    valid_rows: Optional[torch.Tensor] = None):
    """Dynamic per-token quantisation to fp8 e4m3 or int8; returns (q, scales [T, 1])."""
    x2 = _rowmajor_2d(x)
    T, H = x2.shape
    q = torch.empty((T, H), device=x.device, dtype=FP8 if kind == "fp8" else torch.int8)
    s = torch.empty((T, 1), device=x.device, dtype=torch.float32)
    call("b200_per_token_quant", ptr(x2), x2.stride(0), ptr(q), H, ptr(s), ptr(valid_rows), T, H,
         0 if kind == "fp8" else 1, DTYPE_CODE[x.dtype], stream_ptr())
    return q, s


def per_tensor_fp8_quant(x: torch.Tensor):
    xc = x.contiguous()
    q = torch.empty(xc.shape, device=x.device, dtype=FP8)
    ws = torch.empty(1, device=x.device, dtype=torch.float32)
    s = torch.empty(1, device=x.device, dtype=torch.float32)
    call("b200_per_tensor_fp8_quant", ptr(xc), ptr(q), xc.numel(), ptr(ws), ptr(s),
         DTYPE_CODE[x.dtype], stream_ptr())
    return q, s


def int8_dequant(q: torch.Tensor, scale: torch.Tensor, azp: Optional[torch.Tensor] = None,
                 dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    qc = q.contiguous()
    out = torch.empty(qc.shape, device=q.device, dtype=dtype)
    call("b200_int8_dequant", ptr(qc), ptr(out), qc.numel(), ptr(scale), ptr(azp),
         DTYPE_CODE[dtype], stream_ptr())
    return out


def gemm_q8(a: torch.Tensor, b: torch.Tensor, a_scale: torch.Tensor, b_scale: torch.Tensor,
            bias: Optional[torch.Tensor] = None, kind: int = 0,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """8-bit GEMM ``a [M,K] @ b [N,K]^T`` -> bf16.  kind 0: fp8 with per-token ``a_scale [M]``
    and per-channel ``b_scale [N]``; 1: fp8 block scales ``a_scale [M, K/128]``,
    ``b_scale [N/128, K/128]``; 2: int8 with per-token / per-channel scales."""
    M, K = a.shape
    Nn = b.shape[0]
    assert a.element_size() == 1 and b.element_size() == 1 and a.stride(1) == 1
    if out is None:
        out = torch.empty((M, Nn), device=a.device, dtype=torch.bfloat16)
    a_scale = a_scale.contiguous()
    b_scale = b_scale.contiguous()
    lds_a = a_scale.stride(0) if (kind == 1 and a_scale.dim() == 2) else 1
    lds_b = b_scale.stride(0) if (kind == 1 and b_scale.dim() == 2) else 1
    call("b200_gemm_q8", ptr(a), a.stride(0), ptr(b), b.stride(0), ptr(out), out.stride(0), M, Nn,
         K, ptr(a_scale), lds_a, ptr(b_scale), lds_b, ptr(bias), kind, stream_ptr())
    return out


def weight_dequant(qw: torch.Tensor, scales: torch.Tensor, zs: torch.Tensor, out: torch.Tensor,
                   group: int, bits: int) -> torch.Tensor:
    N, K = out.shape
    call("b200_weight_dequant", ptr(qw), ptr(scales), ptr(zs), ptr(out), N, K, group, bits,
         DTYPE_CODE[out.dtype], stream_ptr())
    return out
