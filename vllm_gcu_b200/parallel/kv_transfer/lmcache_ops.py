"""Drop-in for ``lmcache.c_ops``: the functions the LMCache GPU connectors call
(lmcache/csrc/pybind.cpp:44-61).  CUDA tensors run on the kernels of ``csrc/lmcache.cu``; CPU
tensors use index arithmetic in torch, which also serves as the test oracle."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ... import ops
from ...ops import _native
from ...ops._native import DTYPE_CODE, ptr, stream_ptr

_SIGS_DONE = False


def _lib():
    global _SIGS_DONE
    lib = _native.lib()
    if lib is not None and not _SIGS_DONE:
        P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.b200_lmc_multi_layer_kv_transfer.argtypes = [P, P, P, I, I, L, L, I, I, P]
        lib.b200_lmc_single_layer_kv_transfer.argtypes = [P, P, P, P, I, L, L, I, I, P]
        lib.b200_lmc_rerotate_k.argtypes = [P, L, P, P, P, I, I, I, I, I, I, P]
        lib.b200_lmc_calculate_cdf.argtypes = [P, P, I, I, I, I, P]
        lib.b200_lmc_encode.argtypes = [P, P, P, P, I, I, I, I, I, P]
        lib.b200_lmc_decode.argtypes = [P, P, P, P, P, I, I, I, I, I, P]
        lib.b200_alloc_pinned.restype = P
        lib.b200_alloc_pinned.argtypes = [ctypes.c_ulonglong, I]
        lib.b200_free_pinned.argtypes = [P, I]
        lib.b200_gpu_pci_bus_id.argtypes = [I, ctypes.c_char_p, I]
        _SIGS_DONE = True
    return lib


def _check(rc: int, name: str) -> None:
    if rc != 0:
        raise _native.NativeError(f"{name} failed with code {rc}")


def multi_layer_kv_transfer(key_value: torch.Tensor, key_value_ptrs: torch.Tensor,
                            slot_mapping: torch.Tensor, paged_memory_device,
                            page_buffer_size: int, direction: bool, use_mla: bool,
                            layers: Optional[list[torch.Tensor]] = None) -> None:
    """``key_value`` is ``[2, L, T, W]`` (``[L, T, W]`` for MLA); layer i's paged buffer
    ``[2, page_buffer_size, W]`` (``[page_buffer_size, W]`` for MLA) starts at
    ``key_value_ptrs[i]``.  ``direction`` True copies paged -> ``key_value``, False the other
    way.  On CPU the layer tensors must be passed in ``layers`` (raw pointers are opaque)."""
    kvn = 1 if use_mla else 2
    kv = key_value if not use_mla else key_value.unsqueeze(0)
    _, L, T, W = kv.shape
    if key_value.is_cuda:
        rc = _lib().b200_lmc_multi_layer_kv_transfer(
            ptr(key_value), ptr(key_value_ptrs), ptr(slot_mapping), L, T,
            W * key_value.element_size(), page_buffer_size, int(direction), int(use_mla),
            stream_ptr())
        _check(rc, "multi_layer_kv_transfer")
        return
    assert layers is not None, "CPU path needs the layer tensors"
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    for l in range(L):
        paged = layers[l].view(kvn, page_buffer_size, W)
        for k in range(kvn):
            if direction:
                kv[k, l, valid] = paged[k, slots]
            else:
                paged[k, slots] = kv[k, l, valid]


def multi_layer_kv_transfer_unilateral(key_value, key_ptrs, value_ptrs, slot_mapping,
                                       paged_memory_device, page_buffer_size: int,
                                       direction: bool, key_layers=None, value_layers=None) -> None:
    """Variant with separate K and V pointer tables (one paged buffer per layer and side)."""
    L = key_value.shape[1]
    for side, ptrs, lay in ((0, key_ptrs, key_layers), (1, value_ptrs, value_layers)):
        multi_layer_kv_transfer(key_value[side], ptrs, slot_mapping, paged_memory_device,
                                page_buffer_size, direction, True, lay)


def single_layer_kv_transfer(lmc_key_value_cache: torch.Tensor, vllm_key_cache: torch.Tensor,
                             vllm_value_cache: torch.Tensor, slot_mapping: torch.Tensor,
                             direction: bool, token_major: bool = False) -> None:
    """One layer.  Buffer ``[T, 2, W]`` (token major) or ``[2, T, W]``; paged caches
    ``[num_slots, W]`` (any trailing shape)."""
    T = slot_mapping.shape[0]
    W = vllm_key_cache[0].numel() if vllm_key_cache.dim() > 1 else 1
    kc = vllm_key_cache.reshape(-1, W) if vllm_key_cache.dim() == 2 else \
        vllm_key_cache.reshape(-1, vllm_key_cache.shape[-2] * vllm_key_cache.shape[-1]) \
        if vllm_key_cache.dim() == 4 else vllm_key_cache.reshape(-1, vllm_key_cache.shape[-1])
    vc = vllm_value_cache.reshape(kc.shape)
    W = kc.shape[1]
    if lmc_key_value_cache.is_cuda:
        rc = _lib().b200_lmc_single_layer_kv_transfer(
            ptr(lmc_key_value_cache), ptr(kc), ptr(vc), ptr(slot_mapping), T,
            W * kc.element_size(), kc.shape[0], int(direction), int(token_major), stream_ptr())
        _check(rc, "single_layer_kv_transfer")
        return
    buf = lmc_key_value_cache.reshape(T, 2, W) if token_major else \
        lmc_key_value_cache.reshape(2, T, W).transpose(0, 1)
    valid = slot_mapping >= 0
    slots = slot_mapping[valid].long()
    for k, cache in ((0, kc), (1, vc)):
        if direction:
            buf[valid, k] = cache[slots]
        else:
            cache[slots] = buf[valid, k]


def load_and_reshape_flash(key_value: torch.Tensor, key_cache: torch.Tensor,
                           value_cache: torch.Tensor, slot_mapping: torch.Tensor,
                           layer_idx: int) -> None:
    """Paged flash-layout caches of one layer -> ``key_value[:, layer_idx]`` (``[2, L, T, W]``)."""
    T = slot_mapping.shape[0]
    W = key_value.shape[-1]
    tmp = torch.empty((2, T, W), dtype=key_value.dtype, device=key_value.device)
    single_layer_kv_transfer(tmp, key_cache.reshape(-1, W), value_cache.reshape(-1, W),
                             slot_mapping, True, False)
    key_value[:, layer_idx] = tmp


def reshape_and_cache_back_flash(key_value: torch.Tensor, key_cache: torch.Tensor,
                                 value_cache: torch.Tensor, slot_mapping: torch.Tensor,
                                 layer_idx: int) -> None:
    W = key_value.shape[-1]
    tmp = key_value[:, layer_idx].contiguous()
    single_layer_kv_transfer(tmp, key_cache.reshape(-1, W), value_cache.reshape(-1, W),
                             slot_mapping, False, False)


def rotary_embedding_k_fused(old_positions: torch.Tensor, new_positions: torch.Tensor,
                             key: torch.Tensor, head_size: int, cos_sin_cache: torch.Tensor,
                             is_neox: bool) -> None:
    """In place: keys cached at ``old_positions`` become keys at ``new_positions``."""
    T = key.shape[0]
    k2 = key.view(T, -1)
    H = k2.shape[1] // head_size
    rot = cos_sin_cache.shape[-1]
    if key.is_cuda and key.dtype in (torch.bfloat16, torch.float16) \
            and cos_sin_cache.dtype == key.dtype:
        rc = _lib().b200_lmc_rerotate_k(ptr(k2), k2.stride(0), ptr(old_positions),
                                        ptr(new_positions), ptr(cos_sin_cache), T, H, head_size,
                                        rot, int(is_neox), DTYPE_CODE[key.dtype], stream_ptr())
        _check(rc, "rotary_embedding_k_fused")
        return
    half = rot // 2
    cs = cos_sin_cache.float()
    co, so = cs[old_positions.long(), :half], cs[old_positions.long(), half:]
    cn, sn = cs[new_positions.long(), :half], cs[new_positions.long(), half:]
    c = (cn * co + sn * so)[:, None, :]
    s = (sn * co - cn * so)[:, None, :]
    x = k2.float().view(T, H, head_size)
    xr = x[..., :rot]
    if is_neox:
        a, b = xr[..., :half], xr[..., half:]
        out = torch.cat([a * c - b * s, b * c + a * s], -1)
    else:
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([a * c - b * s, b * c + a * s], -1).flatten(-2)
    x = torch.cat([out, x[..., rot:]], -1)
    k2.copy_(x.view(T, -1).to(key.dtype))


def calculate_cdf(input: torch.Tensor, max_bins: int) -> torch.Tensor:
    """CacheGen: per (layer, channel) cumulative bin frequencies scaled to 16 bits.
    input int8 ``[L, T, C]`` -> int16 ``[L, C, max_bins + 1]``."""
    assert max_bins < 64
    L, T, C = input.shape
    out = torch.zeros((L, C, max_bins + 1), dtype=torch.int16, device=input.device)
    if input.is_cuda:
        rc = _lib().b200_lmc_calculate_cdf(ptr(input.contiguous()), ptr(out), L, T, C, max_bins,
                                           stream_ptr())
        _check(rc, "calculate_cdf")
        return out
    onehot = torch.nn.functional.one_hot(input.long().clamp(0, max_bins - 1), max_bins)
    onehot = onehot * ((input >= 0) & (input < max_bins))[..., None]
    hist = onehot.sum(1)                                            # [L, C, bins]
    run = hist.cumsum(-1)
    q = (run * 65535) // max(T, 1)
    out[..., 1:] = q.clamp(max=65535).to(torch.int32).to(torch.int16)
    return out


def alloc_pinned_ptr(size: int, flags: int = 0) -> int:
    p = _lib().b200_alloc_pinned(size, -1)
    if not p:
        raise MemoryError("pinned allocation failed")
    return int(p)


def free_pinned_ptr(p: int) -> None:
    _lib().b200_free_pinned(p, -1)


def alloc_pinned_numa_ptr(size: int, node: int) -> int:
    p = _lib().b200_alloc_pinned(size, max(node, 0))
    if not p:
        raise MemoryError("pinned NUMA allocation failed")
    return int(p)


def free_pinned_numa_ptr(p: int, size: int = 0) -> None:
    _lib().b200_free_pinned(p, 0)


def get_gpu_pci_bus_id(device: int) -> str:
    buf = ctypes.create_string_buffer(32)
    _check(_lib().b200_gpu_pci_bus_id(device, buf, 32), "get_gpu_pci_bus_id")
    return buf.value.decode()


# ---------------------------------------------------------------------------
# CacheGen arithmetic codec
# ---------------------------------------------------------------------------
def _cdf_at(row, i: int, bins: int) -> int:
    return (65536 if i >= bins else int(row[i]) & 0xFFFF) + i


def _encode_stream_py(rows, syms, bins: int) -> bytes:
    """Reference of the device coder (same arithmetic, one stream)."""
    total = 65536 + bins
    low, high, pending = 0, 0xFFFFFFFF, 0
    bits: list[int] = []

    def put(b):
        nonlocal pending
        bits.append(b)
        bits.extend([b ^ 1] * pending)
        pending = 0

    for c, v in enumerate(syms):
        v = min(max(int(v), 0), bins - 1)
        span = high - low + 1
        c_lo, c_hi = _cdf_at(rows[c], v, bins), _cdf_at(rows[c], v + 1, bins)
        high = low + span * c_hi // total - 1
        low = low + span * c_lo // total
        while True:
            if high < 0x80000000:
                put(0)
            elif low >= 0x80000000:
                put(1)
                low -= 0x80000000
                high -= 0x80000000
            elif low >= 0x40000000 and high < 0xC0000000:
                pending += 1
                low -= 0x40000000
                high -= 0x40000000
            else:
                break
            low = (low << 1) & 0xFFFFFFFF
            high = ((high << 1) | 1) & 0xFFFFFFFF
    pending += 1
    put(0 if low < 0x40000000 else 1)
    while len(bits) % 8:
        bits.append(0)
    return bytes(int("".join(map(str, bits[i:i + 8])), 2) for i in range(0, len(bits), 8))


def _decode_stream_py(rows, data: bytes, n: int, bins: int) -> list[int]:
    total = 65536 + bins
    pos = 0

    def get():
        nonlocal pos
        byte = pos >> 3
        b = (data[byte] >> (7 - (pos & 7))) & 1 if byte < len(data) else 0
        pos += 1
        return b

    low, high, code = 0, 0xFFFFFFFF, 0
    for _ in range(32):
        code = (code << 1) | get()
    out = []
    for c in range(n):
        span = high - low + 1
        target = ((code - low + 1) * total - 1) // span
        v = 0
        while v + 1 < bins and _cdf_at(rows[c], v + 1, bins) <= target:
            v += 1
        out.append(v)
        c_lo, c_hi = _cdf_at(rows[c], v, bins), _cdf_at(rows[c], v + 1, bins)
        high = low + span * c_hi // total - 1
        low = low + span * c_lo // total
        while True:
            if high < 0x80000000:
                pass
            elif low >= 0x80000000:
                low -= 0x80000000
                high -= 0x80000000
                code -= 0x80000000
            elif low >= 0x40000000 and high < 0xC0000000:
                low -= 0x40000000
                high -= 0x40000000
                code -= 0x40000000
            else:
                break
            low = (low << 1) & 0xFFFFFFFF
            high = ((high << 1) | 1) & 0xFFFFFFFF
            code = ((code << 1) | get()) & 0xFFFFFFFF
    return out


def encode_fast_new(cdf: torch.Tensor, input_sym: torch.Tensor, output_buffer: torch.Tensor,
                    output_lengths: torch.Tensor) -> None:
    """CacheGen encoder (lmcache/csrc/encode_cuda_new.cpp:29): ``cdf`` int16
    ``[L, C, bins + 1]``, ``input_sym`` int8 ``[L, T, C]``; stream (l, t) is written to
    ``output_buffer[l, t, :]`` (uint8 ``[L, T, max_bytes]``) and its byte count to
    ``output_lengths[l, t]`` (int32; -1 when ``max_bytes`` is too small)."""
    L, T, C = input_sym.shape
    bins = cdf.shape[-1] - 1
    max_bytes = output_buffer.shape[-1]
    if input_sym.is_cuda:
        rc = _lib().b200_lmc_encode(ptr(cdf.contiguous()), ptr(input_sym.contiguous()),
                                    ptr(output_buffer), ptr(output_lengths), L, T, C, bins,
                                    max_bytes, stream_ptr())
        _check(rc, "encode")
        return
    cu = cdf.to(torch.int32) & 0xFFFF
    for l in range(L):
        rows = cu[l].tolist()
        for t in range(T):
            b = _encode_stream_py(rows, input_sym[l, t].tolist(), bins)
            if len(b) > max_bytes:
                output_lengths[l, t] = -1
                continue
            output_buffer[l, t, :len(b)] = torch.tensor(list(b), dtype=torch.uint8)
            output_lengths[l, t] = len(b)


def decode_fast_new(cdf: torch.Tensor, bytestreams: torch.Tensor, lengths: torch.Tensor,
                    output: torch.Tensor) -> None:
    """Inverse of :func:`encode_fast_new` over fixed-size slots
    (lmcache/csrc/decode_cuda_new.cpp:28); ``output`` int8 ``[L, T, C]``."""
    L, T, C = output.shape
    bins = cdf.shape[-1] - 1
    if output.is_cuda:
        rc = _lib().b200_lmc_decode(ptr(cdf.contiguous()), ptr(bytestreams), ptr(lengths), None,
                                    ptr(output), L, T, C, bins, bytestreams.shape[-1],
                                    stream_ptr())
        _check(rc, "decode")
        return
    cu = cdf.to(torch.int32) & 0xFFFF
    for l in range(L):
        rows = cu[l].tolist()
        for t in range(T):
            n = int(lengths[l, t])
            data = bytes(bytestreams[l, t, :max(n, 0)].tolist())
            output[l, t] = torch.tensor(_decode_stream_py(rows, data, C, bins), dtype=torch.int8)


def decode_fast_prefsum(cdf: torch.Tensor, bytestreams: torch.Tensor,
                        lengths_prefsum: torch.Tensor, output: torch.Tensor) -> None:
    """Decoder over packed streams (lmcache/csrc/decode_cuda_prefsum.cpp:27):
    ``bytestreams`` is one uint8 vector, stream s = (l, t) occupies
    ``[lengths_prefsum[s], lengths_prefsum[s + 1])`` (int64 ``[L * T + 1]``)."""
    L, T, C = output.shape
    bins = cdf.shape[-1] - 1
    if output.is_cuda:
        rc = _lib().b200_lmc_decode(ptr(cdf.contiguous()), ptr(bytestreams), None,
                                    ptr(lengths_prefsum.contiguous()), ptr(output), L, T, C, bins,
                                    0, stream_ptr())
        _check(rc, "decode_prefsum")
        return
    cu = cdf.to(torch.int32) & 0xFFFF
    off = lengths_prefsum.tolist()
    for l in range(L):
        rows = cu[l].tolist()
        for t in range(T):
            s = l * T + t
            data = bytes(bytestreams[off[s]:off[s + 1]].tolist())
            output[l, t] = torch.tensor(_decode_stream_py(rows, data, C, bins), dtype=torch.int8)
