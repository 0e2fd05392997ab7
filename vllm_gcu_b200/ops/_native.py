"""ctypes loader for the in-tree native library ``vllm_gcu_b200/_b200.so``.

The library is built by ``python -m vllm_gcu_b200.csrc.build`` (nvcc, sm_100a).
On a machine with a GPU a missing library is an error: the CUDA ops never fall
back to PyTorch silently.  On a CPU-only machine ``lib()`` returns ``None`` and
the op layer uses the torch reference implementations.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path
from typing import Optional

import torch

# VLLM_B200_NATIVE_LIB selects another build of the same library (e.g. a host-sanitizer build,
# see csrc/build.py)
_LIB_PATH = Path(os.environ["VLLM_B200_NATIVE_LIB"]) if os.environ.get("VLLM_B200_NATIVE_LIB") \
    else Path(__file__).resolve().parent.parent / "_b200.so"
_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None
_tried = False

#: number of kernel launches issued through this module (bench.py reports it)
launch_count = 0


class NativeError(RuntimeError):
    """A native entry point returned a non-zero code."""


class KernelTimeoutError(RuntimeError):
    """A bounded device-side wait ran out (the kernel left cleanly)."""


def lib_path() -> Path:
    return _LIB_PATH


def lib() -> Optional[ctypes.CDLL]:
    """Returns the loaded library, or None when there is no GPU and no build."""
    global _lib, _tried
    if _lib is not None or _tried:
        return _lib
    with _lock:
        if _lib is not None or _tried:
            return _lib
        _tried = True
        if not _LIB_PATH.exists():
            if os.environ.get("VLLM_B200_AUTOBUILD", "0") == "1":
                from vllm_gcu_b200.csrc.build import build
                build()
            elif torch.cuda.is_available():
                raise NativeError(
                    f"{_LIB_PATH} is missing; run `python -m vllm_gcu_b200.csrc.build`")
            else:
                return None
        _lib = ctypes.CDLL(str(_LIB_PATH))
        for name in dir(_Sigs):
            if name.startswith("b200_"):
                fn = getattr(_lib, name, None)
                if fn is None:
                    raise NativeError(f"symbol {name} missing from {_LIB_PATH}; rebuild")
                fn.restype = ctypes.c_int
                fn.argtypes = getattr(_Sigs, name)
    return _lib


def available() -> bool:
    return torch.cuda.is_available() and lib() is not None


P = ctypes.c_void_p
I = ctypes.c_int
L = ctypes.c_longlong
F = ctypes.c_float


class _Sigs:
    """Argument types of every exported entry point (checked at load time)."""
    b200_status_take = [P, P]
    b200_sm_count = []
    b200_abi_version = []
    b200_gemm_bf16 = [P, L, P, L, P, L, I, I, I, P, P, L, I, P]
    b200_norm = [P, L, P, L, P, P, P, L, P, P, P, I, I, F, I, I, I, P]
    b200_activation = [P, L, P, L, P, P, P, P, I, I, I, I, I, F, I, P]
    b200_rope_cache_flash = [P, L, P, L, P, L, P, P, I, I, I, P, P, P, L, L, L, I, P, P,
                             I, I, I, I, I, P]
    b200_reshape_and_cache = [P, L, P, L, P, P, P, L, I, I, I, I, I, I, F, F, F, F, I, P]
    b200_mla_rope_cache = [P, L, L, P, L, L, P, L, P, P, P, L, L, P, P, P, P, P, P, P,
                           I, I, I, I, F, I, I, I, P]
    b200_gather_cache = [P, P, P, P, P, I, I, I, L, L, L, I, P]
    b200_copy_blocks = [P, I, P, I, L, P]
    b200_swap_blocks = [P, P, P, I, L, P]
    b200_decode_num_splits = [I, I, I]
    b200_paged_decode = [P, L, P, L, P, P, L, L, L, P, I, I, P, P, P, I, I, I, I, I, F, I, P]
    b200_paged_decode_alibi = [P, L, P, L, P, P, L, L, L, P, I, I, P, P, P, I, I, I, I, I, F, I, P,
                               P]
    b200_varlen_prefill_alibi = [P, L, P, L, P, P, P, P, P, L, L, L, P, I, I, I, I, I, I, I, I, F,
                                 I, I, I, P, P]
    b200_paged_decode_q8kv = [P, L, P, L, P, P, L, L, L, P, I, I, P, P, P, I, I, I, I, I, F, I,
                              I, F, F, F, F, P]
    b200_varlen_prefill_q8kv = [P, L, P, L, P, P, P, P, P, L, L, L, P, I, I, I, I, I, I, I, I, F,
                                I, I, I, I, F, F, F, F, P]
    b200_paged_decode_tma = [P, L, P, L, P, P, L, L, L, P, I, I, P, P, P, I, I, I, I, I, F, I, P]
    b200_varlen_prefill = [P, L, P, L, P, P, P, P, P, L, L, L, P, I, I, I, I, I, I, I, I, F,
                           I, I, I, P]
    b200_fmha_prefill = [P, L, P, L, P, P, P, P, P, L, L, L, P, I, I, I, I, I, I, I, I, F,
                         I, I, I, P]
    b200_merge_attn_states = [P, P, P, P, P, P, I, I, I, I, P]
    b200_mla_attention = [P, P, P, L, P, P, P, I, I, I, I, I, I, I, P, F, P]
    b200_gemm_wna16 = [P, L, P, P, P, P, P, L, I, I, I, I, I, P, P]
    b200_gemm_wna16_workspace = [I, I, I]
    b200_gemm_wna16_grouped = [P, L, P, P, P, P, L, I, I, I, I, I, I, P, P, P, P]
    b200_sample = [P, L, I, I, I, P, P, P, P, P, L, P, P]
    b200_top_k_top_p = [P, L, I, I, I, P, P, P]
    b200_advance_step = [I, I, I, P, P, P, P, P, P, I, I, P]
    b200_feed_tokens = [P, P, P, P, I, P]
    b200_moe_topk = [P, L, P, P, P, I, I, I, I, I, I, I, F, P, I, P, P, I, P]
    b200_moe_align = [P, P, P, P, P, P, P, I, I, I, I, P]
    b200_moe_permute = [P, L, P, L, P, P, I, I, I, I, I, P]
    b200_moe_row_weights = [P, P, P, P, I, I, P]
    b200_moe_unpermute_sum = [P, L, P, P, L, P, L, P, I, I, I, F, I, P]
    b200_get_ep_indices = [P, I, I, I, I, P, P, P, P]
    b200_gemm_bf16_grouped = [P, L, P, L, P, L, I, I, I, I, P, P, P, I, P]
    b200_gemm_skinny = [P, L, P, L, P, L, I, I, I, P, I, P, P, I, P]
    b200_gemm_skinny_workspace = [I, P, P]
    b200_gemm_wide2 = [P, L, P, L, P, L, I, I, I, P, I, P]
    b200_gemm_pair = [P, L, P, L, P, L, I, I, I, P, I, P]
    b200_gemm_pair_split = [P, L, P, L, P, L, I, I, I, P, I, P, P, P]
    b200_gemm_pair_split_workspace = [P, P]
    b200_gemm_skinny_plan = [I, I, I, I, P, P]
    b200_gemm_q8 = [P, L, P, L, P, L, I, I, I, P, L, P, L, P, I, P]
    b200_gemm_q8_grouped = [P, L, P, L, P, L, I, I, I, I, P, L, P, L, P, P, P, I, P]
    b200_per_token_quant = [P, L, P, L, P, P, I, I, I, I, P]
    b200_per_tensor_fp8_quant = [P, P, L, P, P, I, P]
    b200_int8_dequant = [P, P, L, P, P, I, P]
    b200_weight_dequant = [P, P, P, P, I, I, I, I, I, P]
    b200_bgmv = [P, L, P, L, P, P, I, I, I, I, F, I, I, I, P]
    b200_rejection_greedy = [P, P, P, P, P, I, I, P]
    b200_rejection_random = [P, P, P, P, P, P, P, P, I, I, I, P]
    b200_expand_batch_to_tokens = [P, P, P, I, L, L, P]
    b200_sample_recovered_tokens = [P, P, P, P, P, I, I, I, P]


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    """Device (or host) address of a tensor's first element, None for None."""
    if t is None:
        return None
    return t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def call(name: str, *args) -> None:
    """Calls an entry point and raises NativeError on a non-zero return."""
    global launch_count
    l = lib()
    if l is None:
        raise NativeError("native library not loaded")
    rc = getattr(l, name)(*args)
    launch_count += 1
    if rc != 0:
        raise NativeError(f"{name} failed with code {rc}")


def take_status() -> tuple[int, int, int, int]:
    """Synchronises the current stream, returns and clears the status word:
    (code, kernel id, detail, number of reports).  code 0 means no kernel
    reported a timeout or a bounds violation since the last call."""
    l = lib()
    if l is None:
        return (0, 0, 0, 0)
    out = (ctypes.c_uint * 4)()
    rc = l.b200_status_take(ctypes.cast(out, P), stream_ptr())
    if rc != 0:
        raise NativeError(f"b200_status_take failed with CUDA error {rc}")
    return tuple(int(x) for x in out)  # type: ignore[return-value]


def check_status() -> None:
    code, kid, detail, n = take_status()
    if code == 1 or code == 2:
        raise KernelTimeoutError(
            f"device wait timed out: kernel {kid}, detail {detail:#x}, {n} report(s)")
    if code != 0:
        raise NativeError(f"device guard tripped: code {code}, kernel {kid}, detail {detail}")
