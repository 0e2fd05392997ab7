"""Builds the native library ``vllm_gcu_b200/_b200.so`` for sm_100a.

Every ``*.cu`` file in this directory is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a`` into an object and the objects
are linked into one shared library next to the Python package, where
``vllm_gcu_b200.ops._native`` loads it with ctypes.  nvcc cross-compiles, so
the build runs on a machine without a GPU.

Usage: ``python -m vllm_gcu_b200.csrc.build [--force] [--verbose] [-j N] [--sanitize KIND]``

``--sanitize address|thread|undefined`` instruments the host side of the library (launch
wrappers, tensor-map encoding, workspace caches, status word plumbing) with the compiler's
sanitizer and writes ``_b200.<kind>.so`` beside the normal build; run with it through
``VLLM_B200_NATIVE_LIB=<that file>`` and the sanitizer runtime preloaded, e.g.
``LD_PRELOAD=$(gcc -print-file-name=libasan.so) VLLM_B200_NATIVE_LIB=... python -m pytest ...``.
Device code is not instrumented (the device-side checker is a separate tool).
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
OBJ_DIR = CSRC / "build"
LIB_PATH = PKG / "_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or add it to PATH")
    return cand


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha256()
    h.update(extra.encode())
    h.update(path.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(hdr.read_bytes())
    return h.hexdigest()


SANITIZERS = {"address": "-fsanitize=address", "thread": "-fsanitize=thread",
              "undefined": "-fsanitize=undefined"}


def sanitize_flags(kind: str | None) -> list[str]:
    """Extra nvcc flags of a host-sanitizer build (empty for the normal build)."""
    if not kind:
        return []
    if kind not in SANITIZERS:
        raise ValueError(f"unknown sanitizer {kind!r}; known: {sorted(SANITIZERS)}")
    return ["-Xcompiler", f"{SANITIZERS[kind]},-fno-omit-frame-pointer,-g"]


def lib_path_for(kind: str | None) -> Path:
    return LIB_PATH if not kind else PKG / f"_b200.{kind}.so"


def _compile_one(src: Path, force: bool, verbose: bool, sanitize: str | None = None) -> Path:
    obj_dir = OBJ_DIR if not sanitize else CSRC / f"build_{sanitize}"
    obj_dir.mkdir(exist_ok=True)
    obj = obj_dir / (src.stem + ".o")
    stamp = obj_dir / (src.stem + ".sha")
    flags = list(NVCC_FLAGS) + sanitize_flags(sanitize)
    if verbose:
        flags += ["-Xptxas", "-v"]
    dig = _digest(src, " ".join(flags))
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj
    cmd = [nvcc_path(), *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(f"$ {' '.join(cmd)}\n{res.stdout}{res.stderr}\n")
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}")
    stamp.write_text(dig)
    return obj


def build(force: bool = False, verbose: bool = False, jobs: int | None = None,
          sanitize: str | None = None) -> Path:
    """Compiles what changed and links the library.  Returns its path."""
    srcs = sorted(CSRC.glob("*.cu"))
    if not srcs:
        raise RuntimeError("no CUDA sources found")
    jobs = jobs or min(len(srcs), os.cpu_count() or 4)
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, force, verbose, sanitize), srcs))
    newest = max(o.stat().st_mtime for o in objs)
    out = lib_path_for(sanitize)
    if force or not out.exists() or out.stat().st_mtime < newest:
        cmd = [nvcc_path(), "-shared", "-o", str(out), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        if sanitize:
            cmd += ["-Xcompiler", SANITIZERS[sanitize]]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("-j", type=int, default=None)
    ap.add_argument("--sanitize", default=None, choices=sorted(SANITIZERS),
                    help="host-side sanitizer build into _b200.<kind>.so")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.j, a.sanitize))
    from ..utils.shm_ring import build_host_library
    print(build_host_library(a.force))          # host/shm_ring.cpp -> _b200_host.so (g++)


if __name__ == "__main__":
    main()
