"""Builds the native library ``vllm_gcu_b200/_b200.so`` for sm_100a.

Every ``*.cu`` file in this directory is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a`` into an object and the objects
are linked into one shared library next to the Python package, where
``vllm_gcu_b200.ops._native`` loads it with ctypes.  nvcc cross-compiles, so
the build runs on a machine without a GPU.

Usage: ``python -m vllm_gcu_b200.csrc.build [--force] [--verbose] [-j N]``
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


def _compile_one(src: Path, force: bool, verbose: bool) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = OBJ_DIR / (src.stem + ".sha")
    flags = list(NVCC_FLAGS)
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


def build(force: bool = False, verbose: bool = False, jobs: int | None = None) -> Path:
    """Compiles what changed and links the library.  Returns its path."""
    srcs = sorted(CSRC.glob("*.cu"))
    if not srcs:
        raise RuntimeError("no CUDA sources found")
    jobs = jobs or min(len(srcs), os.cpu_count() or 4)
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, force, verbose), srcs))
    newest = max(o.stat().st_mtime for o in objs)
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest:
        cmd = [nvcc_path(), "-shared", "-o", str(LIB_PATH), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB_PATH


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("-j", type=int, default=None)
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.j))


if __name__ == "__main__":
    main()
