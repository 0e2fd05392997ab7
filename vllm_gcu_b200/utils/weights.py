"""Checkpoint I/O: HuggingFace ``*.safetensors`` shards (with or without an index file).

A small self-contained reader / writer of the safetensors container is used when the
``safetensors`` package is absent, so checkpoints load in minimal environments.  The writer
also backs ``save_sharded_state`` (per-rank shards, the counterpart of the reference runner's
``save_sharded_state``, vllm_gcu/worker/model_runner.py:291-315).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from pathlib import Path
from typing import Iterator

import torch

_DTYPES = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
           "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
           "U8": torch.uint8, "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn,
           "F8_E5M2": torch.float8_e5m2, "F64": torch.float64}
_NAMES = {v: k for k, v in _DTYPES.items()}


def read_safetensors(path: str) -> Iterator[tuple[str, torch.Tensor]]:
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    base = 8 + n
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        dt = _DTYPES[meta["dtype"]]
        if hi == lo:
            yield name, torch.empty(meta["shape"], dtype=dt)
            continue
        buf = memoryview(mm)[base + lo:base + hi]
        t = torch.frombuffer(buf, dtype=torch.uint8).view(dt).reshape(meta["shape"])
        yield name, t


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None
                      ) -> None:
    header: dict = {}
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def iter_safetensors(model_dir: str) -> Iterator[tuple[str, torch.Tensor]]:
    """Yields (name, tensor) for every tensor of the checkpoint in ``model_dir``."""
    d = Path(model_dir)
    index = d / "model.safetensors.index.json"
    if index.exists():
        files = sorted(set(json.loads(index.read_text())["weight_map"].values()))
    else:
        files = sorted(p.name for p in d.glob("*.safetensors"))
    if not files:
        # older checkpoints: pickled state dicts (``pytorch_model.bin``, sharded or not)
        bin_index = d / "pytorch_model.bin.index.json"
        if bin_index.exists():
            bins = sorted(set(json.loads(bin_index.read_text())["weight_map"].values()))
        else:
            bins = sorted(p.name for p in list(d.glob("pytorch_model*.bin")) + list(d.glob("*.pt")))
        if not bins:
            raise FileNotFoundError(f"no .safetensors or .bin files in {model_dir}")
        for fn in bins:
            state = torch.load(str(d / fn), map_location="cpu", weights_only=True)
            yield from state.items()
            del state
        return
    for fn in files:
        yield from read_safetensors(str(d / fn))


def save_sharded_state(model: torch.nn.Module, out_dir: str, rank: int,
                       max_shard_bytes: int = 5 << 30) -> list[str]:
    """Writes this rank's parameters as ``model-rank-{rank}-part-{i}.safetensors``."""
    os.makedirs(out_dir, exist_ok=True)
    files, cur, size, part = [], {}, 0, 0
    for name, p in model.state_dict().items():
        nbytes = p.numel() * p.element_size()
        if cur and size + nbytes > max_shard_bytes:
            fn = os.path.join(out_dir, f"model-rank-{rank}-part-{part}.safetensors")
            write_safetensors(fn, cur)
            files.append(fn)
            cur, size, part = {}, 0, part + 1
        cur[name] = p
        size += nbytes
    if cur:
        fn = os.path.join(out_dir, f"model-rank-{rank}-part-{part}.safetensors")
        write_safetensors(fn, cur)
        files.append(fn)
    return files


def load_sharded_state(model: torch.nn.Module, in_dir: str, rank: int) -> None:
    sd = {}
    for p in sorted(Path(in_dir).glob(f"model-rank-{rank}-part-*.safetensors")):
        sd.update(dict(read_safetensors(str(p))))
    model.load_state_dict(sd, strict=False)
