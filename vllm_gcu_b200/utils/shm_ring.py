"""Shared-memory broadcast queue between the executor's front end and its worker processes.

One writer, ``readers`` readers, every reader receives every message in order.  The memory
layout and all ordered accesses live in the native library ``_b200_host.so``
(``csrc/host/shm_ring.cpp``); this module maps the region (a file under ``/dev/shm``), pickles
the messages and offers the waiting styles the executor needs: a blocking ``get`` with a
timeout and a cancel event, ``get_nowait`` and an asyncio ``get_async`` that yields to the
event loop while it waits.  The reference gets the same three from its patch of vLLM's
shared-memory queue (vllm_gcu/patch/patch_0_9_2/shm_broadcast.py:16-101: ``acquire_read_async``
with ``timeout`` and ``cancel``, ``dequeue_async``).

The reader objects are picklable (they travel to spawned workers as process arguments) and
attach to the region on first use.
"""
from __future__ import annotations

import asyncio
import ctypes
import mmap
import os
import pickle
import queue
import subprocess
import threading
import time
from pathlib import Path
from typing import Any, Optional

_PKG = Path(__file__).resolve().parent.parent
_LIB_PATH = _PKG / "_b200_host.so"
_SRC = _PKG / "csrc" / "host" / "shm_ring.cpp"
_lib = None
_lib_lock = threading.Lock()

OK, TIMEOUT, BAD_ARG, TOO_SMALL, NOT_READY = 0, -1, -2, -3, -4


def build_host_library(force: bool = False) -> Path:
    """Compiles the host-only library with the C++ compiler (no CUDA involved)."""
    if not force and _LIB_PATH.exists() and _LIB_PATH.stat().st_mtime >= _SRC.stat().st_mtime:
        return _LIB_PATH
    tmp = _LIB_PATH.with_suffix(f".{os.getpid()}.tmp")
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall",
           "-o", str(tmp), str(_SRC)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building {_LIB_PATH.name} failed:\n{res.stdout}{res.stderr}")
    os.replace(tmp, _LIB_PATH)
    return _LIB_PATH


def host_library():
    """The loaded native library (built on first use when missing or older than its source)."""
    global _lib
    with _lib_lock:
        if _lib is None:
            lib = ctypes.CDLL(str(build_host_library()))
            u32, u64, i64, vp = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int64, ctypes.c_void_p
            lib.b200_ring_bytes.restype = u64
            lib.b200_ring_bytes.argtypes = [u32, u32, u32]
            lib.b200_ring_init.restype = ctypes.c_int
            lib.b200_ring_init.argtypes = [vp, u64, u32, u32, u32]
            lib.b200_ring_write.restype = ctypes.c_int
            lib.b200_ring_write.argtypes = [vp, ctypes.c_char_p, u64, i64]
            for fn in (lib.b200_ring_try_read, lib.b200_ring_read):
                fn.restype = i64
            lib.b200_ring_try_read.argtypes = [vp, u32, vp, u64, ctypes.POINTER(u32),
                                               ctypes.POINTER(u64)]
            lib.b200_ring_read.argtypes = [vp, u32, vp, u64, ctypes.POINTER(u32),
                                           ctypes.POINTER(u64), i64]
            lib.b200_ring_backlog.restype = i64
            lib.b200_ring_backlog.argtypes = [vp, u32]
            _lib = lib
        return _lib


def available() -> bool:
    try:
        host_library()
        return os.path.isdir("/dev/shm")
    except Exception:  # noqa: BLE001 - no compiler / no library: callers fall back to pipes
        return False


class _Region:
    """A mapped ring region; the creator owns (and finally removes) the backing file."""

    def __init__(self, path: str, size: int = 0, create: bool = False):
        self.path, self.owner = path, create
        flags = os.O_RDWR | (os.O_CREAT | os.O_EXCL if create else 0)
        fd = os.open(path, flags, 0o600)
        try:
            if create:
                os.ftruncate(fd, size)
            self.size = os.fstat(fd).st_size
            self.map = mmap.mmap(fd, self.size)
        finally:
            os.close(fd)
        self._anchor = ctypes.c_char.from_buffer(self.map)
        self.base = ctypes.addressof(self._anchor)

    def unlink(self) -> None:
        """Removes the backing file's name; existing mappings stay valid.  Called once every
        reader has attached, so that no file is left behind however the processes end."""
        if self.owner:
            try:
                os.unlink(self.path)
            except FileNotFoundError:
                pass
            self.owner = False

    def close(self) -> None:
        self.base = None          # the native calls answer a null base with an error code
        if self.map is not None:
            self._anchor = None
            try:
                self.map.close()
            except BufferError:
                pass
            self.map = None
        if self.owner:
            try:
                os.unlink(self.path)
            except FileNotFoundError:
                pass
            self.owner = False


_counter = 0


class RingWriter:
    """Creates the ring and writes to it.  ``reader(i)`` gives the picklable i-th reader."""

    def __init__(self, readers: int, slots: int = 256, slot_bytes: int = 16384,
                 write_timeout_s: float = 60.0):
        global _counter
        lib = host_library()
        _counter += 1
        self.readers, self.slots, self.slot_bytes = readers, slots, slot_bytes
        self.write_timeout_s = write_timeout_s
        size = int(lib.b200_ring_bytes(slots, slot_bytes, readers))
        size = (size + mmap.PAGESIZE - 1) // mmap.PAGESIZE * mmap.PAGESIZE
        path = f"/dev/shm/b200_ring_{os.getpid()}_{_counter}_{time.monotonic_ns() & 0xffffff:x}"
        self.region = _Region(path, size, create=True)
        import atexit
        atexit.register(self.region.close)        # normal interpreter exit before unlink()
        rc = lib.b200_ring_init(self.region.base, size, slots, slot_bytes, readers)
        if rc != OK:
            self.region.close()
            raise RuntimeError(f"ring initialisation failed ({rc})")
        self._lock = threading.Lock()

    def reader(self, index: int) -> "RingReader":
        if not 0 <= index < self.readers:
            raise IndexError(index)
        return RingReader(self.region.path, index, self.slot_bytes)

    def put(self, obj: Any, timeout: Optional[float] = None) -> None:
        """Raises ``TimeoutError`` when some reader stayed a full ring behind for ``timeout``
        seconds (the writer treats that as a dead reader)."""
        data = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
        t = self.write_timeout_s if timeout is None else timeout
        with self._lock:
            if self.region.base is None:
                raise RuntimeError("the ring is closed")
            rc = host_library().b200_ring_write(self.region.base, data, len(data),
                                                int(t * 1e9))
        if rc == TIMEOUT:
            raise TimeoutError("a reader of the command ring stopped taking messages")
        if rc != OK:
            raise RuntimeError(f"ring write failed ({rc})")

    def unlink(self) -> None:
        """To be called when all readers have attached (they cannot attach afterwards)."""
        self.region.unlink()

    def backlog(self, index: int) -> int:
        if self.region.base is None:
            raise RuntimeError("the ring is closed")
        return int(host_library().b200_ring_backlog(self.region.base, index))

    def close(self) -> None:
        with self._lock:
            self.region.close()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


class RingReader:
    """One reader's end.  ``get`` / ``get_nowait`` raise ``queue.Empty`` like the standard
    queues, so the worker loop reads a ring or a pipe-backed queue the same way."""

    SLICE_NS = 20_000_000          # a blocking wait re-checks its cancel event this often

    def __init__(self, path: str, index: int, slot_bytes: int):
        self.path, self.index, self.slot_bytes = path, index, slot_bytes
        self._region: Optional[_Region] = None
        self._parts: list[bytes] = []

    def __getstate__(self):
        return {"path": self.path, "index": self.index, "slot_bytes": self.slot_bytes}

    def __setstate__(self, st):
        self.__init__(st["path"], st["index"], st["slot_bytes"])

    def attach(self) -> None:
        """Maps the region now (readers otherwise attach on first use)."""
        self._attach()

    def _attach(self):
        if self._region is None:
            self._region = _Region(self.path)
            self._buf = ctypes.create_string_buffer(self.slot_bytes)
            self._more = ctypes.c_uint32(0)
            self._need = ctypes.c_uint64(0)
        return self._region

    def _chunk(self, wait_ns: int) -> Optional[Any]:
        """Takes at most one chunk; returns the message it completed, else None.  A message
        of pickled ``None`` cannot be told from "nothing yet", so callers send tuples or
        objects, never a bare None."""
        reg, lib = self._attach(), host_library()
        if reg.base is None:
            raise RuntimeError("the ring is closed")
        args = (reg.base, self.index, ctypes.addressof(self._buf), self.slot_bytes,
                ctypes.byref(self._more), ctypes.byref(self._need))
        n = lib.b200_ring_read(*args, wait_ns) if wait_ns > 0 else lib.b200_ring_try_read(*args)
        if n in (NOT_READY, TIMEOUT):
            return None
        if n < 0:
            raise RuntimeError(f"ring read failed ({n})")
        self._parts.append(self._buf.raw[:n])
        if self._more.value:
            return None
        data, self._parts = b"".join(self._parts), []
        return pickle.loads(data)

    def get_nowait(self) -> Any:
        while True:
            had = len(self._parts)
            obj = self._chunk(0)
            if obj is not None:
                return obj
            if len(self._parts) == had:        # nothing arrived
                raise queue.Empty

    def get(self, timeout: Optional[float] = None,
            cancel: Optional[threading.Event] = None) -> Any:
        """Blocks until a message arrives.  ``queue.Empty`` after ``timeout`` seconds,
        ``RuntimeError("cancelled")`` once ``cancel`` is set."""
        end = None if timeout is None else time.monotonic() + timeout
        while True:
            if cancel is not None and cancel.is_set():
                raise RuntimeError("cancelled")
            wait = self.SLICE_NS
            if end is not None:
                left = end - time.monotonic()
                if left <= 0:
                    raise queue.Empty
                wait = max(1, min(wait, int(left * 1e9)))
            obj = self._chunk(wait)
            if obj is not None:
                return obj

    async def get_async(self, timeout: Optional[float] = None,
                        cancel: Optional[threading.Event] = None) -> Any:
        """As :meth:`get`, for coroutines: polls without blocking and hands the event loop
        back between polls (immediately at first, then in steps of up to a millisecond)."""
        end = None if timeout is None else time.monotonic() + timeout
        idle = 0
        while True:
            if cancel is not None and cancel.is_set():
                raise RuntimeError("cancelled")
            had = len(self._parts)
            obj = self._chunk(0)
            if obj is not None:
                return obj
            if len(self._parts) != had:
                continue
            if end is not None and time.monotonic() > end:
                raise TimeoutError
            idle += 1
            await asyncio.sleep(0 if idle < 50 else min(0.001, 0.00002 * (idle - 49)))

    def close(self) -> None:
        if self._region is not None:
            self._buf = None
            self._region.close()
            self._region = None
