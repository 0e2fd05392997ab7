"""Point-to-point KV connector for disaggregated prefill (1P1D and xPyD).

Each engine instance owns a ZMQ ROUTER socket (control + data plane on one connection: the
payload travels as a zero-copy ZMQ frame backed by a pinned host tensor).  Tensor ids are
``request_id#layer_name``.  Modes, as in the reference's ``P2pEcclEngine``
(vllm_gcu/distributed/kv_transfer/v1/p2p_eccl_engine.py:120-235,311-373):

* ``PUT``        – the producer pushes synchronously and waits for the ACK;
* ``PUT_ASYNC``  – pushes from a background sender thread;
* ``GET``        – the producer keeps tensors in an LRU send store, the consumer pulls.

Receive side: tensors are kept on the device up to ``kv_buffer_size`` bytes and spill to a
pinned ``TensorMemoryPool`` above that; a peer that cannot take a tensor answers NACK and
``send_tensor`` returns False (the scheduler then recomputes instead of failing,
vllm_gcu/distributed/kv_transfer/connector.py:184-203).  A heartbeat thread announces the
instance to an optional proxy every 3 s so that the proxy can evict dead instances
(p2p_eccl_engine.py:488-500).
"""
from __future__ import annotations

import threading
import time
from collections import OrderedDict
from typing import Optional

import msgpack
import torch
import zmq

_DT = {"torch.float32": torch.float32, "torch.float16": torch.float16,
       "torch.bfloat16": torch.bfloat16, "torch.int8": torch.int8, "torch.uint8": torch.uint8,
       "torch.int32": torch.int32, "torch.int64": torch.int64,
       "torch.float8_e4m3fn": torch.float8_e4m3fn}


class TensorMemoryPool:
    """Bump allocator with a free list over one pinned host buffer."""

    def __init__(self, size_bytes: int, pin: bool = True):
        self.size = size_bytes
        self.buf = torch.empty(size_bytes, dtype=torch.uint8,
                               pin_memory=pin and torch.cuda.is_available())
        self.free: list[tuple[int, int]] = [(0, size_bytes)]
        self.used: dict[int, int] = {}
        self.lock = threading.Lock()

    def store(self, t: torch.Tensor) -> Optional[int]:
        n = t.numel() * t.element_size()
        n_al = -(-n // 256) * 256
        with self.lock:
            for i, (off, sz) in enumerate(self.free):
                if sz >= n_al:
                    self.free[i] = (off + n_al, sz - n_al)
                    if self.free[i][1] == 0:
                        self.free.pop(i)
                    self.used[off] = n_al
                    break
            else:
                return None
        self.buf[off:off + n].copy_(t.contiguous().view(torch.uint8).view(-1))
        return off

    def load(self, off: int, shape, dtype, device) -> torch.Tensor:
        n = int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size()
        return self.buf[off:off + n].view(dtype).view(shape).to(device, non_blocking=True)

    def release(self, off: int) -> None:
        with self.lock:
            sz = self.used.pop(off, None)
            if sz is not None:
                self.free.append((off, sz))
                self.free.sort()
                merged = []
                for o, s in self.free:
                    if merged and merged[-1][0] + merged[-1][1] == o:
                        merged[-1] = (merged[-1][0], merged[-1][1] + s)
                    else:
                        merged.append((o, s))
                self.free = merged


class P2PKVConnector:
    def __init__(self, host: str = "127.0.0.1", port: int = 0, send_type: str = "PUT",
                 kv_buffer_size: int = 1 << 30, mem_pool_size: int = 1 << 30,
                 device: str = "cpu", proxy_addr: Optional[str] = None, role: str = "kv_both",
                 http_port: int = 0):
        assert send_type in ("PUT", "PUT_ASYNC", "GET")
        self.send_type = send_type
        self.device = torch.device(device)
        self.ctx = zmq.Context.instance()
        self.router = self.ctx.socket(zmq.ROUTER)
        if port == 0:
            self.port = self.router.bind_to_random_port(f"tcp://{host}")
        else:
            self.router.bind(f"tcp://{host}:{port}")
            self.port = int(port)
        self.addr = f"{host}:{self.port}"
        self.peers: dict[str, zmq.Socket] = {}
        self.peer_locks: dict[str, threading.Lock] = {}
        self.recv_store: dict[str, object] = {}
        self.recv_cv = threading.Condition()
        self.buffer_used = 0
        self.kv_buffer_size = kv_buffer_size
        self.pool = TensorMemoryPool(mem_pool_size) if mem_pool_size > 0 else None
        self.send_store: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        self.send_store_bytes = 0
        self.send_q: list = []
        self.send_cv = threading.Condition()
        self.stopped = threading.Event()
        self.stats = {"sent": 0, "received": 0, "nack": 0, "spilled": 0, "get_miss": 0}
        self.listener = threading.Thread(target=self._listen, daemon=True)
        self.listener.start()
        if send_type == "PUT_ASYNC":
            self.sender = threading.Thread(target=self._send_loop, daemon=True)
            self.sender.start()
        if proxy_addr:
            self.proxy_addr, self.role, self.http_port = proxy_addr, role, http_port
            threading.Thread(target=self._ping, daemon=True).start()

    # -- sending -----------------------------------------------------------------------
    def _peer(self, remote: str) -> tuple[zmq.Socket, threading.Lock]:
        if remote not in self.peers:
            s = self.ctx.socket(zmq.DEALER)
            s.setsockopt_string(zmq.IDENTITY, self.addr)
            s.setsockopt(zmq.LINGER, 0)
            s.connect(f"tcp://{remote}")
            self.peers[remote] = s
            self.peer_locks[remote] = threading.Lock()
        return self.peers[remote], self.peer_locks[remote]

    def send_tensor(self, tensor_id: str, tensor: torch.Tensor, remote: str) -> bool:
        if self.send_type == "GET":
            n = tensor.numel() * tensor.element_size()
            self.send_store[tensor_id] = tensor
            self.send_store_bytes += n
            while self.send_store_bytes > self.kv_buffer_size and len(self.send_store) > 1:
                _, old = self.send_store.popitem(last=False)
                self.send_store_bytes -= old.numel() * old.element_size()
            return True
        if self.send_type == "PUT_ASYNC":
            with self.send_cv:
                self.send_q.append((tensor_id, tensor, remote))
                self.send_cv.notify()
            return True
        return self._send_sync(tensor_id, tensor, remote)

    def _send_loop(self) -> None:
        while not self.stopped.is_set():
            with self.send_cv:
                while not self.send_q and not self.stopped.is_set():
                    self.send_cv.wait(0.1)
                if self.stopped.is_set():
                    return
                item = self.send_q.pop(0)
            self._send_sync(*item)

    def _send_sync(self, tensor_id: str, tensor: torch.Tensor, remote: str,
                   timeout_s: float = 30.0) -> bool:
        sock, lock = self._peer(remote)
        host = tensor.detach().to("cpu").contiguous()
        hdr = msgpack.dumps({"cmd": "PUT", "id": tensor_id, "shape": list(host.shape),
                             "dtype": str(host.dtype)})
        payload = host.view(torch.uint8).view(-1).numpy()
        with lock:
            sock.send_multipart([hdr, payload], copy=False)
            if sock.poll(int(timeout_s * 1000)) == 0:
                return False
            ack = sock.recv()
        ok = ack == b"0"
        self.stats["sent" if ok else "nack"] += 1
        return ok

    # -- receiving ---------------------------------------------------------------------
    def _listen(self) -> None:
        poller = zmq.Poller()
        poller.register(self.router, zmq.POLLIN)
        while not self.stopped.is_set():
            if not dict(poller.poll(100)):
                continue
            frames = self.router.recv_multipart()
            ident, hdr = frames[0], msgpack.loads(frames[1])
            if hdr["cmd"] == "PUT":
                ok = self._store(hdr, frames[2])
                self.router.send_multipart([ident, b"0" if ok else b"1"])
            elif hdr["cmd"] == "GET":
                t = self.send_store.get(hdr["id"])
                if t is None:
                    self.stats["get_miss"] += 1
                    self.router.send_multipart([ident, msgpack.dumps({"ret": 1})])
                else:
                    host = t.detach().to("cpu").contiguous()
                    meta = msgpack.dumps({"ret": 0, "shape": list(host.shape),
                                          "dtype": str(host.dtype)})
                    self.router.send_multipart(
                        [ident, meta, host.view(torch.uint8).view(-1).numpy()], copy=False)

    def _store(self, hdr: dict, payload: bytes) -> bool:
        dt = _DT[hdr["dtype"]]
        t = torch.frombuffer(bytearray(payload), dtype=torch.uint8).view(dt).view(hdr["shape"])
        n = t.numel() * t.element_size()
        with self.recv_cv:
            if self.buffer_used + n <= self.kv_buffer_size:
                self.recv_store[hdr["id"]] = t.to(self.device)
                self.buffer_used += n
            else:
                off = self.pool.store(t) if self.pool is not None else None
                if off is None:
                    return False                       # out of memory everywhere: NACK
                self.recv_store[hdr["id"]] = ("pool", off, tuple(hdr["shape"]), dt)
                self.stats["spilled"] += 1
            self.stats["received"] += 1
            self.recv_cv.notify_all()
        return True

    def recv_tensor(self, tensor_id: str, remote: Optional[str] = None,
                    timeout_s: float = 30.0) -> Optional[torch.Tensor]:
        if self.send_type == "GET":
            assert remote is not None
            sock, lock = self._peer(remote)
            with lock:
                sock.send_multipart([msgpack.dumps({"cmd": "GET", "id": tensor_id})])
                if sock.poll(int(timeout_s * 1000)) == 0:
                    return None
                frames = sock.recv_multipart()
            meta = msgpack.loads(frames[0])
            if meta["ret"] != 0:
                return None
            return torch.frombuffer(bytearray(frames[1]), dtype=torch.uint8).view(
                _DT[meta["dtype"]]).view(meta["shape"]).to(self.device)
        end = time.monotonic() + timeout_s
        with self.recv_cv:
            while tensor_id not in self.recv_store:
                left = end - time.monotonic()
                if left <= 0:
                    return None
                self.recv_cv.wait(left)
            item = self.recv_store.pop(tensor_id)
        if isinstance(item, tuple):
            _, off, shape, dt = item
            t = self.pool.load(off, shape, dt, self.device)
            if t.is_cuda:
                torch.cuda.current_stream().synchronize()
            self.pool.release(off)
            return t
        self.buffer_used -= item.numel() * item.element_size()
        return item

    # -- membership ----------------------------------------------------------------------
    def _ping(self) -> None:
        sock = self.ctx.socket(zmq.DEALER)
        sock.setsockopt(zmq.LINGER, 0)
        sock.connect(f"tcp://{self.proxy_addr}")
        msg = msgpack.dumps({"type": "P" if self.role == "kv_producer" else "D",
                             "http_address": f"{self.addr.split(':')[0]}:{self.http_port}",
                             "zmq_address": self.addr})
        while not self.stopped.is_set():
            try:
                sock.send(msg, zmq.NOBLOCK)
            except zmq.ZMQError:
                pass
            self.stopped.wait(3.0)
        sock.close()

    def close(self) -> None:
        self.stopped.set()
        with self.send_cv:
            self.send_cv.notify_all()
        self.listener.join(1.0)
        for s in self.peers.values():
            s.close()
        self.router.close()


def kv_tensor_id(request_id: str, layer_name: str) -> str:
    return f"{request_id}#{layer_name}"
