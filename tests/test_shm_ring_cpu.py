"""Shared-memory broadcast ring (native library + Python queue interface) on the host: order,
chunked large messages, back-pressure, time-outs, cancel, asyncio reads, and two reader
processes."""
import asyncio
import multiprocessing as mp
import queue
import threading
import time

import pytest

from vllm_gcu_b200.utils import shm_ring

pytestmark = pytest.mark.skipif(not shm_ring.available(), reason="no host compiler or /dev/shm")


def test_every_reader_gets_every_message_in_order():
    w = shm_ring.RingWriter(readers=2, slots=4, slot_bytes=128)
    r0, r1 = w.reader(0), w.reader(1)
    try:
        with pytest.raises(queue.Empty):
            r0.get_nowait()
        msgs = [("add", i, list(range(i))) for i in range(3)]
        for m in msgs:
            w.put(m)
        assert [r0.get_nowait() for _ in msgs] == msgs
        assert w.backlog(0) == 0 and w.backlog(1) == 3
        assert [r1.get(timeout=1.0) for _ in msgs] == msgs
        # a message much longer than a slot travels as chunks; slots are reused many times
        big = ("add", "x" * 5000, list(range(700)))
        got = []
        t = threading.Thread(target=lambda: got.extend(r1.get(timeout=5.0) for _ in range(3)))
        t0 = threading.Thread(target=lambda: [r0.get(timeout=5.0) for _ in range(3)])
        t.start(), t0.start()
        for _ in range(3):
            w.put(big, timeout=5.0)
        t.join(), t0.join()
        assert got == [big] * 3
    finally:
        r0.close(), r1.close(), w.close()


def test_timeouts_cancel_and_a_reader_that_stops_taking_messages():
    w = shm_ring.RingWriter(readers=2, slots=2, slot_bytes=64)
    r0, r1 = w.reader(0), w.reader(1)
    try:
        t = time.monotonic()
        with pytest.raises(queue.Empty):
            r0.get(timeout=0.05)
        assert 0.04 < time.monotonic() - t < 1.0
        ev = threading.Event()
        threading.Timer(0.05, ev.set).start()
        with pytest.raises(RuntimeError, match="cancelled"):
            r0.get(timeout=5.0, cancel=ev)
        w.put(("a",)), w.put(("b",))
        assert r0.get_nowait() == ("a",) and r0.get_nowait() == ("b",)
        with pytest.raises(TimeoutError):          # reader 1 never took anything: ring is full
            w.put(("c",), timeout=0.05)
        assert r1.get_nowait() == ("a",)
        w.put(("c",), timeout=1.0)
        assert r0.get(timeout=1.0) == ("c",)
    finally:
        r0.close(), r1.close(), w.close()


def test_async_reader_yields_to_the_event_loop():
    w = shm_ring.RingWriter(readers=1, slots=4, slot_bytes=64)
    r = w.reader(0)

    async def run():
        ticks = 0

        async def ticker():
            nonlocal ticks
            while True:
                ticks += 1
                await asyncio.sleep(0)

        tk = asyncio.create_task(ticker())
        threading.Timer(0.05, lambda: w.put(("late", "y" * 300))).start()
        msg = await r.get_async(timeout=5.0)
        with pytest.raises(TimeoutError):
            await r.get_async(timeout=0.02)
        tk.cancel()
        return msg, ticks

    try:
        msg, ticks = asyncio.run(run())
        assert msg == ("late", "y" * 300) and ticks > 5
    finally:
        r.close(), w.close()


def _reader_proc(reader, n, out_q):
    total = 0
    for _ in range(n):
        kind, i, payload = reader.get(timeout=20.0)
        total += i + len(payload)
    out_q.put((reader.index, total))


def test_two_reader_processes():
    ctx = mp.get_context("spawn")
    w = shm_ring.RingWriter(readers=2, slots=8, slot_bytes=256)
    out_q = ctx.Queue()
    n = 200
    procs = [ctx.Process(target=_reader_proc, args=(w.reader(i), n, out_q)) for i in range(2)]
    try:
        for p in procs:
            p.start()
        want = 0
        for i in range(n):
            payload = b"z" * (i * 7 % 900)
            w.put(("add", i, payload), timeout=20.0)
            want += i + len(payload)
        got = dict(out_q.get(timeout=30.0) for _ in procs)
        assert got == {0: want, 1: want}
    finally:
        for p in procs:
            p.join(10.0)
        w.close()


def test_unlinked_ring_keeps_working_and_leaves_no_file():
    import os
    w = shm_ring.RingWriter(readers=1, slots=4, slot_bytes=64)
    r = w.reader(0)
    path = w.region.path
    try:
        r.attach()
        assert os.path.exists(path)
        w.unlink()
        assert not os.path.exists(path)
        w.put(("still", "works"))
        assert r.get(timeout=1.0) == ("still", "works")
        with pytest.raises(FileNotFoundError):
            w.reader(0).attach()          # nobody can attach after the name is gone
    finally:
        r.close(), w.close()
