"""Multi-process executor: one worker process per GPU, one front-end process.

Every worker hosts a complete engine replica (scheduler + runner) and the replicas advance
in lock-step: rank 0 decides how many queued commands (new requests, aborts) are applied
before the next step and broadcasts that count over the gloo group, so all schedulers see
the same inputs and stay bit-identical while only device collectives cross ranks inside a
step.  Outputs come from rank 0.

With data parallelism (``data_parallel_size > 1``) the ranks form ``dp`` replicas of
``tp * pp`` ranks.  The front end routes each request to the replica with the fewest
requests in flight (the reference patches vLLM's DP load balancer the same way,
vllm_gcu/patch/patch_0_9_2/engine.py:8-44); the command-count agreement runs inside a
replica, rank 0 of every replica returns outputs, and all replicas step together as long
as any of them has work (idle replicas run a zero-token forward so that expert-parallel
collectives line up).

Failure handling (the reference's executor reports worker exceptions as a ``FAILURE``
message and shuts the system down, vllm_gcu/v1/executor/async_multiproc_executor.py:92-171):

* an exception in any worker is sent to the front end as ``("FAILURE", rank, traceback)``;
* the front end watches the process sentinels and a per-worker heartbeat; a worker that
  exits or stops beating marks the executor dead;
* ``SIGTERM`` / ``SIGINT`` in a worker raise ``SystemExit`` once so ``finally`` blocks run;
* after a failure every call raises :class:`EngineDeadError` and ``shutdown`` terminates the
  remaining workers.

``AsyncMultiprocExecutor`` keeps the same process layout and adds an asyncio front end that
streams per-request outputs (used by the API server).
"""
from __future__ import annotations

import asyncio
import multiprocessing as mp
import os
import queue
import signal
import socket
import threading
import time
import traceback
from dataclasses import dataclass, field
from typing import Any, AsyncIterator, Optional, Sequence

from ..config import EngineConfig
from .request import RequestOutput, SamplingParams


class EngineDeadError(RuntimeError):
    """A worker failed; the executor cannot make progress any more."""


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@dataclass
class _Cmd:
    kind: str                       # add | abort | lora | stop | inject
    payload: Any = None


def _rank_address(addr: str, rank: int) -> str:
    """``host:port`` of an instance's rank 0 -> the address of its rank ``rank``."""
    host, _, port = addr.rpartition(":")
    return f"{host}:{int(port) + rank}"


def _worker_main(rank: int, world: int, port: int, cfg: EngineConfig, cmd_q, out_q, hb,
                 backend: Optional[str], parent_pid: int = 0) -> None:
    """Entry point of a worker process.  ``parent_pid``: the front end; a worker that finds
    itself re-parented (the front end was killed) exits instead of holding its GPU."""
    fired = {"v": False}

    def _on_signal(signum, frame):
        if not fired["v"]:
            fired["v"] = True
            raise SystemExit(128 + signum)

    signal.signal(signal.SIGTERM, _on_signal)
    signal.signal(signal.SIGINT, _on_signal)
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    try:
        import torch
        import torch.distributed as dist
        from ..parallel.state import get_state, init_distributed
        from ..utils import redirect_rank_output
        redirect_rank_output(rank)
        from .. import envs
        if envs.CPU_AFFINITY:
            from ..utils import bind_cpu_affinity
            bind_cpu_affinity(rank, world)
        pc = cfg.parallel
        if world > 1:
            init_distributed(pc.tensor_parallel_size, pc.pipeline_parallel_size,
                             pc.data_parallel_size, backend=backend,
                             enable_ep=pc.enable_expert_parallel)
        from .llm import LLMEngine
        engine = LLMEngine(cfg)
        st = get_state()
        ctrl = None
        dp = pc.data_parallel_size
        per_replica = world // dp
        lead = (rank // per_replica) * per_replica           # first rank of this replica
        if world > 1:
            for d in range(dp):                               # every rank joins every new_group
                ranks = list(range(d * per_replica, (d + 1) * per_replica))
                g = dist.new_group(ranks, backend="gloo") if len(ranks) > 1 else None
                if rank in ranks:
                    ctrl = g
        kvc = cfg.additional_config.get("kv_connector")
        connector = None
        if kvc:
            # disaggregated prefill with sharded instances: rank r of one instance talks to rank
            # r of the other, on the instance's base port + r (both sides use the same layout)
            from ..parallel.kv_transfer import P2PKVConnector
            connector = P2PKVConnector(host=kvc.get("host", "127.0.0.1"),
                                       port=int(kvc["port"]) + rank,
                                       send_type=kvc.get("send_type", "PUT_ASYNC"),
                                       device=str(engine.device))
            engine.attach_kv_connector(connector,
                                       recv_timeout_s=float(kvc.get("recv_timeout_s", 30.0)))
        if hasattr(cmd_q, "attach"):
            cmd_q.attach()            # the front end drops the ring's file name after READY
        out_q.put(("READY", rank, engine.runner.num_blocks))
        pending: list[_Cmd] = []
        stop = False
        last_stats, stepped = 0.0, False
        while not stop:
            hb.value = time.monotonic()
            if parent_pid and os.getppid() != parent_pid:
                os._exit(0)                   # the front end is gone
            # 1) agree on the commands applied before this step
            # every rank takes what has arrived (a shared-memory ring is bounded: a rank that
            # left commands in it would hold up the writer), the lead decides how many apply
            while True:
                try:
                    pending.append(cmd_q.get_nowait())
                except queue.Empty:
                    break
            if rank == lead:
                if not pending and not engine.has_unfinished() and not (
                        dp > 1 and engine.dp_global_busy):
                    try:
                        pending.append(cmd_q.get(timeout=0.05))
                    except queue.Empty:
                        pass
                n = len(pending)
            else:
                n = 0
            if ctrl is not None:
                t = torch.tensor([n], dtype=torch.int64)
                dist.broadcast(t, lead, group=ctrl)
                n = int(t.item())
                while len(pending) < n:
                    pending.append(cmd_q.get())
            batch, pending = pending[:n], pending[n:]
            for c in batch:
                if c.kind == "add":
                    rid, prompt, sp, prio, lora = c.payload[:5]
                    mm = c.payload[5] if len(c.payload) > 5 else None
                    kvp = c.payload[6] if len(c.payload) > 6 else None
                    if kvp and kvp.get("remote"):
                        # the front end names the peer instance by its base address
                        kvp = dict(kvp, remote=_rank_address(kvp["remote"], rank))
                    engine.add_request(prompt, sp, request_id=rid, priority=prio, lora_id=lora,
                                       multi_modal_data=mm, kv_transfer_params=kvp)
                elif c.kind == "abort":
                    engine.abort_request(c.payload)
                elif c.kind == "lora":
                    engine.add_lora(*c.payload)
                elif c.kind == "stop":
                    stop = True
                elif c.kind == "inject":
                    # host-side fault injection for tests: ("raise" | "exit", rank)
                    what, target = c.payload
                    if target == rank:
                        if what == "raise":
                            raise RuntimeError("injected worker failure")
                        if what == "exit":
                            os._exit(17)
            if stop:
                break
            # 2) one engine step
            if engine.has_unfinished() or dp > 1:
                outs = engine.step()          # dp > 1: every replica joins the exchange
                stepped = stepped or engine.has_unfinished() or bool(outs)
                if rank == lead and outs:
                    if connector is not None:
                        for o in outs:          # answers name the instance by its base address
                            if o.kv_transfer_params and o.kv_transfer_params.get("remote"):
                                o.kv_transfer_params = dict(
                                    o.kv_transfer_params,
                                    remote=_rank_address(o.kv_transfer_params["remote"], -rank))
                    out_q.put(("OUT", outs))
            if rank == lead and stepped and time.monotonic() - last_stats > 0.5:
                stepped = False
                # the front end's /metrics: scheduler and engine counters of this replica
                last_stats = time.monotonic()
                st_ = dict(engine.scheduler.stats())
                st_.update(engine.stats)
                if engine.spec_metrics is not None:
                    st_["spec_acceptance_rate"] = engine.spec_metrics.acceptance_rate
                out_q.put(("STATS", rank, st_))
        out_q.put(("STOPPED", rank, None))
    except SystemExit:
        raise
    except BaseException:  # noqa: BLE001 - everything is reported to the front end
        try:
            out_q.put(("FAILURE", rank, traceback.format_exc()))
            out_q.close()
            out_q.join_thread()          # flush the message before the process goes away
        finally:
            os._exit(1)


class MultiprocExecutor:
    HEARTBEAT_TIMEOUT_S = 120.0

    def __init__(self, cfg: EngineConfig, backend: Optional[str] = None,
                 start_timeout_s: float = 600.0):
        self.cfg = cfg
        self.world = cfg.parallel.world_size
        ctx = mp.get_context("spawn")
        self.out_q = ctx.Queue()
        self.dp = cfg.parallel.data_parallel_size
        self.per_replica = self.world // self.dp
        # commands travel through one shared-memory broadcast ring per replica (every rank of
        # a replica reads every command of that replica); pipe-backed queues when the native
        # host library is not available or VLLM_B200_SHM_BROADCAST=0
        from .. import envs
        from ..utils import shm_ring
        self.rings = None
        self._use_rings = bool(envs.SHM_BROADCAST) and shm_ring.available()
        if self._use_rings:
            self.rings = [shm_ring.RingWriter(self.per_replica) for _ in range(self.dp)]
            self.cmd_qs = [self.rings[r // self.per_replica].reader(r % self.per_replica)
                           for r in range(self.world)]
        else:
            self.cmd_qs = [ctx.Queue() for _ in range(self.world)]
        self.hbs = [ctx.Value("d", time.monotonic()) for _ in range(self.world)]
        port = _free_port()
        self.procs = [ctx.Process(target=_worker_main, daemon=True,
                                  args=(r, self.world, port, cfg, self.cmd_qs[r], self.out_q,
                                        self.hbs[r], backend, os.getpid()))
                      for r in range(self.world)]
        for p in self.procs:
            p.start()
        self.dead: Optional[str] = None
        self._lock = threading.Lock()
        self._ids = 0
        self._replica_of: dict[str, int] = {}
        self._replica_stats: dict[int, dict] = {}      # lead rank -> latest counters
        self._in_flight = [0] * self.dp
        ready = 0
        deadline = time.monotonic() + start_timeout_s
        while ready < self.world:
            msg = self._get(max(0.1, deadline - time.monotonic()))
            if msg is None:
                self._fail("worker start-up timed out")
            if msg[0] == "READY":
                ready += 1
            elif msg[0] == "FAILURE":
                self._fail(f"worker {msg[1]} failed during start-up:\n{msg[2]}")
        for ring in self.rings or ():
            ring.unlink()             # every reader is attached: no file outlives the processes

    # -- plumbing ------------------------------------------------------------------
    def _get(self, timeout: float):
        """Next message from the workers, or None; checks worker liveness while waiting."""
        end = time.monotonic() + timeout
        while True:
            try:
                return self.out_q.get(timeout=0.05)
            except queue.Empty:
                pass
            self.check_health()
            if time.monotonic() >= end:
                return None

    def _fail(self, why: str) -> None:
        self.dead = why
        self.shutdown()
        raise EngineDeadError(why)

    def check_health(self) -> None:
        if self.dead:
            raise EngineDeadError(self.dead)
        now = time.monotonic()
        for r, p in enumerate(self.procs):
            if not p.is_alive() and p.exitcode not in (0, None):
                # drain a FAILURE message if the worker managed to send one
                detail = ""
                try:
                    while True:
                        m = self.out_q.get_nowait()
                        if m[0] == "FAILURE":
                            detail = "\n" + m[2]
                            break
                except queue.Empty:
                    pass
                self._fail(f"worker {r} exited with code {p.exitcode}{detail}")
            if p.is_alive() and now - self.hbs[r].value > self.HEARTBEAT_TIMEOUT_S:
                self._fail(f"worker {r} stopped responding")

    def _broadcast(self, cmd: _Cmd) -> None:
        if self.dead:
            raise EngineDeadError(self.dead)
        with self._lock:
            for d in range(self.dp):
                self._send(d, cmd)

    def _send(self, replica: int, cmd: _Cmd, timeout: Optional[float] = None) -> None:
        """Hands ``cmd`` to every rank of ``replica`` (caller holds the lock)."""
        if self._use_rings:
            if self.rings is None:
                raise EngineDeadError(self.dead or "the executor was shut down")
            try:
                self.rings[replica].put(cmd, timeout)
            except TimeoutError as e:
                self.dead = self.dead or f"command ring of replica {replica}: {e}"
                raise EngineDeadError(self.dead)
            return
        for r in range(replica * self.per_replica, (replica + 1) * self.per_replica):
            self.cmd_qs[r].put(cmd)

    # -- API -----------------------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int],
                    sampling_params: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, priority: int = 0, lora_id: int = -1,
                    multi_modal_data: Optional[dict] = None,
                    kv_transfer_params: Optional[dict] = None) -> str:
        if request_id is None:
            request_id = f"req-{self._ids}"
            self._ids += 1
        from .llm import check_token_ids
        check_token_ids(prompt_token_ids, self.cfg.model.vocab_size,
                        allow_placeholders=bool(multi_modal_data))
        if sampling_params is not None and sampling_params.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        cmd = _Cmd("add", (request_id, list(prompt_token_ids),
                           sampling_params or SamplingParams(), priority, lora_id,
                           multi_modal_data, kv_transfer_params))
        if self.dp == 1:
            self._broadcast(cmd)
            return request_id
        if self.dead:
            raise EngineDeadError(self.dead)
        with self._lock:
            d = min(range(self.dp), key=lambda i: self._in_flight[i])
            self._in_flight[d] += 1
            self._replica_of[request_id] = d
            self._send(d, cmd)
        return request_id

    def stats(self) -> dict:
        """Latest counters of the replicas (sums; cache usage and acceptance rate as means),
        refreshed about twice a second while the workers step."""
        out: dict = {}
        reps = list(self._replica_stats.values())
        for st_ in reps:
            for k, v in st_.items():
                if isinstance(v, (int, float)):
                    out[k] = out.get(k, 0.0) + v
        for k in ("kv_cache_usage", "spec_acceptance_rate"):
            if k in out and reps:
                out[k] /= len(reps)
        return out

    def abort_request(self, request_id: str) -> None:
        self._broadcast(_Cmd("abort", request_id))

    def add_lora(self, lora_request, tensors=None, config=None) -> None:
        """Loads a LoRA adapter in every worker (each keeps its tensor-parallel shard of the
        full adapter tensors); later requests select it with ``lora_id``.  The command takes its
        place in the same ordered stream as the requests, so a request added afterwards finds
        the adapter loaded on every rank."""
        self._broadcast(_Cmd("lora", (lora_request, tensors, config)))

    def inject_fault(self, what: str, rank: int) -> None:
        """Test hook: make worker ``rank`` raise an exception or exit at its next step."""
        self._broadcast(_Cmd("inject", (what, rank)))

    def poll(self, timeout: float = 0.1) -> list[RequestOutput]:
        """Outputs produced since the last call (blocks up to ``timeout`` for the first)."""
        outs: list[RequestOutput] = []
        msg = self._get(timeout)
        while msg is not None:
            if msg[0] == "OUT":
                outs.extend(msg[1])
                if self.dp > 1:
                    for o in msg[1]:
                        if o.finished:
                            d = self._replica_of.pop(o.request_id, None)
                            if d is not None:
                                self._in_flight[d] -= 1
            elif msg[0] == "FAILURE":
                self._fail(f"worker {msg[1]} failed:\n{msg[2]}")
            elif msg[0] == "STATS":
                self._replica_stats[msg[1]] = msg[2]
            try:
                msg = self.out_q.get_nowait()
            except queue.Empty:
                msg = None
        return outs

    def generate(self, prompts, sampling_params=None, timeout_s: float = 600.0
                 ) -> list[RequestOutput]:
        prompts = list(prompts)
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sps = [sampling_params or SamplingParams()] * len(prompts)
        else:
            sps = list(sampling_params)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, sps)]
        final: dict[str, RequestOutput] = {}
        deadline = time.monotonic() + timeout_s
        while len(final) < len(ids):
            for o in self.poll(0.2):
                if o.finished:
                    final[o.request_id] = o
            if time.monotonic() > deadline:
                self._fail("generate() timed out")
        return [final[i] for i in ids]

    def shutdown(self) -> None:
        for d in range(self.dp):
            try:
                self._send(d, _Cmd("stop"), timeout=1.0)
            except Exception:
                pass
        t_end = time.monotonic() + 5.0
        for p in self.procs:
            p.join(max(0.0, t_end - time.monotonic()))
        for p in self.procs:
            if p.is_alive():
                p.terminate()
        for p in self.procs:
            p.join(2.0)
            if p.is_alive():
                p.kill()
        rings, self.rings = self.rings, None
        for ring in rings or ():
            ring.close()

    def __del__(self):
        try:
            self.shutdown()
        except Exception:
            pass


class AsyncMultiprocExecutor(MultiprocExecutor):
    """asyncio front end: ``generate_stream`` yields the outputs of one request as they are
    produced while other requests run concurrently; a background thread pumps ``poll``."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self._streams: dict[str, asyncio.Queue] = {}
        self._loop: Optional[asyncio.AbstractEventLoop] = None
        self._pump: Optional[threading.Thread] = None
        self._stop_pump = threading.Event()

    def _ensure_pump(self) -> None:
        if self._pump is not None:
            return
        self._loop = asyncio.get_running_loop()

        def run():
            while not self._stop_pump.is_set():
                try:
                    outs = self.poll(0.05)
                except EngineDeadError as e:
                    for q in list(self._streams.values()):
                        self._loop.call_soon_threadsafe(q.put_nowait, e)
                    return
                for o in outs:
                    q = self._streams.get(o.request_id)
                    if q is not None:
                        self._loop.call_soon_threadsafe(q.put_nowait, o)

        self._pump = threading.Thread(target=run, daemon=True)
        self._pump.start()

    def validate_prompt(self, prompt_token_ids: Sequence[int], multimodal: bool = False) -> None:
        """Raises ValueError for a prompt the workers' scheduler would refuse."""
        n = len(prompt_token_ids)
        if n == 0:
            raise ValueError("the prompt is empty")
        limit = self.cfg.scheduler.max_model_len
        if n >= limit:
            raise ValueError(f"prompt of {n} tokens exceeds max_model_len {limit}")
        from .llm import check_token_ids
        check_token_ids(prompt_token_ids, self.cfg.model.vocab_size,
                        allow_placeholders=multimodal)

    async def generate_stream(self, prompt_token_ids: Sequence[int],
                              sampling_params: Optional[SamplingParams] = None,
                              request_id: Optional[str] = None, priority: int = 0,
                              lora_id: int = -1, multi_modal_data: Optional[dict] = None,
                              kv_transfer_params: Optional[dict] = None
                              ) -> AsyncIterator[RequestOutput]:
        self.validate_prompt(prompt_token_ids)
        self._ensure_pump()
        q: asyncio.Queue = asyncio.Queue()
        rid = request_id or f"areq-{self._ids}"
        self._ids += 1
        self._streams[rid] = q
        self.add_request(prompt_token_ids, sampling_params, rid, priority, lora_id,
                         multi_modal_data, kv_transfer_params)
        try:
            while True:
                item = await q.get()
                if isinstance(item, Exception):
                    raise item
                yield item
                if item.finished:
                    break
        except asyncio.CancelledError:
            self.abort_request(rid)
            raise
        finally:
            self._streams.pop(rid, None)

    def shutdown(self) -> None:
        self._stop_pump.set()
        super().shutdown()
