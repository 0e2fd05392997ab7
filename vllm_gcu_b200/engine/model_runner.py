"""Model runner: turns a scheduler decision into device work.

Responsibilities (the reference splits them over ``GCUModelRunner`` and
``AsyncGCUModelRunner``, vllm_gcu/worker/worker_v1.py:30-230 and
vllm_gcu/v1/gcu_async_model_runner.py:99-1081):

* persistent input buffers on the device, filled from pinned host staging with two
  asynchronous copies per step (one int64 block, one int32 block);
* batch layout "decodes first", attention metadata, KV-cache allocation from a memory
  profile;
* device-side next-token feed: a request that continues from a token sampled by the
  previous step takes it from the previous step's on-device output, so the host never
  waits for token ids before launching the next step (async_model_runner.py:370-473);
* CUDA-graph capture of decode-only steps per padded batch size, with batch size 0
  handled eagerly as the dummy step of idle data-parallel ranks (worker_v1.py:52-180);
* fused sampling on the device and an asynchronous device-to-host copy of the ids.
"""
from __future__ import annotations

import time
import zlib
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from ..config import EngineConfig
from ..layers.attention import AttentionMetadata
from ..layers.sampler import RowParallelSampler, Sampler, SamplingTensors
from ..ops import _native
from .scheduler import ScheduledRequest, SchedulerOutput


@dataclass
class StepHandle:
    """Result of a launched step; ``token_ids()`` blocks until the ids are on the host."""
    req_ids: list[str]                     # sampling requests, in output order
    num_sampled: int
    sampled_host: Optional[torch.Tensor]   # pinned int64 [num_sampled * width]
    event: Optional[torch.cuda.Event]
    width: int = 1                         # tokens per request (1 + speculative tokens)
    accepted_host: Optional[torch.Tensor] = None
    draft: Optional[dict[str, list[int]]] = None
    device_ms_events: Optional[tuple] = None
    draft_host: Optional[torch.Tensor] = None
    extra: dict = field(default_factory=dict)

    def draft_tokens(self) -> Optional[dict[str, list[int]]]:
        """Draft tokens proposed by the on-device drafter for every sampling request."""
        if self.draft_host is None or self.num_sampled == 0:
            return None
        self.wait()
        k = int(self.extra.get("draft_width", 1))
        arr = self.draft_host[: self.num_sampled * k].numpy().reshape(self.num_sampled, k)
        return {rid: [int(t) for t in arr[i]] for i, rid in enumerate(self.req_ids)}

    def ready(self) -> bool:
        return self.event is None or self.event.query()

    def wait(self) -> None:
        if self.event is not None:
            self.event.synchronize()

    def token_ids(self) -> dict[str, list[int]]:
        self.wait()
        out: dict[str, list[int]] = {}
        if self.num_sampled == 0:
            return out
        arr = self.sampled_host[: self.num_sampled * self.width].numpy()
        if self.width == 1:
            for i, rid in enumerate(self.req_ids):
                out[rid] = [int(arr[i])]
        else:
            arr = arr.reshape(self.num_sampled, self.width)
            for i, rid in enumerate(self.req_ids):
                row = arr[i]
                out[rid] = [int(t) for t in row if t >= 0]
        return out


def _pad_batch(n: int, sizes: list[int]) -> int:
    for s in sizes:
        if s >= n:
            return s
    return n


class ModelRunner:
    def __init__(self, cfg: EngineConfig, model, device: torch.device):
        self.cfg = cfg
        self.model = model
        self.device = device
        self.is_cuda = device.type == "cuda"
        sc = cfg.scheduler
        self.block_size = cfg.cache.block_size
        self.max_seqs = sc.max_num_seqs
        self.max_tokens = max(sc.max_num_batched_tokens, sc.max_num_seqs)
        self.max_blocks = -(-sc.max_model_len // self.block_size) + 1
        self.kv_caches: list[torch.Tensor] = []
        self.num_blocks = 0
        tp = cfg.parallel.tensor_parallel_size
        # under tensor parallelism every rank samples its slice of the batch rows and the ids
        # are gathered (the reference's DPParallelSampler, vllm_gcu/kernels/sampler.py:13-71)
        self.sampler = (RowParallelSampler if tp > 1 else Sampler)(cfg.model.vocab_size)
        self._greedy_shortcut = tp > 1 and hasattr(model, "greedy_tokens")
        self.max_spec = cfg.speculative.num_speculative_tokens if cfg.speculative.method else 0
        self.rejection = None
        self.drafter = None                        # on-device drafter (DeepSeek MTP)
        self.head_drafter = None                   # Medusa heads / MLP speculator (spec/heads.py)
        self.lora = None                           # LoRAManager when multi-LoRA is enabled
        self.drafter_caches: list[torch.Tensor] = []
        if self.max_spec:
            from ..spec import RejectionSampler
            self.rejection = RejectionSampler()
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.graph_sizes: list[int] = []
        self.graph_pool = None
        self.step_counter = 0
        self.prev_index: dict[str, int] = {}       # req id -> row in prev_sampled
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.graph_launches = 0                    # kernels replayed through CUDA graphs
        self.graph_kernel_counts: dict = {}
        self.timing_events: Optional[list] = None  # set to a list to time every step
        self.timing_meta: list = []                # (decodes, prefills, tokens) per timed step
        self.keep_logits = False                   # debugging / tests: keep last step's logits
        self.keep_hidden = False                   # a pooling request samples in this step:
        self._last_hidden = None                   # keep the sampled rows' final hidden states
        self._features = None                      # per-step sampling extras (penalties, logprobs)
        self._mm_inputs = None                     # (inputs_embeds, mrope positions) of a step
        from .. import envs
        self.nvtx = bool(envs.NVTX) and self.is_cuda
        # shared-prefix (cascade) attention for steps that do not replay a CUDA graph: used
        # when every request of the step starts with at least this many identical cached
        # tokens (0 = never)
        self.cascade_min_tokens = int(cfg.additional_config.get("cascade_min_tokens", 256)) \
            if getattr(cfg, "additional_config", None) is not None else 256
        self.cascade_steps = 0
        self.last_logits: Optional[torch.Tensor] = None
        self._alloc_buffers()

    # -- buffers -------------------------------------------------------------------
    def _alloc_buffers(self) -> None:
        dev, pin = self.device, self.is_cuda
        T, S, MB = self.max_tokens, self.max_seqs, self.max_blocks
        W = 1 + self.max_spec          # sampled positions per request
        # int64 block: input_ids | positions | slot_mapping | sample_indices | seeds | mtp_ids
        self.i64_layout = {"input_ids": (0, T), "positions": (T, T), "slot_mapping": (2 * T, T),
                           "sample_indices": (3 * T, S * W), "seeds": (3 * T + S * W, S),
                           "mtp_ids": (3 * T + S * W + S, T if self.max_spec else 0)}
        n64 = 3 * T + S * W + S + (T if self.max_spec else 0)
        # int32 block: seq_lens | cu_q | feed_dst | feed_src | top_k | num_draft | draft_ids |
        #              block_tables
        o = 0
        self.i32_layout = {}
        for name, n in (("seq_lens", S), ("cu_q", S + 1), ("feed_dst", S), ("feed_src", S),
                        ("top_k", S), ("num_draft", S), ("draft_ids", S * max(self.max_spec, 1)),
                        ("block_tables", S * MB)):
            self.i32_layout[name] = (o, n)
            o += n
        n32 = o
        self.h_i64 = torch.zeros(n64, dtype=torch.int64, pin_memory=pin)
        self.h_i32 = torch.zeros(n32, dtype=torch.int32, pin_memory=pin)
        self.h_f32 = torch.zeros(2 * S, dtype=torch.float32, pin_memory=pin)  # temperature | top_p
        self.d_i64 = torch.zeros(n64, dtype=torch.int64, device=dev)
        self.d_i32 = torch.zeros(n32, dtype=torch.int32, device=dev)
        self.d_f32 = torch.zeros(2 * S, dtype=torch.float32, device=dev)
        self.np_i64 = self.h_i64.numpy()
        self.np_i32 = self.h_i32.numpy()
        self.np_f32 = self.h_f32.numpy()

        def v64(name):
            o, n = self.i64_layout[name]
            return self.d_i64[o:o + n]

        def v32(name):
            o, n = self.i32_layout[name]
            return self.d_i32[o:o + n]

        self.input_ids, self.positions = v64("input_ids"), v64("positions")
        self.slot_mapping, self.sample_indices = v64("slot_mapping"), v64("sample_indices")
        self.seeds = v64("seeds")
        self.seq_lens, self.cu_q = v32("seq_lens"), v32("cu_q")
        self.feed_dst, self.feed_src, self.top_k = v32("feed_dst"), v32("feed_src"), v32("top_k")
        self.block_tables = v32("block_tables").view(S, MB)
        self.temperature, self.top_p = self.d_f32[:S], self.d_f32[S:]
        self.num_draft, self.draft_ids = v32("num_draft"), v32("draft_ids")
        self.mtp_ids = v64("mtp_ids") if self.max_spec else None
        self.sampled = [torch.zeros(S * W, dtype=torch.int64, device=dev) for _ in range(2)]
        self.sampled_host = [torch.zeros(S * W, dtype=torch.int64, pin_memory=pin)
                             for _ in range(2)]
        self.draft_out = torch.zeros(S * max(1, self.max_spec), dtype=torch.int64, device=dev)
        self.draft_host = torch.zeros(S * max(1, self.max_spec), dtype=torch.int64,
                                      pin_memory=pin)
        self.decode_ws: Optional[tuple[torch.Tensor, torch.Tensor]] = None
        # host-side block table, one row per live request
        self.bt_rows: dict[str, int] = {}
        self.free_rows = list(range(S * 2 - 1, -1, -1))
        self.bt_host = np.zeros((S * 2, MB), dtype=np.int32)
        self.bt_len = np.zeros(S * 2, dtype=np.int32)

    # -- KV cache --------------------------------------------------------------------
    def profile_num_blocks(self) -> int:
        """Number of KV blocks that fit next to the weights and the peak activations of a
        full prefill step (vllm_gcu/worker/worker.py:120-191 does the same accounting)."""
        cc = self.cfg.cache
        if cc.num_gpu_blocks is not None:
            return cc.num_gpu_blocks
        bytes_per_block = self.cfg.model.kv_bytes_per_token(
            self.cfg.parallel.tensor_parallel_size) * self.block_size
        bytes_per_block = bytes_per_block * self.model.num_local_layers \
            // max(1, self.cfg.model.num_hidden_layers)
        if not self.is_cuda:
            return max(64, min(4096, (1 << 28) // max(1, bytes_per_block)))
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        self._dummy_forward(self.cfg.scheduler.max_num_batched_tokens)
        torch.cuda.synchronize()
        peak = torch.cuda.max_memory_allocated()
        free, total = torch.cuda.mem_get_info()
        torch.cuda.empty_cache()
        weights_and_act = peak
        budget = int(total * cc.gpu_memory_utilization) - weights_and_act
        # the dummy forward is gone but other processes may hold memory too
        budget = min(budget, int(torch.cuda.mem_get_info()[0] * 0.97))
        n = budget // bytes_per_block
        if n < 16:
            raise RuntimeError(f"not enough GPU memory for the KV cache ({budget} bytes)")
        cap = self.max_seqs * self.max_blocks * 4
        n = int(min(n, cap))
        try:        # the memory budget, as the reference logs it at start-up
            from ..utils import logger
            gib = float(1 << 30)
            logger.info("memory budget: %.1f GiB total x %.2f; weights + peak activations "
                        "%.1f GiB; KV cache %.1f GiB = %d blocks of %d bytes",
                        total / gib, cc.gpu_memory_utilization, weights_and_act / gib,
                        n * bytes_per_block / gib, n, bytes_per_block)
        except Exception:  # noqa: BLE001 - a log line never stops the engine
            pass
        return n

    def init_kv_cache(self, num_blocks: int) -> None:
        spec = self.model.kv_cache_spec()
        mc = self.cfg.model
        dt = mc.dtype
        kvd = (mc.kv_cache_dtype or "auto").lower()
        if self.is_cuda and spec["type"] == "gqa":
            # 8-bit KV cache (fp8 e4m3 or symmetric int8); the attention kernels dequantise on
            # the way into shared memory.  The CPU path keeps the model dtype.
            if kvd.startswith("fp8"):
                dt = torch.float8_e4m3fn
            elif kvd == "int8":
                dt = torch.int8
        if spec["type"] == "mla":
            self.kv_caches = [torch.zeros(num_blocks, self.block_size, spec["width"], dtype=dt,
                                          device=self.device) for _ in range(spec["layers"])]
        else:
            self.kv_caches = [torch.zeros(2, num_blocks, self.block_size, spec["kv_heads"],
                                          spec["head_dim"], dtype=dt, device=self.device)
                              for _ in range(spec["layers"])]
        self.num_blocks = num_blocks
        if self.drafter is not None:
            ds = self.drafter.kv_cache_spec()
            if ds["type"] == "mla":
                self.drafter_caches = [torch.zeros(num_blocks, self.block_size, ds["width"],
                                                   dtype=dt, device=self.device)
                                       for _ in range(ds["layers"])]
            else:
                self.drafter_caches = [torch.zeros(2, num_blocks, self.block_size, ds["kv_heads"],
                                                   ds["head_dim"], dtype=dt, device=self.device)
                                       for _ in range(ds["layers"])]
        if self.is_cuda and spec["type"] == "gqa":
            Hq = mc.num_attention_heads // self.cfg.parallel.tensor_parallel_size
            ns = 32
            self.decode_ws = (
                torch.empty(self.max_seqs * Hq * ns * spec["head_dim"] // 8 + 1024,
                            dtype=torch.float32, device=self.device),
                torch.empty(self.max_seqs * Hq * ns // 8 + 1024, dtype=torch.float32,
                            device=self.device))

    def _decode_splits(self, batch: int, max_seq_len: int) -> int:
        if not self.is_cuda or self.model.kv_cache_spec()["type"] != "gqa":
            return 1
        from ..ops import cuda as C
        kvh = self.model.kv_cache_spec()["kv_heads"]
        s = C.decode_num_splits(batch, kvh, max_seq_len)
        Hq = self.cfg.model.num_attention_heads // self.cfg.parallel.tensor_parallel_size
        while s > 1 and batch * Hq * s * self.cfg.model.head_dim > self.decode_ws[0].numel():
            s -= 1
        return s

    def _dummy_forward(self, num_tokens: int) -> None:
        """Forward over ``num_tokens`` padding tokens that touch no cache slot (memory
        profile; also the keep-alive step of an idle data-parallel rank)."""
        T = max(0, min(num_tokens, self.max_tokens))
        md = AttentionMetadata(
            num_tokens=T, num_decodes=0, num_prefills=0, num_decode_tokens=0,
            positions=self.positions[:T], slot_mapping=torch.full_like(self.slot_mapping[:T], -1),
            block_tables=self.block_tables[:1], seq_lens=self.seq_lens[:1], is_dummy=True)
        caches = self.kv_caches or [None] * self.model.num_local_layers
        with torch.inference_mode():
            hidden = self.model(self.input_ids[:T], md, caches)
            if T > 0 and self.model.is_last_stage:
                self.model.compute_logits(hidden[: min(T, self.max_seqs)])

    def execute_dummy_batch(self) -> None:
        self._dummy_forward(0 if self.cfg.parallel.enable_expert_parallel else 1)

    # -- request bookkeeping -----------------------------------------------------------
    def _row_of(self, s: ScheduledRequest) -> int:
        rid = s.req.request_id
        row = self.bt_rows.get(rid)
        if row is None:
            row = self.free_rows.pop()
            self.bt_rows[rid] = row
            self.bt_len[row] = 0
        if s.is_new:
            self.bt_len[row] = 0
        n0 = int(self.bt_len[row])
        ids = s.req.block_ids
        if len(ids) > n0:
            self.bt_host[row, n0:len(ids)] = ids[n0:]
            self.bt_len[row] = len(ids)
        return row

    def release(self, req_ids) -> None:
        for rid in req_ids:
            row = self.bt_rows.pop(rid, None)
            if row is not None:
                self.free_rows.append(row)
            self.prev_index.pop(rid, None)

    # -- one step ---------------------------------------------------------------------
    def apply_swaps(self, so: SchedulerOutput) -> None:
        """Swap preemption: copies whole KV blocks between the device caches and a host copy
        (pinned, allocated on first use) on the current stream, before this step's kernels can
        overwrite the released blocks.  Copy-in first: a host block freed by it may be the
        target of a copy-out of the same step."""
        if not so.swap_in and not so.swap_out:
            return
        n_cpu = int(self.cfg.cache.num_cpu_blocks)
        if getattr(self, "cpu_caches", None) is None:
            pin = self.is_cuda
            self.cpu_caches = []
            for c in self.kv_caches:
                shape = list(c.shape)
                shape[0 if c.dim() == 3 else 1] = n_cpu
                self.cpu_caches.append(torch.zeros(shape, dtype=c.dtype, device="cpu",
                                                   pin_memory=pin))
        from ..ops import cuda as C, ref
        swap = C.swap_blocks if self.is_cuda else ref.swap_blocks
        m_in = torch.tensor(so.swap_in, dtype=torch.int64).view(-1, 2)
        m_out = torch.tensor(so.swap_out, dtype=torch.int64).view(-1, 2)
        for dev_c, cpu_c in zip(self.kv_caches, self.cpu_caches):
            planes = [(dev_c, cpu_c)] if dev_c.dim() == 3 else [(dev_c[0], cpu_c[0]),
                                                                (dev_c[1], cpu_c[1])]
            for d, h in planes:
                if len(so.swap_in):
                    swap(h, d, m_in)
                if len(so.swap_out):
                    swap(d, h, m_out)
        so.swap_in, so.swap_out = [], []

    def execute(self, so: SchedulerOutput, want_device_timing: bool = False) -> StepHandle:
        self.release(so.finished_req_ids)
        self.release(so.preempted_req_ids)
        self.apply_swaps(so)
        if so.is_empty:
            return StepHandle([], 0, None, None)
        sched = so.scheduled
        decodes = [s for s in sched if s.num_tokens == 1 and s.will_sample]
        prefills = [s for s in sched if not (s.num_tokens == 1 and s.will_sample)]
        order = decodes + prefills
        nd, npf = len(decodes), len(prefills)
        B = nd + npf
        bs = self.block_size
        T_real = nd + sum(s.num_tokens for s in prefills)

        batch_has_lora = self.lora is not None and any(s.req.lora_id >= 0 for s in sched)
        # penalties / log-probabilities need the logits on a side path: no graph for that step
        feat = any(s.req.sampling_params.has_penalties
                   or s.req.sampling_params.logprobs is not None
                   or s.req.sampling_params.prompt_logprobs is not None
                   or s.req.sampling_params.constrained for s in sched)
        self.keep_hidden = any(s.req.sampling_params.pooling for s in sched)
        # Data-parallel replicas pick the graph by the largest token count of any replica in
        # this step (known from the exchange that precedes every step): the expert-parallel
        # receive area inside the graph is sized by the padded batch, so it must cover what
        # the busiest peer can send.
        nd_graph = nd
        if self.cfg.parallel.data_parallel_size > 1 and self.graphs:
            from ..parallel.state import get_state
            nd_graph = max(nd, int(get_state().dp_max_tokens or 0))
        use_graph = (self.is_cuda and npf == 0 and bool(self.graphs)
                     and nd_graph <= self.graph_sizes[-1]
                     and self.drafter is None and self.head_drafter is None
                     and not batch_has_lora and not feat and not self.keep_hidden)
        B_pad = _pad_batch(nd_graph, self.graph_sizes) if use_graph else B
        T = T_real + (B_pad - B)

        i64, i32, f32 = self.np_i64, self.np_i32, self.np_f32
        o_ids, o_pos, o_slot = (self.i64_layout[k][0] for k in ("input_ids", "positions",
                                                                "slot_mapping"))
        o_samp, o_seed = self.i64_layout["sample_indices"][0], self.i64_layout["seeds"][0]
        o_sl, o_cu = self.i32_layout["seq_lens"][0], self.i32_layout["cu_q"][0]
        o_fd, o_fs = self.i32_layout["feed_dst"][0], self.i32_layout["feed_src"][0]
        o_tk, o_bt = self.i32_layout["top_k"][0], self.i32_layout["block_tables"][0]
        MB = self.max_blocks

        rows = np.fromiter((self._row_of(s) for s in order), dtype=np.int64, count=B)
        starts = np.fromiter((s.start for s in order), dtype=np.int64, count=B)
        ntok = np.fromiter((s.num_tokens for s in order), dtype=np.int64, count=B)
        seq_after = starts + ntok
        max_seq_len = int(seq_after.max())
        used_blocks = -(-max_seq_len // bs)

        # token ids / positions
        feed_dst: list[int] = []
        feed_src: list[int] = []
        tok_off = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(ntok, out=tok_off[1:])
        pos = i64[o_pos:o_pos + T_real]
        ids = i64[o_ids:o_ids + T_real]
        if nd:
            # decode fast path: one token per request, either known or fed on the device
            pos[:nd] = starts[:nd]
            dec_ids = [0] * nd
            prev_index = self.prev_index
            for j in range(nd):
                s = order[j]
                req = s.req
                npt = len(req.prompt_token_ids)
                st = s.start
                if st < npt:
                    dec_ids[j] = req.prompt_token_ids[st]
                elif st - npt < len(req.output_token_ids):
                    dec_ids[j] = req.output_token_ids[st - npt]
                else:
                    feed_dst.append(j)
                    feed_src.append(prev_index[req.request_id])
            ids[:nd] = dec_ids
        for j in range(nd, B):
            s = order[j]
            a, b = int(tok_off[j]), int(tok_off[j + 1])
            req = s.req
            known = req.num_tokens
            n_spec = len(s.spec_token_ids)
            pos[a:b] = np.arange(s.start, s.start + s.num_tokens)
            end = s.start + s.num_tokens
            n_known = max(0, min(end, known) - s.start)
            if n_known:
                if s.start + n_known <= req.num_prompt_tokens:
                    ids[a:a + n_known] = req.prompt_token_ids[s.start:s.start + n_known]
                else:
                    ids[a:a + n_known] = [req.token_at(p) for p in range(s.start,
                                                                         s.start + n_known)]
            p = a + n_known
            if p < b - n_spec:
                # exactly one unknown id: the token sampled by the previous step
                src = self.prev_index.get(req.request_id)
                assert src is not None and b - n_spec - p == 1, "token id not available"
                ids[p] = 0
                feed_dst.append(p)
                feed_src.append(src)
                p += 1
            if n_spec:
                ids[b - n_spec:b] = s.spec_token_ids
        # slots
        blk_idx = pos // bs
        tok_rows = np.repeat(rows, ntok)
        i64[o_slot:o_slot + T_real] = (self.bt_host[tok_rows, blk_idx].astype(np.int64) * bs
                                       + pos % bs)
        # multimodal requests: rotary positions differ from sequence positions (M-RoPE)
        mm_step = any(s_.req.mm_embeds is not None or s_.req.mrope_delta for s_ in order)
        mm_chunks = []
        if mm_step:
            deltas = np.fromiter((s_.req.mrope_delta for s_ in order), dtype=np.int64, count=B)
            nprompt = np.fromiter((len(s_.req.prompt_token_ids) for s_ in order), dtype=np.int64,
                                  count=B)
            tok_delta = np.repeat(deltas, ntok)
            pos += np.where(pos >= np.repeat(nprompt, ntok), tok_delta, 0)
            for j, s_ in enumerate(order):
                r_ = s_.req
                if r_.mm_embeds is None and r_.mrope_positions is None:
                    continue
                if s_.start < len(r_.prompt_token_ids):
                    mm_chunks.append((int(tok_off[j]), s_.start,
                                      min(s_.start + s_.num_tokens, len(r_.prompt_token_ids)), r_))
        if T > T_real:
            i64[o_slot + T_real:o_slot + T] = -1
            i64[o_ids + T_real:o_ids + T] = 0
            i64[o_pos + T_real:o_pos + T] = 0
        if self.lora is not None:
            if batch_has_lora:
                tok_lora = np.repeat(np.fromiter((s.req.lora_id for s in order), dtype=np.int64,
                                                 count=B), ntok).tolist()
                smp_lora = [s.req.lora_id for s in order if s.will_sample]
                self.lora.set_batch(tok_lora, smp_lora)
            else:
                self.lora.punica.no_lora = True
        # sampling rows
        samplers = [j for j, s in enumerate(order) if s.will_sample]
        ns = len(samplers)
        nspec = [len(order[j].spec_token_ids) for j in samplers]
        S_max = max(nspec) if nspec else 0
        width = 1 + S_max
        last = tok_off[1:][samplers] - 1 if ns else np.zeros(0, dtype=np.int64)
        if S_max == 0:
            i64[o_samp:o_samp + ns] = last
            if B_pad > B:
                i64[o_samp + ns:o_samp + B_pad] = 0
        else:
            # row (r, i) = i-th verified position of request r; rows past its own draft length
            # repeat its last position and are ignored by the verification kernel
            ns_arr = np.asarray(nspec, dtype=np.int64)
            first = last - ns_arr
            grid = first[:, None] + np.minimum(np.arange(width)[None, :], ns_arr[:, None])
            i64[o_samp:o_samp + ns * width] = grid.reshape(-1)
            o_nd, o_dr = self.i32_layout["num_draft"][0], self.i32_layout["draft_ids"][0]
            i32[o_nd:o_nd + ns] = ns_arr
            dr = np.zeros((ns, S_max), dtype=np.int32)
            for r, j in enumerate(samplers):
                if nspec[r]:
                    dr[r, :nspec[r]] = order[j].spec_token_ids
            i32[o_dr:o_dr + ns * S_max] = dr.reshape(-1)
        sp_list = [order[j].req.sampling_params for j in samplers]
        all_greedy = all(sp.greedy for sp in sp_list)
        if not all_greedy:
            for r, j in enumerate(samplers):
                sp, req = sp_list[r], order[j].req
                f32[r] = sp.temperature
                f32[self.max_seqs + r] = sp.top_p
                i32[o_tk + r] = sp.top_k
                base = sp.seed if sp.seed is not None else zlib.crc32(req.request_id.encode())
                i64[o_seed + r] = (base * 1000003 + order[j].sample_index) & 0x7FFFFFFFFFFFFFFF
        # per-sequence metadata
        i32[o_sl:o_sl + B] = seq_after
        if B_pad > B:
            i32[o_sl + B:o_sl + B_pad] = 0
        cu = np.zeros(npf + 1, dtype=np.int64)
        if npf:
            np.cumsum(ntok[nd:], out=cu[1:])
            i32[o_cu:o_cu + npf + 1] = cu
        nf = len(feed_dst)
        if nf:
            i32[o_fd:o_fd + nf] = feed_dst
            i32[o_fs:o_fs + nf] = feed_src
        bt_view = i32[o_bt:o_bt + self.max_seqs * MB].reshape(self.max_seqs, MB)
        bt_view[:B, :used_blocks] = self.bt_host[rows, :used_blocks]
        if B_pad > B:
            bt_view[B:B_pad, :used_blocks] = 0

        # host -> device
        ev0 = ev1 = None
        if self.is_cuda and (want_device_timing or self.timing_events is not None):
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        if self.drafter is not None:
            # drafter inputs: the step's token ids shifted left by one inside each request; the
            # id that is being sampled right now is patched in on the device
            o_mt = self.i64_layout["mtp_ids"][0]
            mt = i64[o_mt:o_mt + T_real]
            mt[:T_real - 1] = ids[1:T_real]
            for j, s_ in enumerate(order):
                b_ = int(tok_off[j + 1])
                nxt = s_.start + s_.num_tokens
                mt[b_ - 1] = s_.req.token_at(nxt) if nxt < s_.req.num_tokens else 0
            n64 = o_mt + T_real
        else:
            n64 = o_seed + self.max_seqs if not all_greedy else o_samp + max(ns * width, B_pad)
        n32 = o_bt + (max(B_pad, B) - 1) * MB + used_blocks
        self.d_i64[:n64].copy_(self.h_i64[:n64], non_blocking=True)
        self.d_i32[:n32].copy_(self.h_i32[:n32], non_blocking=True)
        self.h2d_bytes += n64 * 8 + n32 * 4
        if not all_greedy:
            self.d_f32.copy_(self.h_f32, non_blocking=True)
            self.h2d_bytes += self.h_f32.numel() * 4
        cur = self.step_counter & 1
        prev_sampled = self.sampled[cur ^ 1]
        if nf:
            if self.is_cuda:
                from ..ops import cuda as C
                C.feed_tokens(self.input_ids, prev_sampled, self.feed_dst, self.feed_src, nf)
            else:
                self.input_ids[self.feed_dst[:nf].long()] = prev_sampled[self.feed_src[:nf].long()]

        out_ids = self.sampled[cur]
        common_prefix = 0
        if (not use_graph and self.cascade_min_tokens > 0 and B >= 4 and not mm_step
                and not self.max_spec and self.model.kv_cache_spec()["type"] == "gqa"):
            nblk = int(starts.min()) // bs          # only tokens that are already in the cache
            if nblk * bs >= self.cascade_min_tokens:
                same = (self.bt_host[rows, :nblk] == self.bt_host[rows[0], :nblk][None, :]).all(0)
                k = nblk if bool(same.all()) else int(np.argmin(same))
                if k * bs >= self.cascade_min_tokens:
                    common_prefix = k * bs
                    self.cascade_steps += 1
        md = AttentionMetadata(
            num_tokens=T, num_decodes=B_pad - npf if use_graph else nd, num_prefills=npf,
            num_decode_tokens=(B_pad if use_graph else nd),
            positions=self.positions[:T], slot_mapping=self.slot_mapping[:T],
            block_tables=self.block_tables[:max(B_pad, B)], seq_lens=self.seq_lens[:max(B_pad, B)],
            cu_q_prefill=self.cu_q[:npf + 1] if npf else None,
            num_q_tiles=int(((ntok[nd:] + 63) // 64).sum()) if npf else 0,
            num_q_tiles_128=int(((ntok[nd:] + 127) // 128).sum()) if npf else 0,
            max_seq_len=max_seq_len,
            decode_splits=self._decode_splits(B_pad if use_graph else max(nd, 1), max_seq_len),
            decode_workspace=self.decode_ws,
            sample_indices=self.sample_indices[:max(ns * width, 1)],
            q_lens_cpu=[int(x) for x in ntok], seq_lens_cpu=[int(x) for x in seq_after],
            common_prefix_len=common_prefix,
            cu_q_all=torch.tensor(tok_off, dtype=torch.int32, device=self.device)
            if common_prefix else None)

        self._features = self._build_features(order, samplers, tok_off) if feat else None
        self._mm_inputs = self._build_mm_inputs(mm_chunks, T) if mm_chunks else None
        if self._mm_inputs is not None:
            md.mrope_positions = self._mm_inputs[1]
        if self.nvtx:
            torch.cuda.nvtx.range_push("decode_step" if npf == 0 else
                                       ("prefill_step" if nd == 0 else "mixed_step"))
        if use_graph:
            key = (B_pad, cur, all_greedy)
            self.graphs[key].replay()
            self.graph_launches += self.graph_kernel_counts.get(key, 0)
        else:
            with torch.inference_mode():
                self._forward_and_sample(md, T, ns, out_ids, all_greedy, width)
        if self.nvtx:
            torch.cuda.nvtx.range_pop()

        # device -> host (asynchronous; consumed by StepHandle.token_ids)
        host = self.sampled_host[cur]
        event = None
        if ns:
            host[:ns * width].copy_(out_ids[:ns * width], non_blocking=True)
            self.d2h_bytes += ns * width * 8
            if self.drafter is not None or self.head_drafter is not None:
                dk = self.head_drafter.k if self.head_drafter is not None else 1
                self.draft_host[:ns * dk].copy_(self.draft_out[:ns * dk], non_blocking=True)
                self.d2h_bytes += ns * dk * 8
        if self.is_cuda:
            if ev1 is not None:
                ev1.record()
                if self.timing_events is not None:
                    self.timing_events.append((ev0, ev1))
                    self.timing_meta.append((nd, npf, T_real))
            event = torch.cuda.Event()
            event.record()
        self.prev_index = {order[j].req.request_id: r for r, j in enumerate(samplers)}
        self.step_counter += 1
        extra = {"num_draft": nspec,
                 "draft_width": self.head_drafter.k if self.head_drafter is not None else 1}
        if self.keep_hidden and ns and self._last_hidden is not None:
            extra["hidden"] = self._last_hidden[:ns * width:width]     # row i = i-th sampler
            self._last_hidden = None
        if self._features is not None:
            extra["logprobs"] = self._features.pop("logprobs_out", None)
            extra["prompt_logprobs"] = self._features.pop("prompt_logprobs_out", None)
            self._features = None
        return StepHandle([order[j].req.request_id for j in samplers], ns, host, event,
                          width, device_ms_events=(ev0, ev1) if ev0 is not None else None,
                          draft_host=self.draft_host if (self.drafter is not None or
                                                         self.head_drafter is not None) else None,
                          extra=extra)

    def _build_mm_inputs(self, mm_chunks, T: int):
        """(inputs_embeds [T, H], mrope_positions [3, T]) of a step that contains multimodal
        prompt tokens: placeholder rows of the token embedding are replaced by the vision
        embeddings of the request, and the prompt part of every such request gets its
        (t, h, w) rotary positions; all other tokens use their 1-D position on all axes."""
        with torch.inference_mode():
            emb = self.model.embed_tokens(self.input_ids[:T]).clone() \
                if self.model.is_first_stage else None
            mpos = self.positions[:T].unsqueeze(0).repeat(3, 1)
            for a, lo, hi, req in mm_chunks:
                if req.mrope_positions is not None:
                    mpos[:, a:a + hi - lo] = req.mrope_positions[:, lo:hi].to(mpos.device)
                if req.mm_embeds is not None and emb is not None:
                    import bisect
                    p0 = bisect.bisect_left(req.mm_positions, lo)
                    p1 = bisect.bisect_left(req.mm_positions, hi)
                    if p1 > p0:
                        rows = torch.tensor([a + p - lo for p in req.mm_positions[p0:p1]],
                                            device=emb.device)
                        emb[rows] = req.mm_embeds[p0:p1].to(device=emb.device, dtype=emb.dtype)
        return emb, mpos

    def _build_features(self, order, samplers, tok_off) -> dict:
        """Host-side description of the per-request sampling extras of this step: penalty
        rows (token histories as index lists), log-probability widths, prompt positions whose
        log-probabilities are wanted (ReadMe-EN.md:283-292 lists the supported options)."""
        f: dict = {}
        V = self.cfg.model.vocab_size
        pen_rows, p_r, p_t, o_r, o_t, pres, freq, rep_ = [], [], [], [], [], [], [], []
        lp_k = []
        for r, j in enumerate(samplers):
            req = order[j].req
            sp = req.sampling_params
            lp_k.append(-1 if sp.logprobs is None else int(sp.logprobs))
            if sp.has_penalties:
                i = len(pen_rows)
                pen_rows.append(r)
                p_r += [i] * len(req.prompt_token_ids)
                p_t += [t for t in req.prompt_token_ids]
                o_r += [i] * len(req.output_token_ids)
                o_t += [t for t in req.output_token_ids]
                pres.append(sp.presence_penalty)
                freq.append(sp.frequency_penalty)
                rep_.append(sp.repetition_penalty)
        dev = self.device
        if pen_rows:
            n = len(pen_rows)
            pm = torch.zeros((n, V), dtype=torch.bool, device=dev)
            oc = torch.zeros((n, V), dtype=torch.int32, device=dev)
            if p_r:
                pm[torch.tensor(p_r, device=dev), torch.tensor(p_t, device=dev).clamp_(0, V - 1)] = True
            if o_r:
                oc.index_put_((torch.tensor(o_r, device=dev),
                               torch.tensor(o_t, device=dev).clamp_(0, V - 1)),
                              torch.ones(len(o_r), dtype=torch.int32, device=dev), accumulate=True)
            f["penalties"] = (torch.tensor(pen_rows, device=dev), pm, oc,
                              torch.tensor(pres, device=dev), torch.tensor(freq, device=dev),
                              torch.tensor(rep_, device=dev))
        if any(k >= 0 for k in lp_k):
            f["logprob_k"] = lp_k
        allow_r, allow_t = [], []
        for r, j in enumerate(samplers):
            req = order[j].req
            nxt = req.allowed_next() if req.sampling_params.constrained else None
            if nxt is not None:
                allow_r.append((r, nxt))
        if allow_r:
            f["allowed"] = allow_r
        # prompt log-probabilities: hidden row of prompt position p predicts token p + 1
        pl = []
        for j, s_ in enumerate(order):
            req = s_.req
            k = req.sampling_params.prompt_logprobs
            if k is None or s_.start >= req.num_prompt_tokens - 1:
                continue
            a = int(tok_off[j])
            n = min(s_.start + s_.num_tokens, req.num_prompt_tokens - 1) - s_.start
            if n > 0:
                pl.append((req.request_id, a, n,
                           req.prompt_token_ids[s_.start + 1:s_.start + 1 + n], int(k)))
        if pl:
            f["prompt_logprobs"] = pl
        return f

    def _apply_features(self, hidden: torch.Tensor, logits: torch.Tensor, ns: int,
                        out_ids: torch.Tensor, before_sampling: bool, width: int = 1
                        ) -> torch.Tensor:
        """``logits`` holds ``width`` rows per sampling request (1 + the longest draft of the
        step).  Requests with sampling extras never carry drafts, so their only live row is
        the first of their group: row ``r * width``."""
        f = self._features
        if before_sampling:
            if "penalties" in f:
                from ..layers.sampler import apply_penalties
                rows, pm, oc, pres, freq, rep_ = f["penalties"]
                rows = rows * width
                sub = logits.index_select(0, rows).float()
                apply_penalties(sub, pm, oc, pres, freq, rep_)
                logits = logits.clone() if not logits.is_contiguous() else logits
                logits.index_copy_(0, rows, sub.to(logits.dtype))
            if "allowed" in f:
                logits = logits.clone()
                for r, ids in f["allowed"]:
                    if not ids:
                        continue
                    keep = torch.tensor(ids, device=logits.device).clamp_(0, logits.shape[1] - 1)
                    row = torch.full_like(logits[r * width], float("-inf"))
                    row[keep] = logits[r * width, keep]
                    logits[r * width] = row
            return logits
        if "logprob_k" in f:
            ks = f["logprob_k"]
            kmax = max(ks)
            first = logits[:ns * width:width]
            ids = out_ids[:ns * width:width].long().clamp_(min=0)
            chosen, tv, ti = self.sampler.logprobs(first, ids, max(kmax, 0))
            f["logprobs_out"] = (chosen.cpu(), tv.cpu(), ti.cpu(), ks)
        if "prompt_logprobs" in f:
            out = {}
            for rid, a, n, targets, k in f["prompt_logprobs"]:
                lg = self.model.compute_logits(hidden[a:a + n]).float()
                lp = torch.log_softmax(lg, dim=-1)
                tgt = torch.tensor(targets, device=lp.device)
                chosen = lp.gather(-1, tgt[:, None]).squeeze(-1).cpu()
                tv, ti = lp.topk(k, dim=-1) if k > 0 else (lp[:, :0], tgt[:, None][:, :0])
                out[rid] = (chosen, tv.cpu(), ti.cpu(), targets)
            f["prompt_logprobs_out"] = out
        return logits

    def _forward_and_sample(self, md: AttentionMetadata, T: int, ns: int, out_ids: torch.Tensor,
                            all_greedy: bool, width: int = 1) -> None:
        from ..parallel.state import get_state
        pp = get_state().pp
        inter = None
        if pp.world_size > 1 and not self.model.is_first_stage:
            inter = self._pp_recv(pp, T)
        mm = getattr(self, "_mm_inputs", None)
        hidden = self.model(self.input_ids[:T], md, self.kv_caches, intermediate=inter,
                            inputs_embeds=mm[0] if mm is not None else None)
        if pp.world_size > 1:
            import torch.distributed as dist
            last = pp.ranks[-1]
            if not self.model.is_last_stage:
                self._pp_send(pp, hidden)
                if ns:      # every stage needs the sampled ids (stop checks, next inputs)
                    dist.broadcast(out_ids[:ns * width], last, group=pp.device_group)
                return
        feats = getattr(self, "_features", None)
        if ns == 0:
            if feats is not None and "prompt_logprobs" in feats and self.model.is_last_stage:
                self._apply_features(hidden, hidden, 0, out_ids, before_sampling=False)
            return
        if md.num_prefills == 0 and width == 1:
            rows = hidden[:ns]          # decode-only: row i is the i-th sampling request
        else:
            rows = hidden.index_select(0, self.sample_indices[:ns * width])
        if self.keep_hidden:
            self._last_hidden = rows.float()
        if (all_greedy and width == 1 and feats is None and not self.keep_logits
                and self.drafter is None and self.head_drafter is None
                and self._greedy_shortcut):
            # greedy decoding under tensor parallelism: each rank reduces its vocabulary block
            # to (max, argmax) per row and only those pairs are exchanged
            out_ids[:ns].copy_(self.model.greedy_tokens(rows))
            if pp.world_size > 1:
                import torch.distributed as dist
                dist.broadcast(out_ids[:ns * width], pp.ranks[-1], group=pp.device_group)
            return
        logits = self.model.compute_logits(rows)
        if self.keep_logits:
            self.last_logits = logits.float().cpu()
        if feats is not None:
            logits = self._apply_features(hidden, logits, ns, out_ids, before_sampling=True,
                                          width=width)
        st = None if all_greedy else SamplingTensors(self.temperature[:ns], self.top_k[:ns],
                                                     self.top_p[:ns], self.seeds[:ns])
        if width == 1:
            self.sampler(logits, st, out=out_ids[:ns])
            if feats is not None:
                self._apply_features(hidden, logits, ns, out_ids, before_sampling=False)
        else:
            self._verify(logits, st, ns, width, out_ids)
            if feats is not None:
                self._apply_features(hidden, logits, ns, out_ids, before_sampling=False,
                                     width=width)
        if self.drafter is not None:
            self._draft_mtp(hidden, md, T, ns, width, out_ids)
        if self.head_drafter is not None:
            self._draft_heads(hidden, ns, width, out_ids)
        if pp.world_size > 1:
            import torch.distributed as dist
            dist.broadcast(out_ids[:ns * width], pp.ranks[-1], group=pp.device_group)

    # -- pipeline hand-off ------------------------------------------------------------------
    # (hidden, residual) travel between stages over NCCL p2p (vllm_gcu/worker/worker_v1.py:
    # 341-360).  On GPUs the transfers run on a side stream tied to the compute stream by
    # events: a stage's compute stream is not held up by its own sends (it can take the next
    # step while they drain), and a receive is posted as soon as the step starts.
    def _pp_side_stream(self):
        if not self.is_cuda:
            return None
        if getattr(self, "_pp_stream", None) is None:
            self._pp_stream = torch.cuda.Stream()
        return self._pp_stream

    def _pp_recv(self, pp, T: int):
        import torch.distributed as dist
        H = self.cfg.model.hidden_size
        x = torch.empty((T, H), dtype=self.cfg.model.dtype, device=self.device)
        r = torch.empty_like(x)
        src = pp.ranks[pp.rank_in_group - 1]
        side = self._pp_side_stream()
        if side is None:
            dist.recv(x, src, group=pp.device_group)
            dist.recv(r, src, group=pp.device_group)
            return x, r
        cur = torch.cuda.current_stream()
        side.wait_stream(cur)                    # the buffers exist before the receives use them
        with torch.cuda.stream(side):
            dist.recv(x, src, group=pp.device_group)
            dist.recv(r, src, group=pp.device_group)
            done = side.record_event()
        x.record_stream(side)
        r.record_stream(side)
        cur.wait_event(done)
        return x, r

    def _pp_send(self, pp, hidden) -> None:
        import torch.distributed as dist
        dst = pp.ranks[pp.rank_in_group + 1]
        h0, h1 = hidden[0].contiguous(), hidden[1].contiguous()
        side = self._pp_side_stream()
        if side is None:
            dist.send(h0, dst, group=pp.device_group)
            dist.send(h1, dst, group=pp.device_group)
            return
        ready = torch.cuda.current_stream().record_event()
        with torch.cuda.stream(side):
            side.wait_event(ready)
            dist.send(h0, dst, group=pp.device_group)
            dist.send(h1, dst, group=pp.device_group)
        h0.record_stream(side)
        h1.record_stream(side)

    def _verify(self, logits: torch.Tensor, st: Optional[SamplingTensors], ns: int, width: int,
                out_ids: torch.Tensor) -> None:
        """Rejection sampling of the draft tokens; writes ``[ns, width]`` ids (-1 padded)."""
        S = width - 1
        draft = self.draft_ids[:ns * S].view(ns, S)
        nd = self.num_draft[:ns]
        if st is None:
            tgt = self.sampler(logits, None).view(ns, width)
            out = self.rejection.greedy(draft, tgt, nd)
        else:
            V = logits.shape[-1]
            t = st.temperature.repeat_interleave(width)
            safe_t = torch.where(t > 0, t, torch.ones_like(t))
            from ..ops import ref as _ref
            masked = _ref.apply_top_k_top_p(
                logits.float() / safe_t[:, None],
                None if st.top_k is None else st.top_k.repeat_interleave(width),
                None if st.top_p is None else st.top_p.repeat_interleave(width)).float()
            probs = masked.softmax(-1).view(ns, width, V)
            greedy_rows = (st.temperature <= 0)
            if bool(greedy_rows.any()):
                onehot = torch.zeros_like(probs)
                onehot.scatter_(-1, logits.view(ns, width, V).argmax(-1, keepdim=True), 1.0)
                probs = torch.where(greedy_rows[:, None, None], onehot, probs)
            idx = nd.long().clamp(max=S)
            bonus_p = probs.gather(1, idx[:, None, None].expand(ns, 1, V)).squeeze(1)
            # the per-request seeds of this step fix the draw (same seeds, same tokens)
            gen = None
            if st.seeds is not None and st.seeds.numel() > 0:
                gen = torch.Generator(device=logits.device)
                gen.manual_seed(int(st.seeds.sum().item()) & 0x7FFFFFFFFFFFFFFF)
            bonus = torch.multinomial(bonus_p.clamp_min(0) + 1e-20, 1, generator=gen).squeeze(1)
            out = self.rejection.random(draft, None, probs[:, :S].contiguous(), bonus, nd,
                                        generator=gen)
        out_ids[:ns * width].copy_(out.reshape(-1))

    def _draft_heads(self, hidden: torch.Tensor, ns: int, width: int, out_ids: torch.Tensor
                     ) -> None:
        """Medusa heads / MLP speculator: drafts from the hidden row of the last accepted
        position and the token emitted there."""
        toks = out_ids[:ns * width].view(ns, width)
        n_emit = (toks >= 0).sum(dim=1).clamp(min=1)
        last_tok = toks.gather(1, (n_emit - 1)[:, None]).squeeze(1)
        rows0 = self.sample_indices[:ns * width].view(ns, width)[:, 0]
        h = hidden.index_select(0, rows0 + n_emit - 1)
        k = self.head_drafter.k
        self.draft_out[:ns * k].copy_(self.head_drafter.propose(h, last_tok).reshape(-1))

    def _draft_mtp(self, hidden: torch.Tensor, md: AttentionMetadata, T: int, ns: int,
                   width: int, out_ids: torch.Tensor) -> None:
        """Runs the MTP module on this step's tokens (ids shifted by one, the freshly emitted
        token patched in at the last accepted position) and takes the draft for the next
        step from the row of the last accepted position."""
        toks = out_ids[:ns * width].view(ns, width)
        n_emit = (toks >= 0).sum(dim=1)                       # accepted drafts + 1
        last_tok = toks.gather(1, (n_emit - 1).clamp(min=0)[:, None]).squeeze(1)
        rows0 = self.sample_indices[:ns * width].view(ns, width)[:, 0]
        row = rows0 + (n_emit - 1).clamp(min=0)               # position of the last accepted token
        ids = self.mtp_ids[:T]
        ids.index_copy_(0, row, last_tok)
        h = self.drafter(ids, hidden, md, self.drafter_caches)
        lg = self.drafter.compute_logits(h.index_select(0, row))
        self.draft_out[:ns].copy_(lg.float().argmax(-1))

    # -- CUDA graphs -----------------------------------------------------------------
    def capture_graphs(self, sizes: Optional[list[int]] = None) -> None:
        """Captures the decode-only step for every padded batch size, for both output
        buffers and for the greedy / sampled variants."""
        if not self.is_cuda or self.cfg.enforce_eager:
            return
        dp = self.cfg.parallel.data_parallel_size > 1
        if dp and any(type(getattr(m, "dispatcher", None)).__name__ == "AllToAllDispatcher"
                      for m in self.model.modules()):
            return      # the library all-to-all sizes its exchange on the host: eager only
        if dp and any(getattr(m, "use_etp", False) for m in self.model.modules()):
            return      # ETP gathers rows of host-known counts over the DP group: eager only
        if sizes is None:
            sizes = [1, 2, 4, 8] + list(range(16, self.max_seqs + 1, 16))
        sizes = sorted({s for s in sizes if s <= self.max_seqs})
        if self.max_seqs not in sizes:
            sizes.append(self.max_seqs)
        self.graph_sizes = sizes
        self.seq_lens.zero_()
        self.slot_mapping.fill_(-1)
        torch.cuda.synchronize()
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream), torch.inference_mode():
            for Bp in reversed(sizes):
                if dp:      # every replica captures the same sizes in the same order, so the
                    from ..parallel.state import get_state     # warm-up exchanges pair up
                    get_state().dp_max_tokens = Bp
                for cur in (0, 1):
                    for greedy in (True, False):
                        md = AttentionMetadata(
                            num_tokens=Bp, num_decodes=Bp, num_prefills=0, num_decode_tokens=Bp,
                            positions=self.positions[:Bp], slot_mapping=self.slot_mapping[:Bp],
                            block_tables=self.block_tables[:Bp], seq_lens=self.seq_lens[:Bp],
                            max_seq_len=self.cfg.scheduler.max_model_len,
                            decode_splits=self._decode_splits(Bp, self.cfg.scheduler.max_model_len),
                            decode_workspace=self.decode_ws,
                            sample_indices=self.sample_indices[:Bp])
                        # warm-up outside the graph (lazy initialisation, autotuning)
                        self._forward_and_sample(md, Bp, Bp, self.sampled[cur], greedy)
                        stream.synchronize()
                        g = torch.cuda.CUDAGraph()
                        n0 = _native.launch_count
                        with torch.cuda.graph(g, pool=self.graph_pool, stream=stream):
                            self._forward_and_sample(md, Bp, Bp, self.sampled[cur], greedy)
                        self.graph_kernel_counts[(Bp, cur, greedy)] = _native.launch_count - n0
                        if self.graph_pool is None:
                            self.graph_pool = g.pool()
                        self.graphs[(Bp, cur, greedy)] = g
        torch.cuda.synchronize()
        _native.check_status()
