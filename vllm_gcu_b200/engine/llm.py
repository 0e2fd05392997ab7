"""Engine front end: ``LLM.generate`` and the step loop.

One engine runs per process (one process per GPU).  Under tensor / pipeline
parallelism every rank runs the same deterministic scheduler on the same requests, so
no control-plane broadcast is needed inside a step; only device collectives cross ranks.
With ``async_scheduling`` the loop keeps two steps in flight: step N+1 is scheduled,
prepared and launched while step N still runs, and the ids of step N are read one
iteration later (the batch queue of vllm_gcu/patch/patch_0_9_2/core.py:102-154 with
depth 2, vllm_gcu/v1/executor/async_multiproc_executor.py:186-191).
"""
from __future__ import annotations

import itertools
import time
from collections import deque
from typing import Iterable, Optional, Sequence, Union

import torch

from ..config import (CacheConfig, EngineConfig, ModelConfig, ParallelConfig, SchedulerConfig,
                      SpeculativeConfig, preset)
from ..models import build_model
from ..parallel.state import get_state, init_distributed
from .model_runner import ModelRunner, StepHandle
from .request import Request, RequestOutput, SamplingParams
from .scheduler import Scheduler, SchedulerOutput


class LLMEngine:
    def __init__(self, cfg: EngineConfig):
        self.cfg = cfg
        pc = cfg.parallel
        if pc.world_size > 1 and not get_state().initialized:
            init_distributed(pc.tensor_parallel_size, pc.pipeline_parallel_size,
                             pc.data_parallel_size, enable_ep=pc.enable_expert_parallel)
        st = get_state()
        if cfg.device == "cuda":
            self.device = torch.device("cuda", st.local_rank if st.world_size > 1
                                       else torch.cuda.current_device())
            torch.cuda.set_device(self.device)
        else:
            self.device = torch.device(cfg.device)
        torch.manual_seed(cfg.seed)
        if pc.data_parallel_size > 1:
            # every replica holds different tokens: MoE layers dispatch (EP) or gather (ETP)
            cfg.model.extra.setdefault("dp_attention", True)
        # engine-level options that the model's layers read from its configuration
        # (``additional_config`` of the reference, vllm_gcu/gcu.py:184-354, and the parallel
        # configuration's expert-placement fields)
        for key in ("num_redundant_experts", "enable_eplb", "expert_map_path", "ep_max_tokens",
                    "ep_backend", "ep_fp8_dispatch", "etp", "sequence_parallel", "q8_experts"):
            if key in cfg.additional_config:
                cfg.model.extra.setdefault(key, cfg.additional_config[key])
        if pc.num_redundant_experts and pc.enable_expert_parallel:
            cfg.model.extra.setdefault("num_redundant_experts", pc.num_redundant_experts)
        if pc.enable_eplb:
            cfg.model.extra.setdefault("enable_eplb", True)
        if pc.enable_sequence_parallel:
            cfg.model.extra.setdefault("sequence_parallel", True)
        self.model = build_model(cfg.model, self.device)
        if cfg.load_format == "dummy":
            self.model.init_random(cfg.seed)
        elif cfg.load_format == "none":
            pass        # the caller loads weights through model.load_weights()
        elif cfg.load_format == "safetensors":
            from ..utils.weights import iter_safetensors
            self.model.load_weights(iter_safetensors(cfg.model_path))
        if cfg.quantization_param_path:
            self.model.load_kv_cache_scales(cfg.quantization_param_path)
        self.model.eval()
        if pc.world_size > 1 and pc.comm_backend == "fused" and self.device.type == "cuda":
            from ..parallel import symm
            symm.attach(cfg)
        self.runner = ModelRunner(cfg, self.model, self.device)
        lora_cfg = cfg.additional_config.get("lora")
        if lora_cfg:
            from ..lora import LoRAManager
            self.runner.lora = LoRAManager(self.model, int(lora_cfg.get("max_loras", 4)),
                                           int(lora_cfg.get("max_lora_rank", 16)),
                                           self.runner.max_tokens, self.runner.max_seqs,
                                           self.device)
        self.proposer = None
        self.spec_metrics = None
        sp = cfg.speculative
        if sp.method:
            from ..spec import NgramProposer, SpecMetrics
            self.spec_metrics = SpecMetrics()
            if cfg.scheduler.async_scheduling:
                # draft tokens come from the previous step's verified output
                cfg.scheduler.async_scheduling = False
            if sp.method == "ngram":
                self.proposer = NgramProposer(sp.num_speculative_tokens, sp.prompt_lookup_max,
                                              sp.prompt_lookup_min)
            elif sp.method in ("mtp", "deepseek_mtp"):
                from ..models.deepseek_mtp import DeepSeekMTP
                if sp.num_speculative_tokens != 1:
                    raise ValueError("the MTP drafter proposes one token per step")
                drafter = DeepSeekMTP(cfg.model, self.device, target=self.model)
                if cfg.load_format == "dummy":
                    drafter.init_random(cfg.seed)
                elif cfg.load_format == "safetensors":
                    from ..utils.weights import iter_safetensors
                    drafter.load_weights(iter_safetensors(cfg.model_path))
                drafter.eval()
                self.runner.drafter = drafter
            elif sp.method == "eagle":
                from ..spec.eagle import EagleDrafter
                if sp.num_speculative_tokens != 1:
                    raise ValueError("the EAGLE drafter proposes one token per step")
                drafter = EagleDrafter(cfg.model, self.device, target=self.model)
                if sp.draft_model:
                    from ..utils.weights import iter_safetensors
                    drafter.load_weights(iter_safetensors(sp.draft_model))
                else:
                    drafter.init_random(cfg.seed)
                self.runner.drafter = drafter.eval()
            elif sp.method in ("medusa", "mlp_speculator"):
                from ..spec import MedusaProposer, MLPSpeculatorProposer
                mc_ = cfg.model
                cls = MedusaProposer if sp.method == "medusa" else MLPSpeculatorProposer
                heads = cls(mc_.hidden_size, mc_.vocab_size, sp.num_speculative_tokens,
                            dtype=mc_.dtype, device=self.device)
                if sp.draft_model:
                    from ..utils.weights import iter_safetensors
                    heads.load_weights(iter_safetensors(sp.draft_model))
                else:
                    heads.init_random(cfg.seed)
                self.runner.head_drafter = heads.eval()
            else:
                raise ValueError(f"unknown speculative method {sp.method!r}")
        num_blocks = self.runner.profile_num_blocks()
        if st.world_size > 1:
            num_blocks = self._agree_min(num_blocks)
        self.runner.init_kv_cache(num_blocks)
        self.runner.capture_graphs(cfg.cuda_graph_sizes)
        self.scheduler = Scheduler(cfg.scheduler, cfg.cache, num_blocks,
                                   separate_prefill_decode=bool(
                                       cfg.additional_config.get("separate_prefill_decode")),
                                   num_lookahead_tokens=sp.num_speculative_tokens
                                   if sp.method else 0)
        self._ids = itertools.count()
        self._want_sync = False
        self.disagg = None               # set by attach_kv_connector()
        self.dp_size = st.dp.world_size
        self.dp_global_busy = self.dp_size > 1     # learnt from the exchange of every step
        if self.dp_size > 1:
            # replicas hold different requests: no replica may run ahead of the exchange
            cfg.scheduler.async_scheduling = False
        self._pending: deque[tuple[SchedulerOutput, StepHandle]] = deque()
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0}

    @staticmethod
    def _agree_min(n: int) -> int:
        """All ranks use the smallest block count any of them can afford
        (vllm_gcu/worker/worker.py:182-189)."""
        import torch.distributed as dist
        st = get_state()
        t = torch.tensor([n], dtype=torch.int64)
        if st.backend == "nccl":
            t = t.cuda()
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return int(t.item())

    # -- requests -------------------------------------------------------------------
    def add_request(self, prompt_token_ids: Sequence[int],
                    sampling_params: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, priority: int = 0,
                    eos_token_id: Optional[int] = None, lora_id: int = -1,
                    multi_modal_data: Optional[dict] = None,
                    kv_transfer_params: Optional[dict] = None) -> str:
        """``multi_modal_data``: processor outputs of a multimodal model
        (``{"pixel_values": [n_patches, C*Tp*P*P], "image_grid_thw": [n_images, 3]}``); the
        prompt must already contain one placeholder token per merged patch."""
        rid = request_id if request_id is not None else f"req-{next(self._ids)}"
        check_token_ids(prompt_token_ids, self.cfg.model.vocab_size,
                        allow_placeholders=bool(multi_modal_data))
        if sampling_params is not None and sampling_params.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if sampling_params is not None:
            sp0 = sampling_params
            V0 = self.cfg.model.vocab_size
            # values the sampling kernels are not written for: top_k beyond the vocabulary or
            # negative (the "disabled" spelling of other servers), top_p outside (0, 1]
            tk = 0 if sp0.top_k is None or sp0.top_k < 0 or sp0.top_k >= V0 else int(sp0.top_k)
            tp_ = float(sp0.top_p) if sp0.top_p is not None else 1.0
            tp_ = 1.0 if not (tp_ == tp_) or tp_ > 1.0 else max(tp_, 1e-6)
            tmp = float(sp0.temperature) if sp0.temperature == sp0.temperature else 0.0
            tmp = min(max(tmp, 0.0), 1e4)
            if (tk, tp_, tmp) != (sp0.top_k, sp0.top_p, sp0.temperature):
                import dataclasses
                sampling_params = dataclasses.replace(sp0, top_k=tk, top_p=tp_, temperature=tmp)
            for name_ in ("logprobs", "prompt_logprobs"):
                k_ = getattr(sampling_params, name_)
                if k_ is not None and not 0 <= int(k_) <= self.MAX_LOGPROBS:
                    raise ValueError(f"{name_} must be between 0 and {self.MAX_LOGPROBS}")
        if sampling_params is not None and sampling_params.constrained:
            # these ids index the logits when the mask is built
            V = self.cfg.model.vocab_size
            ids_ = list(sampling_params.allowed_token_ids or ())
            for c_ in sampling_params.guided_choice or ():
                ids_ += list(c_)
            if ids_ and (min(ids_) < 0 or max(ids_) >= V):
                raise ValueError(f"allowed / choice token ids must lie in [0, {V})")
        if lora_id is not None and lora_id >= 0:
            mgr = self.runner.lora
            if mgr is None or lora_id not in mgr.slots:
                raise ValueError(f"LoRA adapter {lora_id} is not loaded")
        if sampling_params is not None and sampling_params.pooling \
                and sampling_params.max_tokens != 1:
            import dataclasses
            sampling_params = dataclasses.replace(sampling_params, max_tokens=1, min_tokens=0)
        sampling_params = sampling_params or SamplingParams()
        if eos_token_id is None and not sampling_params.ignore_eos:
            # the checkpoint's end-of-sequence ids stop a request like any stop token; the
            # first one is also what a guided request emits once its pattern is complete
            eos = self.cfg.model.eos_token_ids
            if eos:
                eos_token_id = eos[0]
                more = tuple(t for t in eos[1:] if t not in sampling_params.stop_token_ids)
                if more:
                    import dataclasses
                    sampling_params = dataclasses.replace(
                        sampling_params, stop_token_ids=tuple(sampling_params.stop_token_ids) + more)
        req = Request(rid, list(prompt_token_ids), sampling_params,
                      eos_token_id=eos_token_id, priority=priority, lora_id=lora_id)
        if multi_modal_data:
            prep = getattr(self.model, "prepare_request", None)
            if prep is None:
                raise ValueError(f"{self.cfg.model.architecture} takes no multimodal input")
            # second operand: patch grids (Qwen2.5-VL) or tile counts per image (DeepSeek-VL2)
            # or original image sizes (LLaVA-NeXT)
            grids = multi_modal_data.get("image_grid_thw", multi_modal_data.get(
                "images_spatial_crop", multi_modal_data.get("image_sizes")))
            for k, v in prep(req.prompt_token_ids, multi_modal_data["pixel_values"],
                             grids).items():
                setattr(req, k, v)
        if kv_transfer_params:
            req.kv_transfer_params = dict(kv_transfer_params)
            if self.disagg is not None:
                self.disagg.on_add(req)
        sp_ = req.sampling_params
        if sp_.guided_regex is not None or sp_.guided_json is not None:
            if req.eos_token_id is None:     # a guided request ends with EOS once it matches
                req.eos_token_id = getattr(self.cfg.model, "eos_token_id", None)
            req.guide = self._make_guide(sp_, req.eos_token_id)
        self.scheduler.add_request(req)
        if sp_.needs_host_history:
            # these need the ids of every earlier token on the host before the next step
            self._want_sync = True
        return rid

    def set_vocabulary(self, vocab: Sequence[Optional[str]]) -> None:
        """Text of every token id (None for ids that must never be produced by a guided
        request).  Needed by ``guided_regex`` / ``guided_json``."""
        self._vocab = list(vocab)
        self._guides = {}

    def _make_guide(self, sp_: SamplingParams, eos_token_id: Optional[int]):
        from .guided import GuideCursor, RegexGuide, json_schema_to_regex
        vocab = getattr(self, "_vocab", None)
        if vocab is None:
            raise ValueError("guided_regex / guided_json need the vocabulary: call "
                             "set_vocabulary(token_texts) first")
        pattern = sp_.guided_regex if sp_.guided_regex is not None \
            else json_schema_to_regex(sp_.guided_json)
        key = (pattern, eos_token_id)
        guide = self._guides.get(key)
        if guide is None:
            guide = self._guides[key] = RegexGuide(pattern, vocab, eos_token_id)
        return GuideCursor(guide)

    def abort_request(self, request_id: str) -> None:
        self.scheduler.abort_request(request_id)

    def attach_kv_connector(self, connector, recv_timeout_s: float = 30.0):
        """Disaggregated prefill: requests with ``kv_transfer_params`` send their KV to /
        take their KV from the peer instance through ``connector`` (engine/kv_disagg.py)."""
        from .kv_disagg import DisaggCoordinator
        self.disagg = DisaggCoordinator(self, connector, recv_timeout_s)
        self.scheduler.on_free = self.disagg.before_free
        return self.disagg

    def add_lora(self, lora_request, tensors=None, config=None) -> int:
        """Loads a LoRA adapter; requests select it with ``lora_id=lora_request.lora_int_id``."""
        if self.runner.lora is None:
            raise RuntimeError("start the engine with enable_lora=True")
        return self.runner.lora.add_adapter(lora_request, tensors, config)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or bool(self._pending)

    # -- stepping ---------------------------------------------------------------------
    def _dp_exchange(self, num_tokens: int, busy: bool) -> int:
        """Data-parallel attention: every replica publishes its token count and whether it
        still has requests (CPU all-gather over gloo, as the reference does for its DP
        metadata, vllm_gcu/patch/patch_0_9_2/forward_context.py:10-43).  Returns the largest
        token count; ``dp_global_busy`` tells the caller whether any replica has work."""
        import torch.distributed as dist
        st = get_state()
        mine = torch.tensor([num_tokens, int(busy)], dtype=torch.int64)
        parts = [torch.zeros_like(mine) for _ in range(self.dp_size)]
        dist.all_gather(parts, mine, group=st.dp.cpu_group or st.dp.device_group)
        self.dp_global_busy = any(int(p[1]) for p in parts)
        mx = max(int(p[0]) for p in parts)
        st.dp_max_tokens = mx
        return mx

    def _launch(self) -> Optional[tuple[SchedulerOutput, StepHandle]]:
        busy = self.has_unfinished()
        so = self.scheduler.schedule()
        if self.dp_size > 1:
            n_tok = sum(s.num_tokens for s in so.scheduled)
            mx = self._dp_exchange(n_tok, busy)
            if so.is_empty and mx > 0:
                # keep-alive forward: this replica takes part in every expert-parallel
                # collective of the step with zero tokens
                self.runner.execute_dummy_batch()
        if so.is_empty:
            self.runner.release(so.finished_req_ids)
            self.runner.release(so.preempted_req_ids)
            self.runner.apply_swaps(so)
            return None
        handle = self.runner.execute(so)
        self.stats["steps"] += 1
        return so, handle

    def _finish(self, so: SchedulerOutput, handle: StepHandle) -> list[RequestOutput]:
        toks = handle.token_ids()
        draft = handle.draft_tokens()
        if self.spec_metrics is not None:
            for rid, nd in zip(handle.req_ids, handle.extra.get("num_draft", [])):
                if nd:
                    self.spec_metrics.update(nd, len(toks.get(rid, ())))
        lp = None
        raw = handle.extra.get("logprobs")
        if raw is not None:
            chosen, tv, ti, ks = raw
            lp = {}
            for i, rid in enumerate(handle.req_ids):
                if ks[i] < 0:
                    continue
                top = {int(ti[i, c]): float(tv[i, c]) for c in range(ks[i])}
                tok = toks[rid][0] if toks.get(rid) else -1
                top.setdefault(int(tok), float(chosen[i]))
                lp[rid] = top
        pl = handle.extra.get("prompt_logprobs")
        if pl:
            for rid, (chosen, tv, ti, targets) in pl.items():
                req = self.scheduler.requests.get(rid)
                if req is None:
                    continue
                if not hasattr(req, "prompt_logprobs") or req.prompt_logprobs is None:
                    req.prompt_logprobs = [None]          # the first token has no prediction
                for r_, t_ in enumerate(targets):
                    d = {int(ti[r_, c]): float(tv[r_, c]) for c in range(tv.shape[1])}
                    d.setdefault(int(t_), float(chosen[r_]))
                    req.prompt_logprobs.append(d)
        if draft:
            # masks, penalties and log-probabilities are applied to one position per step:
            # such requests take no draft tokens
            reqs = self.scheduler.requests
            draft = {rid: d for rid, d in draft.items()
                     if rid in reqs and not reqs[rid].sampling_params.needs_host_history}
        outs = self.scheduler.update_from_output(so, toks, draft, lp)
        outs = self._apply_stop_strings(so, outs)
        hid = handle.extra.get("hidden")
        if hid is not None:
            so_req = {s.req.request_id: s.req for s in so.scheduled}
            rows = {rid: i for i, rid in enumerate(handle.req_ids)}
            hid = hid.cpu()
            for o in outs:
                i = rows.get(o.request_id)
                r = so_req.get(o.request_id)
                if i is not None and r is not None and r.sampling_params.pooling:
                    o.embedding = hid[i]
        if self.proposer is not None:
            for s in so.scheduled:
                r = s.req
                if r.sampling_params.needs_host_history:
                    continue
                if s.will_sample and not r.finished and r.request_id in self.scheduler.requests:
                    room = r.sampling_params.max_tokens - len(r.output_token_ids) - 1
                    r.spec_token_ids = self.proposer.propose(r.all_token_ids)[:max(0, room)]
        return outs

    MAX_LOGPROBS = 20      # alternatives reported per position, as upstream servers limit it
    detokenizer = None     # callable(token ids) -> text; set by LLM / the server for stop strings

    def _apply_stop_strings(self, so: SchedulerOutput, outs: list[RequestOutput]
                            ) -> list[RequestOutput]:
        """Requests whose sampling parameters name stop strings end as soon as their output
        text contains one; the text is cut in front of it (``include_stop_str_in_output``
        keeps it) and the tokens after the match are dropped from the count that matters to the
        caller only in the text: token ids are returned as generated."""
        if self.detokenizer is None:
            return outs
        by_id = None
        for s in so.scheduled:
            r = s.req
            sp = r.sampling_params
            if not sp.stop or not s.will_sample or not r.output_token_ids:
                continue
            text = self.detokenizer(r.output_token_ids)
            cut = min((text.find(t) + (len(t) if sp.include_stop_str_in_output else 0)
                       for t in sp.stop if t and t in text), default=-1)
            if cut < 0:
                continue
            if by_id is None:
                by_id = {o.request_id: i for i, o in enumerate(outs)}
            final = None
            if r.finished:                       # ended on its own in this very step
                i = by_id.get(r.request_id)
                final = outs[i] if i is not None else None
            else:
                final = self.scheduler.stop_request(r.request_id)
                if final is not None:
                    self.runner.release([r.request_id])
                    i = by_id.get(r.request_id)
                    if i is not None:
                        outs[i] = final
                    else:
                        outs.append(final)
            if final is not None:
                final.outputs[0].text = text[:cut]
                final.outputs[0].finish_reason = "stop"
        return outs

    def step(self) -> list[RequestOutput]:
        """One scheduling round.  With ``num_scheduler_steps = n > 1`` (the reference's
        multi-step scheduler, vllm_gcu/worker/multi_step_worker.py:33-336) the round runs up to
        n engine steps back to back and hands their outputs over together; the steps
        themselves use the device-side next-token feed, so the GPU does not wait for the host
        in between."""
        n = max(1, int(self.cfg.scheduler.num_scheduler_steps))
        if n == 1:
            return self._step_once()
        merged: dict[str, RequestOutput] = {}
        for _ in range(n):
            for o in self._step_once():
                merged[o.request_id] = o
            if not self.has_unfinished():
                break
        return list(merged.values())

    def _step_once(self) -> list[RequestOutput]:
        """Runs (or, with async scheduling, launches and retires) one engine step."""
        from .. import envs
        every = envs.LOG_FORWARD_TIME_EVERY
        if every <= 0:
            return self._step_inner()
        t0 = time.perf_counter()
        n_before = self.stats["steps"]
        outs = self._step_inner()
        if self.stats["steps"] > n_before:
            self.record_step_time(self.scheduler.num_running_last, time.perf_counter() - t0,
                                  every)
        return outs

    def record_step_time(self, batch: int, seconds: float, every: int) -> None:
        """Step wall times by batch size; their medians are logged every ``every`` steps
        (vllm_gcu/patch/patch_0_8_0/forward_context.py:62-92 keeps the same statistic)."""
        log = self.__dict__.setdefault("_step_times", {})
        log.setdefault(int(batch), []).append(seconds)
        total = sum(len(v) for v in log.values())
        if total % every == 0:
            import statistics
            from ..utils import logger
            logger.info("median step time by batch size: %s", ", ".join(
                f"{b}: {statistics.median(v) * 1e3:.2f} ms ({len(v)})"
                for b, v in sorted(log.items())))

    def _step_inner(self) -> list[RequestOutput]:
        outs: list[RequestOutput] = []
        if self._want_sync and self.cfg.scheduler.async_scheduling:
            # a request whose next token depends on host-side history has arrived: retire
            # every step in flight first, then run in lock-step until no such request is left
            while self._pending:
                outs += self._finish(*self._pending.popleft())
            self.cfg.scheduler.async_scheduling = False
            self.scheduler.async_mode = False
            self._async_suspended = True
        if not self.cfg.scheduler.async_scheduling:
            item = self._launch()
            if item is not None:
                outs += self._finish(*item)
            if getattr(self, "_async_suspended", False) and not any(
                    r.sampling_params.needs_host_history
                    for r in self.scheduler.requests.values()):
                self._want_sync = False
                self._async_suspended = False
                self.cfg.scheduler.async_scheduling = True
                self.scheduler.async_mode = True
            return outs
        item = self._launch() if self.scheduler.has_unfinished() else None
        if item is not None:
            self._pending.append(item)
        if self._pending and (len(self._pending) >= 2 or item is None):
            outs = self._finish(*self._pending.popleft())
        return outs

    def generate(self, prompts: Iterable[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 ) -> list[RequestOutput]:
        prompts = list(prompts)
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sps = [sampling_params or SamplingParams()] * len(prompts)
        else:
            sps = list(sampling_params)
        order = []
        for p, sp in zip(prompts, sps):
            if isinstance(p, dict):      # {"prompt_token_ids": [...], "multi_modal_data": {...}}
                order.append(self.add_request(p["prompt_token_ids"], sp,
                                              multi_modal_data=p.get("multi_modal_data")))
            else:
                order.append(self.add_request(p, sp))
        final: dict[str, RequestOutput] = {}
        prev, self.scheduler.emit_partial = self.scheduler.emit_partial, False
        try:
            while self.has_unfinished() or self.dp_global_busy:
                for ro in self.step():
                    if ro.finished:
                        final[ro.request_id] = ro
        finally:
            self.scheduler.emit_partial = prev
        return [final[r] for r in order]


    def embed(self, prompts: Iterable[Sequence[int]], normalize: bool = True) -> torch.Tensor:
        """Embeddings from a decoder checkpoint (gte-Qwen2 in the reference's model table,
        docs/source/user_guide/support_matrix/supported_models.md:22): the final-norm hidden
        state of each prompt's last token, L2-normalised, as a float32 [n, hidden] tensor on
        the host.  Prompts run through the normal scheduler (chunked prefill, prefix cache,
        batching) as one-token requests; the sampled token is discarded."""
        prompts = [list(p) for p in prompts]
        outs = self.generate(prompts, SamplingParams(temperature=0.0, max_tokens=1,
                                                     ignore_eos=True, pooling=True))
        vec = torch.stack([o.embedding for o in outs])
        if normalize:
            vec = torch.nn.functional.normalize(vec, dim=-1)
        return vec


def check_token_ids(prompt_token_ids, vocab_size: int, allow_placeholders: bool = False) -> None:
    """Raises ValueError for a token id outside the vocabulary: such an id would index past the
    embedding table.  Prompts with multimodal data may carry placeholder ids beyond the text
    vocabulary (their rows are replaced by the vision embeddings), negative ids never."""
    if len(prompt_token_ids) == 0:
        return
    lo, hi = min(prompt_token_ids), max(prompt_token_ids)
    if lo < 0 or (hi >= vocab_size and not allow_placeholders):
        bad = lo if lo < 0 else hi
        raise ValueError(f"token id {bad} is outside the vocabulary of {vocab_size} entries")


def decode_text(tokenizer, token_ids) -> str:
    """Output text without special tokens (the end-of-sequence marker that ended a request is
    part of its token ids, not of its text)."""
    try:
        return tokenizer.decode(list(token_ids), skip_special_tokens=True)
    except TypeError:                       # tokenizers without that option
        return tokenizer.decode(list(token_ids))


def chat_template_ids(tokenizer, messages) -> list[int]:
    """Prompt ids of a conversation rendered with the tokenizer's chat template.  Depending on
    the tokenizer library's version the call returns the ids or an encoding that holds them."""
    out = tokenizer.apply_chat_template(list(messages), tokenize=True, add_generation_prompt=True)
    if hasattr(out, "keys"):
        out = out["input_ids"]
    if out and isinstance(out[0], (list, tuple)):
        out = out[0]
    return [int(t) for t in out]


class LLM:
    """Convenience wrapper mirroring the offline-inference entry point users of the
    reference call (``vllm.LLM``): build from a preset / HF config / checkpoint directory and
    call :meth:`generate` with token-id prompts."""

    def __init__(self, model: Union[str, ModelConfig], tensor_parallel_size: int = 1,
                 pipeline_parallel_size: int = 1, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 8192, max_model_len: Optional[int] = None,
                 block_size: int = 16, gpu_memory_utilization: float = 0.9,
                 enable_prefix_caching: bool = True, async_scheduling: bool = False,
                 num_scheduler_steps: int = 1,
                 enforce_eager: bool = False, device: str = "auto", seed: int = 0,
                 num_gpu_blocks: Optional[int] = None, num_cpu_blocks: int = 0,
                 scheduling_policy: str = "fcfs",
                 load_format: Optional[str] = None, comm_backend: str = "fused",
                 enable_expert_parallel: bool = False, dtype: Optional[str] = None,
                 cuda_graph_sizes: Optional[list[int]] = None,
                 speculative_method: Optional[str] = None, num_speculative_tokens: int = 0,
                 speculative_model: Optional[str] = None,
                 prompt_lookup_max: int = 4, prompt_lookup_min: int = 1,
                 enable_lora: bool = False, max_loras: int = 4, max_lora_rank: int = 16,
                 additional_config: Optional[dict] = None, tokenizer=None,
                 quantization_param_path: Optional[str] = None, mm_processor=None,
                 **model_overrides):
        model_path = None
        if isinstance(model, ModelConfig):
            mc = model
        else:
            import os
            if os.path.isdir(model):
                mc = ModelConfig.from_pretrained(model, **model_overrides)
                model_path = model
            else:
                mc = preset(model, **model_overrides)
        if dtype is not None:
            from ..config import to_dtype
            mc.dtype = to_dtype(dtype)
        additional_config = dict(additional_config or {})
        if enable_lora:
            additional_config["lora"] = {"max_loras": max_loras, "max_lora_rank": max_lora_rank}
        cfg = EngineConfig(
            model=mc,
            cache=CacheConfig(block_size=block_size, gpu_memory_utilization=gpu_memory_utilization,
                              enable_prefix_caching=enable_prefix_caching,
                              num_gpu_blocks=num_gpu_blocks, num_cpu_blocks=num_cpu_blocks),
            scheduler=SchedulerConfig(max_num_seqs=max_num_seqs,
                                      max_num_batched_tokens=max_num_batched_tokens,
                                      max_model_len=max_model_len or mc.max_position_embeddings,
                                      policy=scheduling_policy, async_scheduling=async_scheduling,
                                      num_scheduler_steps=num_scheduler_steps),
            parallel=ParallelConfig(tensor_parallel_size=tensor_parallel_size,
                                    pipeline_parallel_size=pipeline_parallel_size,
                                    comm_backend=comm_backend,
                                    enable_expert_parallel=enable_expert_parallel),
            speculative=SpeculativeConfig(speculative_method, num_speculative_tokens,
                                          prompt_lookup_max, prompt_lookup_min,
                                          speculative_model),
            device=device, seed=seed, enforce_eager=enforce_eager,
            cuda_graph_sizes=cuda_graph_sizes,
            load_format=load_format or ("safetensors" if model_path else "dummy"),
            model_path=model_path, additional_config=additional_config or {},
            quantization_param_path=quantization_param_path)
        self.engine = LLMEngine(cfg)
        # text in / text out: a tokenizer object (``encode`` / ``decode``) or a directory
        # with tokenizer files; by default the tokenizer next to the checkpoint
        self.tokenizer = None
        if tokenizer is None and model_path:
            tokenizer = model_path
        if isinstance(tokenizer, str):
            try:
                from transformers import AutoTokenizer
                self.tokenizer = AutoTokenizer.from_pretrained(tokenizer)
            except Exception:
                self.tokenizer = None
        elif tokenizer is not None:
            self.tokenizer = tokenizer
        if self.tokenizer is not None:
            tok_ = self.tokenizer
            self.engine.detokenizer = lambda ids: decode_text(tok_, ids)
        # images given as PIL objects (``multi_modal_data={"image": ...}``) go through the
        # checkpoint's HuggingFace processor when it has one (entrypoints/multimodal.py)
        self.mm_processor = mm_processor
        if mm_processor is None and model_path:
            from ..entrypoints.multimodal import default_processor
            self.mm_processor = default_processor(model_path, self.engine.model, self.tokenizer)

    def _encode(self, prompt):
        """Prompts may be token-id lists, dicts with ``prompt_token_ids`` or text."""
        if isinstance(prompt, dict) and "image" in (prompt.get("multi_modal_data") or {}) \
                and "prompt" in prompt:
            if self.mm_processor is None or not hasattr(self.mm_processor, "from_text"):
                raise ValueError("raw images need a multimodal processor "
                                 "(LLM(..., mm_processor=...))")
            images = prompt["multi_modal_data"]["image"]
            images = list(images) if isinstance(images, (list, tuple)) else [images]
            ids, mm = self.mm_processor.from_text(prompt["prompt"], images)
            return {"prompt_token_ids": ids, "multi_modal_data": mm}
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("text prompts need a tokenizer (LLM(..., tokenizer=...))")
            return list(self.tokenizer.encode(prompt))
        if isinstance(prompt, dict) and "prompt" in prompt and "prompt_token_ids" not in prompt:
            d = dict(prompt)
            d["prompt_token_ids"] = self._encode(d.pop("prompt"))
            return d
        return prompt

    def _decode_outputs(self, outs):
        if self.tokenizer is not None:
            for o in outs:
                for c in o.outputs:
                    if not c.text:           # a stop string already cut this one's text
                        c.text = decode_text(self.tokenizer, c.token_ids)
        return outs

    def chat(self, messages, sampling_params=None) -> list[RequestOutput]:
        """One conversation (list of ``{"role", "content"}``) or a list of conversations,
        rendered with the tokenizer's chat template."""
        if self.tokenizer is None or not hasattr(self.tokenizer, "apply_chat_template"):
            raise ValueError("chat() needs a tokenizer with a chat template")
        convs = messages if messages and isinstance(messages[0], list) else [messages]
        prompts = [chat_template_ids(self.tokenizer, c) for c in convs]
        return self.generate(prompts, sampling_params)

    def set_vocabulary(self, vocab) -> None:
        """Token texts (index = token id) or a tokenizer; enables ``guided_regex`` /
        ``guided_json`` requests."""
        if hasattr(vocab, "decode"):
            from .guided import vocabulary_of
            vocab = vocabulary_of(vocab, self.engine.cfg.model.vocab_size)
        self.engine.set_vocabulary(vocab)

    def embed(self, prompts, normalize: bool = True):
        """Last-token embeddings of text or token-id prompts from a decoder checkpoint
        (:meth:`LLMEngine.embed`)."""
        if isinstance(prompts, str):
            prompts = [prompts]
        return self.engine.embed([self._encode(p) for p in prompts], normalize=normalize)

    def generate(self, prompts, sampling_params=None) -> list[RequestOutput]:
        """One ``RequestOutput`` per prompt.  ``n`` / ``best_of`` > 1 run that many sampled
        continuations per prompt (sharing the prompt's KV blocks through the prefix cache)
        and return the ``n`` with the highest cumulative log-probability; ``use_beam_search``
        routes to :meth:`beam_search` (best-of and beam search are listed as functional in
        docs/source/user_guide/support_matrix/supported_features.md:11-64)."""
        if isinstance(prompts, str):
            prompts = [prompts]
        prompts = [self._encode(p) for p in prompts]
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sps = [sampling_params or SamplingParams()] * len(prompts)
        else:
            sps = list(sampling_params)
        if any(sp.guided_regex is not None or sp.guided_json is not None for sp in sps) \
                and getattr(self.engine, "_vocab", None) is None and self.tokenizer is not None:
            self.set_vocabulary(self.tokenizer)
        if all(sp.n == 1 and not sp.best_of and not sp.use_beam_search for sp in sps):
            return self._decode_outputs(self.engine.generate(prompts, sps))
        import dataclasses
        flat_p, flat_sp, owner = [], [], []
        results: list[Optional[RequestOutput]] = [None] * len(prompts)
        for i, (p, sp) in enumerate(zip(prompts, sps)):
            if sp.use_beam_search:
                results[i] = self.beam_search(p, max(sp.best_of or sp.n, 1), sp.max_tokens,
                                              num_return=sp.n, eos_token_id=None)
                continue
            k = max(sp.best_of or sp.n, sp.n)
            for c in range(k):
                seed = (sp.seed if sp.seed is not None else 0) * 7919 + c + 1
                flat_sp.append(dataclasses.replace(
                    sp, n=1, best_of=None, seed=seed,
                    logprobs=sp.logprobs if sp.logprobs is not None else (0 if k > sp.n else None)))
                flat_p.append(p)
                owner.append(i)
        outs = self.engine.generate(flat_p, flat_sp) if flat_p else []
        grouped: dict[int, list] = {}
        for o, i in zip(outs, owner):
            grouped.setdefault(i, []).append(o)
        for i, group in grouped.items():
            comps = [g.outputs[0] for g in group]
            if len(comps) > sps[i].n:
                comps.sort(key=lambda c: -(c.cumulative_logprob or 0.0))
                comps = comps[:sps[i].n]
            for idx, c in enumerate(comps):
                c.index = idx
            results[i] = RequestOutput(group[0].request_id, group[0].prompt_token_ids, comps, True,
                                       group[0].num_cached_tokens, group[0].prompt_logprobs)
        return self._decode_outputs(results)          # type: ignore[arg-type]

    def beam_search(self, prompt: Sequence[int], beam_width: int, max_tokens: int,
                    num_return: int = 1, eos_token_id: Optional[int] = None,
                    length_penalty: float = 1.0) -> RequestOutput:
        """Beam search on top of the engine: every step scores the live beams with one
        single-token request each (``logprobs = 2 * beam_width``); the shared prefixes are
        served by the prefix cache, so a step costs one decode token per beam."""
        from .request import CompletionOutput
        beams = [(list(prompt), 0.0)]
        done: list[tuple[list[int], float]] = []
        n_prompt = len(prompt)
        sp = SamplingParams(max_tokens=1, temperature=0.0, logprobs=2 * beam_width,
                            ignore_eos=True)
        for _ in range(max_tokens):
            outs = self.engine.generate([b[0] for b in beams], sp)
            cand = []
            for (toks, score), o in zip(beams, outs):
                lp = o.outputs[0].logprobs[0]
                for tid, l in lp.items():
                    cand.append((toks + [tid], score + l))
            cand.sort(key=lambda c: -c[1])
            beams = []
            for toks, score in cand:
                if eos_token_id is not None and toks[-1] == eos_token_id:
                    done.append((toks, score))
                else:
                    beams.append((toks, score))
                if len(beams) >= beam_width:
                    break
            if not beams:
                break
        done += beams

        def norm(item):
            toks, score = item
            return score / (max(len(toks) - n_prompt, 1) ** length_penalty)
        done.sort(key=lambda c: -norm(c))
        comps = [CompletionOutput(i, toks[n_prompt:], "length", None, score)
                 for i, (toks, score) in enumerate(done[:num_return])]
        return RequestOutput("beam", list(prompt), comps, True)
