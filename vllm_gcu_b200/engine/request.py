"""Requests, sampling parameters and outputs of the engine."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass
class SamplingParams:
    """Per-request sampling options (the subset the reference documents as supported,
    ReadMe-EN.md:283-292: top-p / top-k, presence / frequency / repetition penalty,
    ignore-eos, stop handling, logprobs)."""
    max_tokens: int = 16
    min_tokens: int = 0
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    seed: Optional[int] = None
    ignore_eos: bool = False
    stop_token_ids: tuple[int, ...] = ()
    # stop strings: generation ends when the output text contains one (needs an engine that can
    # detokenise: LLM with a tokenizer, or the server); the text is cut in front of it
    stop: tuple[str, ...] = ()
    include_stop_str_in_output: bool = False
    logprobs: Optional[int] = None
    prompt_logprobs: Optional[int] = None
    n: int = 1
    best_of: Optional[int] = None
    use_beam_search: bool = False
    # constrained decoding: only these token ids may be sampled / the output must be one of
    # these token sequences (the token-level form of guided "choice" decoding)
    allowed_token_ids: Optional[tuple[int, ...]] = None
    guided_choice: Optional[tuple[tuple[int, ...], ...]] = None
    # grammar-guided decoding (engine/guided.py): the output text must match the pattern /
    # be a JSON document of the schema; needs an engine that knows its vocabulary
    guided_regex: Optional[str] = None
    guided_json: Optional[Any] = None
    # pooling request (embedding from a decoder checkpoint): the output carries the final
    # hidden state of the last prompt token; the request ends after its first step
    pooling: bool = False
    extra_args: dict[str, Any] = field(default_factory=dict)

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def constrained(self) -> bool:
        return (self.allowed_token_ids is not None or self.guided_choice is not None
                or self.guided_regex is not None or self.guided_json is not None)

    def allowed_next(self, output_token_ids: list) -> Optional[list]:
        """Token ids that may follow ``output_token_ids`` (None = unconstrained)."""
        if self.guided_choice is not None:
            n = len(output_token_ids)
            nxt = sorted({c[n] for c in self.guided_choice
                          if len(c) > n and list(c[:n]) == list(output_token_ids)})
            return nxt
        if self.allowed_token_ids is not None:
            return list(self.allowed_token_ids)
        return None

    @property
    def has_penalties(self) -> bool:
        return (self.presence_penalty != 0.0 or self.frequency_penalty != 0.0
                or self.repetition_penalty != 1.0)

    @property
    def needs_host_history(self) -> bool:
        """True when sampling the next token needs every earlier token id on the host
        (penalty histories, guide state, allowed-token masks) or reads the logits back
        (log-probabilities).  Such a request never runs ahead of its own results and never
        carries draft tokens."""
        return (self.has_penalties or self.constrained or self.logprobs is not None
                or self.prompt_logprobs is not None)


class RequestStatus(enum.IntEnum):
    WAITING = 0
    RUNNING = 1
    PREEMPTED = 2
    SWAPPED = 3
    FINISHED_STOPPED = 4
    FINISHED_LENGTH = 5
    FINISHED_ABORTED = 6

    @property
    def finished(self) -> bool:
        return self >= RequestStatus.FINISHED_STOPPED


@dataclass(eq=False)      # identity semantics: requests live in lists and sets
class Request:
    request_id: str
    prompt_token_ids: list[int]
    sampling_params: SamplingParams
    eos_token_id: Optional[int] = None
    arrival_time: float = field(default_factory=time.monotonic)
    priority: int = 0
    lora_id: int = -1
    is_idle: bool = False                     # keep-alive request of a DP replica
    kv_transfer_params: Optional[dict] = None
    kv_transfer_params_out: Optional[dict] = None   # prefill instance: what the decode one needs
    # multimodal inputs: embeddings of the placeholder tokens (row i belongs to prompt position
    # mm_positions[i]), M-RoPE (t, h, w) positions of the prompt ``[3, n_prompt]`` and the
    # offset added to the position of every later token
    mm_embeds: Optional[Any] = None
    mm_positions: Optional[list] = None
    mrope_positions: Optional[Any] = None
    mrope_delta: int = 0
    cache_salt: Optional[int] = None          # separates prefix-cache entries (image content)
    guide: Optional[Any] = None               # GuideCursor of a grammar-guided request
    cpu_block_ids: list = field(default_factory=list)   # host blocks while swapped out

    # mutable state -------------------------------------------------------
    status: RequestStatus = RequestStatus.WAITING
    output_token_ids: list[int] = field(default_factory=list)
    num_computed_tokens: int = 0              # tokens whose KV is in the cache
    num_output_placeholders: int = 0          # async scheduling: tokens scheduled, id unknown
    num_cached_tokens: int = 0                # prefix-cache hit length (first schedule)
    spec_token_ids: list[int] = field(default_factory=list)
    block_ids: list[int] = field(default_factory=list)
    num_preemptions: int = 0
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    logprobs: list[Any] = field(default_factory=list)          # per output token: {id: logprob}
    prompt_logprobs: Optional[list] = None                     # per prompt token (first: None)

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_tokens(self) -> int:
        """Known tokens (prompt + generated)."""
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def num_tokens_with_placeholders(self) -> int:
        return self.num_tokens + self.num_output_placeholders

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    @property
    def finished(self) -> bool:
        return self.status.finished

    def allowed_next(self) -> Optional[list]:
        """Token ids the next sampled token must come from (None = unconstrained)."""
        if self.guide is not None:
            return self.guide.allowed_next(self.output_token_ids)
        return self.sampling_params.allowed_next(self.output_token_ids)

    def token_at(self, i: int) -> int:
        n = len(self.prompt_token_ids)
        return self.prompt_token_ids[i] if i < n else self.output_token_ids[i - n]


@dataclass
class CompletionOutput:
    index: int
    token_ids: list[int]
    finish_reason: Optional[str] = None
    logprobs: Optional[list] = None
    cumulative_logprob: Optional[float] = None
    text: Optional[str] = None                # filled when the LLM has a tokenizer


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: list[int]
    outputs: list[CompletionOutput]
    finished: bool
    num_cached_tokens: int = 0
    prompt_logprobs: Optional[list] = None
    metrics: dict[str, float] = field(default_factory=dict)
    kv_transfer_params: Optional[dict] = None       # disaggregated prefill: for the decode side
    embedding: Optional[Any] = None                 # pooling requests: float32 [hidden] on the host


def check_stop(req: Request, max_model_len: int) -> bool:
    """Applies the stop conditions to the last appended token.  Returns True when the
    request finished (status updated)."""
    sp = req.sampling_params
    n_out = len(req.output_token_ids)
    if n_out == 0:
        return False
    last = req.output_token_ids[-1]
    if n_out >= sp.min_tokens:
        if not sp.ignore_eos and req.eos_token_id is not None and last == req.eos_token_id:
            req.status = RequestStatus.FINISHED_STOPPED
            return True
        if last in sp.stop_token_ids:
            req.status = RequestStatus.FINISHED_STOPPED
            return True
    if sp.guided_choice is not None and any(
            list(c) == req.output_token_ids for c in sp.guided_choice) and not any(
            len(c) > n_out and list(c[:n_out]) == req.output_token_ids for c in sp.guided_choice):
        req.status = RequestStatus.FINISHED_STOPPED      # a complete choice, no longer one
        return True
    if req.guide is not None and (last == req.eos_token_id
                                  or req.guide.finished(req.output_token_ids)):
        req.status = RequestStatus.FINISHED_STOPPED      # pattern matched, nothing can follow
        return True
    if n_out >= sp.max_tokens or req.num_tokens >= max_model_len:
        req.status = RequestStatus.FINISHED_LENGTH
        return True
    return False
