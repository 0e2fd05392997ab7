"""Disaggregated prefill (1 prefill instance -> 1 decode instance) on top of the
point-to-point KV connector.

Flow (the reference's v1 ``P2pEcclConnector``: vllm_gcu/v1/p2p_eccl_engine.py:120-373 and its
v0 ``SimpleConnector`` wiring, vllm_gcu/distributed/kv_transfer/connector.py:122-128):

* the **prefill instance** runs the prompt, emits the first token and, when the request
  finishes, gathers the KV of every layer for the prompt tokens by slot mapping (the LMCache
  multi-layer kernel) and sends it under the request id (``PUT`` / ``PUT_ASYNC``) or keeps it
  for a later ``GET``;
* the **decode instance** receives a request that names the prefill request, takes blocks
  for ``n_prompt - 1`` tokens, scatters the received KV into its paged cache and starts at
  the last prompt token: one single-token step produces the first output token, then decode
  continues as usual.  If nothing arrives in time the request falls back to a local prefill.

Request side: ``kv_transfer_params = {"do_remote_decode": True, "remote": "host:port"}`` on
the prefill instance; ``{"do_remote_prefill": True, "remote": ..., "remote_request_id": ...}``
on the decode instance.  The finished output of the prefill instance carries the parameters
for the decode instance (``RequestOutput.kv_transfer_params``), as the reference's patched
NIXL scheduler side does (vllm_gcu/patch/patch_0_9_2/nixl_connector.py:98-155).

Two switches of that patch are kept (``VLLM_B200_NIXL_ENABLE_*``, nixl_connector.py:71-90,
127-143):

* *full KV transfer* – the KV of a partly filled last block travels too.  This connector
  moves rows per token, so that is what it always does; with the switch off the decode
  instance takes whole blocks only and recomputes the rest, which is the stock behaviour the
  patch changes.
* *first-token reuse* – the prefill instance hands its first output token over with the
  parameters; the decode instance appends it to the prompt, takes the KV of the whole prompt
  and starts decoding at that token: no prompt token is computed twice.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..parallel.kv_transfer import lmcache_ops


def _layer_views(runner):
    """Per layer: paged buffer viewed as [kv, slots, W], plus slot count and width."""
    caches = runner.kv_caches
    c0 = caches[0]
    mla = c0.dim() == 3
    if mla:
        slots, W = c0.shape[0] * c0.shape[1], c0.shape[2]
    else:
        slots, W = c0.shape[1] * c0.shape[2], c0.shape[3] * c0.shape[4]
    return caches, mla, slots, W


def _slot_mapping(block_ids, n_tokens: int, block_size: int, device) -> torch.Tensor:
    pos = torch.arange(n_tokens)
    blocks = torch.tensor(block_ids, dtype=torch.long)[pos // block_size]
    return (blocks * block_size + pos % block_size).to(device)


def extract_kv(runner, block_ids, n_tokens: int) -> torch.Tensor:
    """KV of the first ``n_tokens`` of a request: ``[2, L, n, W]`` (``[L, n, W]`` for MLA)."""
    caches, mla, slots, W = _layer_views(runner)
    L = len(caches)
    dev = caches[0].device
    shape = (L, n_tokens, W) if mla else (2, L, n_tokens, W)
    buf = torch.empty(shape, dtype=caches[0].dtype, device=dev)
    sm = _slot_mapping(block_ids, n_tokens, runner.block_size, dev)
    ptrs = torch.tensor([c.data_ptr() for c in caches], dtype=torch.int64, device=dev)
    lmcache_ops.multi_layer_kv_transfer(buf, ptrs, sm, dev, slots, True, mla,
                                        layers=None if dev.type == "cuda" else list(caches))
    return buf


def inject_kv(runner, block_ids, kv: torch.Tensor) -> None:
    caches, mla, slots, W = _layer_views(runner)
    dev = caches[0].device
    kv = kv.to(device=dev, dtype=caches[0].dtype).contiguous()
    n = kv.shape[-2]
    sm = _slot_mapping(block_ids, n, runner.block_size, dev)
    ptrs = torch.tensor([c.data_ptr() for c in caches], dtype=torch.int64, device=dev)
    lmcache_ops.multi_layer_kv_transfer(kv, ptrs, sm, dev, slots, False, mla,
                                        layers=None if dev.type == "cuda" else list(caches))


class DisaggCoordinator:
    """Glue between an engine and its :class:`P2PKVConnector`."""

    def __init__(self, engine, connector, recv_timeout_s: float = 30.0):
        self.engine = engine
        self.connector = connector
        self.recv_timeout_s = recv_timeout_s
        self.stats = {"sent": 0, "injected": 0, "fallback": 0}

    # -- decode instance ------------------------------------------------------------
    def on_add(self, req) -> None:
        p = req.kv_transfer_params or {}
        if not p.get("do_remote_prefill"):
            return
        from .. import envs
        n_prompt = req.num_prompt_tokens
        first = p.get("first_token") if envs.NIXL_ENABLE_FIRST_TOKEN_REUSE else None
        if first is not None:
            n = n_prompt                             # the whole prompt; next input = first token
        else:
            n = n_prompt - 1                         # the last prompt token gives the first output
        if not envs.NIXL_ENABLE_FULL_KV_TRANSFER and first is None:
            n = min(n, n_prompt // self.engine.runner.block_size * self.engine.runner.block_size)
        if n <= 0:
            return
        kv = self.connector.recv_tensor(p.get("remote_request_id", req.request_id),
                                        p.get("remote"), timeout_s=self.recv_timeout_s)
        sched = self.engine.scheduler
        if kv is None or kv.shape[-2] < n:
            self.stats["fallback"] += 1
            return                                   # local prefill
        if first is not None:
            req.prompt_token_ids.append(int(first))
            self.stats["first_token_reused"] = self.stats.get("first_token_reused", 0) + 1
        blocks = sched.kv.allocate_slots(req, n)
        if blocks is None:
            self.stats["fallback"] += 1
            return
        inject_kv(self.engine.runner, req.block_ids, kv[..., :n, :])
        req.num_computed_tokens = n
        req.num_cached_tokens = n
        self.stats["injected"] += 1

    # -- prefill instance -------------------------------------------------------------
    def before_free(self, req) -> None:
        """Called when a request finishes, while its blocks are still allocated."""
        p = req.kv_transfer_params or {}
        if not p.get("do_remote_decode") or not req.block_ids:
            return
        n = min(req.num_prompt_tokens, req.num_computed_tokens)
        kv = extract_kv(self.engine.runner, req.block_ids, n)
        if kv.is_cuda:
            torch.cuda.current_stream().synchronize()
        self.connector.send_tensor(req.request_id, kv.cpu() if self.connector.device.type == "cpu"
                                   else kv, p.get("remote", ""))
        self.stats["sent"] += 1
        from .. import envs
        out = {"do_remote_prefill": True, "do_remote_decode": False,
               "remote": getattr(self.connector, "addr", None),
               "remote_request_id": req.request_id, "num_tokens": n,
               "tp_size": self.engine.cfg.parallel.tensor_parallel_size, "first_token": None}
        if envs.NIXL_ENABLE_FIRST_TOKEN_REUSE and req.output_token_ids:
            out["first_token"] = int(req.output_token_ids[0])
        req.kv_transfer_params_out = out
