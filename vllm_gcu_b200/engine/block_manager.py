"""Paged KV-cache block pool with automatic prefix caching.

A block holds ``block_size`` tokens.  Full blocks are content-addressed by a
chained hash ``h_i = hash(h_{i-1}, tokens_i, extra)`` so a new request can reuse
the longest cached prefix; blocks with reference count zero stay in the hash
table on an LRU free list until their memory is needed.

The reference obtains the same capability from upstream vLLM's KV-cache manager
(automatic prefix caching is listed as functional in
docs/source/user_guide/support_matrix/supported_features.md:11-64); the async
scheduler only caches tokens whose ids are known
(vllm_gcu/v1/core/sched/async_scheduler.py:550-554), which ``cache_full_blocks``
honours through its ``num_tokens`` argument.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Optional, Sequence


@dataclass
class Block:
    block_id: int
    ref_cnt: int = 0
    block_hash: Optional[int] = None


def hash_block(parent: Optional[int], tokens: Sequence[int], extra: tuple = ()) -> int:
    return hash((parent, tuple(tokens), extra))


class BlockPool:
    def __init__(self, num_blocks: int, block_size: int, enable_prefix_caching: bool = True):
        assert num_blocks > 0
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.enable_prefix_caching = enable_prefix_caching
        self.blocks = [Block(i) for i in range(num_blocks)]
        # LRU order: front = evict first.  Holds every block with ref_cnt == 0.
        self.free: "OrderedDict[int, None]" = OrderedDict((i, None) for i in range(num_blocks))
        self.cached: dict[int, int] = {}            # block hash -> block id
        self.hits = 0
        self.queries = 0

    # -- queries -----------------------------------------------------------
    @property
    def num_free_blocks(self) -> int:
        return len(self.free)

    @property
    def usage(self) -> float:
        return 1.0 - len(self.free) / self.num_blocks

    def blocks_needed(self, num_tokens: int, have: int) -> int:
        return max(0, -(-num_tokens // self.block_size) - have)

    # -- prefix cache --------------------------------------------------------
    def block_hashes(self, token_ids: Sequence[int], extra: tuple = ()) -> list[int]:
        bs = self.block_size
        out: list[int] = []
        parent: Optional[int] = None
        for i in range(len(token_ids) // bs):
            parent = hash_block(parent, token_ids[i * bs:(i + 1) * bs], extra)
            out.append(parent)
        return out

    def find_cached_prefix(self, token_ids: Sequence[int], extra: tuple = ()) -> list[int]:
        """Block ids of the longest cached prefix, never covering the last token (the
        model must compute at least one token to produce logits)."""
        if not self.enable_prefix_caching:
            return []
        self.queries += 1
        usable = (len(token_ids) - 1) // self.block_size
        ids: list[int] = []
        for h in self.block_hashes(token_ids, extra)[:usable]:
            bid = self.cached.get(h)
            if bid is None:
                break
            ids.append(bid)
        if ids:
            self.hits += 1
        return ids

    def touch(self, block_ids: Sequence[int]) -> None:
        """Takes a reference on blocks (removing them from the free list if idle)."""
        for bid in block_ids:
            b = self.blocks[bid]
            if b.ref_cnt == 0:
                self.free.pop(bid, None)
            b.ref_cnt += 1

    # -- allocation ----------------------------------------------------------
    def allocate(self, n: int) -> Optional[list[int]]:
        if n > len(self.free):
            return None
        out = []
        for _ in range(n):
            bid, _ = self.free.popitem(last=False)
            b = self.blocks[bid]
            if b.block_hash is not None:            # evict from the prefix cache
                if self.cached.get(b.block_hash) == bid:
                    del self.cached[b.block_hash]
                b.block_hash = None
            b.ref_cnt = 1
            out.append(bid)
        return out

    def release(self, block_ids: Sequence[int]) -> None:
        """Drops one reference per block; tail blocks are freed first so that the
        head of a prefix outlives its tail in the LRU order."""
        for bid in reversed(list(block_ids)):
            b = self.blocks[bid]
            assert b.ref_cnt > 0, f"double free of block {bid}"
            b.ref_cnt -= 1
            if b.ref_cnt == 0:
                if b.block_hash is not None:
                    self.free[bid] = None            # most recently used end
                else:
                    self.free[bid] = None
                    self.free.move_to_end(bid, last=False)  # uncached: reuse first

    def cache_full_blocks(self, block_ids: Sequence[int], token_ids: Sequence[int],
                          num_tokens: int, extra: tuple = ()) -> None:
        """Registers every full block among the first ``num_tokens`` tokens."""
        if not self.enable_prefix_caching:
            return
        nfull = min(num_tokens, len(token_ids)) // self.block_size
        parent: Optional[int] = None
        bs = self.block_size
        for i in range(nfull):
            b = self.blocks[block_ids[i]]
            if b.block_hash is not None:
                parent = b.block_hash
                continue
            h = hash_block(parent, token_ids[i * bs:(i + 1) * bs], extra)
            parent = h
            if h not in self.cached:
                self.cached[h] = b.block_id
                b.block_hash = h

    def reset_prefix_cache(self) -> bool:
        if any(b.ref_cnt > 0 for b in self.blocks):
            return False
        for b in self.blocks:
            b.block_hash = None
        self.cached.clear()
        return True


class KVCacheManager:
    """Per-request block bookkeeping on top of a :class:`BlockPool`."""

    def __init__(self, num_blocks: int, block_size: int, enable_prefix_caching: bool = True,
                 watermark_blocks: int = 0):
        self.pool = BlockPool(num_blocks, block_size, enable_prefix_caching)
        self.block_size = block_size
        self.watermark = watermark_blocks

    @staticmethod
    def _extra(req) -> tuple:
        """What besides the token ids identifies a block's content: the LoRA adapter and the
        salt of multimodal requests (same placeholder ids, different image)."""
        salt = getattr(req, "cache_salt", None)
        if salt is not None:
            return (req.lora_id, salt)
        return (req.lora_id,) if req.lora_id >= 0 else ()

    def get_computed_blocks(self, req) -> tuple[list[int], int]:
        extra = self._extra(req)
        ids = self.pool.find_cached_prefix(req.all_token_ids, extra)
        return ids, len(ids) * self.block_size

    def allocate_slots(self, req, num_new_tokens: int,
                       new_computed_blocks: Sequence[int] = (),
                       num_lookahead_tokens: int = 0) -> Optional[list[int]]:
        """Makes sure ``req`` owns blocks for ``num_computed + num_new (+ lookahead)``
        tokens.  Returns the newly appended block ids, or None when the pool cannot
        supply them (nothing is changed in that case)."""
        if not new_computed_blocks and (req.num_computed_tokens + num_new_tokens
                                        + num_lookahead_tokens) <= len(req.block_ids) * self.block_size:
            return []                       # the blocks already owned cover this step
        num_computed = req.num_computed_tokens + len(new_computed_blocks) * self.block_size \
            if new_computed_blocks else req.num_computed_tokens
        total = num_computed + num_new_tokens + num_lookahead_tokens
        have = len(req.block_ids) + len(new_computed_blocks)
        need = self.pool.blocks_needed(total, have)
        idle_hits = sum(1 for b in new_computed_blocks if self.pool.blocks[b].ref_cnt == 0)
        if need + idle_hits > self.pool.num_free_blocks - (self.watermark if not req.block_ids
                                                            else 0):
            return None
        if new_computed_blocks:
            self.pool.touch(new_computed_blocks)
            req.block_ids.extend(new_computed_blocks)
        new_ids = self.pool.allocate(need) if need else []
        assert new_ids is not None
        req.block_ids.extend(new_ids)
        return list(new_computed_blocks) + new_ids

    def cache_blocks(self, req, num_tokens: int) -> None:
        """Registers the full blocks among the first ``num_tokens`` tokens of ``req``.
        Incremental: only blocks completed since the previous call are hashed."""
        pool = self.pool
        if not pool.enable_prefix_caching:
            return
        bs = self.block_size
        nfull = min(num_tokens, req.num_tokens) // bs
        done = getattr(req, "_hashed_blocks", 0)
        if nfull <= done:
            return
        extra = self._extra(req)
        parent = getattr(req, "_last_hash", None)
        if done == 0:
            parent = None
        npt = req.num_prompt_tokens
        for i in range(done, nfull):
            a, b = i * bs, (i + 1) * bs
            if b <= npt:
                toks = req.prompt_token_ids[a:b]
            elif a >= npt:
                toks = req.output_token_ids[a - npt:b - npt]
            else:
                toks = req.prompt_token_ids[a:] + req.output_token_ids[:b - npt]
            blk = pool.blocks[req.block_ids[i]]
            if blk.block_hash is not None:
                parent = blk.block_hash
                continue
            h = hash_block(parent, toks, extra)
            parent = h
            if h not in pool.cached:
                pool.cached[h] = blk.block_id
                blk.block_hash = h
        req._hashed_blocks = nfull
        req._last_hash = parent

    def free(self, req) -> None:
        self.pool.release(req.block_ids)
        req.block_ids = []
        req._hashed_blocks = 0
        req._last_hash = None

    @property
    def usage(self) -> float:
        return self.pool.usage
