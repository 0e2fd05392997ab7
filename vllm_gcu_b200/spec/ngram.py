"""Prompt-lookup (n-gram) proposer: the draft continues the most recent earlier occurrence
of the current suffix of the sequence (the reference's ``[ngram]`` speculative method,
models/qwen/qwen.md:9-30, legacy runner vllm_gcu/v1/worker/gcu_model_runner.py:1111-1144)."""
from __future__ import annotations

from typing import Sequence

import numpy as np


class NgramProposer:
    def __init__(self, num_speculative_tokens: int, max_n: int = 4, min_n: int = 1):
        assert 1 <= min_n <= max_n
        self.k = num_speculative_tokens
        self.max_n, self.min_n = max_n, min_n

    def propose(self, token_ids: Sequence[int]) -> list[int]:
        """Longest suffix (length max_n .. min_n) that occurred before; returns the up to ``k``
        tokens that followed its latest earlier occurrence, or [] when nothing matches."""
        arr = np.asarray(token_ids, dtype=np.int64)
        L = arr.shape[0]
        for n in range(min(self.max_n, L - 1), self.min_n - 1, -1):
            suffix = arr[L - n:]
            # candidate start positions of earlier occurrences: windows [i, i + n), i + n < L
            limit = L - n
            if limit <= 0:
                continue
            windows = np.lib.stride_tricks.sliding_window_view(arr[: L - 1], n)
            hits = np.nonzero((windows == suffix).all(axis=1))[0]
            hits = hits[hits + n <= L - 1]
            if hits.size == 0:
                continue
            start = int(hits[-1]) + n
            out = arr[start:start + self.k]
            if out.size:
                return [int(t) for t in out]
        return []
