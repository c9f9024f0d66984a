"""Prompt-lookup (n-gram) drafter: find the most recent earlier occurrence of the last n tokens
and propose what followed it.  Pure host code, vectorised with numpy (the reference uses vLLM's
numba n-gram proposer, reference: src/vllm_torchtpu/runner/tpu_runner.py:88,706)."""
from __future__ import annotations

import numpy as np


def find_ngram_continuation(tokens: np.ndarray, n_min: int, n_max: int, k: int) -> list:
    L = len(tokens)
    for n in range(min(n_max, L - 1), n_min - 1, -1):
        if n <= 0 or L < n + 1:
            continue
        pat = tokens[L - n:]
        # windows ending before the last position
        win = np.lib.stride_tricks.sliding_window_view(tokens[:L - 1], n)
        hits = np.nonzero((win == pat).all(axis=1))[0]
        if hits.size:
            start = int(hits[-1]) + n
            cont = tokens[start:start + k]
            if cont.size:
                return cont.tolist()
    return []


class NgramProposer:
    def __init__(self, num_speculative_tokens: int, n_min: int = 2, n_max: int = 4, suffix: bool = False):
        self.num_speculative_tokens = num_speculative_tokens
        self.n_min, self.n_max = n_min, (n_max if not suffix else 16)
        self.stats = {"proposed": 0, "requests": 0}

    def propose(self, out, sampled: dict) -> dict:
        """Drafts for every request that just produced a token and keeps decoding."""
        drafts = {}
        for s in out.scheduled:
            req = s.request
            if req.request_id not in sampled or req.status.finished:
                continue
            toks = np.asarray(req.all_token_ids + list(sampled[req.request_id]), dtype=np.int64)
            room = req.sampling_params.max_tokens - len(req.output_token_ids) - len(sampled[req.request_id]) - 1
            k = min(self.num_speculative_tokens, max(0, room))
            if k <= 0:
                continue
            d = find_ngram_continuation(toks, self.n_min, self.n_max, k)
            if d:
                drafts[req.request_id] = d
                self.stats["proposed"] += len(d)
            self.stats["requests"] += 1
        return drafts
