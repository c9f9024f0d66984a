"""Prefix-aware admission: among the first ``lookahead`` waiting requests, admit
the one with the fewest tokens that are not already in the prefix cache, so that
requests sharing a hot prefix run while it is still cached
(reference: src/vllm_torchtpu/core/prefix_aware_scheduler.py:14-139)."""
from __future__ import annotations

from itertools import islice

from ..engine.scheduler import Scheduler


class PrefixAwareScheduler(Scheduler):
    lookahead = 32

    def _uncached_tokens(self, req) -> int:
        if req.num_computed_tokens > 0 or req.block_ids:
            return req.num_tokens - req.num_computed_tokens
        pool = self.kv.pool
        q, h = pool.queries, pool.hits
        _, cached = self.kv.get_computed_blocks(req)
        pool.queries, pool.hits = q, h          # a probe is not a hit-rate sample
        return req.num_tokens - cached

    def _select_waiting(self):
        if not self.waiting:
            return None
        if not self.kv.pool.enable_caching:
            return self.waiting[0]
        window = list(islice(self.waiting, self.lookahead))
        best = min(range(len(window)), key=lambda i: (self._uncached_tokens(window[i]), i))
        return window[best]
