"""Pipeline-parallel chunk scheduler.

A step moves through the pipeline one stage at a time, so (a) a lone prompt that
is run as one full step leaves every other stage idle, and (b) steps of equal
token count are not steps of equal time: a chunk deep inside a long prompt attends
to all tokens before it.  Two policies fix that, as in the reference
(reference: src/vllm_torchtpu/core/pp_chunks.py:14-140, core/pp_chunk_scheduler.py:61):

* lone-prompt chunking: while the pending prefill work cannot fill every stage
  with a full step, a step is held to that work spread over the stages;
* equal-cost chunking: every step gets a time budget and prefill chunks are sized
  against a cost model ``t = linear(tokens) + attn * Σ (chunk·prefix + chunk²/2)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from statistics import median
from typing import Optional, Sequence

from .. import envs
from ..engine.scheduler import Scheduler


def chunk_granularity(block_size: int, max_tokens: int, block_aligned: bool = False) -> int:
    """Chunks are cut at multiples of an eighth of a step (whole KV blocks when required)."""
    g = max(max_tokens // 8, 1)
    if block_aligned and block_size <= max_tokens:
        g = -(-g // block_size) * block_size
    return g


def step_limit(pending: int, pp_size: int, granularity: int, step: int) -> Optional[int]:
    """Token cap of a step while ``pending`` prefill tokens cannot fill all stages."""
    if pending <= 0:
        return None
    share = -(-pending // pp_size)
    if share >= step:
        return None
    return min(-(-share // granularity) * granularity, step)


@dataclass
class StepCostModel:
    """Per-stage step time model fitted from a few timed forwards."""
    linear_ms_per_token: float
    linear_ms_base: float
    attn_ms_per_pair: float          # per (chunk token x context token)
    target_ms: float

    @staticmethod
    def fit(samples: Sequence[tuple], max_tokens: int, slack: float) -> "StepCostModel":
        """``samples`` = (tokens, prefix, milliseconds).  Prefix-free samples give the linear part,
        pairs of samples of one bucket at two prefixes give the attention slope (median)."""
        free = sorted((t, ms) for t, p, ms in samples if p == 0)
        if len(free) >= 2:
            (t0, m0), (t1, m1) = free[0], free[-1]
            slope = (m1 - m0) / max(1, t1 - t0)
            base = m0 - slope * t0
        else:
            slope, base = (free[0][1] / free[0][0], 0.0) if free else (0.0, 0.0)
        slopes = []
        by_tokens: dict = {}
        for t, p, ms in samples:
            by_tokens.setdefault(t, []).append((p, ms))
        for t, pts in by_tokens.items():
            pts.sort()
            if len(pts) >= 2 and pts[-1][0] > pts[0][0]:
                slopes.append((pts[-1][1] - pts[0][1]) / (t * (pts[-1][0] - pts[0][0])))
        attn = max(0.0, median(slopes)) if slopes else 0.0
        # remove each prefix-free sample's own causal attention from the linear fit
        target = (base + slope * max_tokens + attn * max_tokens * max_tokens / 2) * (1.0 + slack)
        return StepCostModel(slope, base, attn, target)

    def cost(self, chunks: Sequence[tuple]) -> float:
        """``chunks`` = (chunk tokens, prefix tokens) of every request in the step."""
        tokens = sum(c for c, _ in chunks)
        pairs = sum(c * p + c * c / 2 for c, p in chunks)
        return self.linear_ms_base + self.linear_ms_per_token * tokens + self.attn_ms_per_pair * pairs

    def max_chunk(self, prefix: int, used: Sequence[tuple], granularity: int, cap: int) -> int:
        """Largest granule-multiple chunk behind ``prefix`` that keeps the step within target."""
        best = 0
        c = granularity
        while c <= cap:
            if self.cost(list(used) + [(c, prefix)]) > self.target_ms:
                break
            best = c
            c += granularity
        return best


class PipelineChunkScheduler(Scheduler):
    def __init__(self, *a, pp_size: int = 1, cost_model: Optional[StepCostModel] = None, **kw):
        super().__init__(*a, **kw)
        self.pp_size = pp_size
        self.cost_model = cost_model
        self.granularity = chunk_granularity(self.block_size, self.cfg.max_num_batched_tokens)
        self.lone_prompt = True
        self.equal_cost = envs.B200_PP_EQUAL_COST_CHUNKS

    def _pending_prefill(self) -> int:
        n = sum(r.num_tokens - r.num_computed_tokens for r in self.waiting)
        n += sum(max(0, r.num_prompt_tokens - r.num_computed_tokens) for r in self.running)
        return n

    def schedule(self):
        full = self.cfg.max_num_batched_tokens
        stages = envs.B200_PP_LONE_PROMPT_CHUNKS or self.pp_size
        limit = step_limit(self._pending_prefill(), stages, self.granularity, full) \
            if self.lone_prompt and self.pp_size > 1 else None
        saved_budget, saved_thr = self.cfg.max_num_batched_tokens, self.cfg.long_prefill_token_threshold
        try:
            if limit is not None:
                decodes = sum(1 for r in self.running if not r.is_prefill)
                self.cfg.max_num_batched_tokens = min(full, limit + decodes)
            if self.equal_cost and self.cost_model is not None:
                # the deepest prefix among prefilling requests bounds the chunk of this step
                deepest = max([r.num_computed_tokens for r in list(self.running) + list(self.waiting)
                               if r.is_prefill] or [0])
                cap = self.cost_model.max_chunk(deepest, [], self.granularity, self.cfg.max_num_batched_tokens)
                if cap:
                    self.cfg.long_prefill_token_threshold = cap
            return super().schedule()
        finally:
            self.cfg.max_num_batched_tokens = saved_budget
            self.cfg.long_prefill_token_threshold = saved_thr
