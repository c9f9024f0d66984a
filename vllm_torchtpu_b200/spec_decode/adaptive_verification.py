"""Adaptive draft verification: how many of the proposed draft tokens a step verifies.

Every draft slot is scored by its survival probability, the running product of the drafter's
per-position confidences.  A step verifies the globally best ``budget`` slots, with the budget
chosen to maximise expected emitted tokens per millisecond under a table of step costs measured
at start-up.  Survival only falls along a request, so each request keeps a prefix of its drafts
and verification stays lossless: the trimmed drafts are simply never proposed.  Under data-parallel
lockstep every rank pads to the largest rank's token count, so once that count is agreed a rank
re-admits its best trimmed drafts into the padding (``expand``).
(reference: src/vllm_torchtpu/spec_decode/adaptive_verification.py:14-530)
"""
from __future__ import annotations

import bisect
from dataclasses import dataclass, field
from typing import Optional, Sequence

_OVERHEAD_EMA = 0.05     # smoothing of the measured per-step time that the table leaves out
_STALL_FACTOR = 4.0      # a step this many times slower (or faster) than predicted is not calibrated against


def validate_adaptive_verification_config(cfg) -> None:
    """Adaptive verification needs the drafter's confidences and one batch layout on every rank
    that runs the model: it excludes LoRA steps and pipeline parallelism."""
    sc = getattr(cfg, "speculative", None) or {}
    if not sc.get("enable_adaptive_verification"):
        return
    if getattr(cfg, "enable_lora", False):
        raise ValueError("adaptive verification is not compatible with LoRA; pass "
                         "enable_adaptive_verification=false in the speculative config")
    if getattr(cfg.parallel, "pipeline_parallel_size", 1) > 1:
        raise ValueError("adaptive verification is not compatible with pipeline parallelism")
    if sc.get("method", "ngram") in ("ngram", "suffix"):
        raise ValueError("adaptive verification needs a drafter that reports confidences (eagle3, mtp, "
                         "dflash, dspark)")


class StepCostTable:
    """Step time in milliseconds as a function of the number of token rows in the step, from
    (rows, ms) samples; linear between samples, flat beyond the ends' slope."""

    def __init__(self, samples: Sequence[tuple]):
        pts = sorted((int(n), float(ms)) for n, ms in samples)
        if not pts:
            raise ValueError("StepCostTable needs at least one sample")
        self.rows = [n for n, _ in pts]
        self.ms = [m for _, m in pts]

    @classmethod
    def profile(cls, run_step, row_counts: Sequence[int], repeats: int = 3) -> "StepCostTable":
        """``run_step(rows)`` runs one decode-shaped step of that many rows and returns its time in ms."""
        samples = []
        for n in row_counts:
            times = sorted(run_step(n) for _ in range(repeats))
            samples.append((n, times[len(times) // 2]))
        return cls(samples)

    def cost(self, rows: int) -> float:
        r, m = self.rows, self.ms
        if len(r) == 1:
            return m[0]
        i = bisect.bisect_left(r, rows)
        i = min(max(i, 1), len(r) - 1)
        x0, x1, y0, y1 = r[i - 1], r[i], m[i - 1], m[i]
        return max(0.0, y0 + (y1 - y0) * (rows - x0) / max(1, x1 - x0))


@dataclass
class AdaptiveVerificationManager:
    cost_table: StepCostTable
    max_drafts_per_request: int
    overhead_ms: float = 0.0
    stats: dict = field(default_factory=lambda: {"proposed": 0, "verified": 0, "steps": 0})

    @staticmethod
    def survival(confidences: Sequence[float]) -> list:
        out, p = [], 1.0
        for c in confidences:
            p *= min(1.0, max(0.0, float(c)))
            out.append(p)
        return out

    def select(self, confidences: dict, base_rows: Optional[int] = None) -> dict:
        """``confidences[request_id]`` = the drafter's probability of each proposed token, in order.
        Returns how many leading drafts of each request to verify."""
        reqs = list(confidences)
        n_req = len(reqs)
        base = n_req if base_rows is None else base_rows       # one target row per request without drafts
        slots = []
        for rid in reqs:
            for pos, s in enumerate(self.survival(confidences[rid][: self.max_drafts_per_request])):
                slots.append((s, rid, pos))
        slots.sort(key=lambda t: -t[0])
        best_b, best_rate, gain = 0, n_req / max(1e-9, self.cost_table.cost(base) + self.overhead_ms), 0.0
        for b, (s, _, _) in enumerate(slots, start=1):
            gain += s
            rate = (n_req + gain) / max(1e-9, self.cost_table.cost(base + b) + self.overhead_ms)
            if rate > best_rate:
                best_b, best_rate = b, rate
        keep = {rid: 0 for rid in reqs}
        for s, rid, pos in slots[:best_b]:
            keep[rid] = max(keep[rid], pos + 1)       # survival falls along a request: a prefix
        self.stats["proposed"] += len(slots)
        self.stats["verified"] += sum(keep.values())
        self.stats["steps"] += 1
        return keep

    def expand(self, keep: dict, confidences: dict, extra_rows: int) -> dict:
        """Re-admit the best trimmed drafts into ``extra_rows`` of padding that the step runs anyway."""
        keep = dict(keep)
        while extra_rows > 0:
            best, best_s = None, -1.0
            for rid, conf in confidences.items():
                k = keep.get(rid, 0)
                if k < min(len(conf), self.max_drafts_per_request):
                    s = self.survival(conf[: k + 1])[-1]
                    if s > best_s:
                        best, best_s = rid, s
            if best is None:
                break
            keep[best] = keep.get(best, 0) + 1
            extra_rows -= 1
        return keep

    def trim(self, drafts: dict, confidences: dict, base_rows: Optional[int] = None) -> dict:
        """Drafts (request id -> token list) cut to the selected prefixes; requests whose drafter gave
        no confidences keep all their drafts."""
        scored = {rid: confidences[rid] for rid in drafts if rid in confidences}
        keep = self.select(scored, base_rows)
        out = {}
        for rid, toks in drafts.items():
            toks = list(toks)[: keep[rid]] if rid in keep else list(toks)
            if toks:
                out[rid] = toks
        return out

    def observe(self, rows: int, measured_ms: float) -> None:
        """Calibrate the per-step overhead that the table does not contain (host work, sampling)."""
        predicted = self.cost_table.cost(rows) + self.overhead_ms
        if predicted <= 0 or measured_ms > _STALL_FACTOR * predicted or measured_ms * _STALL_FACTOR < predicted:
            return
        self.overhead_ms += _OVERHEAD_EMA * (measured_ms - predicted)
        self.overhead_ms = max(0.0, self.overhead_ms)
