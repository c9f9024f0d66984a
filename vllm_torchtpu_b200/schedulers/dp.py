"""Data-parallel aware scheduler.

With DP attention + expert parallelism every DP rank must run the same padded
step shape, so one rank admitting a long prefill stalls the decodes of all the
others.  This scheduler aligns prefill admission across ranks: a rank may admit
new prefills only in steps where the group agreed to (``throttle_prefills``),
which the engine derives from a host-side MAX all-reduce of each rank's pending
prefill tokens.  Same intent as the reference's DP scheduler
(reference: src/vllm_torchtpu/core/tpu_scheduler.py:22-57).
"""
from __future__ import annotations

from ..engine.scheduler import Scheduler


class DpScheduler(Scheduler):
    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self._prefill_allowed = True
        self.prefill_interval = 1
        self._steps_since_prefill = 0

    def pending_prefill_tokens(self) -> int:
        n = sum(r.num_tokens - r.num_computed_tokens for r in self.waiting)
        n += sum(max(0, r.num_prompt_tokens - r.num_computed_tokens) for r in self.running)
        return n

    def throttle_prefills(self, group_pending: list, *, max_decode_gap: int = 4) -> None:
        """``group_pending[i]`` = pending prefill tokens of DP rank i (from the lockstep all-reduce).
        Prefills are admitted by everyone in the same steps: when any rank has prefill work and
        at least ``max_decode_gap`` decode-only steps have passed (or nothing is decoding)."""
        any_pending = any(p > 0 for p in group_pending)
        if not any_pending:
            self._prefill_allowed = True
            return
        self._steps_since_prefill += 1
        if not self.running or self._steps_since_prefill >= max_decode_gap:
            self._prefill_allowed = True
            self._steps_since_prefill = 0
        else:
            self._prefill_allowed = False

    def _may_admit_prefill(self, req, budget: int) -> bool:
        return self._prefill_allowed
