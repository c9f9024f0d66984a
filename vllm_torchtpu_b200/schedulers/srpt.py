"""Shortest-remaining-prefill-first admission with a hold-back budget: short
prompts jump ahead of long ones (lower mean TTFT), but a request that has been
passed over ``max_skips`` times is admitted next regardless, so long prompts do
not starve (reference: src/vllm_torchtpu/core/experimental/srpt_prefill_scheduler.py)."""
from __future__ import annotations

from .. import envs
from ..engine.scheduler import Scheduler


class SrptPrefillScheduler(Scheduler):
    max_skips = 16

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self._skips: dict = {}
        self.hold_back = envs.B200_SRPT_HOLD_BACK

    def _select_waiting(self):
        if not self.waiting:
            return None
        starving = [r for r in self.waiting if self._skips.get(r.request_id, 0) >= self.max_skips]
        if starving:
            pick = starving[0]
        else:
            pick = min(self.waiting, key=lambda r: (r.num_tokens - r.num_computed_tokens, r.arrival_time))
        for r in self.waiting:
            if r is not pick and r.arrival_time < pick.arrival_time:
                self._skips[r.request_id] = self._skips.get(r.request_id, 0) + 1
        self._skips.pop(pick.request_id, None)
        return pick

    def _may_admit_prefill(self, req, budget: int) -> bool:
        # keep `hold_back` tokens of every step's budget for decodes that arrive later in the step
        return budget > self.hold_back
