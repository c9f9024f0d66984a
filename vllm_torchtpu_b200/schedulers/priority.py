"""Priority admission: the waiting request with the smallest ``priority`` value is admitted first (ties by
arrival), and when the KV cache runs out the running request with the largest value is preempted first (the
base scheduler's victim rule).  ``priority`` comes with the request (``LLMEngine.add_request(..., priority=)``,
``"priority"`` in the server's request body); the upstream engine's ``--scheduling-policy priority``."""
from __future__ import annotations

from ..engine.scheduler import Scheduler


class PriorityScheduler(Scheduler):
    def _select_waiting(self):
        if not self.waiting:
            return None
        return min(self.waiting, key=lambda r: (r.priority, r.arrival_time))
