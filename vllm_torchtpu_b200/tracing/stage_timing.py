"""Non-blocking stage timers: CUDA events recorded around a stage and read back only
once complete, so timing a step never synchronises the device
(reference: src/vllm_torchtpu/runner/stage_timing.py:35-89)."""
from __future__ import annotations

from collections import defaultdict, deque

import torch


class RunnerStageTiming:
    def __init__(self, keep: int = 1024):
        self._open: dict = {}
        self._pending: deque = deque()
        self.samples = defaultdict(lambda: deque(maxlen=keep))

    def start(self, stage: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._open[stage] = ev

    def stop(self, stage: str) -> None:
        start = self._open.pop(stage, None)
        if start is None:
            return
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        self._pending.append((stage, start, end))

    def drain(self) -> None:
        """Collect finished measurements without waiting for unfinished ones."""
        while self._pending and self._pending[0][2].query():
            stage, a, b = self._pending.popleft()
            self.samples[stage].append(a.elapsed_time(b))

    def summary(self) -> dict:
        self.drain()
        out = {}
        for k, v in self.samples.items():
            if v:
                s = sorted(v)
                out[k] = {"n": len(s), "p50_ms": s[len(s) // 2], "max_ms": s[-1]}
        return out
