"""Start/stop profiling sessions (the ``/start_profile`` / ``/stop_profile`` RPC surface,
reference: src/vllm_torchtpu/worker/tpu_worker.py:715-818, profiler_trace.py:14-33).

Options come from the profile prefix ``key:value;key:value`` (reference:
src/vllm_torchtpu/tracing/options.py:48-80): ``dir``, ``python`` (0/1 with_stack),
``shapes`` (0/1), ``memory`` (0/1).  Each rank writes ``<dir>/rank_<N>/trace.json``.
The phase-based profiler captures one trace per inference phase, picked from the batch
composition of the steps it sees (reference: src/vllm_torchtpu/runner/utils.py:63-415)."""
from __future__ import annotations

import os
import time

import torch

from .. import envs
from . import annotation


def parse_profile_options(prefix: str) -> dict:
    opts = {"dir": envs.B200_PROFILE_DIR or "/tmp/b200_profile", "python": False, "shapes": False,
            "memory": False}
    for part in (prefix or "").split(";"):
        if ":" not in part:
            continue
        k, v = part.split(":", 1)
        k, v = k.strip(), v.strip()
        if k == "dir":
            opts["dir"] = v
        elif k in ("python", "shapes", "memory"):
            opts[k] = v.lower() in ("1", "true", "yes")
        else:
            raise ValueError(f"unknown profile option {k!r}")
    return opts


class ProfileSession:
    def __init__(self, opts: dict, rank: int = 0):
        self.out_dir = os.path.join(opts["dir"], f"rank_{rank}")
        os.makedirs(self.out_dir, exist_ok=True)
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self.prof = torch.profiler.profile(activities=acts, with_stack=opts["python"],
                                           record_shapes=opts["shapes"], profile_memory=opts["memory"])
        self.prof.__enter__()
        annotation.set_active(True)
        self.t0 = time.time()

    def stop(self) -> str:
        annotation.set_active(False)
        self.prof.__exit__(None, None, None)
        path = os.path.join(self.out_dir, f"trace_{int(self.t0)}.json")
        self.prof.export_chrome_trace(path)
        return path


def start_profile(prefix: str = "") -> ProfileSession:
    return ProfileSession(parse_profile_options(prefix), int(os.environ.get("RANK", "0")))


def classify_phase(num_prefill_tokens: int, num_decode_tokens: int) -> str:
    total = num_prefill_tokens + num_decode_tokens
    if total == 0:
        return "idle"
    frac = num_prefill_tokens / total
    if frac >= 0.8:
        return "prefill_heavy"
    if frac <= 0.2:
        return "decode_heavy"
    return "balanced"


class PhaseBasedProfiler:
    """Captures ``steps_per_phase`` steps of each phase once, then stays out of the way."""

    def __init__(self, out_dir: str, steps_per_phase: int = 5):
        self.out_dir, self.steps = out_dir, steps_per_phase
        self.done: set = set()
        self.current = None
        self.session = None
        self.left = 0
        self.stats = {"prefill_heavy": 0, "decode_heavy": 0, "balanced": 0, "idle": 0}

    def on_step(self, num_prefill_tokens: int, num_decode_tokens: int) -> None:
        phase = classify_phase(num_prefill_tokens, num_decode_tokens)
        self.stats[phase] += 1
        if self.session is not None:
            self.left -= 1
            if self.left <= 0 or phase != self.current:
                self.session.stop()
                self.done.add(self.current)
                self.session, self.current = None, None
            return
        if phase != "idle" and phase not in self.done:
            self.current, self.left = phase, self.steps
            self.session = ProfileSession({"dir": os.path.join(self.out_dir, phase), "python": False,
                                           "shapes": False, "memory": False},
                                          int(os.environ.get("RANK", "0")))
