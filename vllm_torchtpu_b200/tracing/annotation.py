"""Trace annotations: ``torch.profiler.record_function`` ranges (plus NVTX when a GPU is
present) that cost nothing unless a profiling session is active
(reference: src/vllm_torchtpu/tracing/annotation.py:27-50)."""
from __future__ import annotations

import contextlib

import torch

_active = 0


def set_active(on: bool) -> None:
    global _active
    _active += 1 if on else -1
    _active = max(_active, 0)


def is_active() -> bool:
    return _active > 0


@contextlib.contextmanager
def trace_annotation(name: str, **fields):
    if not is_active():
        yield
        return
    label = name if not fields else name + " " + " ".join(f"{k}={v}" for k, v in fields.items())
    nvtx = torch.cuda.is_available()
    if nvtx:
        torch.cuda.nvtx.range_push(label)
    try:
        with torch.profiler.record_function(label):
            yield
    finally:
        if nvtx:
            torch.cuda.nvtx.range_pop()
