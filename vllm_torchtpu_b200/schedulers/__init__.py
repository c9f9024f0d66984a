"""Opt-in scheduling policies on top of the base continuous-batching scheduler.

Counterparts of the reference's engine-side schedulers
(reference: src/vllm_torchtpu/core/tpu_scheduler.py:22-57,
core/pp_chunk_scheduler.py:61, core/prefix_aware_scheduler.py:14-139,
core/experimental/srpt_prefill_scheduler.py)."""
from __future__ import annotations


def get_scheduler_class(name: str):
    if name == "dp":
        from .dp import DpScheduler
        return DpScheduler
    if name == "pp_chunk":
        from .pp_chunk import PipelineChunkScheduler
        return PipelineChunkScheduler
    if name == "prefix_aware":
        from .prefix_aware import PrefixAwareScheduler
        return PrefixAwareScheduler
    if name == "srpt":
        from .srpt import SrptPrefillScheduler
        return SrptPrefillScheduler
    if name == "priority":
        from .priority import PriorityScheduler
        return PriorityScheduler
    raise ValueError(f"unknown scheduler {name!r}")
