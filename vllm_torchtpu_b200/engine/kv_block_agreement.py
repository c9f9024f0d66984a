"""Agreement on the KV block count across the ranks of an engine.

Every rank profiles its own free memory, so the counts differ by a few blocks.  The ranks of one pipeline
stage hold the same layers and must end up with the same count: the stage takes its minimum, but a spread
beyond the tolerance (4 blocks or 0.5 %, whichever is larger) means the ranks do not see the same model or
the same memory, which is reported instead of being papered over.  Stages hold different layers, so their
counts are compared only after each has settled; the engine uses the minimum over stages because the
scheduler addresses every stage with one block table.
(reference: src/vllm_torchtpu/executors/kv_block_override.py:37-134)"""
from __future__ import annotations

ABS_TOLERANCE = 4
REL_TOLERANCE = 0.005


def within_tolerance(counts, abs_tol: int = ABS_TOLERANCE, rel_tol: float = REL_TOLERANCE) -> bool:
    lo, hi = min(counts), max(counts)
    return hi - lo <= max(abs_tol, int(rel_tol * hi))


def reconcile(counts_by_rank: dict, stage_of_rank: dict, abs_tol: int = ABS_TOLERANCE,
              rel_tol: float = REL_TOLERANCE) -> int:
    """counts_by_rank: rank -> profiled block count; stage_of_rank: rank -> pipeline stage.  Returns the
    count every rank adopts; raises ``ValueError`` naming the stage whose ranks disagree."""
    if not counts_by_rank:
        raise ValueError("no block counts to reconcile")
    stages: dict = {}
    for rank, n in counts_by_rank.items():
        stages.setdefault(stage_of_rank.get(rank, 0), {})[rank] = int(n)
    settled = []
    for stage in sorted(stages):
        per_rank = stages[stage]
        if not within_tolerance(list(per_rank.values()), abs_tol, rel_tol):
            raise ValueError(f"pipeline stage {stage}: ranks profiled KV block counts {per_rank} that differ by "
                             f"more than max({abs_tol}, {rel_tol:.1%}); they do not hold the same layers or "
                             "do not see the same free memory")
        settled.append(min(per_rank.values()))
    return min(settled)


def agree_over_group(num_blocks: int, rank: int, stage: int, cpu_group) -> int:
    """Collective form: gathers (rank, stage, count) over the gloo group and reconciles."""
    import torch.distributed as dist
    every = [None] * dist.get_world_size(group=cpu_group)
    dist.all_gather_object(every, (rank, stage, int(num_blocks)), group=cpu_group)
    return reconcile({r: n for r, _, n in every}, {r: s for r, s, _ in every})
