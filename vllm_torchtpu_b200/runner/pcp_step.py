"""Prefill context parallelism inside the engine.

The ranks of a PCP group hold the same model and are handed the same requests.  A long prefill chunk is cut
into 2P pieces and rank r computes pieces r and 2P-1-r (the head-tail split that equalises causal work,
``parallel/pcp.py`` ``HeadTailPlan``): each piece enters the step as a request of its own - same block table,
``seq_len`` = end of the piece, ``q_len`` = its length - so the paged attention kernels need nothing new.  What
the pieces of the other ranks contribute is their keys and values: in every attention layer the k / v columns
of the local QKV projection are all-gathered, appended behind the local rows (with empty queries) and the
usual RoPE + cache-write kernel stores them into this rank's pages, so every rank's cache ends up complete and
decode steps run on any of them without communication.  Linear layers, norms and the MLP run on a rank's own
tokens only: prefill compute is divided by P.

The piece that ends a chunk is always on rank 0 (it owns piece 2P-1), so the hidden state of a chunk's last
token - the row that is sampled - is broadcast from rank 0 to the rows that stand in for it on the other
ranks; every rank then samples the same token and the schedulers stay in step.

Decode tokens and chunks shorter than ``min_tokens`` are computed by every rank (replicated): they are too
small to split.  Requests that read all their prompt rows (prompt logprobs, pooling, multimodal items,
speculative drafts) are replicated too.
(reference: src/vllm_torchtpu/runner/pcp/manager.py:136-206, runner/pcp/head_tail_sharding_plan.py,
layers/core/pcp_sequence_layout.py, pcp_workspace.py - there the KV of remote pieces is streamed through a
workspace and attention runs over it; here the cache itself is completed)"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

import numpy as np
import torch


def piece_bounds(lo: int, n: int, P: int) -> list:
    """2P consecutive pieces of [lo, lo + n), sizes differing by at most one, none empty for n >= 2P."""
    return [(lo + i * n // (2 * P), lo + (i + 1) * n // (2 * P)) for i in range(2 * P)]


def splittable(s) -> bool:
    sp = s.request.sampling_params
    return not (s.spec_token_ids or sp.prompt_logprobs is not None or sp.pooling)


@dataclass
class PcpStepPlan:
    counts: list                 # split tokens per rank
    own: int                     # this rank's split tokens: the last rows of its token list
    others_idx: torch.Tensor     # rows of the gathered [P * max(counts)] buffer held by other ranks
    others_pos: torch.Tensor     # their positions (int32)
    others_slots: torch.Tensor   # their cache slots (int32)
    mute: list                   # local pieces that end no chunk: they sample nothing and store no token
    fix: list                    # local pieces that stand in for a chunk's end: their sampling row is rank 0's
    mute_rows: Optional[list] = None             # rows of the two lists in the step's request order, filled by
    fix_rows: Optional[torch.Tensor] = None      # ``bind_rows`` once the runner has ordered the requests

    @property
    def max_count(self) -> int:
        return max(self.counts)


def split_step(scheds: list, P: int, rank: int, min_tokens: int, slot_of: dict, block_table, block_size: int,
               device, has_mm=lambda rid: False):
    """(local request list, plan) for one step, or (scheds, None) when nothing is worth splitting.  The local
    list keeps the replicated requests in place and appends two pieces per split request."""
    split = [s for s in scheds if s.num_new_tokens >= max(min_tokens, 4 * P) and splittable(s)
             and not has_mm(s.request.request_id)]
    if not split:
        return scheds, None
    ids = {id(s) for s in split}
    local = [s for s in scheds if id(s) not in ids]
    per_rank_pos, per_rank_slot = [[] for _ in range(P)], [[] for _ in range(P)]
    mute, fix = [], []
    for s in split:
        b = piece_bounds(s.start, s.num_new_tokens, P)
        row = block_table[slot_of[s.request.request_id]]
        for r in range(P):
            for lo, hi in (b[r], b[2 * P - 1 - r]):
                pos = np.arange(lo, hi, dtype=np.int64)
                per_rank_pos[r].append(pos)
                per_rank_slot[r].append(row[pos // block_size].astype(np.int64) * block_size + pos % block_size)
        (h_lo, h_hi), (t_lo, t_hi) = b[rank], b[2 * P - 1 - rank]
        head = replace(s, start=h_lo, num_new_tokens=h_hi - h_lo, samples=False, is_new=False, new_block_ids=[])
        # the second piece stands in for the chunk's end on every rank (rank 0 really holds it)
        tail = replace(s, start=t_lo, num_new_tokens=t_hi - t_lo, is_new=False, new_block_ids=[])
        mute.append(head)
        fix.append(tail)
        local += [head, tail]
    pos = [np.concatenate(p) for p in per_rank_pos]
    slots = [np.concatenate(p) for p in per_rank_slot]
    counts = [len(p) for p in pos]
    mx = max(counts)
    others = [r for r in range(P) if r != rank]
    idx = np.concatenate([r * mx + np.arange(counts[r]) for r in others]) if others else np.zeros(0, np.int64)
    t32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(device)       # noqa: E731
    plan = PcpStepPlan(counts, counts[rank], torch.from_numpy(idx).to(device),
                       t32(np.concatenate([pos[r] for r in others])), t32(np.concatenate([slots[r] for r in others])),
                       mute, fix)
    return local, plan


def bind_rows(plan: PcpStepPlan, ordered: list, device) -> None:
    """``ordered``: the step's requests in the order the runner laid them out (decodes first)."""
    where = {id(s): i for i, s in enumerate(ordered)}
    plan.mute_rows = [where[id(s)] for s in plan.mute]
    plan.fix_rows = torch.tensor([where[id(s)] for s in plan.fix], dtype=torch.long, device=device)


def gather_remote_kv(plan: PcpStepPlan, qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                     q_width: int, num_tokens: int, comm):
    """qkv [T_pad, q_width + kv_width] of the local rows -> (extended qkv, positions, slots): the local rows
    followed by the other ranks' split rows, whose query columns are zero and whose k / v columns come from an
    all-gather.  ``num_tokens`` local rows are real; the split ones are the last ``plan.own`` of them."""
    T = num_tokens
    kv_own = qkv[T - plan.own:T, q_width:]
    if plan.own < plan.max_count:
        kv_own = torch.cat([kv_own, kv_own.new_zeros(plan.max_count - plan.own, kv_own.shape[1])])
    every = comm.all_gather(kv_own.contiguous(), dim=0)
    theirs = every.index_select(0, plan.others_idx)
    ext = torch.cat([theirs.new_zeros(theirs.shape[0], q_width), theirs], dim=1)
    return (torch.cat([qkv[:T], ext]), torch.cat([positions[:T], plan.others_pos]),
            torch.cat([slots[:T], plan.others_slots]))


def broadcast_sample_rows(plan: PcpStepPlan, h: torch.Tensor, comm):
    """Hidden states of the sampling rows: the rows of split requests take rank 0's values."""
    rows = plan.fix_rows
    part = h.index_select(0, rows).contiguous()
    part = comm.broadcast(part, src=0)
    h = h.clone()
    h[rows] = part
    return h
