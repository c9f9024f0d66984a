"""Decode context parallelism: the KV cache of a sequence is sharded by position
over the DCP ranks (interleaved in units of ``interleave`` tokens), every rank
attends its shard for ALL heads, and partial results are merged by their
log-sum-exp.

Dataflow per attention layer, as in the reference
(reference: src/vllm_torchtpu/layers/adapter/cp_attention.py:274-349,
distributed/dcp_comm.py:23-104): all-gather the q heads of the DCP group →
attention over the local KV shard returning (out, lse) → all-gather lse,
weight the partial outputs, reduce-scatter them back to head shards.  The merge
is ``o = Σ_r softmax_r(lse) · o_r`` with a guard for shards that saw no key.
An all-to-all variant exchanges (out, lse) per head shard instead of
gather+reduce-scatter for small token counts.
"""
from __future__ import annotations

import torch

from .. import envs, ops
from ..ops import reference as ref
from .communicator import get_dcp_comm


def dcp_local_positions(seq_len: int, rank: int, size: int, interleave: int = 1) -> torch.Tensor:
    """Global positions of the tokens whose KV lives on ``rank``."""
    pos = torch.arange(seq_len)
    return pos[(pos // interleave) % size == rank]


def dcp_local_len(seq_len: int, rank: int, size: int, interleave: int = 1) -> int:
    full, rem = divmod(seq_len, interleave * size)
    extra = min(max(rem - rank * interleave, 0), interleave)
    return full * interleave + extra


def dcp_owner(position: int, size: int, interleave: int = 1) -> int:
    return (position // interleave) % size


def cp_lse_ag_out_rs(out: torch.Tensor, lse: torch.Tensor, comm, fp32_out: bool = True) -> torch.Tensor:
    """Merge partial attention of all DCP ranks and return this rank's head shard.

    out: [T, H_all, D] partial over the local KV shard; lse: [T, H_all] natural log.
    Returns [T, H_all / size, D]."""
    size = comm.size
    if size == 1:
        return out
    lses = comm.all_gather(lse.unsqueeze(0).contiguous(), dim=0)          # [size, T, H]
    m = lses.max(0).values
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    w_all = torch.exp(lses - m)
    w_all = torch.where(torch.isfinite(lses), w_all, torch.zeros_like(w_all))
    denom = w_all.sum(0).clamp_min(1e-38)
    w = w_all[comm.rank] / denom                                           # [T, H]
    weighted = torch.where(w[..., None] > 0, out.float() * w[..., None], torch.zeros_like(out, dtype=torch.float32))
    if not fp32_out:
        weighted = weighted.to(out.dtype)
    # reduce-scatter over the head dimension
    T, H, D = weighted.shape
    x = weighted.reshape(T, size, H // size, D).permute(1, 0, 2, 3).contiguous()   # [size, T, H/size, D]
    red = comm.reduce_scatter(x.reshape(size * T, H // size, D), dim=0)
    return red.reshape(T, H // size, D).to(out.dtype)


def cp_lse_a2a(out: torch.Tensor, lse: torch.Tensor, comm) -> torch.Tensor:
    """All-to-all variant: every rank receives all partials of its head shard and merges them locally."""
    size = comm.size
    T, H, D = out.shape
    o = comm.all_to_all(out.reshape(T, size, H // size, D).permute(1, 0, 2, 3).contiguous(), 0, 0)
    l = comm.all_to_all(lse.reshape(T, size, H // size).permute(1, 0, 2).contiguous(), 0, 0)
    o = o.reshape(size, T, H // size, D)
    l = l.reshape(size, T, H // size)
    merged, _ = ref.merge_attn_states([o[i] for i in range(size)], [l[i] for i in range(size)])
    return merged


def dcp_attention(layer, q: torch.Tensor, kv_cache: torch.Tensor, meta) -> torch.Tensor:
    """q: [T, Hq_local, D] (this TP rank's heads).  KV for local positions only is in ``kv_cache``
    and ``meta`` already describes the LOCAL shard (seq_lens / block tables of local tokens;
    causality is preserved because the newest token's KV is visible to its owner only after
    the write, and the new-token contribution is merged with the same LSE rule)."""
    comm = get_dcp_comm()
    q_all = comm.all_gather(q.contiguous(), dim=1)                # all heads of the group
    out, lse = ops.paged_attention(q_all, kv_cache, meta, layer.scale, sliding_window=layer.sliding_window,
                                   softcap=layer.softcap, return_lse=True)
    if envs.B200_DCP_LSE_MERGE_A2A and q.shape[0] <= envs.B200_DCP_LSE_MERGE_A2A_MAX_TOKENS:
        return cp_lse_a2a(out, lse, comm)
    return cp_lse_ag_out_rs(out, lse, comm, envs.B200_DCP_RS_OUT_FP32)
