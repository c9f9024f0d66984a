"""Prefill context parallelism (ring attention).

A long prompt is split over the PCP ranks; every rank computes the queries of its own token
shard and the K/V shards travel round the ring (each rank pulls the previous rank's shard over
NVLink while it computes on the one it holds), with online-softmax merging of the partial
results, so no rank ever materialises the whole KV.  Two pieces of planning are shared with the
reference: tokens are packed rank-major interleaved in units of ``cp_kv_cache_interleave_size``,
and for causal balance rank r takes chunks r and 2P-1-r of the prompt ("head-tail" split)
(reference: src/vllm_torchtpu/runner/pcp/head_tail_sharding_plan.py, manager.py:136-206;
kernels/experimental/pcp_streaming_rpa/README.md:1-121).

``ring_attention`` is written against a transport interface (``exchange(kv) -> kv of previous
rank``) so the math and the schedule are tested on CPU with an in-process ring; on GPUs the
exchange is a peer copy out of the neighbour's symmetric buffer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ..ops import reference as ref


class PcpStaticSupportValidator:
    """Static admissibility of a PCP configuration
    (reference: src/vllm_torchtpu/platforms/pcp_validation.py)."""

    def __init__(self, cfg):
        self.cfg = cfg

    def validate(self) -> None:
        m, p, c = self.cfg.model, self.cfg.parallel, self.cfg.cache
        pcp = p.prefill_context_parallel_size
        if pcp & (pcp - 1):
            raise ValueError("prefill_context_parallel_size must be a power of two")
        if p.cp_kv_cache_interleave_size % c.block_size and c.block_size % p.cp_kv_cache_interleave_size:
            raise ValueError("cp_kv_cache_interleave_size must divide or be a multiple of block_size")
        if self.cfg.scheduler.max_num_batched_tokens % (2 * pcp):
            raise ValueError("max_num_batched_tokens must be a multiple of 2 * pcp (head-tail chunks)")
        if m.sliding_window:
            raise ValueError("sliding-window models are not supported under PCP")
        if self.cfg.speculative:
            raise ValueError("speculative decoding is not supported under PCP")
        if m.is_mla or getattr(m, "is_hybrid_gdn", False):
            raise ValueError("PCP in the engine splits GQA attention layers; latent-attention and linear-attention "
                             "models are not supported")
        if p.enable_expert_parallel or p.data_parallel_size > 1:
            raise ValueError("PCP ranks compute different numbers of rows per step; expert parallelism and "
                             "data-parallel lockstep need equal rows and are not supported together with it")
        if p.decode_context_parallel_size > 1:
            raise ValueError("PCP completes every rank's KV cache; it is not combined with a position-sharded "
                             "cache (DCP)")


@dataclass
class HeadTailPlan:
    """Token ranges of a prompt of ``n`` tokens held by each of ``P`` ranks: the prompt is cut into
    2P chunks and rank r owns chunks r and 2P-1-r, which equalises causal attention work."""
    n: int
    P: int

    def chunk_bounds(self) -> list:
        c = -(-self.n // (2 * self.P))
        return [(min(i * c, self.n), min((i + 1) * c, self.n)) for i in range(2 * self.P)]

    def ranges(self, rank: int) -> list:
        b = self.chunk_bounds()
        return [b[rank], b[2 * self.P - 1 - rank]]

    def positions(self, rank: int) -> torch.Tensor:
        return torch.cat([torch.arange(lo, hi) for lo, hi in self.ranges(rank)])

    def work(self, rank: int) -> int:
        """Causal (query, key) pairs of a rank."""
        return int(sum((hi * (hi + 1) - lo * (lo + 1)) // 2 for lo, hi in self.ranges(rank)))


def interleaved_owner(position: int, P: int, interleave: int) -> int:
    """Rank that stores the KV of ``position`` under rank-major interleaved packing."""
    return (position // interleave) % P


def ring_attention(q: torch.Tensor, q_pos: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                   kv_pos: torch.Tensor, scale: float, P: int,
                   exchange: Callable[[tuple], tuple]) -> torch.Tensor:
    """q [Tq, H, D] with absolute positions q_pos; local k/v [Tk, Hkv, D] with kv_pos.
    ``exchange((k, v, pos))`` returns the shard currently held by the previous rank.  After P steps
    every rank has seen every shard once; partial results are merged by their log-sum-exp."""
    Hq, Hkv = q.shape[1], k.shape[1]
    G = Hq // Hkv
    outs, lses = [], []
    cur = (k, v, kv_pos)
    for step in range(P):
        nxt = exchange(cur) if step < P - 1 else None      # overlaps with the compute below on GPUs
        kk, vv, pp = cur
        if kk.shape[0] > 0:
            s = torch.einsum("qhd,khd->hqk", q.float(), kk.float().repeat_interleave(G, dim=1)) * scale
            mask = pp[None, :] <= q_pos[:, None]
            s = s.masked_fill(~mask[None], float("-inf"))
            l = torch.logsumexp(s, dim=-1)
            p_ = torch.exp(s - l[..., None])
            p_ = torch.where(torch.isfinite(l)[..., None], p_, torch.zeros_like(p_))
            o = torch.einsum("hqk,khd->qhd", p_, vv.float().repeat_interleave(G, dim=1))
            outs.append(o.to(q.dtype))
            lses.append(l.t().contiguous())
        cur = nxt
    out, _ = ref.merge_attn_states(outs, lses)
    return out


class InProcessRing:
    """P simulated ranks in one process (tests): exchange hands each rank its predecessor's shard."""

    def __init__(self, P: int):
        self.P = P
        self.slots: list = [None] * P

    def run(self, fn_per_rank: list) -> list:
        """Each element is a generator-style callable taking ``exchange``; runs them in lockstep."""
        import threading
        results = [None] * self.P
        barrier = threading.Barrier(self.P)
        boxes = [None] * self.P

        def make_exchange(r):
            def exchange(item):
                boxes[r] = item
                barrier.wait()
                got = boxes[(r - 1) % self.P]
                barrier.wait()
                return got
            return exchange

        def work(r):
            results[r] = fn_per_rank[r](make_exchange(r))

        ths = [threading.Thread(target=work, args=(r,)) for r in range(self.P)]
        [t.start() for t in ths]
        [t.join() for t in ths]
        return results
