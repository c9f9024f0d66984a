"""Block moves between engines whose tensor-parallel degrees differ.

A rank's paged KV block is ``[2, heads_of_this_rank, block_size, head_dim]``.  With ``H`` KV heads and ``tp``
ranks a rank holds ``max(1, H / tp)`` heads, starting at head ``(rank // replicas) · heads_per_rank`` where
``replicas = max(1, tp / H)`` ranks share a head when there are fewer heads than ranks.  A consumer rank
therefore needs, from every producer rank whose head range meets its own, one piece of the K half and one
piece of the V half of each block: a ``Span`` with two chunks.  Latent (MLA) caches are the same on every
rank of an engine: the consumer takes whole blocks from one producer rank.

``plan_pull`` is evaluated by the consumer (what to fetch from whom) and, with the roles swapped, by the
producer (which consumer ranks will acknowledge a transfer before its blocks may be freed).
(reference: src/vllm_torchtpu/distributed/kv_transfer/tpu_connector.py:1063 — heterogeneous resharding
PCP/TP/DCP→TP/DP of the native connector; raiden/byte_spans.py)"""
from __future__ import annotations

from dataclasses import asdict, dataclass


@dataclass(frozen=True)
class KVGeometry:
    """How one rank of an engine lays out a KV block."""
    tp: int = 1
    rank: int = 0
    num_kv_heads: int = 1           # of the model; 0 for a latent (MLA) cache without a head axis
    head_bytes: int = 0             # block_size · head_dim · element size (bytes of one head in one half)
    block_bytes: int = 0            # of this rank's block

    @property
    def latent(self) -> bool:
        return self.num_kv_heads == 0

    def heads_per_rank(self) -> int:
        return max(1, self.num_kv_heads // self.tp)

    def head_range(self, rank: int | None = None) -> tuple:
        r = self.rank if rank is None else rank
        replicas = max(1, self.tp // max(1, self.num_kv_heads))
        h = self.heads_per_rank()
        lo = (r // replicas) * h
        return lo, lo + h

    def to_dict(self) -> dict:
        return asdict(self)

    @staticmethod
    def from_dict(d: dict) -> "KVGeometry":
        return KVGeometry(**{k: d[k] for k in ("tp", "rank", "num_kv_heads", "head_bytes", "block_bytes")})

    @staticmethod
    def of_cache(layer, tp: int, rank: int, num_kv_heads: int) -> "KVGeometry":
        """Geometry of a rank whose per-layer cache tensor is ``layer`` ([blocks, 2, heads, block_size, dim]
        or a latent [blocks, block_size, width])."""
        block_bytes = layer[0].numel() * layer.element_size()
        if layer.dim() != 5:
            return KVGeometry(tp, rank, 0, 0, block_bytes)
        return KVGeometry(tp, rank, num_kv_heads, layer.shape[3] * layer.shape[4] * layer.element_size(), block_bytes)


@dataclass(frozen=True)
class Span:
    src_off: int
    dst_off: int
    nbytes: int
    chunks: int = 1
    src_stride: int = 0
    dst_stride: int = 0


def same_layout(a: KVGeometry, b: KVGeometry) -> bool:
    return a.block_bytes == b.block_bytes and (a.latent or a.head_range() == b.head_range())


def plan_pull(consumer: KVGeometry, producer: KVGeometry) -> list:
    """[(producer rank, Span)] that fills every block of ``consumer``'s rank from the producer engine
    (``producer.rank`` is ignored: all its ranks are considered)."""
    if consumer.latent != producer.latent:
        raise ValueError("latent and per-head caches cannot feed each other")
    if consumer.latent:
        if consumer.block_bytes != producer.block_bytes:
            raise ValueError("latent caches differ in block size")
        # spread the consumer ranks over the producer ranks
        return [(consumer.rank % producer.tp, Span(0, 0, consumer.block_bytes))]
    if consumer.num_kv_heads != producer.num_kv_heads or consumer.head_bytes != producer.head_bytes:
        raise ValueError(f"KV geometry differs: consumer {consumer}, producer {producer}")
    c_lo, c_hi = consumer.head_range()
    hb = consumer.head_bytes
    c_half, p_half = consumer.heads_per_rank() * hb, producer.heads_per_rank() * hb
    plan, covered = [], c_lo
    replicas = max(1, producer.tp // producer.num_kv_heads)
    for pr in range(producer.tp):
        p_lo, p_hi = producer.head_range(pr)
        lo, hi = max(c_lo, p_lo), min(c_hi, p_hi)
        if lo >= hi or lo != covered:
            continue                                     # no overlap, or a replica of a range already planned
        if replicas > 1:
            pr = pr + consumer.rank % replicas            # replicas of a head: spread the readers
        plan.append((pr, Span((lo - p_lo) * hb, (lo - c_lo) * hb, (hi - lo) * hb, 2, p_half, c_half)))
        covered = hi
    if covered != c_hi:
        raise ValueError(f"producer ranks do not cover heads [{c_lo}, {c_hi}) of the consumer")
    return plan


def readers_of(producer: KVGeometry, consumer_tp: int, consumer_proto: KVGeometry) -> list:
    """Consumer ranks that fetch from ``producer``'s rank (they each acknowledge the transfer)."""
    out = []
    for cr in range(consumer_tp):
        c = KVGeometry(consumer_tp, cr, consumer_proto.num_kv_heads, consumer_proto.head_bytes,
                       _block_bytes(consumer_proto, consumer_tp))
        if any(pr == producer.rank for pr, _ in plan_pull(c, producer)):
            out.append(cr)
    return out


def _block_bytes(proto: KVGeometry, tp: int) -> int:
    if proto.latent:
        return proto.block_bytes
    return 2 * max(1, proto.num_kv_heads // tp) * proto.head_bytes
