"""Paged KV-cache block pool with hash-chained prefix caching.

Blocks are reference-counted.  A full block gets a content hash chained on its
predecessor's hash; freed hashed blocks stay in an LRU list so a later request
with the same prefix can revive them.  Block 0 is reserved as the null block
that padded table entries point at.
"""
from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from typing import Optional


def hash_block(parent: Optional[int], tokens: tuple, extra: tuple = ()) -> int:
    """Identity of a full KV block: SHA-256 over the parent block's identity, the block's token ids
    and the request attributes that change the KV contents (``extra``: LoRA adapter name, model /
    dtype namespace), truncated to 128 bits.  Stable across processes, unlike ``hash()``
    (reference: the chained block hashes of the prefix cache the plugin inherits from vLLM)."""
    h = hashlib.sha256()
    h.update(b"\0" * 16 if parent is None else int(parent).to_bytes(16, "little"))
    h.update(struct.pack(f"<{len(tokens)}q", *tokens))
    if extra:
        h.update(repr(tuple(extra)).encode())
    return int.from_bytes(h.digest()[:16], "little")


class KVBlock:
    __slots__ = ("block_id", "ref_cnt", "block_hash")

    def __init__(self, block_id: int):
        self.block_id = block_id
        self.ref_cnt = 0
        self.block_hash: Optional[int] = None


class BlockPool:
    def __init__(self, num_blocks: int, block_size: int, enable_caching: bool = False):
        if num_blocks < 2:
            raise ValueError("need at least 2 KV blocks")
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.enable_caching = enable_caching
        self.blocks = [KVBlock(i) for i in range(num_blocks)]
        # free list ordered by eviction priority (front = evict first)
        self.free: "OrderedDict[int, None]" = OrderedDict((i, None) for i in range(1, num_blocks))
        self.cached: dict[int, int] = {}          # hash -> block id
        self.blocks[0].ref_cnt = 1                # null block
        self.hits = 0
        self.queries = 0

    @property
    def num_free_blocks(self) -> int:
        return len(self.free)

    @property
    def usage(self) -> float:
        return 1.0 - len(self.free) / (self.num_blocks - 1)

    def _pop_free(self) -> KVBlock:
        bid, _ = self.free.popitem(last=False)
        blk = self.blocks[bid]
        if blk.block_hash is not None:
            if self.cached.get(blk.block_hash) == bid:
                del self.cached[blk.block_hash]
            blk.block_hash = None
        return blk

    def allocate(self, n: int) -> list[int]:
        if n > len(self.free):
            raise RuntimeError(f"out of KV blocks: want {n}, free {len(self.free)}")
        out = []
        for _ in range(n):
            blk = self._pop_free()
            blk.ref_cnt = 1
            out.append(blk.block_id)
        return out

    def touch(self, block_ids: list[int]) -> None:
        for bid in block_ids:
            blk = self.blocks[bid]
            if blk.ref_cnt == 0:
                self.free.pop(bid, None)
            blk.ref_cnt += 1

    def release(self, block_ids: list[int]) -> None:
        # free in reverse so that the tail of a sequence is evicted before its head
        for bid in reversed(block_ids):
            if bid == 0:
                continue
            blk = self.blocks[bid]
            blk.ref_cnt -= 1
            assert blk.ref_cnt >= 0, f"double free of block {bid}"
            if blk.ref_cnt == 0:
                self.free[bid] = None
                if blk.block_hash is None:
                    self.free.move_to_end(bid, last=False)

    # ---- prefix caching ---------------------------------------------------
    def lookup_prefix(self, token_ids: list, extra: tuple = ()) -> list[int]:
        """Longest run of cached full blocks for ``token_ids`` (never the last
        token: at least one token must be computed to produce logits)."""
        if not self.enable_caching:
            return []
        bs = self.block_size
        usable = (len(token_ids) - 1) // bs
        out, parent = [], None
        self.queries += usable
        for i in range(usable):
            h = hash_block(parent, tuple(token_ids[i * bs:(i + 1) * bs]), extra)
            bid = self.cached.get(h)
            if bid is None:
                break
            out.append(bid)
            parent = h
        self.hits += len(out)
        return out

    def cache_full_blocks(self, token_ids: list, block_ids: list[int], num_computed: int,
                          extra: tuple = ()) -> None:
        if not self.enable_caching:
            return
        bs = self.block_size
        parent = None
        for i in range(num_computed // bs):
            blk = self.blocks[block_ids[i]]
            if blk.block_hash is not None:
                parent = blk.block_hash
                continue
            h = hash_block(parent, tuple(token_ids[i * bs:(i + 1) * bs]), extra)
            blk.block_hash = h
            self.cached.setdefault(h, blk.block_id)
            parent = h

    def reset_prefix_cache(self) -> None:
        for blk in self.blocks:
            blk.block_hash = None
        self.cached.clear()


class KVCacheManager:
    """Per-request block tables over a BlockPool."""

    def __init__(self, num_blocks: int, block_size: int, enable_caching: bool = False,
                 sliding_window: Optional[int] = None):
        self.pool = BlockPool(num_blocks, block_size, enable_caching)
        self.block_size = block_size
        self.sliding_window = sliding_window

    def blocks_needed(self, num_tokens: int) -> int:
        return -(-num_tokens // self.block_size)

    def get_computed_blocks(self, request) -> tuple[list[int], int]:
        extra = (request.sampling_params.lora_name,) if request.sampling_params.lora_name else ()
        ids = self.pool.lookup_prefix(request.all_token_ids, extra)
        return ids, len(ids) * self.block_size

    def can_allocate(self, request, num_new_tokens: int, cached_blocks: Optional[list] = None) -> bool:
        have = len(request.block_ids) + (len(cached_blocks) if cached_blocks else 0)
        need = self.blocks_needed(request.num_computed_tokens + num_new_tokens) - have
        if cached_blocks:
            need += sum(1 for b in cached_blocks if self.pool.blocks[b].ref_cnt == 0)
        return need <= self.pool.num_free_blocks

    def allocate_slots(self, request, num_new_tokens: int, cached_blocks: Optional[list] = None,
                       lookahead: int = 0) -> Optional[list[int]]:
        """Grow ``request.block_ids`` to hold ``num_computed + num_new (+lookahead)``
        tokens.  Returns the newly added block ids or None if the pool is short."""
        if cached_blocks:
            assert not request.block_ids
            self.pool.touch(cached_blocks)
            request.block_ids = list(cached_blocks)
        total = request.num_computed_tokens + num_new_tokens + lookahead
        need = self.blocks_needed(total) - len(request.block_ids)
        if need > self.pool.num_free_blocks:
            if cached_blocks:
                self.pool.release(request.block_ids)
                request.block_ids = []
            return None
        new = self.pool.allocate(need) if need > 0 else []
        request.block_ids.extend(new)
        return new

    def cache_blocks(self, request, num_computed: int) -> None:
        extra = (request.sampling_params.lora_name,) if request.sampling_params.lora_name else ()
        self.pool.cache_full_blocks(request.all_token_ids, request.block_ids, num_computed, extra)

    def free(self, request) -> None:
        self.pool.release(request.block_ids)
        request.block_ids = []
