"""Scheduler blocks split into kernel blocks.

The scheduler may count the KV cache in larger blocks than the attention kernels page it in (coarser
prefix-cache hashing and fewer allocator operations with, say, 128-token blocks, while the kernels keep
16-token pages).  Scheduler block ``b`` then owns the kernel blocks ``b * m .. b * m + m - 1`` of the pool
(``m`` = tokens per scheduler block / tokens per kernel block), and the block-table rows the kernels read
list kernel blocks.  (reference: src/vllm_torchtpu/runner/kernel_block_table.py:37-108)"""
from __future__ import annotations

import numpy as np


class KernelBlockTable:
    def __init__(self, max_reqs: int, max_kernel_blocks: int, kernel_blocks_per_block: int = 1):
        if kernel_blocks_per_block < 1:
            raise ValueError("a scheduler block holds at least one kernel block")
        self.m = kernel_blocks_per_block
        self.table = np.zeros((max_reqs, max_kernel_blocks), dtype=np.int32)
        self.num_blocks = np.zeros(max_reqs, dtype=np.int32)       # kernel blocks per row
        self._offsets = np.arange(self.m, dtype=np.int32)

    def expand(self, block_ids) -> np.ndarray:
        """Kernel block ids of the given scheduler blocks, in order."""
        ids = np.asarray(block_ids, dtype=np.int32)
        if self.m == 1:
            return ids
        return (ids[:, None] * self.m + self._offsets[None, :]).reshape(-1)

    def set_row(self, slot: int, block_ids) -> None:
        k = self.expand(block_ids)
        self.table[slot, :len(k)] = k
        self.num_blocks[slot] = len(k)

    def append(self, slot: int, new_block_ids) -> None:
        if len(new_block_ids) == 0:
            return
        k = self.expand(new_block_ids)
        n = int(self.num_blocks[slot])
        self.table[slot, n:n + len(k)] = k
        self.num_blocks[slot] = n + len(k)
