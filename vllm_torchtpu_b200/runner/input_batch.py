"""Persistent batch state on the host and the packed staging buffers.

The runner keeps one row per live request (token ids, block table, sampling
parameters) in numpy arrays so that preparing a step is a handful of vectorised
operations, and packs every per-step array into one pinned host buffer that
mirrors one device buffer: a step costs two host→device copies (scalars+token
arrays, block tables) regardless of batch size.  The reference keeps equivalent
CPU staging buffers and a decode fast path
(reference: src/vllm_torchtpu/runner/tpu_runner.py:1071-1182, 3393-3938).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch


class InputBatch:
    def __init__(self, max_reqs: int, max_model_len: int, block_size: int, kernel_blocks_per_block: int = 1):
        self.max_reqs = max_reqs
        self.max_model_len = max_model_len
        self.block_size = block_size
        # rows list kernel blocks; a scheduler block may cover several (its last one may be partly unused)
        self.max_blocks = -(-max_model_len // block_size) + kernel_blocks_per_block
        self.req_ids: list = [None] * max_reqs
        self.slot_of: dict = {}
        self.free_slots = list(range(max_reqs - 1, -1, -1))
        self.token_ids = np.zeros((max_reqs, max_model_len + 8), dtype=np.int32)
        self.num_known = np.zeros(max_reqs, dtype=np.int32)
        from .kernel_block_table import KernelBlockTable
        self.kbt = KernelBlockTable(max_reqs, self.max_blocks, kernel_blocks_per_block)
        self.block_table = self.kbt.table
        self.num_blocks = self.kbt.num_blocks
        self.temperature = np.zeros(max_reqs, dtype=np.float32)
        self.top_k = np.zeros(max_reqs, dtype=np.int32)
        self.top_p = np.ones(max_reqs, dtype=np.float32)
        self.lora_id = np.zeros(max_reqs, dtype=np.int32)

    def add(self, req, block_ids: list) -> int:
        rid = req.request_id
        if rid in self.slot_of:
            slot = self.slot_of[rid]
        else:
            slot = self.free_slots.pop()
            self.slot_of[rid] = slot
            self.req_ids[slot] = rid
        toks = req.all_token_ids
        n = len(toks)
        self.token_ids[slot, :n] = toks
        self.num_known[slot] = n
        self.kbt.set_row(slot, block_ids)
        sp = req.sampling_params
        self.temperature[slot] = sp.temperature
        self.top_k[slot] = sp.top_k if sp.top_k and sp.top_k > 0 else 0
        self.top_p[slot] = sp.top_p
        return slot

    def append_blocks(self, slot: int, new_block_ids: list) -> None:
        if not new_block_ids:
            return
        self.kbt.append(slot, new_block_ids)

    def append_token(self, slot: int, token: int) -> None:
        n = int(self.num_known[slot])
        self.token_ids[slot, n] = token
        self.num_known[slot] = n + 1

    def remove(self, rid: str) -> None:
        slot = self.slot_of.pop(rid, None)
        if slot is None:
            return
        self.req_ids[slot] = None
        self.num_known[slot] = 0
        self.num_blocks[slot] = 0
        self.free_slots.append(slot)


class StepBuffers:
    """One pinned host buffer + one device buffer with identical layout.

    int32 region:  input_ids[T] positions[T] slot_mapping[T] token_src[T]
                   query_start_loc[R+1] seq_lens[R] logits_indices[R] top_k[R] batch_slots[R]
    fp32 region:   temperature[R] top_p[R]
    block tables:  [R, max_blocks] int32 (separate copy)
    """

    def __init__(self, token_cap: int, req_cap: int, max_blocks: int, device):
        self.T, self.R, self.max_blocks = token_cap, req_cap, max_blocks
        T, R = token_cap, req_cap
        pad = lambda n: (n + 3) // 4 * 4        # keep every array 16-byte aligned
        sizes = [("input_ids", T), ("positions", T), ("slot_mapping", T), ("token_src", T),
                 ("query_start_loc", R + 1), ("seq_lens", R), ("logits_indices", T), ("top_k", T),
                 ("batch_slots", R), ("temperature", T), ("top_p", T), ("rng_step", 2), ("global_seq_lens", R),
                 ("num_valid", 1)]
        self.offsets, off = {}, 0
        for name, n in sizes:
            self.offsets[name] = (off, n)
            off += pad(n)
        self.small_len = off
        is_cuda = torch.device(device).type == "cuda"
        self.host = torch.zeros(off, dtype=torch.int32, pin_memory=is_cuda)
        self.host_bt = torch.zeros((R, max_blocks), dtype=torch.int32, pin_memory=is_cuda)
        self.dev = torch.zeros(off, dtype=torch.int32, device=device)
        self.dev_bt = torch.zeros((R, max_blocks), dtype=torch.int32, device=device)
        self.np = self.host.numpy()
        self.np_bt = self.host_bt.numpy()
        self.h2d_bytes = 0

    def host_view(self, name: str, n: Optional[int] = None, dtype=np.int32) -> np.ndarray:
        off, cap = self.offsets[name]
        v = self.np[off:off + (cap if n is None else n)]
        return v if dtype == np.int32 else v.view(dtype)

    def dev_view(self, name: str, n: Optional[int] = None, dtype=torch.int32) -> torch.Tensor:
        off, cap = self.offsets[name]
        v = self.dev[off:off + (cap if n is None else n)]
        return v if dtype == torch.int32 else v.view(dtype)

    def upload(self, num_bt_rows: int) -> int:
        """Copy the staged step to the device (async on the current stream). Returns bytes copied."""
        self.dev.copy_(self.host, non_blocking=True)
        n = self.small_len * 4
        if num_bt_rows > 0:
            self.dev_bt[:num_bt_rows].copy_(self.host_bt[:num_bt_rows], non_blocking=True)
            n += num_bt_rows * self.max_blocks * 4
        self.h2d_bytes += n
        return n
