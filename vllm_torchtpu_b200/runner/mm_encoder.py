"""Multimodal encoder manager: runs the vision encoder for the images / video chunks that the
scheduled requests need, under a patch budget and with padded batch shapes.

* Items (one image, or one temporal chunk of a video) are packed into encoder batches whose total
  patch count stays within ``max_patches_per_batch``; the total is padded up to a bucket (a fixed
  list of sizes) with a dummy item so that the encoder sees few distinct shapes.
* A video is split along time into chunks of at most ``max_patches_per_batch`` patches (whole
  frame groups), each chunk being an independent attention segment — the patches of a chunk attend
  to each other only.
* Outputs are cached per (request, item) until the request's prompt has consumed them; the runner
  asks for the embedding rows that fall into the token range a step computes and writes them over
  the placeholder-token embeddings.
(reference: src/vllm_torchtpu/runner/mm_encoder_manager.py — vision-encoder token-budget buckets;
runner/mm_video_chunking.py — temporal video chunking.)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


def patch_buckets(max_patches: int, smallest: int = 256) -> list:
    out, b = [], smallest
    while b < max_patches:
        out.append(b)
        b *= 2
    out.append(max_patches)
    return out


def chunk_video(num_frames: int, patches_per_frame: int, max_patches: int, temporal_patch: int = 2) -> list:
    """Split a video into (first_frame, num_frames) chunks of whole temporal-patch groups whose patch
    count fits the budget.  A frame group that alone exceeds the budget is an error."""
    group = max(1, temporal_patch)
    per_group = patches_per_frame          # one temporal patch group yields this many patches
    if per_group > max_patches:
        raise ValueError(f"one frame group has {per_group} patches, the encoder budget is {max_patches}")
    groups_total = -(-num_frames // group)
    per_chunk = max(1, max_patches // per_group)
    chunks, g = [], 0
    while g < groups_total:
        n = min(per_chunk, groups_total - g)
        first = g * group
        chunks.append((first, min(n * group, num_frames - first)))
        g += n
    return chunks


@dataclass
class MMItem:
    request_id: str
    index: int                     # position among the request's multimodal items
    patches: torch.Tensor          # [num_patches, patch_dim]
    prompt_offset: int             # first placeholder token of the item in the prompt
    num_tokens: int = 0            # placeholder tokens (= patches // merge), set by the manager


@dataclass
class MMEncoderManager:
    encoder: object
    max_patches_per_batch: int = 8192
    buckets: list = field(default_factory=list)
    cache: dict = field(default_factory=dict)          # (request id, item index) -> [tokens, hidden]
    items: dict = field(default_factory=dict)          # request id -> [MMItem]
    stats: dict = field(default_factory=lambda: {"batches": 0, "items": 0, "patches": 0, "padded_patches": 0})

    def __post_init__(self):
        if not self.buckets:
            self.buckets = patch_buckets(self.max_patches_per_batch)

    # ---- request lifecycle ------------------------------------------------------
    def add_request(self, request_id: str, items: list) -> None:
        merge = self.encoder.cfg.merge
        for it in items:
            n = it.patches.shape[0]
            if n > self.max_patches_per_batch:
                raise ValueError(f"item with {n} patches exceeds the encoder budget {self.max_patches_per_batch}; "
                                 "split videos with chunk_video")
            if n % merge:
                raise ValueError(f"patch count {n} is not a multiple of the merge size {merge}")
            it.num_tokens = n // merge
        self.items[request_id] = sorted(items, key=lambda it: it.prompt_offset)

    def remove_request(self, request_id: str) -> None:
        for it in self.items.pop(request_id, []):
            self.cache.pop((request_id, it.index), None)

    # ---- scheduling ---------------------------------------------------------------
    def needed(self, request_id: str, start: int, end: int) -> list:
        """Items of the request whose placeholder range intersects prompt tokens [start, end) and that
        have not been encoded yet."""
        return [it for it in self.items.get(request_id, [])
                if it.prompt_offset < end and it.prompt_offset + it.num_tokens > start
                and (request_id, it.index) not in self.cache]

    def plan_batches(self, items: list) -> list:
        """First-fit packing in arrival order into batches within the patch budget."""
        batches, cur, total = [], [], 0
        for it in items:
            n = it.patches.shape[0]
            if cur and total + n > self.max_patches_per_batch:
                batches.append(cur)
                cur, total = [], 0
            cur.append(it)
            total += n
        if cur:
            batches.append(cur)
        return batches

    def _bucket(self, n: int) -> int:
        for b in self.buckets:
            if b >= n:
                return b
        return n

    def encode(self, items: list) -> None:
        """Run the encoder for ``items`` (batched, padded to a bucket) and cache the embeddings."""
        merge = self.encoder.cfg.merge
        for batch in self.plan_batches(items):
            counts = [it.patches.shape[0] for it in batch]
            total = sum(counts)
            pad = self._bucket(total) - total
            pad -= pad % merge
            mats = [it.patches for it in batch]
            if pad > 0:
                mats.append(torch.zeros((pad, mats[0].shape[1]), dtype=mats[0].dtype, device=mats[0].device))
                counts.append(pad)            # the padding is its own attention segment
            outs = self.encoder.forward(torch.cat(mats, 0), counts)
            for it, emb in zip(batch, outs):
                self.cache[(it.request_id, it.index)] = emb
            self.stats["batches"] += 1
            self.stats["items"] += len(batch)
            self.stats["patches"] += total
            self.stats["padded_patches"] += total + max(0, pad)

    # ---- consumption ----------------------------------------------------------------
    def gather(self, request_id: str, start: int, end: int) -> list:
        """(row offset inside [start, end), embedding rows) pairs for the placeholder tokens of the
        request that fall into prompt tokens [start, end); encodes what is missing first."""
        missing = self.needed(request_id, start, end)
        if missing:
            self.encode(missing)
        out = []
        for it in self.items.get(request_id, []):
            lo, hi = max(start, it.prompt_offset), min(end, it.prompt_offset + it.num_tokens)
            if lo < hi:
                emb = self.cache[(request_id, it.index)]
                out.append((lo - start, emb[lo - it.prompt_offset: hi - it.prompt_offset]))
        return out

    def merge_into(self, hidden: torch.Tensor, request_id: str, start: int, row0: int, num_rows: int) -> None:
        """Overwrite the placeholder-token embeddings of one request's rows of a step:
        ``hidden[row0 : row0 + num_rows]`` holds prompt tokens [start, start + num_rows)."""
        for off, emb in self.gather(request_id, start, start + num_rows):
            hidden[row0 + off: row0 + off + emb.shape[0]] = emb.to(hidden.dtype)

    def release_consumed(self, request_id: str, computed_tokens: int) -> None:
        """Drop cached embeddings whose placeholder range lies entirely before ``computed_tokens``."""
        for it in self.items.get(request_id, []):
            if it.prompt_offset + it.num_tokens <= computed_tokens:
                self.cache.pop((request_id, it.index), None)
