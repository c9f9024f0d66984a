"""KV offload connector: full KV blocks of finished requests are copied to a pinned host slab
(optionally spilled to disk), keyed by the prefix-cache hash chain; a later request with the same
prefix loads them back instead of recomputing.

Save path: ``request_finished`` keeps the blocks alive; the worker half waits for a device event
recorded after the producing forward (save fence), then copies the blocks GPU→host on a side
stream with the block-copy kernel and commits the slots.  Failed saves are retried
``B200_OFFLOAD_SAVE_RETRIES`` times.  Load path: synchronous host→GPU copy before the forward of
the admitting step.  Same life cycle as the reference's offloading connector
(reference: src/vllm_torchtpu/offload/raiden_connector.py:14-570, raiden_store.py:227-2722).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .. import envs
from ..engine.block_manager import hash_block
from ..logger import init_logger
from .base import Connector, ConnectorMetadata, SchedulerConnectorBase, WorkerConnectorBase
from .transport import PoolInfo, copy_blocks, nan_blocks

logger = init_logger(__name__)


class HostKVStore:
    """Pinned host slab [layer][slot][block_bytes] + the native slot index."""

    def __init__(self, num_layers: int, block_shape: tuple, dtype, capacity: int, pin: bool,
                 disk_dir: str = "", namespace: str = ""):
        from ..ops import cuda
        self.lib = cuda.lib()
        self.lib.b200_store_create.restype = ctypes.c_void_p
        self.h = ctypes.c_void_p(self.lib.b200_store_create(ctypes.c_int(capacity)))
        self.capacity = capacity
        self.layers = [torch.zeros((capacity,) + tuple(block_shape), dtype=dtype, pin_memory=pin)
                       for _ in range(num_layers)]
        self.pool = PoolInfo("host-store", self.layers)
        # spilled blocks of another model, KV dtype or block geometry must never be read back: each
        # (namespace, layers, shape, dtype) gets a directory of its own
        self.disk_dir = ""
        if disk_dir:
            import hashlib
            tag = hashlib.sha256(repr((namespace, num_layers, tuple(block_shape), str(dtype))).encode()).hexdigest()
            self.disk_dir = os.path.join(disk_dir, tag[:16])
            os.makedirs(self.disk_dir, exist_ok=True)

    @staticmethod
    def key(h: int) -> int:
        return h & 0xFFFFFFFFFFFFFFFF

    def lookup_prefix(self, hashes: list, pin: bool = True) -> list:
        n = len(hashes)
        if n == 0:
            return []
        keys = (ctypes.c_uint64 * n)(*[self.key(h) for h in hashes])
        out = (ctypes.c_int * n)()
        k = self.lib.b200_store_lookup_prefix(self.h, keys, ctypes.c_int(n), out, ctypes.c_int(1 if pin else 0))
        return list(out[:k])

    def reserve(self, h: int) -> int:
        return self.lib.b200_store_reserve(self.h, ctypes.c_uint64(self.key(h)))

    def commit(self, slot: int, ok: bool = True) -> None:
        self.lib.b200_store_commit(self.h, ctypes.c_int(slot), ctypes.c_int(1 if ok else 0))

    def unpin(self, slots: list) -> None:
        if slots:
            arr = (ctypes.c_int * len(slots))(*slots)
            self.lib.b200_store_unpin(self.h, arr, ctypes.c_int(len(slots)))

    def stats(self) -> dict:
        out = (ctypes.c_uint64 * 4)()
        self.lib.b200_store_stats(self.h, out)
        return {"hits": out[0], "misses": out[1], "evictions": out[2], "stored": out[3],
                "pinned": int(self.lib.b200_store_pinned(self.h))}

    # ---- disk tier: one file per evicted-but-wanted block is kept simple on purpose ----
    def spill(self, h: int, slot: int) -> None:
        if self.disk_dir:
            torch.save([l[slot].clone() for l in self.layers], os.path.join(self.disk_dir, f"{self.key(h):016x}.pt"))

    def unspill(self, h: int, slot: int) -> bool:
        p = os.path.join(self.disk_dir, f"{self.key(h):016x}.pt") if self.disk_dir else ""
        if not p or not os.path.exists(p):
            return False
        for l, t in zip(self.layers, torch.load(p, weights_only=True)):
            l[slot].copy_(t)
        return True

    def close(self):
        if self.h:
            self.lib.b200_store_destroy(self.h)
            self.h = None


def block_hashes(token_ids: list, block_size: int, n_blocks: int, extra: tuple = ()) -> list:
    out, parent = [], None
    for i in range(n_blocks):
        parent = hash_block(parent, tuple(token_ids[i * block_size:(i + 1) * block_size]), extra)
        out.append(parent)
    return out


def _kv_identity(request) -> tuple:
    """What, besides the tokens, decides the contents of a request's KV blocks; the same tuple the
    GPU prefix cache hashes (engine/block_manager.py)."""
    name = request.sampling_params.lora_name
    return (name,) if name else ()


class OffloadSchedulerHalf(SchedulerConnectorBase):
    def __init__(self, store: HostKVStore, block_size: int):
        self.store, self.bs = store, block_size
        self._loads, self._saves = [], []
        self._pending_load: dict = {}
        # prompt tokens looked up in / served from the host store (admitted requests only)
        self.stats = {"external_queries": 0, "external_hits": 0}

    def request_not_admitted(self, request) -> None:
        """The scheduler asked for matches but could not admit the request in this step: give the
        pinned host slots back (the next attempt looks them up again)."""
        prev = self._pending_load.pop(request.request_id, None)
        if prev is not None:
            self.store.unpin(prev[1])

    def get_num_new_matched_tokens(self, request, num_cached: int):
        self.request_not_admitted(request)          # a repeated query must not leak the earlier pins
        usable = (request.num_tokens - 1) // self.bs
        hashes = block_hashes(request.all_token_ids, self.bs, usable, _kv_identity(request))
        slots = self.store.lookup_prefix(hashes, pin=True)
        have = num_cached // self.bs
        if len(slots) <= have:
            self.store.unpin(slots)
            return 0, False
        self.store.unpin(slots[:have])
        self._pending_load[request.request_id] = (have, slots[have:])
        return (len(slots) - have) * self.bs, False

    def update_state_after_alloc(self, request, block_ids, num_external):
        have, slots = self._pending_load.pop(request.request_id)
        self.stats["external_queries"] += getattr(request, "num_prompt_tokens", request.num_tokens)
        self.stats["external_hits"] += len(slots) * self.bs
        self._loads.append((request.request_id, slots, list(block_ids)[have:have + len(slots)]))

    def request_finished(self, request, block_ids):
        n_full = min(request.num_computed_tokens, request.num_tokens) // self.bs
        if request.error or n_full == 0:
            return False, None
        hashes = block_hashes(request.all_token_ids, self.bs, n_full, _kv_identity(request))
        self._saves.append((request.request_id, hashes, list(block_ids)[:n_full]))
        return True, None

    def build_connector_meta(self, out):
        m = ConnectorMetadata()
        m.loads, self._loads = self._loads, []
        m.sends, self._saves = self._saves, []
        return m


class OffloadWorkerHalf(WorkerConnectorBase):
    def __init__(self, store: HostKVStore, gpu_pool: PoolInfo, is_cuda: bool):
        self.store, self.gpu, self.is_cuda = store, gpu_pool, is_cuda
        self._done: list = []
        self._jobs: list = []            # (request_id, event, slots)
        self.stream = torch.cuda.Stream() if is_cuda else None
        self.failed_saves = 0
        self.nan_blocked = 0

    def start_load_kv(self, meta: Optional[ConnectorMetadata]) -> None:
        if meta is None:
            return
        for rid, slots, local in meta.loads:
            copy_blocks(self.store.pool, self.gpu, slots, local)        # stream-ordered before the forward
            if self.is_cuda:
                torch.cuda.current_stream().synchronize()
            self.store.unpin(slots)

    def save_kv(self, meta: Optional[ConnectorMetadata]) -> None:
        if meta is None:
            return
        for rid, hashes, blocks in meta.sends:
            todo_slots, todo_blocks = [], []
            # a block with a NaN / Inf is never stored, nor are the blocks behind it in the hash chain
            bad = set(nan_blocks(self.gpu, list(blocks))) if envs.B200_KV_SAVE_NAN_CHECK else set()
            if bad:
                self.nan_blocked += len(bad)
                cut = min(i for i, b in enumerate(blocks) if b in bad)
                hashes, blocks = hashes[:cut], blocks[:cut]
                logger.warning("request %s: %d KV blocks hold non-finite values, not stored", rid, len(bad))
            for h, b in zip(hashes, blocks):
                slot = self.store.reserve(h)
                if slot >= 0:
                    todo_slots.append(slot)
                    todo_blocks.append(b)
            ok = self._copy_with_retries(todo_blocks, todo_slots)
            for s in todo_slots:
                self.store.commit(s, ok)
            self._done.append(rid)

    def _copy_with_retries(self, blocks, slots) -> bool:
        if not blocks:
            return True
        for attempt in range(1 + envs.B200_OFFLOAD_SAVE_RETRIES):
            try:
                if self.is_cuda:
                    fence = torch.cuda.Event()
                    fence.record()                       # the forward that produced the blocks
                    with torch.cuda.stream(self.stream):
                        self.stream.wait_event(fence)
                        copy_blocks(self.gpu, self.store.pool, blocks, slots)
                    self.stream.synchronize()
                else:
                    copy_blocks(self.gpu, self.store.pool, blocks, slots)
                return True
            except RuntimeError as e:
                self.failed_saves += 1
                logger.warning("offload save attempt %d failed: %r", attempt + 1, e)
        return False

    def get_finished_sending(self) -> list:
        out, self._done = self._done, []
        return out


def create_offloading_connector(cfg, runner, **kw) -> Connector:
    extra = (cfg.kv_transfer or {}).get("kv_connector_extra_config", {})
    layers = runner.kv_caches
    block_shape = tuple(layers[0].shape[1:])
    per_block = layers[0][0].numel() * layers[0].element_size() * len(layers)
    gb = float(extra.get("dram_gb", envs.B200_OFFLOAD_DRAM_GB or 1.0))
    capacity = int(extra.get("num_blocks", max(8, int(gb * 2**30) // per_block)))
    is_cuda = layers[0].is_cuda
    store = HostKVStore(len(layers), block_shape, layers[0].dtype, capacity, pin=is_cuda,
                        disk_dir=extra.get("disk_dir", envs.B200_OFFLOAD_DISK_DIR),
                        namespace=f"{cfg.model.name}/{cfg.model_path or ''}")
    c = Connector(OffloadSchedulerHalf(store, cfg.cache.block_size),
                  OffloadWorkerHalf(store, PoolInfo("gpu", layers), is_cuda))
    c.store = store
    return c
