"""Adapter registry: add / remove / pin / list adapters, LRU slot assignment, per-layer stacked
A/B tensors with one row per slot that the linears index by token
(reference: src/vllm_torchtpu/worker/tpu_worker.py:898-908, lora/lora_manager.py)."""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass
class LoRAAdapter:
    name: str
    rank: int
    alpha: float
    weights: dict = field(default_factory=dict)    # "<layer name>" -> (A [r, K], B [N, r])

    @property
    def scale(self) -> float:
        return self.alpha / self.rank


class LoRAManager:
    def __init__(self, max_loras: int, max_rank: int, dtype=torch.bfloat16, device="cpu"):
        self.max_loras, self.max_rank, self.dtype, self.device = max_loras, max_rank, dtype, device
        self.adapters: dict = {}
        self.slot_of: "OrderedDict[str, int]" = OrderedDict()
        self.pinned: set = set()
        self.free_slots = list(range(max_loras - 1, -1, -1))
        self.layers: dict = {}                     # layer name -> (A [slots, r, K], B [slots, N, r])
        self.scales = torch.zeros(max_loras, dtype=torch.float32, device=device)

    def register_layer(self, name: str, in_features: int, out_features: int) -> None:
        if not hasattr(self, "shard_fns"):
            self.shard_fns = {}
        self.layers[name] = (torch.zeros(self.max_loras, self.max_rank, in_features, dtype=self.dtype, device=self.device),
                             torch.zeros(self.max_loras, out_features, self.max_rank, dtype=self.dtype, device=self.device))

    def add_adapter(self, ad: LoRAAdapter) -> bool:
        if ad.rank > self.max_rank:
            raise ValueError(f"adapter rank {ad.rank} exceeds max_lora_rank {self.max_rank}")
        if ad.name in self.adapters:
            return False
        self.adapters[ad.name] = ad
        return True

    def remove_adapter(self, name: str) -> bool:
        if name not in self.adapters:
            return False
        self.pinned.discard(name)
        if name in self.slot_of:
            self.free_slots.append(self.slot_of.pop(name))
        del self.adapters[name]
        return True

    def pin_adapter(self, name: str) -> bool:
        if name not in self.adapters:
            return False
        self.activate(name)
        self.pinned.add(name)
        return True

    def list_adapters(self) -> list:
        return sorted(self.adapters)

    def activate(self, name: str) -> int:
        """Slot of an adapter, loading it into a slot (evicting the least recently used unpinned one)."""
        if name in self.slot_of:
            self.slot_of.move_to_end(name)
            return self.slot_of[name]
        if name not in self.adapters:
            raise KeyError(f"unknown LoRA adapter {name!r}")
        if not self.free_slots:
            victim = next((n for n in self.slot_of if n not in self.pinned), None)
            if victim is None:
                raise RuntimeError("every LoRA slot is pinned")
            self.free_slots.append(self.slot_of.pop(victim))
        slot = self.free_slots.pop()
        ad = self.adapters[name]
        for lname, (A, B) in self.layers.items():
            A[slot].zero_()
            B[slot].zero_()
            if lname in ad.weights:
                a, b = ad.weights[lname]
                if lname in self.shard_fns:          # tensor parallelism: this rank's part
                    a, b = self.shard_fns[lname](a, b)
                A[slot, :a.shape[0], :] = a.to(self.dtype)
                B[slot, :, :b.shape[1]] = b.to(self.dtype)
        self.scales[slot] = ad.scale
        self.slot_of[name] = slot
        return slot

    def token_indices(self, lora_names: list, num_new_tokens: list) -> Optional[torch.Tensor]:
        """Per-token slot ids (-1 = base model) for a step."""
        if not any(lora_names):
            return None
        ids = []
        for name, n in zip(lora_names, num_new_tokens):
            ids += [self.activate(name) if name else -1] * n
        return torch.tensor(ids, dtype=torch.int64, device=self.device)
