"""Connects the adapter registry to the model's linears and to the step loop.

Every linear gets the list of adapter targets that land in its output columns (a fused q/k/v or
gate/up projection has one target per Hugging Face sub-projection, at its column offset).  Before a
step the runner publishes the per-token slot ids; ``apply`` adds the low-rank update after the base
projection.  Steps without any adapter request publish nothing and run the unmodified (graph) path
(reference: src/vllm_torchtpu/lora/torch_punica_tpu.py, lora/lora_manager.py)."""
from __future__ import annotations

from typing import Optional

import torch

from .manager import LoRAManager
from .ops import lora_apply

FUSED_TARGETS = {"qkv_proj": ("q_proj", "k_proj", "v_proj"), "gate_up_proj": ("gate_proj", "up_proj")}

_step_idx: Optional[torch.Tensor] = None         # [T_pad] slot per token row, -1 = base model
_manager: Optional[LoRAManager] = None


def attach(model, manager: LoRAManager) -> None:
    from ..parallel.state import get_state
    if get_state().tp.size > 1:
        raise NotImplementedError("LoRA adapters are wired for tensor_parallel_size == 1")
    global _manager
    _manager = manager
    for lin in model.named_linears():
        prefix, leaf = lin.name.rsplit(".", 1)
        targets = []
        if leaf in FUSED_TARGETS:
            sizes = getattr(lin, "shard_sizes", None) or lin.output_sizes
            off = 0
            for sub, size in zip(FUSED_TARGETS[leaf], sizes):
                key = f"{prefix}.{sub}"
                manager.register_layer(key, lin.in_features, size)
                targets.append((key, off))
                off += size
        else:
            manager.register_layer(lin.name, lin.in_features, lin.out_features)
            targets.append((lin.name, 0))
        lin.lora_targets = targets


def set_step(idx: Optional[torch.Tensor]) -> None:
    global _step_idx
    _step_idx = idx


def active() -> bool:
    return _step_idx is not None


def apply(lin, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """y += scale * (x A^T) B^T per token adapter, for every target inside this linear."""
    if _step_idx is None or not getattr(lin, "lora_targets", None):
        return y
    x2 = x.reshape(-1, x.shape[-1])
    y2 = y.reshape(-1, y.shape[-1])
    idx = _step_idx[: x2.shape[0]]
    for key, off in lin.lora_targets:
        A, B = _manager.layers[key]
        lora_apply(x2, y2, A, B, idx, _manager.scales, col_offset=off)
    return y
