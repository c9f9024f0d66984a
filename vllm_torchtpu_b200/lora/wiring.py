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


def _column_shard_fn(lin, sub_index: int):
    """Adapter weights of one logical sub-projection of a column-parallel linear -> this rank's part.
    A (rank x in) is kept whole; B (out x rank) is cut exactly like the base weight's rows, by running
    the linear's own sharding over a full-height matrix that holds B at the sub-projection's rows."""
    full_sizes = list(lin.output_sizes)
    local_sizes = list(getattr(lin, "shard_sizes", None) or lin.output_sizes)
    off_full, off_local = sum(full_sizes[:sub_index]), sum(local_sizes[:sub_index])

    def fn(a, b):
        if b.shape[0] == local_sizes[sub_index] and lin.tp_size == 1:
            return a, b
        full = torch.zeros((sum(full_sizes), b.shape[1]), dtype=b.dtype)
        full[off_full:off_full + full_sizes[sub_index]] = b
        local = lin.shard_of(full)
        return a, local[off_local:off_local + local_sizes[sub_index]]
    return fn


def _row_shard_fn(lin):
    """Row-parallel linear: A (rank x in) is cut along the input features like the base weight, B is
    kept whole; every rank's update is a partial sum that the layer's all-reduce completes."""
    def fn(a, b):
        return lin.shard_of(a), b
    return fn


def attach(model, manager: LoRAManager) -> None:
    """Under tensor parallelism the adapter matrices are sharded like the base weights: column-parallel
    layers cut B by output rows, row-parallel layers cut A by input columns and add their partial
    update before the all-reduce."""
    global _manager
    _manager = manager
    for lin in model.named_linears():
        prefix, leaf = lin.name.rsplit(".", 1)
        targets = []
        tp = getattr(lin, "tp_size", 1)
        row_parallel = hasattr(lin, "reduce_results")
        if leaf in FUSED_TARGETS:
            sizes = getattr(lin, "shard_sizes", None) or lin.output_sizes
            off = 0
            for i, (sub, size) in enumerate(zip(FUSED_TARGETS[leaf], sizes)):
                key = f"{prefix}.{sub}"
                manager.register_layer(key, lin.in_features, size)
                if tp > 1:
                    manager.shard_fns[key] = _column_shard_fn(lin, i)
                targets.append((key, off))
                off += size
        else:
            manager.register_layer(lin.name, lin.in_features, lin.out_features)
            if tp > 1:
                if row_parallel:
                    manager.shard_fns[lin.name] = _row_shard_fn(lin)
                elif hasattr(lin, "output_sizes"):
                    manager.shard_fns[lin.name] = _column_shard_fn(lin, 0)
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
