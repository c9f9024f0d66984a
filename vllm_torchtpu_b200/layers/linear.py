"""Tensor-parallel linear layers.

Weights are stored ``[out_features, in_features]`` (K-major rows), which is the
layout the tcgen05 GEMM consumes directly as its 128-row operand.  Column
parallel layers shard ``out``, row parallel layers shard ``in`` and reduce
across the TP group; the bias of a row-parallel layer is added after the
reduction so every rank runs the same program
(reference: src/vllm_torchtpu/layers/adapter/linear.py:25-66).

Each layer owns a quantisation method object (``quantization/``) that creates,
loads and applies its weights.
"""
from __future__ import annotations

import zlib
from typing import Optional, Sequence

import torch

from .. import envs, ops
from ..parallel.communicator import get_tp_comm
from ..parallel.state import get_state


def seeded_normal(name: str, shape: Sequence[int], std: float, dtype, device, seed: int = 0) -> torch.Tensor:
    """Deterministic N(0, std) init keyed by the parameter name, identical on every rank."""
    g = torch.Generator(device=device)
    g.manual_seed((zlib.crc32(name.encode()) + 7919 * seed) & 0x7FFFFFFF)
    # fp32 draw then cast keeps CPU and GPU runs of tiny models comparable within a device
    return (torch.randn(tuple(shape), generator=g, device=device, dtype=torch.float32) * std).to(dtype)


class LinearBase:
    def __init__(self, name: str, in_features: int, out_features: int, *, bias: bool = False,
                 dtype=torch.bfloat16, device="cpu", quant_config=None):
        from ..quantization import get_linear_method
        self.name = name
        self.in_features = in_features          # per-rank sizes
        self.out_features = out_features
        self.dtype = dtype
        self.device = device
        self.bias: Optional[torch.Tensor] = None
        self.has_bias = bias
        self.method = get_linear_method(quant_config, name)
        self.method.create_weights(self)

    # full (unsharded) shapes, for loaders
    full_in: int = 0
    full_out: int = 0

    def shard_of(self, full_weight: torch.Tensor) -> torch.Tensor:
        return full_weight

    def init_dummy(self, std: float, seed: int) -> None:
        self.method.init_dummy(self, std, seed)
        if self.has_bias:
            self.bias = torch.zeros(self.out_features, dtype=self.dtype, device=self.device)

    def load_weight(self, full_weight: torch.Tensor, **kw) -> None:
        self.method.load_weight(self, full_weight, **kw)

    def weight_bytes(self) -> int:
        return self.method.weight_bytes(self)

    lora_targets = None          # set by lora.wiring.attach: [(adapter target name, column offset)]

    lora_in_forward = False      # row-parallel layers under TP add the update before their all-reduce

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        y = self.forward(x)
        if self.lora_targets and not self.lora_in_forward:
            from ..lora import wiring
            if wiring.active():
                y = wiring.apply(self, x, y)
        return y


class ReplicatedLinear(LinearBase):
    def __init__(self, name, in_features, out_features, **kw):
        self.full_in, self.full_out = in_features, out_features
        super().__init__(name, in_features, out_features, **kw)

    def forward(self, x):
        return self.method.apply(self, x, self.bias)


class ColumnParallelLinear(LinearBase):
    """``output_sizes`` lists the logical sub-matrices packed along ``out``
    (q/k/v or gate/up); each is sharded over TP separately."""

    def __init__(self, name, in_features, output_sizes, *, tp_size=None, tp_rank=None,
                 replicate_sizes: Sequence[bool] = (), **kw):
        st = get_state()
        self.tp_size = tp_size if tp_size is not None else st.tp.size
        self.tp_rank = tp_rank if tp_rank is not None else st.tp.rank_in_group
        if isinstance(output_sizes, int):
            output_sizes = [output_sizes]
        self.output_sizes = list(output_sizes)
        self.shard_sizes = [s // self.tp_size for s in self.output_sizes]
        self.full_in, self.full_out = in_features, sum(self.output_sizes)
        super().__init__(name, in_features, sum(self.shard_sizes), **kw)

    def shard_of(self, full_weight):
        parts, off = [], 0
        for s, sh in zip(self.output_sizes, self.shard_sizes):
            parts.append(full_weight[off + self.tp_rank * sh: off + (self.tp_rank + 1) * sh])
            off += s
        return torch.cat(parts, 0) if len(parts) > 1 else parts[0]

    def forward(self, x):
        return self.method.apply(self, x, self.bias)


class RowParallelLinear(LinearBase):
    def __init__(self, name, in_features, out_features, *, tp_size=None, tp_rank=None,
                 reduce_results: bool = True, **kw):
        st = get_state()
        self.tp_size = tp_size if tp_size is not None else st.tp.size
        self.tp_rank = tp_rank if tp_rank is not None else st.tp.rank_in_group
        self.reduce_results = reduce_results
        # set by a decoder layer whose next op is add + RMSNorm: small outputs may then be returned
        # as a pending reduction that the norm kernel completes
        self.defer_reduce = False
        self.lora_in_forward = self.tp_size > 1 and reduce_results
        self.full_in, self.full_out = in_features, out_features
        super().__init__(name, in_features // self.tp_size, out_features, **kw)

    def shard_of(self, full_weight):
        k = self.in_features
        return full_weight[:, self.tp_rank * k:(self.tp_rank + 1) * k]

    def forward_quantised(self, xq, xs):
        """Forward on an activation the caller has already quantised for this layer's method (block-scaled
        fp8: e4m3 rows with 1x128 scales, e.g. SiLU*mul fused into the quantisation kernel).  GPU only, no
        LoRA on this layer."""
        m = self.method
        if self.tp_size == 1 or not self.reduce_results:
            return m.apply_quantised(self, xq, xs, self.bias)
        comm = get_tp_comm()
        fused = comm.heap is not None and comm.heap.fused_tp is not None
        if (fused and self.defer_reduce and self.bias is None
                and m.can_push(comm.heap.fused_tp, xq.shape[0], self.out_features)):
            return m.apply_push_quantised(self, xq, xs, comm)
        y = comm.all_reduce(m.apply_quantised(self, xq, xs, None))
        return y + self.bias if self.bias is not None else y

    def forward(self, x):
        if self.tp_size == 1 or not self.reduce_results:
            return self.method.apply(self, x, self.bias)
        comm = get_tp_comm()
        if self.lora_targets:
            from ..lora import wiring
            if wiring.active():
                # the low-rank update of this rank's input shard is a partial sum like the base product
                y = wiring.apply(self, x, self.method.apply(self, x, None))
                y = comm.all_reduce(y)
                return y + self.bias if self.bias is not None else y
        fused = x.is_cuda and comm.heap is not None and comm.heap.fused_tp is not None
        if (fused and self.defer_reduce and self.bias is None and not self.lora_targets
                and hasattr(self.method, "apply_push")):
            ft, T = comm.heap.fused_tp, x.numel() // x.shape[-1]
            can = getattr(self.method, "can_push", None)
            if can(ft, T, self.out_features) if can is not None else ft.can_push(T, self.out_features):
                return self.method.apply_push(self, x, comm)
        if fused and self.method.supports_fused_reduce:
            y = self.method.apply_fused_all_reduce(self, x, comm)
        else:
            y = comm.all_reduce(self.method.apply(self, x, None))
        if self.bias is not None:
            y = y + self.bias
        return y
