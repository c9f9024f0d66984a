"""Unquantised (bf16/fp16/fp32) linear and MoE methods."""
from __future__ import annotations

import torch

from .. import ops


class LinearMethodBase:
    supports_fused_reduce = False

    def create_weights(self, layer) -> None:
        raise NotImplementedError

    def init_dummy(self, layer, std: float, seed: int) -> None:
        raise NotImplementedError

    def load_weight(self, layer, full_weight, **kw) -> None:
        raise NotImplementedError

    def apply(self, layer, x, bias=None):
        raise NotImplementedError

    def weight_bytes(self, layer) -> int:
        raise NotImplementedError


class UnquantizedLinearMethod(LinearMethodBase):
    supports_fused_reduce = True

    def create_weights(self, layer) -> None:
        layer.weight = None

    def init_dummy(self, layer, std, seed) -> None:
        from ..layers.linear import seeded_normal
        full = seeded_normal(layer.name, (layer.full_out, layer.full_in), std, layer.dtype,
                             layer.device, seed)
        layer.weight = layer.shard_of(full).contiguous()

    def load_weight(self, layer, full_weight, **kw) -> None:
        layer.weight = layer.shard_of(full_weight).to(device=layer.device, dtype=layer.dtype).contiguous()

    def apply(self, layer, x, bias=None):
        return ops.gemm(x, layer.weight, bias)

    def apply_fused_all_reduce(self, layer, x, comm):
        return ops.cuda_ops().gemm_all_reduce(x, layer.weight, comm.heap)

    def apply_push(self, layer, x, comm):
        return ops.cuda_ops().gemm_push(x, layer.weight, comm.heap)

    def weight_bytes(self, layer) -> int:
        return layer.weight.numel() * layer.weight.element_size()


def dequant_expert_pieces(moe, pieces, scales):
    """fp8 checkpoint pieces with their ``weight_scale_inv`` grids -> float tensors (others pass through)."""
    out = []
    for w, sc in zip(pieces, scales):
        if w.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            if sc is None:
                raise ValueError(f"{moe.name}: fp8 expert weights without weight_scale_inv")
            from .fp8 import dequantize_weight_block
            w = dequantize_weight_block(w, sc.float(), tuple(getattr(moe.cfg, "weight_block_size", (128, 128))))
        out.append(w)
    return out


def expert_tp_shard(moe, gate, up, down):
    """Rows of gate / up and columns of down that belong to this rank when the experts' intermediate
    dimension is sharded over tensor parallelism (no expert parallelism)."""
    I, r, n = moe.intermediate_size, moe.tp_rank, moe.tp_size
    if n == 1:
        return gate, up, down
    return gate[r * I:(r + 1) * I], up[r * I:(r + 1) * I], down[:, r * I:(r + 1) * I]


def padded_hidden(moe) -> int:
    """Rows of the down projection: the hidden size rounded up to the GEMM kernels' 128-row tile (hidden sizes
    such as 2880 are not a multiple of it); the extra rows are zero and the output is cut back."""
    return (moe.hidden_size + 127) // 128 * 128


class UnquantizedMoEMethod:
    name = "unquantized"

    def create_weights(self, moe) -> None:
        moe.w13 = None      # [E_local, 2I, H]
        moe.w2 = None       # [E_local, H, I]

    def init_dummy(self, moe, std, seed) -> None:
        from ..layers.linear import seeded_normal
        E, I, H = moe.num_experts, moe.intermediate_size, moe.hidden_size
        lo, hi = moe.expert_range
        w13 = []
        w2 = []
        for e in range(lo, hi):
            w13.append(seeded_normal(f"{moe.name}.experts.{e}.w13", (2 * I, H), std, moe.dtype, moe.device, seed))
            w2.append(seeded_normal(f"{moe.name}.experts.{e}.w2", (H, I), std, moe.dtype, moe.device, seed))
        moe.w13 = torch.stack(w13).contiguous()
        moe.w2 = torch.stack(w2).contiguous()
        if padded_hidden(moe) != H:
            moe.w2 = torch.nn.functional.pad(moe.w2, (0, 0, 0, padded_hidden(moe) - H)).contiguous()

    def load_expert(self, moe, local_e, gate, up, down, scales=(None, None, None)) -> None:
        """Unsharded checkpoint matrices of one expert; the intermediate dimension is sliced for this
        TP rank here.  Block-scaled fp8 pieces (``scales`` given) are expanded first."""
        gate, up, down = expert_tp_shard(moe, *dequant_expert_pieces(moe, (gate, up, down), scales))
        I = moe.intermediate_size
        moe.w13[local_e, :I] = gate.to(moe.w13.dtype)
        moe.w13[local_e, I:] = up.to(moe.w13.dtype)
        moe.w2[local_e, :moe.hidden_size] = down.to(moe.w2.dtype)

    def alloc(self, moe) -> None:
        E, I, H = moe.num_local_experts, moe.intermediate_size, moe.hidden_size
        moe.w13 = torch.zeros(E, 2 * I, H, dtype=moe.dtype, device=moe.device)
        moe.w2 = torch.zeros(E, padded_hidden(moe), I, dtype=moe.dtype, device=moe.device)

    def apply(self, moe, x, topk_ids, topk_w):
        kw = dict(act=moe.activation, b13=getattr(moe, "b13", None), b2=getattr(moe, "b2", None))
        if x.is_cuda:
            return ops.cuda_ops().moe_experts(x, moe.w13, moe.w2, topk_ids, topk_w, moe.expert_range[0], **kw)
        return ops.ref.moe_experts(x, moe.w13, moe.w2, topk_ids, topk_w, moe.expert_range[0], **kw)

    def apply_fused_ep(self, moe, x, topk_ids, topk_w, comm):
        return ops.cuda_ops().moe_experts_ep(x, moe.w13, moe.w2, topk_ids, topk_w, comm.heap, moe.num_experts)

    def weight_bytes(self, moe) -> int:
        return sum(t.numel() * t.element_size() for t in (moe.w13, moe.w2))
