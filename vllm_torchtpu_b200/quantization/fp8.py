"""fp8 (e4m3) quantisation: per-tensor, and 128x128 block-scaled weights with
dynamic 1x128 activation scales.

Checkpoint layout handled: HF fp8 checkpoints carry ``weight`` (e4m3, [N, K]) and
``weight_scale_inv`` ([ceil(N/128), ceil(K/128)] fp32, dequant = w * scale) or a
per-tensor ``weight_scale``.  The runtime layout keeps [N, K] K-major rows (what the
tcgen05 GEMM consumes) and the scale grid as is; TP sharding slices both on block
boundaries (reference: src/vllm_torchtpu/layers/adapter/quantization/fp8.py:1256-1318,
1600-1627).  Activations are quantised per token per 128 columns at run time
(reference: src/vllm_torchtpu/layers/adapter/linear_common.py:69-133).
``online_fp8`` quantises bf16 checkpoints at load time.
"""
from __future__ import annotations

import torch

from .. import envs, ops
from .unquantized import LinearMethodBase

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


def quantize_weight_block(w: torch.Tensor, block=(128, 128)):
    """[N,K] -> (e4m3 [N,K], scale_inv [ceil(N/bn), ceil(K/bk)] fp32) with dequant = q * scale_inv."""
    N, K = w.shape
    bn, bk = block
    nb, kb = -(-N // bn), -(-K // bk)
    wp = torch.zeros(nb * bn, kb * bk, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, bn, kb, bk)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX)
    q = q.view(nb * bn, kb * bk)[:N, :K].to(FP8)
    return q.contiguous(), scale.contiguous()


def dequantize_weight_block(q: torch.Tensor, scale_inv: torch.Tensor, block=(128, 128)) -> torch.Tensor:
    N, K = q.shape
    bn, bk = block
    s = scale_inv.repeat_interleave(bn, 0)[:N].repeat_interleave(bk, 1)[:, :K]
    return q.float() * s


def quantize_act_1x128(x: torch.Tensor, group: int = 128):
    """[T,K] -> (e4m3 [T,K], scales [T, ceil(K/group)] fp32), dynamic per token per group."""
    T, K = x.shape
    g = -(-K // group)
    xp = torch.zeros(T, g * group, dtype=torch.float32, device=x.device)
    xp[:, :K] = x.float()
    xg = xp.view(T, g, group)
    amax = xg.abs().amax(-1).clamp_min(1e-12)
    scale = amax / FP8_MAX
    q = (xg / scale[..., None]).clamp(-FP8_MAX, FP8_MAX).view(T, g * group)[:, :K].to(FP8)
    return q.contiguous(), scale.contiguous()


def fp8_block_gemm_reference(x, wq, w_scale_inv, block=(128, 128), out_dtype=None):
    """Oracle of the block-scaled GEMM: quantise activations 1x128, multiply the e4m3 values, apply
    the product of activation and weight scales per K block (fp32 accumulate)."""
    xq, xs = quantize_act_1x128(x, block[1])
    T, K = x.shape
    N = wq.shape[0]
    bk = block[1]
    acc = torch.zeros(T, N, dtype=torch.float32, device=x.device)
    ws_rows = w_scale_inv.repeat_interleave(block[0], 0)[:N]          # [N, kb]
    for kb in range(-(-K // bk)):
        sl = slice(kb * bk, min(K, (kb + 1) * bk))
        part = xq[:, sl].float() @ wq[:, sl].float().t()
        acc += part * xs[:, kb:kb + 1] * ws_rows[:, kb][None, :]
    return acc.to(out_dtype or x.dtype)


class Fp8BlockLinearMethod(LinearMethodBase):
    """128x128 block-scaled e4m3 weights, dynamic 1x128 e4m3 activations."""

    def __init__(self, block=(128, 128)):
        self.block = tuple(block)

    def create_weights(self, layer) -> None:
        layer.weight = None
        layer.weight_scale_inv = None

    def init_dummy(self, layer, std, seed) -> None:
        from ..layers.linear import seeded_normal
        full = seeded_normal(layer.name, (layer.full_out, layer.full_in), std, torch.bfloat16, layer.device, seed)
        self._set(layer, layer.shard_of(full))

    def _set(self, layer, w_shard):
        q, s = quantize_weight_block(w_shard, self.block)
        layer.weight, layer.weight_scale_inv = q, s

    def load_weight(self, layer, full_weight, scale_inv=None, **kw) -> None:
        if full_weight.dtype != FP8:
            self._set(layer, layer.shard_of(full_weight.to(layer.device)))
            return
        # checkpoint already quantised: slice weight and scale grid consistently
        if scale_inv is None:
            raise ValueError(f"{layer.name}: fp8 checkpoint weight without weight_scale_inv")
        w = layer.shard_of(full_weight.to(layer.device))
        deq_full_rows = layer.shard_of(dequantize_weight_block(full_weight.to(layer.device),
                                                               scale_inv.to(layer.device).float(), self.block))
        bn, bk = self.block
        aligned = (w.shape[0] % bn == 0 or w.shape[0] == full_weight.shape[0]) and \
                  (w.shape[1] % bk == 0 or w.shape[1] == full_weight.shape[1])
        if aligned and envs.B200_REQUANTIZE_BLOCK_SIZE is None:
            layer.weight, layer.weight_scale_inv = w.contiguous(), self._slice_scales(layer, scale_inv)
            if layer.weight_scale_inv is None:
                layer.weight, layer.weight_scale_inv = quantize_weight_block(deq_full_rows, self.block)
        else:
            layer.weight, layer.weight_scale_inv = quantize_weight_block(deq_full_rows, self.block)

    def _slice_scales(self, layer, scale_inv):
        """Scale grid of this rank's shard, or None when some 128x128 block of the shard mixes
        elements of several checkpoint blocks (e.g. half a k block packed next to half a v block)."""
        bn, bk = self.block
        ids = torch.arange(scale_inv.numel(), dtype=torch.float32).view_as(scale_inv)
        full_idx = ids.repeat_interleave(bn, 0)[:layer.full_out].repeat_interleave(bk, 1)[:, :layer.full_in]
        shard_idx = layer.shard_of(full_idx)
        N, K = shard_idx.shape
        nb, kb = -(-N // bn), -(-K // bk)
        first = shard_idx[::bn, ::bk]
        expect = first.repeat_interleave(bn, 0)[:N].repeat_interleave(bk, 1)[:, :K]
        if first.shape != (nb, kb) or not torch.equal(expect, shard_idx):
            return None
        return scale_inv.to(layer.device).float().flatten()[first.long().to(layer.device)].contiguous()

    def apply(self, layer, x, bias=None):
        if x.is_cuda:
            return ops.cuda_ops().fp8_block_gemm(x, layer.weight, layer.weight_scale_inv, bias, self.block)
        y = fp8_block_gemm_reference(x, layer.weight, layer.weight_scale_inv, self.block)
        return y if bias is None else (y.float() + bias.float()).to(y.dtype)

    def apply_quantised(self, layer, xq, xs, bias=None):
        """The product on an activation that is already e4m3 with 1x128 scales (GPU)."""
        y = torch.empty((xq.shape[0], layer.weight.shape[0]), dtype=torch.bfloat16, device=xq.device)
        return ops.cuda_ops().fp8_block_gemm_quantised(xq, xs, layer.weight, layer.weight_scale_inv, y, bias)

    def apply_push_quantised(self, layer, xq, xs, comm):
        return ops.cuda_ops().fp8_block_gemm_push_quantised(xq, xs, layer.weight, layer.weight_scale_inv, comm.heap)

    def can_push(self, fused_tp, T: int, N: int) -> bool:
        # the consumer derives the token tile from T; the fp8 kernel's largest token tile is 128
        return T <= 128 and fused_tp.can_push(T, N)

    def apply_push(self, layer, x, comm):
        """Row-parallel product whose partial goes to every rank from the GEMM epilogue (decode-sized
        outputs); the add + RMSNorm that follows sums what arrived."""
        return ops.cuda_ops().fp8_block_gemm_push(x, layer.weight, layer.weight_scale_inv, comm.heap)

    def weight_bytes(self, layer) -> int:
        return layer.weight.numel() + layer.weight_scale_inv.numel() * 4


class OnlineFp8LinearMethod(Fp8BlockLinearMethod):
    """bf16 checkpoint quantised to block-scaled fp8 while loading."""


class Fp8PerTensorLinearMethod(LinearMethodBase):
    """Per-tensor weight scale, dynamic per-token activation scale."""

    def create_weights(self, layer) -> None:
        layer.weight = None
        layer.weight_scale = None

    def _set(self, layer, w):
        s = w.float().abs().max().clamp_min(1e-12) / FP8_MAX
        layer.weight = (w.float() / s).clamp(-FP8_MAX, FP8_MAX).to(FP8).contiguous()
        layer.weight_scale = s.reshape(1).float()

    def init_dummy(self, layer, std, seed) -> None:
        from ..layers.linear import seeded_normal
        full = seeded_normal(layer.name, (layer.full_out, layer.full_in), std, torch.bfloat16, layer.device, seed)
        self._set(layer, layer.shard_of(full))

    def load_weight(self, layer, full_weight, weight_scale=None, **kw) -> None:
        w = layer.shard_of(full_weight.to(layer.device))
        if full_weight.dtype == FP8 and weight_scale is not None:
            layer.weight, layer.weight_scale = w.contiguous(), weight_scale.to(layer.device).float().reshape(1)
        else:
            self._set(layer, w)

    def apply(self, layer, x, bias=None):
        if x.is_cuda and x.dtype == torch.bfloat16:
            if not hasattr(layer, "_ws_grid"):       # the per-tensor scale repeated over the GEMM's block grid
                N, K = layer.weight.shape
                layer._ws_grid = layer.weight_scale.reshape(1, 1).float().expand(
                    -(-N // 128), -(-K // 128)).contiguous()
            return ops.cuda_ops().fp8_per_tensor_gemm(x, layer.weight, layer.weight_scale, bias, layer._ws_grid)
        xf = x.float()
        xs = xf.abs().amax(-1, keepdim=True).clamp_min(1e-12) / FP8_MAX
        xq = (xf / xs).clamp(-FP8_MAX, FP8_MAX).to(FP8)
        if x.is_cuda:
            y = ops.cuda_ops().fp8_rowwise_gemm(xq, xs, layer.weight, layer.weight_scale, x.dtype)
        else:
            y = ((xq.float() @ layer.weight.float().t()) * xs * layer.weight_scale).to(x.dtype)
        return y if bias is None else (y.float() + bias.float()).to(y.dtype)

    def weight_bytes(self, layer) -> int:
        return layer.weight.numel() + 4


class Fp8BlockMoEMethod:
    """Experts with block-scaled e4m3 weights (grouped block-scaled GEMM)."""
    name = "fp8_block"

    def __init__(self, block=(128, 128), online: bool = False):
        self.block = tuple(block)
        self.online = online

    def create_weights(self, moe) -> None:
        moe.w13 = moe.w2 = moe.w13_scale = moe.w2_scale = None

    def init_dummy(self, moe, std, seed) -> None:
        from ..layers.linear import seeded_normal
        I, H = moe.intermediate_size, moe.hidden_size
        lo, hi = moe.expert_range
        q13, s13, q2, s2 = [], [], [], []
        for e in range(lo, hi):
            a, b = quantize_weight_block(seeded_normal(f"{moe.name}.experts.{e}.w13", (2 * I, H), std,
                                                       torch.bfloat16, moe.device, seed), self.block)
            c, d = quantize_weight_block(seeded_normal(f"{moe.name}.experts.{e}.w2", (H, I), std,
                                                       torch.bfloat16, moe.device, seed), self.block)
            q13.append(a); s13.append(b); q2.append(c); s2.append(d)
        moe.w13, moe.w13_scale = torch.stack(q13), torch.stack(s13)
        moe.w2, moe.w2_scale = torch.stack(q2), torch.stack(s2)

    def alloc(self, moe) -> None:
        E, I, H = moe.num_local_experts, moe.intermediate_size, moe.hidden_size
        bn, bk = self.block
        moe.w13 = torch.zeros(E, 2 * I, H, dtype=FP8, device=moe.device)
        moe.w2 = torch.zeros(E, H, I, dtype=FP8, device=moe.device)
        moe.w13_scale = torch.ones(E, -(-2 * I // bn), -(-H // bk), dtype=torch.float32, device=moe.device)
        moe.w2_scale = torch.ones(E, -(-H // bn), -(-I // bk), dtype=torch.float32, device=moe.device)

    def load_expert(self, moe, local_e, gate, up, down, scales=(None, None, None)) -> None:
        """One expert from the checkpoint (unsharded matrices).  Pieces that are already e4m3 with a
        scale grid are kept bit-exact when this rank's slice starts and ends on block boundaries;
        anything else (bf16 checkpoints, unaligned TP slices) goes through dequantise + quantise."""
        from .unquantized import dequant_expert_pieces, expert_tp_shard
        I, r, n = moe.intermediate_size, moe.tp_rank, moe.tp_size
        bn, bk = self.block
        dev = moe.device
        all_fp8 = all(w.dtype == FP8 and s is not None for w, s in zip((gate, up, down), scales))
        if all_fp8 and I % bn == 0 and I % bk == 0:
            g, u, d = expert_tp_shard(moe, gate, up, down)
            gs, us, ds = scales
            rb, cb = I // bn, I // bk
            if n > 1:
                gs, us, ds = gs[r * rb:(r + 1) * rb], us[r * rb:(r + 1) * rb], ds[:, r * cb:(r + 1) * cb]
            moe.w13[local_e, :I], moe.w13[local_e, I:] = g.to(dev), u.to(dev)
            moe.w2[local_e] = d.to(dev)
            moe.w13_scale[local_e, :rb], moe.w13_scale[local_e, rb:] = gs.to(dev).float(), us.to(dev).float()
            moe.w2_scale[local_e] = ds.to(dev).float()
            return
        g, u, d = expert_tp_shard(moe, *dequant_expert_pieces(moe, (gate, up, down), scales))
        q13, s13 = quantize_weight_block(torch.cat([g, u], 0).to(dev).float(), self.block)
        q2, s2 = quantize_weight_block(d.to(dev).float(), self.block)
        moe.w13[local_e], moe.w13_scale[local_e] = q13, s13
        moe.w2[local_e], moe.w2_scale[local_e] = q2, s2

    def apply(self, moe, x, topk_ids, topk_w):
        if getattr(moe, "activation", "silu") != "silu":
            raise NotImplementedError("block-scaled fp8 experts are built for the SiLU gate only")
        if x.is_cuda:
            return ops.cuda_ops().moe_experts_fp8(x, moe.w13, moe.w13_scale, moe.w2, moe.w2_scale, topk_ids,
                                                  topk_w, moe.expert_range[0], self.block)
        w13 = torch.stack([dequantize_weight_block(moe.w13[e], moe.w13_scale[e], self.block)
                           for e in range(moe.w13.shape[0])]).to(x.dtype)
        w2 = torch.stack([dequantize_weight_block(moe.w2[e], moe.w2_scale[e], self.block)
                          for e in range(moe.w2.shape[0])]).to(x.dtype)
        return ops.ref.moe_experts(x, w13, w2, topk_ids, topk_w, moe.expert_range[0])

    def apply_fused_ep(self, moe, x, topk_ids, topk_w, comm):
        return ops.cuda_ops().moe_experts_ep_fp8(x, moe.w13, moe.w13_scale, moe.w2, moe.w2_scale, topk_ids, topk_w,
                                                 comm.heap, moe.num_experts)

    def weight_bytes(self, moe) -> int:
        return moe.w13.numel() + moe.w2.numel() + 4 * (moe.w13_scale.numel() + moe.w2_scale.numel())
