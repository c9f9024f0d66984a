"""4-bit float weight formats.

* mxfp4: e2m1 values, one e8m0 (power-of-two) scale per 32 elements along K
  (reference: src/vllm_torchtpu/layers/core/quantization.py:106-195, 334-360).
* nvfp4: e2m1 values, one e4m3 scale per 16 elements plus a per-tensor fp32 scale
  (reference: src/vllm_torchtpu/layers/adapter/quantization/nvfp4.py).

Two nibbles are packed per byte (low nibble = even index).  Activations stay bf16
(W4A16): the GPU kernel expands a weight tile to bf16 in shared memory in front of
the tensor-core mainloop; the CPU path dequantises the whole weight.
"""
from __future__ import annotations

import torch

from .. import ops
from .unquantized import LinearMethodBase

E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                            -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def _nearest_e2m1(x: torch.Tensor) -> torch.Tensor:
    """Codes 0..15 of the e2m1 value nearest to x (ties to the smaller magnitude code)."""
    mags = E2M1_VALUES[:8].to(x.device)
    idx = (x.abs()[..., None] - mags).abs().argmin(-1)
    return (idx + (x < 0).long() * 8).to(torch.uint8)


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).to(torch.uint8)


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    lo, hi = packed & 0xF, packed >> 4
    return torch.stack([lo, hi], dim=-1).flatten(-2)


def quantize_mxfp4(w: torch.Tensor, group: int = 32):
    N, K = w.shape
    assert K % group == 0
    g = w.float().view(N, K // group, group)
    amax = g.abs().amax(-1).clamp_min(2.0 ** -126)
    exp = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    scale = torch.exp2(exp)
    codes = _nearest_e2m1(g / scale[..., None]).view(N, K)
    return pack_nibbles(codes), (exp + 127).to(torch.uint8)          # e8m0 biased exponent


def dequantize_mxfp4(packed: torch.Tensor, e8m0: torch.Tensor, group: int = 32) -> torch.Tensor:
    codes = unpack_nibbles(packed).long()
    vals = E2M1_VALUES.to(packed.device)[codes]
    scale = torch.exp2(e8m0.float() - 127.0).repeat_interleave(group, dim=-1)
    return vals * scale


def quantize_nvfp4(w: torch.Tensor, group: int = 16):
    N, K = w.shape
    assert K % group == 0
    wf = w.float()
    global_scale = wf.abs().max().clamp_min(1e-12) / (448.0 * 6.0)
    g = wf.view(N, K // group, group)
    bs = (g.abs().amax(-1) / 6.0 / global_scale).clamp(2.0 ** -9, 448.0).to(torch.float8_e4m3fn)
    scale = bs.float() * global_scale
    codes = _nearest_e2m1(g / scale[..., None].clamp_min(1e-30)).view(N, K)
    return pack_nibbles(codes), bs, global_scale.reshape(1).float()


def dequantize_nvfp4(packed, block_scale, global_scale, group: int = 16) -> torch.Tensor:
    codes = unpack_nibbles(packed).long()
    vals = E2M1_VALUES.to(packed.device)[codes]
    scale = (block_scale.float() * global_scale).repeat_interleave(group, dim=-1)
    return vals * scale


class _Fp4Base(LinearMethodBase):
    def create_weights(self, layer) -> None:
        layer.weight = None
        layer.weight_scale = None
        layer.weight_global_scale = None

    def init_dummy(self, layer, std, seed) -> None:
        from ..layers.linear import seeded_normal
        full = seeded_normal(layer.name, (layer.full_out, layer.full_in), std, torch.bfloat16, layer.device, seed)
        self._set(layer, layer.shard_of(full))

    def load_weight(self, layer, full_weight, **kw) -> None:
        if full_weight.dtype == torch.uint8:
            raise NotImplementedError("pre-packed fp4 checkpoints are re-sharded by the loader")
        self._set(layer, layer.shard_of(full_weight.to(layer.device)))

    fmt = None            # name of the kernel format, set by the subclasses

    def apply(self, layer, x, bias=None):
        if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 64 == 0:
            # W4A16 on the tensor cores: the packed weight is expanded tile by tile in shared memory
            return ops.cuda_ops().w4a16_gemm(x, layer.weight, layer.weight_scale, self.fmt,
                                             layer.weight_global_scale, bias)
        w = self.dequant(layer).to(x.dtype)
        y = ops.gemm(x, w)
        return y if bias is None else (y.float() + bias.float()).to(y.dtype)

    def weight_bytes(self, layer) -> int:
        return layer.weight.numel() + layer.weight_scale.numel()


class Mxfp4LinearMethod(_Fp4Base):
    fmt = "mxfp4"

    def _set(self, layer, w):
        layer.weight, layer.weight_scale = quantize_mxfp4(w)

    def dequant(self, layer):
        return dequantize_mxfp4(layer.weight, layer.weight_scale)


class Nvfp4LinearMethod(_Fp4Base):
    fmt = "nvfp4"

    def _set(self, layer, w):
        layer.weight, layer.weight_scale, layer.weight_global_scale = quantize_nvfp4(w)

    def dequant(self, layer):
        return dequantize_nvfp4(layer.weight, layer.weight_scale, layer.weight_global_scale)


class Mxfp4MoEMethod:
    """mxfp4 experts (W4A16): packed e2m1 + e8m0 per 32, expanded to bf16 per expert tile."""
    name = "mxfp4"

    def create_weights(self, moe) -> None:
        moe.w13 = moe.w2 = moe.w13_scale = moe.w2_scale = None

    def init_dummy(self, moe, std, seed) -> None:
        from ..layers.linear import seeded_normal
        I, H = moe.intermediate_size, moe.hidden_size
        lo, hi = moe.expert_range
        a, b, c, d = [], [], [], []
        for e in range(lo, hi):
            q, s = quantize_mxfp4(seeded_normal(f"{moe.name}.experts.{e}.w13", (2 * I, H), std, torch.bfloat16,
                                                moe.device, seed))
            a.append(q); b.append(s)
            q, s = quantize_mxfp4(seeded_normal(f"{moe.name}.experts.{e}.w2", (H, I), std, torch.bfloat16,
                                                moe.device, seed))
            c.append(q); d.append(s)
        moe.w13, moe.w13_scale, moe.w2, moe.w2_scale = map(torch.stack, (a, b, c, d))
        from .unquantized import padded_hidden
        if padded_hidden(moe) != H:          # zero rows up to the kernels' tile (e8m0 scale byte 0 = 2^-127)
            extra = padded_hidden(moe) - H
            moe.w2 = torch.nn.functional.pad(moe.w2, (0, 0, 0, extra)).contiguous()
            moe.w2_scale = torch.nn.functional.pad(moe.w2_scale, (0, 0, 0, extra)).contiguous()

    def alloc(self, moe) -> None:
        E, I, H = moe.num_local_experts, moe.intermediate_size, moe.hidden_size
        moe.w13 = torch.zeros(E, 2 * I, H // 2, dtype=torch.uint8, device=moe.device)
        from .unquantized import padded_hidden
        Hp = padded_hidden(moe)
        moe.w2 = torch.zeros(E, Hp, I // 2, dtype=torch.uint8, device=moe.device)
        moe.w13_scale = torch.zeros(E, 2 * I, H // 32, dtype=torch.uint8, device=moe.device)
        moe.w2_scale = torch.zeros(E, Hp, I // 32, dtype=torch.uint8, device=moe.device)

    def load_expert(self, moe, local_e, gate, up, down, scales=(None, None, None)) -> None:
        """One expert from a bf16 (or block-scaled fp8) checkpoint, quantised to mxfp4 here."""
        from .unquantized import dequant_expert_pieces, expert_tp_shard
        g, u, d = expert_tp_shard(moe, *dequant_expert_pieces(moe, (gate, up, down), scales))
        q, s = quantize_mxfp4(torch.cat([g, u], 0).to(moe.device).float())
        moe.w13[local_e], moe.w13_scale[local_e] = q, s
        q, s = quantize_mxfp4(d.to(moe.device).float())
        moe.w2[local_e, :moe.hidden_size], moe.w2_scale[local_e, :moe.hidden_size] = q, s

    def load_packed_expert(self, moe, local_e, w13_q, w13_s, w2_q, w2_s) -> None:
        """One expert that is mxfp4 in the checkpoint already: packed nibbles [rows, K / 2] and e8m0 scales
        [rows, K / 32], gate rows first in w13; stored as they are."""
        if moe.tp_size != 1:
            raise NotImplementedError("packed mxfp4 experts are loaded unsharded (expert parallelism or one rank)")
        moe.w13[local_e], moe.w13_scale[local_e] = w13_q.to(moe.device), w13_s.to(moe.device)
        moe.w2[local_e, :moe.hidden_size] = w2_q.to(moe.device)
        moe.w2_scale[local_e, :moe.hidden_size] = w2_s.to(moe.device)

    def apply(self, moe, x, topk_ids, topk_w):
        I, H = moe.intermediate_size, moe.hidden_size
        kw = dict(act=moe.activation, b13=getattr(moe, "b13", None), b2=getattr(moe, "b2", None))
        if x.is_cuda and x.dtype == torch.bfloat16 and H % 64 == 0 and I % 64 == 0:
            # K of both GEMMs a multiple of 64; N = 2I a multiple of 128, N = hidden padded to 128 at load
            return ops.cuda_ops().moe_experts_w4a16(x, moe.w13, moe.w13_scale, moe.w2, moe.w2_scale, topk_ids, topk_w,
                                                    moe.expert_range[0], "mxfp4", **kw)
        w13 = dequantize_mxfp4(moe.w13, moe.w13_scale).to(x.dtype)
        w2 = dequantize_mxfp4(moe.w2, moe.w2_scale).to(x.dtype)
        if x.is_cuda:
            return ops.cuda_ops().moe_experts(x, w13, w2, topk_ids, topk_w, moe.expert_range[0], **kw)
        return ops.ref.moe_experts(x, w13, w2, topk_ids, topk_w, moe.expert_range[0], **kw)

    def weight_bytes(self, moe) -> int:
        return sum(t.numel() for t in (moe.w13, moe.w2, moe.w13_scale, moe.w2_scale))
