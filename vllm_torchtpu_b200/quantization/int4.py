"""Group-quantised 4-bit integer weights (AWQ / GPTQ style, W4A16): unsigned nibbles with a
per-group scale (fp16 precision) and zero point along K.  On the GPU the weight stays packed and runs on
the W4A16 tcgen05 kernel (``ops/cuda_fp4.py: w4a16_int4_gemm``); the CPU path dequantises in front of the GEMM."""
from __future__ import annotations

import torch

from .. import ops
from .fp4 import pack_nibbles, unpack_nibbles
from .unquantized import LinearMethodBase


def quantize_int4_group(w: torch.Tensor, group: int = 128):
    N, K = w.shape
    assert K % group == 0
    g = w.float().view(N, K // group, group)
    lo, hi = g.amin(-1), g.amax(-1)
    scale = ((hi - lo) / 15.0).clamp_min(1e-7).half().float()      # checkpoints carry fp16 scales
    zero = torch.round(-lo / scale).clamp(0, 15)
    q = torch.round(g / scale[..., None] + zero[..., None]).clamp(0, 15).to(torch.uint8).view(N, K)
    return pack_nibbles(q), scale.float(), zero.to(torch.uint8)


def dequantize_int4_group(packed, scale, zero, group: int = 128):
    q = unpack_nibbles(packed).float()
    s = scale.repeat_interleave(group, dim=-1)
    z = zero.float().repeat_interleave(group, dim=-1)
    return (q - z) * s


class Int4GroupLinearMethod(LinearMethodBase):
    def __init__(self, fmt: str = "awq", group: int = 128):
        self.fmt, self.group = fmt, group

    def create_weights(self, layer) -> None:
        layer.weight = layer.weight_scale = layer.weight_zero = None

    def init_dummy(self, layer, std, seed) -> None:
        from ..layers.linear import seeded_normal
        full = seeded_normal(layer.name, (layer.full_out, layer.full_in), std, torch.bfloat16, layer.device, seed)
        self._set(layer, layer.shard_of(full))

    def _set(self, layer, w):
        g = self.group if w.shape[1] % self.group == 0 else w.shape[1]
        layer.group = g
        layer.weight, layer.weight_scale, layer.weight_zero = quantize_int4_group(w, g)
        layer.weight_scale_h = layer.weight_scale.half().contiguous() if layer.weight.is_cuda else None

    def load_weight(self, layer, full_weight, **kw) -> None:
        self._set(layer, layer.shard_of(full_weight.to(layer.device)))

    def apply(self, layer, x, bias=None):
        if x.is_cuda and x.dtype == torch.bfloat16 and getattr(layer, "weight_scale_h", None) is not None:
            from ..ops import cuda_fp4
            return cuda_fp4.w4a16_int4_gemm(x, layer.weight, layer.weight_scale_h, layer.weight_zero, layer.group,
                                            bias)
        w = dequantize_int4_group(layer.weight, layer.weight_scale, layer.weight_zero, layer.group).to(x.dtype)
        y = ops.gemm(x, w)
        return y if bias is None else (y.float() + bias.float()).to(y.dtype)

    def weight_bytes(self, layer) -> int:
        return layer.weight.numel() + layer.weight_scale.numel() * 4 + layer.weight_zero.numel()
