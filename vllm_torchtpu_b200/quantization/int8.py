"""W8A8 int8: per-output-channel symmetric weight scales, dynamic per-token activation
scales (the compressed-tensors W8A8-int8 scheme;
reference: src/vllm_torchtpu/layers/adapter/quantization/compressed_tensors/, kernels/quantized_matmul/)."""
from __future__ import annotations

import torch

from .. import ops
from .unquantized import LinearMethodBase


def quantize_weight_int8(w: torch.Tensor):
    s = w.float().abs().amax(dim=1, keepdim=True).clamp_min(1e-12) / 127.0
    q = torch.round(w.float() / s).clamp(-127, 127).to(torch.int8)
    return q.contiguous(), s.squeeze(1).float().contiguous()


def quantize_act_int8(x: torch.Tensor):
    s = x.float().abs().amax(dim=-1, keepdim=True).clamp_min(1e-12) / 127.0
    q = torch.round(x.float() / s).clamp(-127, 127).to(torch.int8)
    return q, s.float()


def int8_gemm_reference(x, wq, w_scale):
    xq, xs = quantize_act_int8(x)
    acc = xq.to(torch.int32).float() @ wq.to(torch.int32).float().t()       # exact in fp32 for K < 2^10ish blocks
    return (acc * xs * w_scale[None, :]).to(x.dtype)


class Int8LinearMethod(LinearMethodBase):
    def create_weights(self, layer) -> None:
        layer.weight = None
        layer.weight_scale = None

    def init_dummy(self, layer, std, seed) -> None:
        from ..layers.linear import seeded_normal
        full = seeded_normal(layer.name, (layer.full_out, layer.full_in), std, torch.bfloat16, layer.device, seed)
        layer.weight, layer.weight_scale = quantize_weight_int8(layer.shard_of(full))

    def load_weight(self, layer, full_weight, weight_scale=None, **kw) -> None:
        w = layer.shard_of(full_weight.to(layer.device))
        if full_weight.dtype == torch.int8 and weight_scale is not None:
            ws = weight_scale.to(layer.device).float().reshape(-1)
            rows = layer.shard_of(ws[:, None].expand(-1, layer.full_in))[:, 0] if ws.numel() == layer.full_out else ws
            layer.weight, layer.weight_scale = w.contiguous(), rows.contiguous()
        else:
            layer.weight, layer.weight_scale = quantize_weight_int8(w)

    def apply(self, layer, x, bias=None):
        if x.is_cuda:
            y = ops.cuda_ops().int8_gemm(x, layer.weight, layer.weight_scale)
        else:
            y = int8_gemm_reference(x, layer.weight, layer.weight_scale)
        return y if bias is None else (y.float() + bias.float()).to(y.dtype)

    def weight_bytes(self, layer) -> int:
        return layer.weight.numel() + layer.weight_scale.numel() * 4
