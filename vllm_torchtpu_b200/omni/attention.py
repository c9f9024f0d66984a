"""Attention for diffusion transformers: dense, bidirectional, long sequences (a 480p video is ~33 k tokens).

bf16 self-attention without a mask runs on the package's tcgen05 prefill kernel with the causal mask off
(the kernel behind the vision encoders); anything else (a mask, causal, cross-attention with a different
key length, another dtype, a head size the kernel does not take) goes to PyTorch SDPA with a warning that is
logged once per reason (reference: src/vllm_torchtpu/omni/attention.py:60-136)."""
from __future__ import annotations

from typing import Optional

import torch

from ..logger import init_logger

logger = init_logger(__name__)
_warned: set = set()


def _fallback_reason(q, k, causal, attn_mask) -> Optional[str]:
    if not q.is_cuda:
        return "not on a GPU"
    if causal:
        return "causal=True"
    if attn_mask is not None:
        return "attn_mask is not None"
    if q.dtype != torch.bfloat16:
        return f"dtype {q.dtype} (bfloat16 needed)"
    if q.shape[1] != k.shape[1]:
        return "query and key lengths differ"
    if q.shape[-1] not in (64, 128):
        return f"head_dim {q.shape[-1]}"
    return None


def sdpa_bshd(q, k, v, scale=None, causal=False, attn_mask=None):
    """PyTorch SDPA on [B, S, H, D] tensors; fewer key heads than query heads are repeated."""
    Hq, Hkv = q.shape[2], k.shape[2]
    if Hq != Hkv:
        k, v = k.repeat_interleave(Hq // Hkv, dim=2), v.repeat_interleave(Hq // Hkv, dim=2)
    o = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=attn_mask, is_causal=causal, scale=scale)
    return o.transpose(1, 2)


def diffusion_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None,
                        causal: bool = False, attn_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [B, Sq, Hq, D], k / v [B, Sk, Hkv, D] -> [B, Sq, Hq, D]."""
    if q.shape[2] % k.shape[2] != 0:
        raise ValueError(f"num_heads ({q.shape[2]}) must be a multiple of num_kv_heads ({k.shape[2]})")
    why = _fallback_reason(q, k, causal, attn_mask)
    if why is not None:
        if q.is_cuda and why not in _warned:
            _warned.add(why)
            logger.warning("diffusion attention falls back to PyTorch SDPA (%s)", why)
        return sdpa_bshd(q, k, v, scale, causal, attn_mask)
    from .. import ops
    B, S, Hq, D = q.shape
    cu = [i * S for i in range(B + 1)]
    o = ops.cuda_ops().encoder_attention(q.reshape(B * S, Hq, D), k.reshape(B * S, -1, D), v.reshape(B * S, -1, D),
                                         cu, scale)
    return o.view(B, S, Hq, D)
