"""Attention backend object in the shape an external omni runtime asks for: a named backend whose
implementation takes [B, S, H, D] query / key / value and optional metadata carrying a mask
(reference: src/vllm_torchtpu/omni/attention.py:40-136)."""
from __future__ import annotations

from .attention import diffusion_attention


class B200DiffusionAttentionImpl:
    def __init__(self, num_heads: int, head_size: int, softmax_scale: float = None, causal: bool = False,
                 num_kv_heads: int = None, **_):
        self.num_heads, self.head_size = num_heads, head_size
        self.softmax_scale = softmax_scale if softmax_scale is not None else head_size ** -0.5
        self.causal = causal
        self.num_kv_heads = num_kv_heads or num_heads

    def forward(self, query, key, value, attn_metadata=None):
        mask = getattr(attn_metadata, "attn_mask", None) if attn_metadata is not None else None
        return diffusion_attention(query, key, value, self.softmax_scale, self.causal, mask)


class B200DiffusionAttentionBackend:
    accept_output_buffer = False

    @staticmethod
    def get_name() -> str:
        return "B200_TCGEN05_ATTN"

    @staticmethod
    def get_impl_cls():
        return B200DiffusionAttentionImpl

    @staticmethod
    def get_supported_head_sizes() -> list:
        return [64, 128]
