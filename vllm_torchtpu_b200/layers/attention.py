"""GQA attention layer over the paged KV cache.

One call does what the reference's attention op does in one kernel
(reference: src/vllm_torchtpu/layers/adapter/attention.py:1464-1698): optional
per-head q/k RMSNorm, RoPE, write of this step's K/V into the request's pages,
then ragged paged attention over the mixed decode/prefill batch.  Under decode
context parallelism the cache is sharded by position and partial results are
merged by their log-sum-exp (``parallel/dcp.py``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..runner.attn_metadata import AttentionMetadata


class PagedAttention:
    def __init__(self, num_q_heads: int, num_kv_heads: int, head_dim: int, inv_freq: torch.Tensor, *,
                 scale: Optional[float] = None, rope_interleaved: bool = False,
                 q_norm_w=None, k_norm_w=None, eps: float = 1e-6, sliding_window=None,
                 softcap=None, sinks=None, k_scale: float = 1.0, v_scale: float = 1.0):
        self.num_q_heads = num_q_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.inv_freq = inv_freq
        self.scale = scale if scale is not None else head_dim ** -0.5
        self.rope_interleaved = rope_interleaved
        self.q_norm_w, self.k_norm_w, self.eps = q_norm_w, k_norm_w, eps
        self.sliding_window, self.softcap, self.sinks = sliding_window, softcap, sinks
        self.k_scale, self.v_scale = k_scale, v_scale

    def forward(self, qkv: torch.Tensor, kv_cache: torch.Tensor, meta: AttentionMetadata) -> torch.Tensor:
        positions, slots = meta.positions, meta.slot_mapping
        T_local = qkv.shape[0]
        if meta.pcp is not None:
            # prefill context parallelism: the k / v columns of the other ranks' pieces are gathered and stored
            # with this rank's own, so the pages are complete before the attention reads them
            from ..parallel.communicator import get_pcp_comm
            from ..runner.pcp_step import gather_remote_kv
            qkv, positions, slots = gather_remote_kv(meta.pcp, qkv, positions, slots,
                                                     self.num_q_heads * self.head_dim, meta.num_tokens, get_pcp_comm())
        q = ops.rope_and_cache(qkv, positions, self.inv_freq, kv_cache, slots,
                               self.num_q_heads, self.num_kv_heads, self.head_dim,
                               self.rope_interleaved, self.q_norm_w, self.k_norm_w, self.eps,
                               self.k_scale, self.v_scale)
        if meta.pcp is not None:
            q = q[:T_local]
        if meta.dcp_size > 1:
            from ..parallel.dcp import dcp_attention
            out = dcp_attention(self, q, kv_cache, meta)
        else:
            out = ops.paged_attention(q, kv_cache, meta, self.scale, sliding_window=self.sliding_window,
                                      softcap=self.softcap, sinks=self.sinks,
                                      k_scale=self.k_scale, v_scale=self.v_scale)
        return out.reshape(out.shape[0], self.num_q_heads * self.head_dim)
