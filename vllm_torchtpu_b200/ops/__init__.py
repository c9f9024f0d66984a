"""Op entry points used by layers.

CUDA tensors go to the hand-written sm_100a kernels (``ops.cuda``, loaded from
the in-tree shared library; a missing library on a GPU box is an error, never a
silent fallback).  CPU tensors go to the plain-PyTorch statements in
``ops.reference`` so the whole engine also runs in CPU unit tests.
"""
from __future__ import annotations

import torch

from . import reference as ref

_cuda = None


def cuda_ops():
    global _cuda
    if _cuda is None:
        from . import cuda as _c
        _cuda = _c
    return _cuda


def _on_gpu(t: torch.Tensor) -> bool:
    return t.is_cuda


def rms_norm(x, weight, eps):
    return cuda_ops().rms_norm(x, weight, eps) if _on_gpu(x) else ref.rms_norm(x, weight, eps)


def materialize(x):
    """A row-parallel output whose cross-rank sum is still pending becomes a tensor."""
    return x.materialize() if hasattr(x, "materialize") else x


def fused_add_rms_norm(x, residual, weight, eps):
    if hasattr(x, "add_rms_norm"):          # pushed partials: the sum rides in this kernel
        return x.add_rms_norm(residual, weight, eps)
    if _on_gpu(x):
        return cuda_ops().fused_add_rms_norm(x, residual, weight, eps)
    return ref.fused_add_rms_norm(x, residual, weight, eps)


def gated_act_and_mul(x, spec: str = "silu"):
    if spec == "silu":
        return silu_and_mul(x)
    return cuda_ops().gated_act_and_mul(x, spec) if _on_gpu(x) else ref.gated_act_and_mul(x, spec)


def silu_and_mul(x):
    return cuda_ops().silu_and_mul(x) if _on_gpu(x) else ref.silu_and_mul(x)


def gemm(x, w, bias=None, out=None):
    return cuda_ops().gemm(x, w, bias, out=out) if _on_gpu(x) else ref.gemm(x, w, bias)


def embedding(ids, table):
    return cuda_ops().embedding(ids, table) if _on_gpu(table) else ref.embedding(ids, table)


def rope_and_cache(qkv, positions, inv_freq, kv_cache, slot_mapping, num_q_heads, num_kv_heads,
                   head_dim, interleaved=False, q_norm_w=None, k_norm_w=None, eps=1e-6,
                   k_scale=1.0, v_scale=1.0):
    f = cuda_ops().rope_and_cache if _on_gpu(qkv) else ref.rope_and_cache
    return f(qkv, positions, inv_freq, kv_cache, slot_mapping, num_q_heads, num_kv_heads, head_dim,
             interleaved, q_norm_w, k_norm_w, eps, k_scale, v_scale)


def paged_attention(q, kv_cache, meta, scale, *, sliding_window=None, softcap=None, sinks=None,
                    k_scale=1.0, v_scale=1.0, return_lse=False):
    if _on_gpu(q):
        return cuda_ops().paged_attention(q, kv_cache, meta, scale, sliding_window=sliding_window,
                                          softcap=softcap, sinks=sinks, k_scale=k_scale,
                                          v_scale=v_scale, return_lse=return_lse)
    return ref.paged_attention(q, kv_cache, meta.block_tables, meta.seq_lens, meta.query_start_loc,
                               scale, num_reqs=meta.num_reqs, sliding_window=sliding_window,
                               softcap=softcap, sinks=sinks, k_scale=k_scale, v_scale=v_scale,
                               return_lse=return_lse, global_seq_lens=meta.global_seq_lens,
                               dcp_size=meta.dcp_size, dcp_rank=meta.dcp_rank,
                               dcp_interleave=meta.dcp_interleave)


def mla_write_cache(cache, kv_c, k_pe, slot_mapping):
    if _on_gpu(cache):
        return cuda_ops().mla_write_cache(cache, kv_c, k_pe, slot_mapping)
    return ref.mla_write_cache(cache, kv_c, k_pe, slot_mapping)


def mla_paged_attention(q_latent, cache, meta, scale, kv_lora_rank, *, topk_indices=None, return_lse=False):
    if _on_gpu(q_latent):
        return cuda_ops().mla_paged_attention(q_latent, cache, meta, scale, kv_lora_rank,
                                              topk_indices=topk_indices, return_lse=return_lse)
    return ref.mla_paged_attention(q_latent, cache, meta.block_tables, meta.seq_lens, meta.query_start_loc,
                                   scale, kv_lora_rank, num_reqs=meta.num_reqs, topk_indices=topk_indices,
                                   return_lse=return_lse)


def sample(logits, temperature, top_k, top_p, uniform=None, all_greedy=False):
    if _on_gpu(logits):
        return cuda_ops().sample(logits, temperature, top_k, top_p, uniform, all_greedy)
    return ref.sample(logits, temperature, top_k, top_p, None if all_greedy else uniform)


def moe_route(router_logits, top_k, **kw):
    if _on_gpu(router_logits):
        return cuda_ops().moe_route(router_logits, top_k, **kw)
    return ref.moe_route(router_logits, top_k, **kw)


# ---- launch accounting ---------------------------------------------------------
_launches = 0


def count_launch(n: int = 1) -> None:
    """Every wrapper of a hand-written kernel calls this once per launch."""
    global _launches
    _launches += n


def launch_count() -> int:
    return _launches
