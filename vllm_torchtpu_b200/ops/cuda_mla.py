"""Bindings of the MLA kernels (``csrc/attention_mla.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong

import torch

from . import count_launch
from . import cuda as _c


def mla_write_cache(cache, kv_c, k_pe, slot_mapping):
    """cache [blocks, block_size, L + R] row of slot s = kv_c[t] ‖ k_pe[t] (slot < 0: skipped)."""
    _c._require_bf16(cache, kv_c, k_pe)
    T, L = kv_c.shape
    R = k_pe.shape[-1]
    assert cache.is_contiguous() and cache.shape[-1] == L + R and kv_c.stride(-1) == 1 and k_pe.stride(-1) == 1
    slots = slot_mapping.to(torch.int32).contiguous()
    _c._check(_c.lib().b200_mla_write_cache(
        _c._p(cache), _c._p(kv_c), _c._p(k_pe), _c._p(slots), c_int(T), c_int(L), c_int(R), c_int(kv_c.stride(0)),
        c_int(k_pe.stride(0)), c_longlong(cache.shape[0] * cache.shape[1]), _c._stream()), "mla_write_cache")
    count_launch()


def mla_paged_attention(q_latent, cache, meta, scale, kv_lora_rank: int, *, topk_indices=None,
                        return_lse: bool = False):
    """Absorbed-query MLA over the paged latent cache; dense, or sparse when ``topk_indices`` [T, K] is given."""
    _c._require_bf16(q_latent, cache)
    q = q_latent.contiguous()
    T, H, Dq = q.shape
    nb, bs, _ = cache.shape
    out = torch.zeros((T, H, kv_lora_rank), dtype=q.dtype, device=q.device)
    lse = torch.full((T, H), float("-inf"), dtype=torch.float32, device=q.device) if return_lse else None
    topk = None
    K = 0
    if topk_indices is not None:
        topk = topk_indices.to(torch.int32).contiguous()
        K = topk.shape[1]
    _c._check(_c.lib().b200_mla_attention(
        _c._p(q), _c._p(cache), _c._p(out), _c._p(lse), _c._p(meta.block_tables), _c._p(meta.seq_lens),
        _c._p(meta.query_start_loc), _c._p(topk), c_int(K), c_int(T), c_int(meta.num_reqs), c_int(H), c_int(Dq),
        c_int(kv_lora_rank), c_int(meta.block_tables.shape[1]), c_int(bs), c_longlong(nb), c_float(scale),
        _c._stream()), "mla_attention")
    count_launch()
    if return_lse:
        return out, lse
    return out
