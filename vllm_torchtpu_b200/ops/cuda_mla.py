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
    # split-KV when the batch alone leaves SMs idle (decode): about three CTAs per SM and at least four
    # 16-row chunks per split.  Inside a captured graph the choice depends on the batch shape only (lengths
    # change between replays; a split without keys contributes lse = -inf).
    groups = (H + 15) // 16
    splits = 1
    if T * groups < 2 * _c._sms:
        splits = max(1, min(16, (3 * _c._sms) // max(1, T * groups)))
        if not torch.cuda.is_current_stream_capturing():
            n_kv = K if topk is not None else max(1, int(meta.max_seq_len or 0))
            splits = max(1, min(splits, n_kv // 64))
    part_o = part_lse = None
    if splits > 1:
        part_o = torch.empty((splits, T, H, kv_lora_rank), dtype=q.dtype, device=q.device)
        part_lse = torch.empty((splits, T, H), dtype=torch.float32, device=q.device)
    _c._check(_c.lib().b200_mla_attention(
        _c._p(q), _c._p(cache), _c._p(out), _c._p(lse), _c._p(meta.block_tables), _c._p(meta.seq_lens),
        _c._p(meta.query_start_loc), _c._p(topk), c_int(K), c_int(T), c_int(meta.num_reqs), c_int(H), c_int(Dq),
        c_int(kv_lora_rank), c_int(meta.block_tables.shape[1]), c_int(bs), c_longlong(nb), c_float(scale),
        c_int(splits), _c._p(part_o), _c._p(part_lse), _c._stream()), "mla_attention")
    count_launch(2 if splits > 1 else 1)
    if return_lse:
        return out, lse
    return out


def permute_rows(src, dst, A: int, B: int, D: int, src_strides, dst_strides):
    """dst[b, a, :D] = src[a, b, :D] with explicit element strides (src: (stride_a, stride_b), dst likewise)."""
    _c._require_bf16(src, dst)
    _c._check(_c.lib().b200_permute_rows(
        _c._p(src), _c._p(dst), c_int(A), c_int(B), c_int(D), c_longlong(src_strides[0]), c_longlong(src_strides[1]),
        c_longlong(dst_strides[0]), c_longlong(dst_strides[1]), _c._stream()), "permute_rows")
    count_launch()


def rope_rows(src, dst, positions, inv_freq, T: int, H: int, interleaved: bool, src_strides, dst_strides):
    """Rotary embedding of 2 * len(inv_freq) dims of src[t, h] into dst[t, h] (element strides (t, h))."""
    _c._require_bf16(src, dst)
    pos = positions if positions.dtype == torch.int32 else positions.to(torch.int32)
    _c._check(_c.lib().b200_rope_rows(
        _c._p(src), _c._p(dst), _c._p(pos), _c._p(inv_freq), c_int(T), c_int(H), c_int(inv_freq.numel()),
        c_int(1 if interleaved else 0), c_longlong(src_strides[0]), c_longlong(src_strides[1]),
        c_longlong(dst_strides[0]), c_longlong(dst_strides[1]), _c._stream()), "rope_rows")
    count_launch()


_head_offsets: dict = {}


def mla_absorb(q, kv, positions, inv_freq, w_uk_t, nope: int, rope: int, kv_lora: int, interleaved: bool):
    """Query side of absorbed MLA on this package's kernels.

    q [T, H, nope + rope] and kv [T, kv_lora + rope] (the k_pe columns) ->
    q_latent [T, H, kv_lora + rope] (q_nope . W_UK per head through the grouped tcgen05 GEMM with heads as
    groups, then the rotated rope dims) and k_pe [T, rope] rotated."""
    T, H, Dq = q.shape
    dev = q.device
    assert q.is_contiguous() and kv.stride(-1) == 1
    q_hm = torch.empty((H * T, nope), dtype=q.dtype, device=dev)
    permute_rows(q, q_hm, T, H, nope, (H * Dq, Dq), (nope, T * nope))
    ql_hm = _c.grouped_gemm(q_hm, w_uk_t, head_offsets(H, T, dev), False, T)
    q_latent = torch.empty((T, H, kv_lora + rope), dtype=q.dtype, device=dev)
    permute_rows(ql_hm, q_latent, H, T, kv_lora, (T * kv_lora, kv_lora), (kv_lora + rope, H * (kv_lora + rope)))
    rope_rows(q[:, :, nope:], q_latent[:, :, kv_lora:], positions, inv_freq, T, H, interleaved, (H * Dq, Dq),
              (H * (kv_lora + rope), kv_lora + rope))
    k_pe = torch.empty((T, rope), dtype=q.dtype, device=dev)
    rope_rows(kv[:, kv_lora:], k_pe, positions, inv_freq, T, 1, interleaved, (kv.stride(0), 0), (rope, 0))
    return q_latent, k_pe


def mla_unabsorb(o_lat, w_uv_t):
    """o_lat [T, H, L] x W_UV per head -> [T, H * v] (grouped tcgen05 GEMM, heads as groups)."""
    T, H, L = o_lat.shape
    v = w_uv_t.shape[1]
    dev = o_lat.device
    o_hm = torch.empty((H * T, L), dtype=o_lat.dtype, device=dev)
    permute_rows(o_lat, o_hm, T, H, L, (H * L, L), (L, T * L))
    y_hm = _c.grouped_gemm(o_hm, w_uv_t, head_offsets(H, T, dev), False, T)
    y = torch.empty((T, H * v), dtype=o_lat.dtype, device=dev)
    permute_rows(y_hm, y, H, T, v, (T * v, v), (v, H * v))
    return y


def head_offsets(H: int, T: int, device):
    """Row offsets [0, T, 2T, ...] of the head-major layout, kept per (H, T) so that graph capture sees a
    fixed address."""
    key = (H, T, str(device))
    t = _head_offsets.get(key)
    if t is None:
        t = (torch.arange(H + 1, dtype=torch.int32, device=device) * T).contiguous()
        _head_offsets[key] = t
    return t
