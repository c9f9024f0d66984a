"""Bindings of the small kernels in ``csrc/misc_ops.cu``: LoRA bgmv, token bitmask, pool row copies,
fp8 KV quantisation, TurboQuant 4-bit KV encode/decode."""
from __future__ import annotations

from ctypes import c_float, c_int, c_size_t, c_void_p

import torch

from . import count_launch
from . import cuda as _c


def bgmv_shrink(x, A, idx):
    _c._require_bf16(x, A)
    x = x.contiguous()
    T, K = x.shape
    r = A.shape[1]
    h = torch.empty(T, r, dtype=torch.float32, device=x.device)
    A, idx = A.contiguous(), idx.to(torch.int32).contiguous()                             # kept alive
    _c._check(_c.lib().b200_bgmv_shrink(_c._p(x), _c._p(A), _c._p(idx), _c._p(h),
                                        c_int(T), c_int(K), c_int(r), c_int(x.stride(0)), _c._stream()),
              "bgmv_shrink")
    count_launch()
    return h


def bgmv_expand(h, B, idx, y, scale, col_offset: int = 0):
    _c._require_bf16(B, y)
    assert y.stride(-1) == 1 and h.is_contiguous()
    T, r = h.shape
    N = B.shape[1]
    B, idx, scale = B.contiguous(), idx.to(torch.int32).contiguous(), scale.float().contiguous()
    _c._check(_c.lib().b200_bgmv_expand(_c._p(h), _c._p(B), _c._p(idx),
                                        _c._p(scale), _c._p(y), c_int(T), c_int(N), c_int(r),
                                        c_int(y.stride(0)), c_int(col_offset), _c._stream()), "bgmv_expand")
    count_launch()
    return y


def apply_token_bitmask(logits, bitmask, rows=None):
    """In place: logits[row, v] = -inf where bit v of bitmask[m] is 0 (row = rows[m] or m)."""
    assert logits.stride(-1) == 1
    bm = bitmask.to(device=logits.device, dtype=torch.int32).contiguous()
    rw = None if rows is None else rows.to(device=logits.device, dtype=torch.int64).contiguous()
    _c._check(_c.lib().b200_apply_token_bitmask(
        _c._p(logits), c_int(_c._logit_dtype(logits)), c_int(logits.stride(0)), _c._p(bm), c_int(bm.shape[1]),
        _c._p(rw), c_int(bm.shape[0]), c_int(logits.shape[1]), _c._stream()), "apply_token_bitmask")
    count_launch()
    return logits


def copy_rows(dst, src, dst_idx, src_idx):
    """dst[dst_idx[i]] = src[src_idx[i]] for pools whose rows (dim 0) are contiguous blocks of a
    multiple of 16 bytes: mamba / GDN state slots, KV pool blocks (negative index: skipped)."""
    assert dst.is_contiguous() and src.is_contiguous() and dst.dtype == src.dtype
    row_bytes = dst[0].numel() * dst.element_size()
    assert row_bytes == src[0].numel() * src.element_size()
    n = dst_idx.numel()
    di, si = dst_idx.to(torch.int32).contiguous(), src_idx.to(torch.int32).contiguous()   # kept alive
    _c._check(_c.lib().b200_copy_rows(_c._p(dst), _c._p(src), _c._p(di), _c._p(si), c_int(n),
                                      c_size_t(row_bytes), _c._stream()), "copy_rows")
    count_launch()
    return dst


def quantize_kv_fp8(x, scale: float):
    _c._require_bf16(x)
    x = x.contiguous()
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    _c._check(_c.lib().b200_kv_quant_fp8(_c._p(x), _c._p(q), c_size_t(x.numel()), c_float(scale), c_int(0),
                                         _c._stream()), "kv_quant_fp8")
    count_launch()
    return q


def dequantize_kv_fp8(q, scale: float):
    q = q.contiguous()
    x = torch.empty(q.shape, dtype=torch.bfloat16, device=q.device)
    _c._check(_c.lib().b200_kv_quant_fp8(_c._p(x), _c._p(q), c_size_t(q.numel()), c_float(scale), c_int(1),
                                         _c._stream()), "kv_dequant_fp8")
    count_launch()
    return x


def tq4_encode(k, v):
    _c._require_bf16(k, v)
    rows, D = k.shape
    assert D == 128 and v.shape == k.shape
    dev = k.device
    kc = torch.empty(rows, 64, dtype=torch.uint8, device=dev)
    vc = torch.empty(rows, 64, dtype=torch.uint8, device=dev)
    kn = torch.empty(rows, dtype=torch.bfloat16, device=dev)
    vm = torch.empty(rows, 2, dtype=torch.bfloat16, device=dev)
    k, v = k.contiguous(), v.contiguous()
    _c._check(_c.lib().b200_tq4_encode(_c._p(k), _c._p(v), _c._p(kc), _c._p(kn),
                                       _c._p(vc), _c._p(vm), c_int(rows), _c._stream()), "tq4_encode")
    count_launch()
    return kc, kn, vc, vm


def tq4_decode(kc, kn, vc, vm):
    rows = kc.shape[0]
    k = torch.empty(rows, 128, dtype=torch.bfloat16, device=kc.device)
    v = torch.empty_like(k)
    _c._check(_c.lib().b200_tq4_decode(_c._p(kc), _c._p(kn), _c._p(vc), _c._p(vm), _c._p(k), _c._p(v),
                                       c_int(rows), _c._stream()), "tq4_decode")
    count_launch()
    return k, v


def kv_write(key, value, kv_cache, slot_mapping):
    """Write already-rotated keys / values [T, Hkv, D] (bf16, unit stride in D) into the paged cache
    [blocks, 2, Hkv, block_size, D] at ``slot_mapping`` (int32 or int64; negative slots are skipped)."""
    from ctypes import c_longlong
    _c._require_bf16(key, value, kv_cache)
    T, Hkv, D = key.shape
    assert key.stride(2) == 1 and value.stride(2) == 1 and key.stride(1) == D and value.stride(1) == D
    nb, _, _, bs, _ = kv_cache.shape
    s64 = slot_mapping if slot_mapping.dtype == torch.int64 else None
    s32 = slot_mapping if slot_mapping.dtype == torch.int32 else None
    if s64 is None and s32 is None:
        raise TypeError("slot_mapping must be int32 or int64")
    n = min(T, slot_mapping.numel())
    _c._check(_c.lib().b200_kv_write(_c._p(key), _c._p(value), _c._p(kv_cache), _c._p(s64), _c._p(s32), c_int(n),
                                     c_int(Hkv), c_int(D), c_int(bs), c_longlong(nb), c_longlong(key.stride(0)),
                                     c_longlong(value.stride(0)), _c._stream()), "kv_write")
    count_launch()
