"""Bindings of the Gated DeltaNet kernels."""
from __future__ import annotations

from ctypes import c_int

import torch

from . import count_launch
from . import cuda as _c


def gdn_forward(mixed, a, b, meta, conv_pool, rec_pool, conv_w, A_log, dt_bias, Hk, Hv, dk, dv):
    """mixed [T, 2*Hk*dk + Hv*dv] bf16 (may be a column slice), a/b [T, Hv] -> o [T, Hv, dv]."""
    _c._require_bf16(mixed, a, b, conv_w)
    T, C = mixed.shape
    dev = mixed.device
    R = meta.padded_num_reqs if meta.padded_num_reqs is not None else meta.num_reqs
    conv_out = torch.empty((T, C), dtype=torch.bfloat16, device=dev)
    qn = torch.empty((T, Hk, dk), dtype=torch.float32, device=dev)
    kn = torch.empty_like(qn)
    g = torch.empty((T, Hv), dtype=torch.float32, device=dev)
    beta = torch.empty_like(g)
    out = torch.zeros((T, Hv, dv), dtype=torch.bfloat16, device=dev)
    _c._check(_c.lib().b200_gdn_forward(
        _c._p(mixed), c_int(mixed.stride(0)), _c._p(a), _c._p(b), c_int(a.stride(0)), _c._p(conv_w),
        _c._p(A_log), _c._p(dt_bias), _c._p(conv_pool), _c._p(rec_pool), _c._p(conv_out), _c._p(qn), _c._p(kn),
        _c._p(g), _c._p(beta), _c._p(out), _c._p(meta.query_start_loc), _c._p(meta.seq_lens),
        _c._p(meta.state_slots), c_int(R), c_int(T), c_int(Hk), c_int(Hv), c_int(dk), c_int(dv),
        c_int(conv_w.shape[1]), _c._stream()), "gdn_forward")
    count_launch(3)
    return out


def kda_forward(q, k, v, a, b, meta, rec_pool, A_log, dt_bias, lower_bound=None):
    """Kimi Delta Attention (per-channel decay).  q, k [T, Hk, dk], v [T, Hv, dv], a [T, Hv, dk], b [T, Hv]
    bf16; A_log [Hv], dt_bias [Hv, dk] fp32; rec_pool [slots, Hv, dk, dv] fp32 -> o [T, Hv, dv]."""
    from ctypes import c_float
    _c._require_bf16(q, k, v, a, b)
    q, k, v, a, b = (t.contiguous() for t in (q, k, v, a, b))
    T, Hk, dk = q.shape
    Hv, dv = v.shape[1], v.shape[2]
    dev = q.device
    R = meta.padded_num_reqs if meta.padded_num_reqs is not None else meta.num_reqs
    qn = torch.empty((T, Hk, dk), dtype=torch.float32, device=dev)
    kn = torch.empty_like(qn)
    g = torch.empty((T, Hv, dk), dtype=torch.float32, device=dev)
    beta = torch.empty((T, Hv), dtype=torch.float32, device=dev)
    out = torch.zeros((T, Hv, dv), dtype=torch.bfloat16, device=dev)
    A_log = A_log.float().contiguous()
    dt_bias = dt_bias.float().contiguous()
    lb = float(lower_bound) if lower_bound is not None else 0.0
    _c._check(_c.lib().b200_kda_forward(
        _c._p(q), _c._p(k), _c._p(v), _c._p(a), _c._p(b), _c._p(A_log), _c._p(dt_bias), c_float(lb),
        _c._p(rec_pool), _c._p(qn), _c._p(kn), _c._p(g), _c._p(beta), _c._p(out), _c._p(meta.query_start_loc),
        _c._p(meta.seq_lens), _c._p(meta.state_slots), c_int(R), c_int(T), c_int(Hk), c_int(Hv), c_int(dk),
        c_int(dv), _c._stream()), "kda_forward")
    count_launch(2)
    return out


def short_conv(x, meta, conv_pool, conv_w):
    """Causal depth-wise conv (kernel 4) + SiLU with the carried window; x [T, C] bf16 (row stride free)."""
    _c._require_bf16(x, conv_w)
    T, C = x.shape
    R = meta.padded_num_reqs if meta.padded_num_reqs is not None else meta.num_reqs
    y = torch.zeros((T, C), dtype=torch.bfloat16, device=x.device)
    _c._check(_c.lib().b200_short_conv(
        _c._p(x), c_int(x.stride(0)), _c._p(conv_w), _c._p(conv_pool), _c._p(y), _c._p(meta.query_start_loc),
        _c._p(meta.seq_lens), _c._p(meta.state_slots), c_int(R), c_int(C), c_int(conv_w.shape[1]), _c._stream()),
        "short_conv")
    count_launch()
    return y
