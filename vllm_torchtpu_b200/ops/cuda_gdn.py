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
