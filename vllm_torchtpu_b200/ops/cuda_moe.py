"""Bindings of the MoE kernels and the SwiGLU / grouped tcgen05 GEMM variants."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from . import count_launch
from . import cuda as _c


def gemm_swiglu(x, w, out=None):
    """silu(x @ w[:I].T) * (x @ w[I:].T) in one tcgen05 kernel; w is [2I, K]."""
    _c._require_bf16(x, w)
    if x.stride(-1) != 1:
        x = x.contiguous()
    x2 = x.reshape(-1, x.shape[-1])
    T, K = x2.shape
    I = w.shape[0] // 2
    y = out if out is not None else torch.empty((T, I), dtype=x.dtype, device=x.device)
    if T == 0:
        return y
    ws = _c.Workspace.get(x.device)
    _c._check(_c.lib().b200_gemm_bf16_swiglu(
        _c._p(x2), _c._p(w), _c._p(y), c_int(T), c_int(I), c_int(K), c_int(x2.stride(0)), c_int(w.stride(0)),
        c_int(y.stride(0)), _c._p(ws.status), c_int(_c._sms), _c._stream()), "gemm_swiglu")
    count_launch()
    return y


def grouped_gemm(x_perm, w, group_off, swiglu: bool, avg_rows: int, out=None):
    """Rows [group_off[e], group_off[e+1]) of x_perm times w[e] ([N,K] or [2N,K] when swiglu)."""
    _c._require_bf16(x_perm, w)
    R, K = x_perm.shape
    E = w.shape[0]
    N = w.shape[1] // 2 if swiglu else w.shape[1]
    y = out if out is not None else torch.empty((R, N), dtype=x_perm.dtype, device=x_perm.device)
    if R == 0:
        return y
    ws = _c.Workspace.get(x_perm.device)
    _c._check(_c.lib().b200_grouped_gemm_bf16(
        _c._p(x_perm), _c._p(w), _c._p(y), _c._p(group_off), c_int(E), c_int(R), c_int(N), c_int(K),
        c_int(1 if swiglu else 0), c_int(max(1, avg_rows)), _c._p(ws.status), c_int(_c._sms), _c._stream()),
        "grouped_gemm")
    count_launch()
    return y


def moe_route(router_logits, top_k, scoring="softmax", renormalize=True, routed_scaling=1.0, score_bias=None,
              n_group=1, topk_group=1):
    T, E = router_logits.shape
    ids = torch.empty((T, top_k), dtype=torch.int32, device=router_logits.device)
    w = torch.empty((T, top_k), dtype=torch.float32, device=router_logits.device)
    _c._check(_c.lib().b200_moe_route(
        _c._p(router_logits), c_int(_c._logit_dtype(router_logits)), c_int(router_logits.stride(0)), c_int(T),
        c_int(E), c_int(top_k), c_int(1 if scoring == "sigmoid" else 0), c_int(1 if renormalize else 0),
        c_float(routed_scaling), _c._p(score_bias), c_int(n_group), c_int(topk_group), _c._p(ids), _c._p(w),
        _c._stream()), "moe_route")
    count_launch()
    return ids, w


def moe_permute(x, topk_ids, e_lo: int, e_local: int):
    T, H = x.shape
    k = topk_ids.shape[1]
    dev = x.device
    group_off = torch.empty(e_local + 1, dtype=torch.int32, device=dev)
    row_src = torch.empty(T * k, dtype=torch.int32, device=dev)
    inv_pos = torch.empty(T * k, dtype=torch.int32, device=dev)
    x_perm = torch.empty((T * k, H), dtype=x.dtype, device=dev)
    _c._check(_c.lib().b200_moe_permute(
        _c._p(x), _c._p(topk_ids), c_int(T), c_int(k), c_int(H), c_int(e_lo), c_int(e_local), _c._p(group_off),
        _c._p(row_src), _c._p(inv_pos), _c._p(x_perm), _c._stream()), "moe_permute")
    count_launch(2)
    return x_perm, group_off, row_src, inv_pos


def moe_unpermute(y, inv_pos, topk_w, T: int):
    H = y.shape[1]
    k = topk_w.shape[1]
    out = torch.empty((T, H), dtype=y.dtype, device=y.device)
    _c._check(_c.lib().b200_moe_unpermute(_c._p(y), _c._p(inv_pos), _c._p(topk_w), _c._p(out), c_int(T),
                                          c_int(H), c_int(k), c_int(y.shape[0]), _c._stream()),
              "moe_unpermute")
    count_launch()
    return out


def moe_experts(x, w13, w2, topk_ids, topk_w, expert_offset: int = 0):
    """Σ_k w_k · FFN_e(x) over the local experts: permute → grouped SwiGLU GEMM → grouped GEMM →
    weighted un-permute.  w13: [E_local, 2I, H] (gate rows first), w2: [E_local, H, I]."""
    T, H = x.shape
    E_local = w13.shape[0]
    k = topk_ids.shape[1]
    x_perm, group_off, _, inv_pos = moe_permute(x.contiguous(), topk_ids.contiguous(), expert_offset, E_local)
    avg = (T * k + E_local - 1) // E_local
    act = grouped_gemm(x_perm, w13, group_off, True, avg)
    y = grouped_gemm(act, w2, group_off, False, avg)
    return moe_unpermute(y, inv_pos, topk_w.contiguous(), T)
