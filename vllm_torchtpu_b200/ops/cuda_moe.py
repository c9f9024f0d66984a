"""Bindings of the MoE kernels and the SwiGLU / grouped tcgen05 GEMM variants."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from .. import envs
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
    if 0 < envs.B200_GEMM_2SM_MIN_T <= T:
        _c._check(_c.lib().b200_gemm_bf16_swiglu_2sm(
            _c._p(x2), _c._p(w), _c._p(y), c_int(T), c_int(I), c_int(K), c_int(x2.stride(0)), c_int(w.stride(0)),
            c_int(y.stride(0)), _c._p(ws.status), c_int(_c._sms), _c._stream()), "gemm_swiglu_2sm")
        count_launch()
        return y
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


ROUTE_SIM = {"": 0, "off": 0, "uniform": 1, "hash": 2}


def moe_route_post(ids, w, num_experts: int, num_valid=None, sim: str = ""):
    """In place: rows from ``num_valid[0]`` (device int32) on lose their experts; ``sim`` replaces the
    router's choice by a balanced ("uniform") or hashed assignment with weights 1 / k."""
    T, k = ids.shape
    _c._check(_c.lib().b200_moe_route_post(_c._p(ids), _c._p(w), c_int(T), c_int(k), c_int(num_experts),
                                           _c._p(num_valid), c_int(ROUTE_SIM[sim]), _c._stream()), "moe_route_post")
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


def group_bias_add(y, bias, group_off):
    """In place: y[r] += bias[e] for the rows of expert e (rows grouped by expert through ``group_off``)."""
    _c._require_bf16(y, bias)
    R, N = y.shape
    _c._check(_c.lib().b200_group_bias_add(_c._p(y), _c._p(bias), _c._p(group_off), c_int(R), c_int(N),
                                           c_int(y.stride(0)), c_int(bias.shape[0]), _c._stream()), "group_bias_add")
    count_launch()
    return y


def moe_experts(x, w13, w2, topk_ids, topk_w, expert_offset: int = 0, act: str = "silu", b13=None, b2=None):
    """Σ_k w_k · FFN_e(x) over the local experts: permute → grouped SwiGLU GEMM → grouped GEMM →
    weighted un-permute.  w13: [E_local, 2I, H] (gate rows first), w2: [E_local, H, I]."""
    T, H = x.shape
    E_local = w13.shape[0]
    k = topk_ids.shape[1]
    x_perm, group_off, _, inv_pos = moe_permute(x.contiguous(), topk_ids.contiguous(), expert_offset, E_local)
    avg = (T * k + E_local - 1) // E_local
    if act == "silu" and b13 is None:
        h = grouped_gemm(x_perm, w13, group_off, True, avg)          # SiLU * mul in the GEMM epilogue
    else:
        # other gated activations / expert biases: one grouped GEMM over the stacked [gate; up] rows, bias,
        # then the activation kernel
        h = grouped_gemm(x_perm, w13, group_off, False, avg)
        if b13 is not None:
            group_bias_add(h, b13, group_off)
        h = _c.gated_act_and_mul(h, act)
    y = grouped_gemm(h, w2, group_off, False, avg)
    if b2 is not None:
        group_bias_add(y, b2, group_off)
    out = moe_unpermute(y, inv_pos, topk_w.contiguous(), T)
    return out if out.shape[1] == H else out[:, :H].contiguous()      # down projection padded to the tile width


# ----------------------------------------------------------------- expert parallel, fused plane
class EpState:
    """Heap regions and local scratch of the fused expert-parallel plane (one per EP heap).

    ``cap`` rows can be received per call; a call that would need more sets the device status word
    (``ops.cuda.check_status``) and drops the excess rows.  The worst case is world * T_max * k rows
    (every row of every rank routed to one owner: random-init routers of deep models come close); that
    is the default, and a positive ``capacity_factor`` keeps that multiple of the balanced load instead."""

    def __init__(self, heap, max_tokens: int, top_k: int, hidden: int, inter: int, num_experts: int,
                 capacity_factor: float):
        import ctypes
        world = heap.world
        self.heap, self.max_tokens, self.k, self.H, self.E = heap, max_tokens, top_k, hidden, num_experts
        worst = world * max_tokens * top_k
        self.cap = worst if capacity_factor <= 0 else int(min(worst, max(1024, capacity_factor * max_tokens * top_k)))
        self.cnt = heap.alloc("ep_cnt", world * num_experts * 4)
        self.cnt_flag = heap.alloc("ep_cnt_flag", world * 4)
        self.data_flag = heap.alloc("ep_data_flag", world * 4)
        self.ret_flag = heap.alloc("ep_ret_flag", world * 4)
        self.recv_x = heap.alloc("ep_recv_x", self.cap * hidden * 2)
        self.recv_route = heap.alloc("ep_recv_route", self.cap * 8)
        self.ret = heap.alloc("ep_ret", max_tokens * top_k * hidden * 2)
        self.layout = (ctypes.c_ulonglong * 7)(self.cnt.offset, self.cnt_flag.offset, self.data_flag.offset,
                                               self.ret_flag.offset, self.recv_x.offset, self.recv_route.offset,
                                               self.ret.offset)
        dev = heap.device
        self.ctrl = torch.zeros(4, dtype=torch.int32, device=dev)
        self.fill = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self.group_off = torch.zeros(num_experts // world + 1, dtype=torch.int32, device=dev)
        self.act = torch.zeros(self.cap, inter, dtype=torch.bfloat16, device=dev)

    def fp8_scratch(self, inter: int) -> dict:
        """Local buffers of the fp8 expert pipeline (quantised rows, scales, gate|up product), made on
        first use outside graph capture."""
        if getattr(self, "_fp8", None) is None:
            dev, cap, H = self.heap.device, self.cap, self.H
            f8 = torch.float8_e4m3fn
            self._fp8 = {
                "xq1": torch.zeros(cap, H, dtype=f8, device=dev),
                "xs1": torch.zeros(cap, (H + 127) // 128, dtype=torch.float32, device=dev),
                "h": torch.zeros(cap, 2 * inter, dtype=torch.bfloat16, device=dev),
                "xq2": torch.zeros(cap, inter, dtype=f8, device=dev),
                "xs2": torch.zeros(cap, (inter + 127) // 128, dtype=torch.float32, device=dev)}
        return self._fp8

    @staticmethod
    def heap_bytes(max_tokens, top_k, hidden, num_experts, world, capacity_factor) -> int:
        worst = world * max_tokens * top_k
        cap = worst if capacity_factor <= 0 else int(min(worst, max(1024, capacity_factor * max_tokens * top_k)))
        return (cap * hidden * 2 + cap * 8 + max_tokens * top_k * hidden * 2 + world * num_experts * 4
                + (1 << 20))


def moe_experts_ep(x, w13, w2, topk_ids, topk_w, heap, num_experts: int, phase_events: list = None):
    """MoE expert computation under expert parallelism with the dispatch / combine all-to-all done by
    NVLink stores inside the pipeline: rows are PUT into the owners' receive buffers, the owners run
    the grouped tcgen05 GEMMs on what they received, and the epilogue of the second GEMM stores each
    output row into the return slot of the rank the token came from."""
    import ctypes
    from ctypes import c_size_t, c_ulonglong
    _c._require_bf16(x, w13, w2)
    st = heap.ep_state
    T, H = x.shape
    k = topk_ids.shape[1]
    E_local, I = w13.shape[0], w2.shape[2]
    if T > st.max_tokens or k != st.k or H != st.H or num_experts != st.E:
        raise RuntimeError("fused EP plane was configured for a different shape")

    def mark():
        # measurement aid: an event after every phase (dispatch, first GEMM, routed GEMM, combine)
        if phase_events is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            phase_events.append(e)
    mark()
    L = _c.lib()
    ws = _c.Workspace.get(x.device)
    spin = ctypes.c_uint(min(heap.spin_limit, 2**31 - 1))
    x = x.contiguous()
    ids = topk_ids.contiguous()
    _c._check(L.b200_ep_dispatch(heap.peers_c, c_int(heap.rank), c_int(heap.world), st.layout, _c._p(st.ctrl),
                                 _c._p(st.fill), _c._p(st.group_off), _c._p(x), _c._p(ids), c_int(T), c_int(k),
                                 c_int(H), c_int(num_experts), c_int(st.cap), _c._p(ws.status), spin,
                                 _c._stream()), "ep_dispatch")
    count_launch(3)
    mark()
    recv_x = heap.tensor(st.recv_x, (st.cap, H), torch.bfloat16)
    avg = max(1, (T * k) // max(1, E_local))
    grouped_gemm(recv_x, w13, st.group_off, True, avg, out=st.act)
    mark()
    _c._check(L.b200_grouped_gemm_bf16_routed(
        _c._p(st.act), _c._p(w2), _c._p(st.group_off), c_int(E_local), c_int(st.cap), c_int(H), c_int(I),
        c_int(avg), heap.peers_c, c_int(heap.rank), c_int(heap.world),
        c_void_p(heap.local_ptr + st.recv_route.offset), c_ulonglong(st.ret.offset),
        c_ulonglong(st.ret_flag.offset), _c._p(st.ctrl), _c._p(ws.status), c_int(_c._sms), _c._stream()),
        "grouped_gemm_routed")
    count_launch()
    mark()
    out = torch.empty((T, H), dtype=x.dtype, device=x.device)
    topk_w = topk_w.contiguous()
    _c._check(L.b200_ep_combine(c_void_p(heap.local_ptr), c_ulonglong(st.ret.offset),
                                c_ulonglong(st.ret_flag.offset), _c._p(st.ctrl), _c._p(ids),
                                _c._p(topk_w), _c._p(out), c_int(T), c_int(k), c_int(H),
                                c_int(num_experts), c_int(heap.world), _c._p(ws.status), spin, _c._stream()),
              "ep_combine")
    count_launch()
    mark()
    return out
