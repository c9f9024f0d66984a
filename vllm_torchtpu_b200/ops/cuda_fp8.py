"""Bindings of the block-scaled fp8 tcgen05 GEMM family."""
from __future__ import annotations

from ctypes import c_int, c_ulonglong, c_void_p

import torch

from . import count_launch
from . import cuda as _c

FP8 = torch.float8_e4m3fn


def quant_act_1x128(x):
    """bf16 [T, K] -> (e4m3 [T, K], fp32 scales [T, ceil(K/128)])."""
    _c._require_bf16(x)
    if x.stride(-1) != 1:
        x = x.contiguous()
    T, K = x.shape
    xq = torch.empty((T, K), dtype=FP8, device=x.device)
    xs = torch.empty((T, (K + 127) // 128), dtype=torch.float32, device=x.device)
    if T:
        _c._check(_c.lib().b200_quant_rows_1x128(_c._p(x), _c._p(xq), _c._p(xs), c_int(T), c_int(K),
                                                 c_int(x.stride(0)), c_void_p(0), c_int(0), c_int(_c._sms),
                                                 _c._stream()), "quant_rows_1x128")
        count_launch()
    return xq, xs


def quant_rows_1x128(x, K: int, rows=None, swiglu: bool = False, out=None):
    """Quantise the first ``rows[0]`` rows (device int32; all rows when None) of bf16 ``x`` to e4m3 with
    1x128 scales.  With ``swiglu`` the rows hold [gate(K) | up(K)] and SiLU(gate) * up is quantised, so
    the activation never goes back to memory in bf16.  ``out``: (xq [T, K], xs [T, ceil(K/128)])."""
    _c._require_bf16(x)
    assert x.stride(-1) == 1 and x.shape[1] == (2 * K if swiglu else K)
    T = x.shape[0]
    if out is None:
        out = (torch.empty((T, K), dtype=FP8, device=x.device),
               torch.empty((T, (K + 127) // 128), dtype=torch.float32, device=x.device))
    xq, xs = out
    _c._check(_c.lib().b200_quant_rows_1x128(_c._p(x), _c._p(xq), _c._p(xs), c_int(T), c_int(K), c_int(x.stride(0)),
                                             _c._p(rows), c_int(1 if swiglu else 0), c_int(_c._sms),
                                             _c._stream()), "quant_rows_1x128")
    count_launch()
    return xq, xs


def _grouped_fp8_launch(xq, xs, wq, w_scale, group_off, avg_rows: int, y):
    R, K = xq.shape
    E, N = wq.shape[0], wq.shape[1]
    ws = _c.Workspace.get(xq.device)
    from .. import envs
    if envs.B200_FP8_ROWS_MIN_TILES >= 0 and avg_rows >= 256 and use_rows_kernel(R, N):
        _c._check(_c.lib().b200_grouped_gemm_fp8_block_rows(
            _c._p(xq), _c._p(xs), _c._p(wq), _c._p(w_scale), _c._p(y), _c._p(group_off), c_int(E), c_int(R),
            c_int(N), c_int(K), _c._p(ws.status), c_int(_c._sms), _c._stream()), "grouped_gemm_fp8_block_rows")
        count_launch()
        return y
    _c._check(_c.lib().b200_grouped_gemm_fp8_block(
        _c._p(xq), _c._p(xs), _c._p(wq), _c._p(w_scale), _c._p(y), _c._p(group_off), c_int(E), c_int(R),
        c_int(N), c_int(K), c_int(max(1, avg_rows)), _c._p(ws.status), c_int(_c._sms), _c._stream()),
        "grouped_gemm_fp8_block")
    count_launch()
    return y


def use_rows_kernel(T: int, N: int) -> bool:
    """The many-token kernel (tokens on the TMEM lanes, one scale scalar per thread and K block) pays off
    once its 128 x 256 tiles fill most of the SMs; below that the weight-major kernel with split-K does."""
    from .. import envs
    min_tiles = envs.B200_FP8_ROWS_MIN_TILES
    return min_tiles >= 0 and T > 128 and (-(-T // 128)) * (-(-N // 256)) >= min_tiles


_last_quant = None       # (tensor kept alive, key, xq, xs): the activation most recently quantised


def quant_act_shared(x2):
    """``quant_act_1x128`` that recognises the activation it quantised last: projections that read the same
    tensor (q_a / kv_a of MLA, a shared expert next to the router) quantise it once.  The tensor is kept
    alive while cached, so its address cannot be handed to another tensor; an in-place write bumps its
    version and misses."""
    global _last_quant
    key = (x2.data_ptr(), tuple(x2.shape), tuple(x2.stride()), x2._version)
    if _last_quant is not None and _last_quant[1] == key:
        return _last_quant[2], _last_quant[3]
    xq, xs = quant_act_1x128(x2)
    _last_quant = (x2, key, xq, xs)
    return xq, xs


def fp8_block_gemm(x, wq, w_scale_inv, bias=None, block=(128, 128), out=None):
    """x bf16 [T,K]; wq e4m3 [N,K]; w_scale_inv fp32 [ceil(N/128), ceil(K/128)] -> bf16 [T,N]."""
    if tuple(block) != (128, 128):
        raise NotImplementedError("the fp8 kernel is built for 128x128 weight blocks")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    T, K = x2.shape
    N = wq.shape[0]
    xq, xs = quant_act_shared(x2)
    y = out if out is not None else torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return y.reshape(*lead, N)
    fp8_block_gemm_quantised(xq, xs, wq, w_scale_inv, y, bias)
    return y.reshape(*lead, N)


def fp8_block_gemm_quantised(xq, xs, wq, w_scale_inv, y, bias=None):
    """The GEMM alone on operands that are already e4m3 with their scales; picks the kernel by shape."""
    T, K = xq.shape
    N = wq.shape[0]
    ws = _c.Workspace.get(xq.device)
    fn, name = ((_c.lib().b200_gemm_fp8_block_rows, "gemm_fp8_block_rows") if use_rows_kernel(T, N)
                else (_c.lib().b200_gemm_fp8_block, "gemm_fp8_block"))
    _c._check(fn(_c._p(xq), _c._p(xs), _c._p(wq), _c._p(w_scale_inv), _c._p(y), _c._p(bias), c_int(T), c_int(N),
                 c_int(K), c_int(y.stride(0)), _c._p(ws.status), c_int(_c._sms), _c._stream()), name)
    count_launch()
    return y


def fp8_block_gemm_push(x, wq, w_scale_inv, heap):
    """Row-parallel block-scaled fp8 ``x @ wq.T`` whose bf16 partial is pushed to every rank of ``heap``
    from the GEMM epilogue; returns the :class:`PendingReduce` the next add + RMSNorm (or
    ``materialize``) completes.  For at most 128 tokens within ``FusedTP.can_push``."""
    x2 = x.reshape(-1, x.shape[-1])
    xq, xs = quant_act_shared(x2)
    return fp8_block_gemm_push_quantised(xq, xs, wq, w_scale_inv, heap, x.shape[:-1])


def fp8_block_gemm_push_quantised(xq, xs, wq, w_scale_inv, heap, lead_shape=None):
    """The push GEMM on an activation that is already e4m3 with 1x128 scales."""
    st = heap.fused_tp
    T, K = xq.shape
    N = wq.shape[0]
    part = st.parts[st.flip]
    st.flip ^= 1
    ws = _c.Workspace.get(xq.device)
    _c._check(_c.lib().b200_gemm_fp8_block_push(
        _c._p(xq), _c._p(xs), _c._p(wq), _c._p(w_scale_inv), c_int(T), c_int(N), c_int(K),
        heap.peers_c, c_int(heap.rank), c_int(heap.world), c_ulonglong(part.offset),
        c_ulonglong(st.part_bytes), c_ulonglong(st.tile_flags.offset), c_int(_c.FusedTP.MAX_TILES),
        _c._p(st.ctrl), _c._p(ws.status), c_int(_c._sms), _c._stream()), "gemm_fp8_block_push")
    count_launch()
    return _c.PendingReduce(heap, part, T, N, lead_shape if lead_shape is not None else (T,))


def fp8_per_tensor_gemm(x, wq, w_scale, bias=None, ws_grid=None):
    """W8A8 with one weight scale per tensor and one activation scale per token: the activation is
    quantised by one kernel (row amax -> e4m3), the product runs on the block-scaled tcgen05 kernel
    with both scales repeated over its K blocks (dequantisation happens block by block either way)."""
    _c._require_bf16(x)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    T, K = x2.shape
    N = wq.shape[0]
    kb = (K + 127) // 128
    y = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return y.reshape(*lead, N)
    xq = torch.empty((T, K), dtype=FP8, device=x.device)
    xs_b = torch.empty((T, kb), dtype=torch.float32, device=x.device)
    _c._check(_c.lib().b200_quant_act_rowwise(_c._p(x2), _c._p(xq), _c._p(xs_b), c_int(T), c_int(K),
                                              c_int(x2.stride(0)), c_int(kb), _c._stream()), "quant_act_rowwise")
    count_launch()
    if ws_grid is None:
        ws_grid = w_scale.reshape(1, 1).float().expand((N + 127) // 128, kb).contiguous()
    fp8_block_gemm_quantised(xq, xs_b, wq, ws_grid, y, bias)
    return y.reshape(*lead, N)


def fp8_rowwise_gemm(xq, xs, wq, w_scale, out_dtype):
    """Operands already quantised (per-row activation scales xs [T], per-tensor weight scale)."""
    xq = xq.contiguous()
    T, K = xq.shape
    N = wq.shape[0]
    kb = (K + 127) // 128
    xs_b = xs.reshape(T, 1).float().expand(T, kb).contiguous()
    ws_b = w_scale.reshape(1, 1).float().expand((N + 127) // 128, kb).contiguous()
    y = torch.empty((T, N), dtype=torch.bfloat16, device=xq.device)
    fp8_block_gemm_quantised(xq, xs_b, wq, ws_b, y)
    return y.to(out_dtype)


def grouped_fp8_gemm(x_perm, wq, w_scale, group_off, avg_rows: int):
    """x_perm bf16 [R,K] sorted by expert; wq e4m3 [E,N,K]; w_scale fp32 [E, N/128, ceil(K/128)]."""
    R, K = x_perm.shape
    E, N = wq.shape[0], wq.shape[1]
    xq, xs = quant_act_1x128(x_perm)
    y = torch.empty((R, N), dtype=torch.bfloat16, device=x_perm.device)
    return _grouped_fp8_launch(xq, xs, wq, w_scale, group_off, avg_rows, y)


def moe_experts_fp8(x, w13, w13_scale, w2, w2_scale, topk_ids, topk_w, expert_offset, block=(128, 128)):
    """fp8 experts: permute -> grouped fp8 GEMM (gate|up) -> SiLU*mul -> grouped fp8 GEMM -> un-permute."""
    from . import cuda_moe
    T, H = x.shape
    E_local = w13.shape[0]
    k = topk_ids.shape[1]
    x_perm, group_off, _, inv_pos = cuda_moe.moe_permute(x.contiguous(), topk_ids.contiguous(), expert_offset,
                                                         E_local)
    avg = (T * k + E_local - 1) // E_local
    h = grouped_fp8_gemm(x_perm, w13, w13_scale, group_off, avg)
    aq, a_s = quant_rows_1x128(h, w2.shape[2], swiglu=True)       # SiLU*mul fused into the quantisation
    y = torch.empty((h.shape[0], w2.shape[1]), dtype=torch.bfloat16, device=x.device)
    _grouped_fp8_launch(aq, a_s, w2, w2_scale, group_off, avg, y)
    return cuda_moe.moe_unpermute(y, inv_pos, topk_w.contiguous(), T)


def moe_experts_ep_fp8(x, w13, w13_scale, w2, w2_scale, topk_ids, topk_w, heap, num_experts: int):
    """Block-scaled fp8 experts under expert parallelism on the fused plane: bf16 rows are PUT into the
    owners' receive buffers, the owners quantise what arrived (the row count stays on the device), run
    the grouped fp8 tcgen05 GEMMs with SiLU*mul fused into the second quantisation, and the epilogue of
    the second GEMM stores every output row into the return slot of the rank the token came from."""
    import ctypes
    from . import cuda_moe
    st = heap.ep_state
    T, H = x.shape
    k = topk_ids.shape[1]
    E_local, I = w13.shape[0], w2.shape[2]
    if T > st.max_tokens or k != st.k or H != st.H or num_experts != st.E:
        raise RuntimeError("fused EP plane was configured for a different shape")
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
    bound = st.cap               # rows the receive buffer holds; the live count is group_off[E_local]
    f8 = st.fp8_scratch(I)
    rows = st.group_off[E_local:]
    recv_x = heap.tensor(st.recv_x, (st.cap, H), torch.bfloat16)[:bound]
    avg = max(1, (T * k) // max(1, E_local))
    xq, xs = quant_rows_1x128(recv_x, H, rows=rows, out=(f8["xq1"][:bound], f8["xs1"][:bound]))
    h = _grouped_fp8_launch(xq, xs, w13, w13_scale, st.group_off, avg, f8["h"][:bound])
    aq, a_s = quant_rows_1x128(h, I, rows=rows, swiglu=True, out=(f8["xq2"][:bound], f8["xs2"][:bound]))
    _c._check(L.b200_grouped_gemm_fp8_block_routed(
        _c._p(aq), _c._p(a_s), _c._p(w2), _c._p(w2_scale), _c._p(st.group_off), c_int(E_local), c_int(bound),
        c_int(H), c_int(I), c_int(avg), heap.peers_c, c_int(heap.rank), c_int(heap.world),
        c_void_p(heap.local_ptr + st.recv_route.offset), c_ulonglong(st.ret.offset),
        c_ulonglong(st.ret_flag.offset), _c._p(st.ctrl), _c._p(ws.status), c_int(_c._sms), _c._stream()),
        "grouped_gemm_fp8_routed")
    count_launch()
    out = torch.empty((T, H), dtype=x.dtype, device=x.device)
    topk_w = topk_w.contiguous()
    _c._check(L.b200_ep_combine(c_void_p(heap.local_ptr), c_ulonglong(st.ret.offset),
                                c_ulonglong(st.ret_flag.offset), _c._p(st.ctrl), _c._p(ids),
                                _c._p(topk_w), _c._p(out), c_int(T), c_int(k), c_int(H),
                                c_int(num_experts), c_int(heap.world), _c._p(ws.status), spin, _c._stream()),
              "ep_combine")
    count_launch()
    return out


def quant_act_int8(x):
    """bf16 [T, K] -> (int8 [T, K], fp32 per-token scales [T])."""
    _c._require_bf16(x)
    if x.stride(-1) != 1:
        x = x.contiguous()
    T, K = x.shape
    xq = torch.empty((T, K), dtype=torch.int8, device=x.device)
    xs = torch.empty((T,), dtype=torch.float32, device=x.device)
    _c._check(_c.lib().b200_quant_act_int8(_c._p(x), _c._p(xq), _c._p(xs), c_int(T), c_int(K), c_int(x.stride(0)),
                                           _c._stream()), "quant_act_int8")
    count_launch()
    return xq, xs


def int8_gemm(x, wq, w_scale, bias=None):
    """W8A8: x bf16 [T,K] is quantised per token, wq int8 [N,K] has per-output-channel scales [N];
    tcgen05 kind::i8 with exact s32 sums -> bf16 [T,N]."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    T, K = x2.shape
    N = wq.shape[0]
    if K % 16:
        raise NotImplementedError("int8 GEMM needs K % 16 == 0")
    xq, xs = quant_act_int8(x2)
    y = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return y.reshape(*lead, N)
    ws = _c.Workspace.get(x.device)
    wq, w_scale = wq.contiguous(), w_scale.float().contiguous()
    _c._check(_c.lib().b200_gemm_int8(
        _c._p(xq), _c._p(xs), _c._p(wq), _c._p(w_scale), _c._p(y), _c._p(bias),
        c_int(T), c_int(N), c_int(K), c_int(y.stride(0)), _c._p(ws.status), c_int(_c._sms), _c._stream()),
        "gemm_int8")
    count_launch()
    return y.reshape(*lead, N)
