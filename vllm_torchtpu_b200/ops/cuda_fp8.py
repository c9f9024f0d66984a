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
    _c._check(_c.lib().b200_quant_act_1x128(_c._p(x), _c._p(xq), _c._p(xs), c_int(T), c_int(K),
                                            c_int(x.stride(0)), _c._stream()), "quant_act_1x128")
    count_launch()
    return xq, xs


def fp8_block_gemm(x, wq, w_scale_inv, bias=None, block=(128, 128), out=None):
    """x bf16 [T,K]; wq e4m3 [N,K]; w_scale_inv fp32 [ceil(N/128), ceil(K/128)] -> bf16 [T,N]."""
    if tuple(block) != (128, 128):
        raise NotImplementedError("the fp8 kernel is built for 128x128 weight blocks")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    T, K = x2.shape
    N = wq.shape[0]
    xq, xs = quant_act_1x128(x2)
    y = out if out is not None else torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return y.reshape(*lead, N)
    ws = _c.Workspace.get(x.device)
    _c._check(_c.lib().b200_gemm_fp8_block(
        _c._p(xq), _c._p(xs), _c._p(wq), _c._p(w_scale_inv), _c._p(y), _c._p(bias), c_int(T), c_int(N),
        c_int(K), c_int(y.stride(0)), _c._p(ws.status), c_int(_c._sms), _c._stream()), "gemm_fp8_block")
    count_launch()
    return y.reshape(*lead, N)


def fp8_block_gemm_push(x, wq, w_scale_inv, heap):
    """Row-parallel block-scaled fp8 ``x @ wq.T`` whose bf16 partial is pushed to every rank of ``heap``
    from the GEMM epilogue; returns the :class:`PendingReduce` the next add + RMSNorm (or
    ``materialize``) completes.  For at most 128 tokens within ``FusedTP.can_push``."""
    st = heap.fused_tp
    x2 = x.reshape(-1, x.shape[-1])
    T, K = x2.shape
    N = wq.shape[0]
    xq, xs = quant_act_1x128(x2)
    part = st.parts[st.flip]
    st.flip ^= 1
    ws = _c.Workspace.get(x.device)
    _c._check(_c.lib().b200_gemm_fp8_block_push(
        _c._p(xq), _c._p(xs), _c._p(wq), _c._p(w_scale_inv), c_int(T), c_int(N), c_int(K),
        heap.peers_c, c_int(heap.rank), c_int(heap.world), c_ulonglong(part.offset),
        c_ulonglong(st.part_bytes), c_ulonglong(st.tile_flags.offset), c_int(_c.FusedTP.MAX_TILES),
        _c._p(st.ctrl), _c._p(ws.status), c_int(_c._sms), _c._stream()), "gemm_fp8_block_push")
    count_launch()
    return _c.PendingReduce(heap, part, T, N, x.shape[:-1])


def fp8_rowwise_gemm(xq, xs, wq, w_scale, out_dtype):
    """Per-tensor weight scale, per-row activation scale: expressed through the block kernel by
    broadcasting both scales over the K blocks (dequant happens block by block either way)."""
    xq = xq.contiguous()
    T, K = xq.shape
    N = wq.shape[0]
    kb = (K + 127) // 128
    xs_b = xs.reshape(T, 1).float().expand(T, kb).contiguous()
    ws_b = w_scale.reshape(1, 1).float().expand((N + 127) // 128, kb).contiguous()
    y = torch.empty((T, N), dtype=torch.bfloat16, device=xq.device)
    ws = _c.Workspace.get(xq.device)
    _c._check(_c.lib().b200_gemm_fp8_block(
        _c._p(xq), _c._p(xs_b), _c._p(wq), _c._p(ws_b), _c._p(y), c_void_p(0), c_int(T), c_int(N),
        c_int(K), c_int(y.stride(0)), _c._p(ws.status), c_int(_c._sms), _c._stream()), "gemm_fp8_block")
    count_launch()
    return y.to(out_dtype)


def grouped_fp8_gemm(x_perm, wq, w_scale, group_off, avg_rows: int):
    """x_perm bf16 [R,K] sorted by expert; wq e4m3 [E,N,K]; w_scale fp32 [E, N/128, ceil(K/128)]."""
    R, K = x_perm.shape
    E, N = wq.shape[0], wq.shape[1]
    xq, xs = quant_act_1x128(x_perm)
    y = torch.empty((R, N), dtype=torch.bfloat16, device=x_perm.device)
    ws = _c.Workspace.get(x_perm.device)
    _c._check(_c.lib().b200_grouped_gemm_fp8_block(
        _c._p(xq), _c._p(xs), _c._p(wq), _c._p(w_scale), _c._p(y), _c._p(group_off), c_int(E), c_int(R),
        c_int(N), c_int(K), c_int(max(1, avg_rows)), _c._p(ws.status), c_int(_c._sms), _c._stream()),
        "grouped_gemm_fp8_block")
    count_launch()
    return y


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
    a = _c.silu_and_mul(h)
    y = grouped_fp8_gemm(a, w2, w2_scale, group_off, avg)
    return cuda_moe.moe_unpermute(y, inv_pos, topk_w.contiguous(), T)


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
