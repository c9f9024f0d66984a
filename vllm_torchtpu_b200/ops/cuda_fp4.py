"""Bindings of the W4A16 tcgen05 GEMM (``csrc/gemm_w4a16_tcgen05.cu``): packed e2m1 weights with mxfp4 or
nvfp4 group scales, or unsigned 4-bit integers with group scales and zero points (AWQ / GPTQ), bf16 activations.  The weight stays 4-bit in HBM; tiles are expanded in shared memory."""
from __future__ import annotations

from ctypes import c_int

import torch

from . import count_launch
from . import cuda as _c

FMT = {"mxfp4": 0, "nvfp4": 1}
DEQUANT_FROM_TOKENS = 1024


def dequant_w4(w_packed, scales, fmt: str, global_scale=None):
    """Packed e2m1 [..., rows, K / 2] with its group scales -> bf16 [..., rows, K]."""
    from ctypes import c_longlong
    K = w_packed.shape[-1] * 2
    rows = w_packed.numel() // w_packed.shape[-1]
    out = torch.empty(w_packed.shape[:-1] + (K,), dtype=torch.bfloat16, device=w_packed.device)
    _c._check(_c.lib().b200_dequant_w4(_c._p(w_packed), _c._p(scales), _c._p(global_scale), _c._p(out),
                                       c_longlong(rows), c_int(K), c_int(FMT[fmt]), _c._stream()), "dequant_w4")
    count_launch()
    return out


def w4a16_gemm(x, w_packed, scales, fmt: str, global_scale=None, bias=None):
    """x bf16 [..., K]; w_packed uint8 [N, K / 2]; scales uint8 [N, K / 32] (mxfp4) or float8_e4m3fn
    [N, K / 16] (nvfp4, with global_scale fp32[1]) -> bf16 [..., N].  K % 64 == 0."""
    _c._require_bf16(x, bias)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    T, K = x2.shape
    N = w_packed.shape[0]
    if T >= DEQUANT_FROM_TOKENS:
        # many tokens: one pass over the weight into a bf16 scratch, then the bf16 tcgen05 GEMM (the fused
        # kernel would expand every weight tile once per token tile)
        return _c.gemm(x2, dequant_w4(w_packed, scales, fmt, global_scale), bias).reshape(*lead, N)
    y = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return y.reshape(*lead, N)
    ws = _c.Workspace.get(x.device)
    _c._check(_c.lib().b200_gemm_w4a16(
        _c._p(x2), _c._p(w_packed), _c._p(scales), _c._p(global_scale), _c._p(y), _c._p(bias), c_int(T), c_int(N),
        c_int(K), c_int(x2.stride(0)), c_int(N), c_int(FMT[fmt]), _c._p(ws.status), c_int(_c._sms), _c._stream()),
        "gemm_w4a16")
    count_launch()
    return y.reshape(*lead, N)


def dequant_int4(w_packed, scales, zeros, group: int):
    """Packed unsigned nibbles [rows, K / 2], fp16 scales and uint8 zero points [rows, K / group] -> bf16 [rows, K]."""
    from ctypes import c_longlong
    K = w_packed.shape[-1] * 2
    rows = w_packed.numel() // w_packed.shape[-1]
    out = torch.empty(w_packed.shape[:-1] + (K,), dtype=torch.bfloat16, device=w_packed.device)
    _c._check(_c.lib().b200_dequant_int4(_c._p(w_packed), _c._p(scales), _c._p(zeros), _c._p(out), c_longlong(rows),
                                         c_int(K), c_int(group), _c._stream()), "dequant_int4")
    count_launch()
    return out


def int4_kernel_ok(K: int, group: int) -> bool:
    return K % 64 == 0 and group >= 32 and group & (group - 1) == 0 and K % group == 0


def w4a16_int4_gemm(x, w_packed, scales, zeros, group: int, bias=None):
    """AWQ / GPTQ style weights on the W4A16 kernel: x bf16 [..., K]; w_packed uint8 [N, K / 2] (low nibble = even
    k), scales fp16 [N, K / group], zeros uint8 [N, K / group]; value = (nibble - zero) * scale -> bf16 [..., N]."""
    _c._require_bf16(x, bias)
    if scales.dtype != torch.float16 or zeros.dtype != torch.uint8:
        raise TypeError("int4 weights take fp16 scales and uint8 zero points")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    T, K = x2.shape
    N = w_packed.shape[0]
    if T >= DEQUANT_FROM_TOKENS or not int4_kernel_ok(K, group):
        return _c.gemm(x2, dequant_int4(w_packed, scales, zeros, group), bias).reshape(*lead, N)
    y = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
    if T == 0:
        return y.reshape(*lead, N)
    ws = _c.Workspace.get(x.device)
    _c._check(_c.lib().b200_gemm_w4a16_int4(
        _c._p(x2), _c._p(w_packed), _c._p(scales), _c._p(zeros), _c._p(y), _c._p(bias), c_int(T), c_int(N), c_int(K),
        c_int(x2.stride(0)), c_int(N), c_int(group), _c._p(ws.status), c_int(_c._sms), _c._stream()),
        "gemm_w4a16_int4")
    count_launch()
    return y.reshape(*lead, N)


def grouped_w4a16_gemm(x_perm, w_packed, scales, group_off, avg_rows: int, fmt: str, global_scale=None):
    """Rows [group_off[e], group_off[e+1]) of x_perm [R, K] times expert e's packed weight
    w_packed [E, N, K / 2] (scales [E, N, K / G]; nvfp4: global_scale fp32[E]) -> bf16 [R, N]."""
    _c._require_bf16(x_perm)
    R, K = x_perm.shape
    E, N = w_packed.shape[0], w_packed.shape[1]
    y = torch.empty((R, N), dtype=torch.bfloat16, device=x_perm.device)
    if R == 0:
        return y
    ws = _c.Workspace.get(x_perm.device)
    _c._check(_c.lib().b200_grouped_gemm_w4a16(
        _c._p(x_perm), _c._p(w_packed), _c._p(scales), _c._p(global_scale), _c._p(y), _c._p(group_off), c_int(E),
        c_int(R), c_int(N), c_int(K), c_int(max(1, avg_rows)), c_int(FMT[fmt]), _c._p(ws.status), c_int(_c._sms),
        _c._stream()), "grouped_gemm_w4a16")
    count_launch()
    return y


def moe_experts_w4a16(x, w13, w13_scale, w2, w2_scale, topk_ids, topk_w, expert_offset: int, fmt: str = "mxfp4",
                      act: str = "silu", b13=None, b2=None):
    """4-bit experts: permute -> grouped W4A16 GEMM (gate | up) -> SiLU*mul -> grouped W4A16 GEMM -> un-permute."""
    from . import cuda_moe
    T, H = x.shape
    E_local = w13.shape[0]
    k = topk_ids.shape[1]
    x_perm, group_off, _, inv_pos = cuda_moe.moe_permute(x.contiguous(), topk_ids.contiguous(), expert_offset, E_local)
    avg = (T * k + E_local - 1) // E_local
    h = grouped_w4a16_gemm(x_perm, w13, w13_scale, group_off, avg, fmt)
    if b13 is not None:
        cuda_moe.group_bias_add(h, b13, group_off)
    a = _c.silu_and_mul(h) if act == "silu" else _c.gated_act_and_mul(h, act)
    y = grouped_w4a16_gemm(a, w2, w2_scale, group_off, avg, fmt)
    if b2 is not None:
        cuda_moe.group_bias_add(y, b2, group_off)
    out = cuda_moe.moe_unpermute(y, inv_pos, topk_w.contiguous(), T)
    return out if out.shape[1] == H else out[:, :H].contiguous()      # down projection padded to the tile width
