"""Fused q/k RMSNorm (over all heads * head_dim channels) + interleaved RoPE."""
from __future__ import annotations

import torch

from .rope import apply_rotary_interleaved


def qk_norm_rope_reference(qkv, wq, wk, cos, sin, num_q_heads, num_kv_heads, head_dim, eps=1e-6):
    """Plain PyTorch statement of the fused op; the normalised value is rounded to the input dtype before the
    rotation, as the kernel does (reference: src/vllm_torchtpu/kernels/diffusion_attention/qk_norm_rope.py:14-24)."""
    T = qkv.shape[0]
    Cq, Ck = num_q_heads * head_dim, num_kv_heads * head_dim
    out = []
    for x, w, H in ((qkv[:, :Cq], wq, num_q_heads), (qkv[:, Cq:Cq + Ck], wk, num_kv_heads)):
        xf = x.float()
        y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(qkv.dtype)
        out.append(apply_rotary_interleaved(y.view(T, H, head_dim), cos, sin))
    return out[0], out[1]


def qk_norm_rope(qkv, wq, wk, cos, sin, num_q_heads, num_kv_heads, head_dim, eps=1e-6):
    """qkv [T, >= (Hq + Hkv) * D] (q columns first, then k) -> q [T, Hq, D], k [T, Hkv, D].  One kernel on a
    GPU in bf16; the PyTorch statement elsewhere."""
    if not (qkv.is_cuda and qkv.dtype == torch.bfloat16):
        return qk_norm_rope_reference(qkv, wq, wk, cos, sin, num_q_heads, num_kv_heads, head_dim, eps)
    from ctypes import c_float, c_int, c_longlong

    from ..ops import cuda as C
    if qkv.stride(-1) != 1 or qkv.stride(0) % 8 or qkv.data_ptr() % 16:
        qkv = qkv.contiguous()             # the kernel reads 16-byte vectors
    T = qkv.shape[0]
    Cq, Ck = num_q_heads * head_dim, num_kv_heads * head_dim
    q = torch.empty((T, num_q_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    k = torch.empty((T, num_kv_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    cos, sin = cos.float().contiguous(), sin.float().contiguous()
    if cos.shape != (T, head_dim // 2) or sin.shape != cos.shape:
        raise ValueError(f"cos / sin must be [{T}, {head_dim // 2}], got {tuple(cos.shape)}")
    wq, wk = wq.to(torch.bfloat16).contiguous(), wk.to(torch.bfloat16).contiguous()
    C._check(C.lib().b200_qk_norm_rope(C._p(qkv), c_longlong(qkv.stride(0)), C._p(wq), C._p(wk), C._p(cos), C._p(sin),
                                       C._p(q), C._p(k), c_int(T), c_int(Cq), c_int(Ck), c_int(head_dim),
                                       c_float(eps), C._stream()), "qk_norm_rope")
    C.count_launch()
    return q, k
