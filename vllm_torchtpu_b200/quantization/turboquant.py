"""TurboQuant 4-bit KV-cache quantisation (the ``turboquant_4bit_nc`` preset), head_dim 128.

Keys: ``k / |k|`` is rotated by the orthonormal Walsh-Hadamard matrix ``H`` and every coordinate is
snapped to the nearest of 16 Lloyd-Max levels of a unit normal divided by sqrt(D); the stored bf16
norm carries the correction ``|k| / |centroid vector|``.  Because ``q . k == (q H) . (k H)`` an
attention kernel may rotate the query once instead of un-rotating keys; ``decode`` below returns
keys in the original basis.  Values: per-row asymmetric uniform 4-bit codes with bf16
``(scale, zero)``.  Storage per row: 64 + 64 code bytes + 6 metadata bytes instead of 512
(reference: src/vllm_torchtpu/layers/core/turboquant.py:14-60)."""
from __future__ import annotations

import math

import torch

LEVELS = torch.tensor([-2.7326, -2.0690, -1.6181, -1.2562, -0.9424, -0.6568, -0.3881, -0.1284,
                       0.1284, 0.3881, 0.6568, 0.9424, 1.2562, 1.6181, 2.0690, 2.7326])
KEY_NORM_EPS = 1e-8
CENTROID_NORM_EPS = 1e-16
VALUE_SCALE_MIN = 1e-8


def hadamard(n: int, device=None) -> torch.Tensor:
    """Orthonormal Walsh-Hadamard matrix (Sylvester order), n a power of two."""
    h = torch.ones(1, 1, device=device)
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h / math.sqrt(n)


def _pack(codes: torch.Tensor) -> torch.Tensor:
    c = codes.to(torch.uint8)
    return (c[..., 0::2] | (c[..., 1::2] << 4)).contiguous()


def _unpack(packed: torch.Tensor) -> torch.Tensor:
    out = torch.empty(*packed.shape[:-1], packed.shape[-1] * 2, dtype=torch.uint8, device=packed.device)
    out[..., 0::2] = packed & 15
    out[..., 1::2] = packed >> 4
    return out


def encode(k: torch.Tensor, v: torch.Tensor):
    """k, v [rows, D] → (k_codes u8 [rows, D/2], k_norm bf16 [rows], v_codes u8 [rows, D/2],
    v_meta bf16 [rows, 2])."""
    D = k.shape[-1]
    lv = LEVELS.to(k.device)
    kf = k.float()
    norm = kf.norm(dim=-1, keepdim=True)
    rot = (kf / norm.clamp_min(KEY_NORM_EPS)) @ hadamard(D, k.device)
    bounds = 0.5 * (lv[:-1] + lv[1:])
    codes = torch.bucketize((rot * math.sqrt(D)).contiguous(), bounds, right=False)
    cent = lv[codes] / math.sqrt(D)
    k_norm = (norm.squeeze(-1) * torch.rsqrt((cent * cent).sum(-1) + CENTROID_NORM_EPS)).to(torch.bfloat16)
    vf = v.float()
    mx, mn = vf.amax(-1, keepdim=True), vf.amin(-1, keepdim=True)
    scale = ((mx - mn) / 15.0).clamp_min(VALUE_SCALE_MIN).to(torch.bfloat16).float()
    zero = mn.to(torch.bfloat16).float()
    vc = torch.round((vf - zero) / scale).clamp(0, 15)
    v_meta = torch.cat([scale, zero], -1).to(torch.bfloat16)
    return _pack(codes), k_norm, _pack(vc), v_meta


def decode(k_codes, k_norm, v_codes, v_meta, dtype=torch.bfloat16):
    D = k_codes.shape[-1] * 2
    lv = LEVELS.to(k_codes.device)
    cent = lv[_unpack(k_codes).long()] / math.sqrt(D)
    k = (cent @ hadamard(D, k_codes.device)) * k_norm.float()[:, None]
    v = _unpack(v_codes).float() * v_meta[:, :1].float() + v_meta[:, 1:].float()
    return k.to(dtype), v.to(dtype)


def quantize_kv_fp8(x: torch.Tensor, scale: float) -> torch.Tensor:
    """bf16 → e4m3 with a per-tensor scale (reference: layers/core/quantization.py:91 ``quantize_kv``)."""
    return (x.float() / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)


def dequantize_kv_fp8(q: torch.Tensor, scale: float, dtype=torch.bfloat16) -> torch.Tensor:
    return (q.float() * scale).to(dtype)
