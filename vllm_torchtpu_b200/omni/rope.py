"""Rotary embeddings of diffusion transformers.

A video token has three coordinates (frame, row, column); the head dimension is split into three bands and
each band rotates by its own coordinate.  The angles are therefore not ``position * inv_freq`` and are handed
to the kernels as per-token cos / sin tables of half the head dimension.  The rotation is the interleaved one:
channel pairs (2i, 2i + 1) turn together (reference: src/vllm_torchtpu/omni/rope.py:1-80 — the same rotation,
written there as a signed pair-swap matmul for the systolic array; on a GPU the swap is a register move inside
the fused kernel)."""
from __future__ import annotations

import torch


def axes_split(head_dim: int) -> tuple:
    """Pairs per axis (frame, row, column) as Wan splits them: the two spatial axes get a third of the
    head each (rounded down to whole pairs), the frame axis the rest."""
    half = head_dim // 2
    hw = head_dim // 6
    return half - 2 * hw, hw, hw


def rope_table_3d(grid: tuple, head_dim: int, theta: float = 10000.0, device="cpu") -> tuple:
    """cos, sin fp32 [F * H * W, head_dim / 2] for a (frames, rows, columns) token grid in row-major order."""
    F, H, W = grid
    parts = []
    coords = torch.meshgrid(torch.arange(F), torch.arange(H), torch.arange(W), indexing="ij")
    for n_pairs, pos in zip(axes_split(head_dim), coords):
        if n_pairs == 0:
            continue
        inv = 1.0 / (theta ** (torch.arange(0, n_pairs, dtype=torch.float64) * 2 / (2 * n_pairs)))
        parts.append(pos.reshape(-1, 1).double() * inv[None])
    ang = torch.cat(parts, -1)
    return ang.cos().float().to(device), ang.sin().float().to(device)


def rope_table_1d(num_tokens: int, head_dim: int, theta: float = 10000.0, device="cpu") -> tuple:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim // 2, dtype=torch.float64) * 2 / head_dim))
    ang = torch.arange(num_tokens, dtype=torch.float64)[:, None] * inv[None]
    return ang.cos().float().to(device), ang.sin().float().to(device)


def apply_rotary_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [..., T, H, D]; cos / sin [T, D / 2].  fp32 math, one rounding to x's dtype."""
    xf = x.float().unflatten(-1, (-1, 2))
    a, b = xf[..., 0], xf[..., 1]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.stack([a * c - b * s, b * c + a * s], -1).flatten(-2).to(x.dtype)
