"""Batched gather matrix-vector products for LoRA.

shrink:  h[t] = x[t] @ A[idx[t]]^T          A: [slots, r, K]
expand:  y[t] += scale[idx[t]] * h[t] @ B[idx[t]]^T   B: [slots, N, r]
Tokens with idx < 0 have no adapter.  The formulation groups tokens by slot (a handful of slots
are live at a time) so each group is one dense GEMM; the reference uses a one-hot contraction
for the same effect (reference: src/vllm_torchtpu/lora/lora_ops.py:14-101)."""
from __future__ import annotations

import torch


def _cuda_ok(*ts) -> bool:
    return all(t.is_cuda for t in ts) and all(t.dtype == torch.bfloat16 for t in ts)


def bgmv_shrink(x: torch.Tensor, A: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    if _cuda_ok(x, A) and x.shape[-1] % 8 == 0:
        from ..ops import cuda_misc
        return cuda_misc.bgmv_shrink(x, A, idx)
    T, r = x.shape[0], A.shape[1]
    h = torch.zeros(T, r, dtype=torch.float32, device=x.device)
    for s in torch.unique(idx[idx >= 0]).tolist():
        m = idx == s
        h[m] = x[m].float() @ A[s].float().t()
    return h


def bgmv_expand(h: torch.Tensor, B: torch.Tensor, idx: torch.Tensor, y: torch.Tensor,
                scale: torch.Tensor, col_offset: int = 0) -> torch.Tensor:
    N = B.shape[1]
    if _cuda_ok(B, y) and h.is_cuda and y.stride(-1) == 1 and y.dim() == 2:
        from ..ops import cuda_misc
        return cuda_misc.bgmv_expand(h.contiguous(), B, idx, y, scale, col_offset)
    for s in torch.unique(idx[idx >= 0]).tolist():
        m = idx == s
        y[m, col_offset:col_offset + N] = (y[m, col_offset:col_offset + N].float() +
                                           float(scale[s]) * (h[m] @ B[s].float().t())).to(y.dtype)
    return y


def lora_apply(x, y, A, B, idx, scale, col_offset: int = 0):
    """y[:, off:off+N] += scale * (x @ A^T) @ B^T per token adapter."""
    if idx is None or (not idx.is_cuda and not bool((idx >= 0).any())):
        return y                     # (on the GPU the kernels skip rows without an adapter: no host sync)
    return bgmv_expand(bgmv_shrink(x, A, idx), B, idx, y, scale, col_offset)
