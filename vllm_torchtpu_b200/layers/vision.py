"""Vision encoder (ViT) blocks on the bidirectional varlen attention op.

An image (or a temporal chunk of video frames) arrives as a matrix of flattened patches; a linear
patch embedding, ``depth`` pre-norm transformer blocks (LayerNorm → fused QKV → bidirectional
attention inside each image → projection; LayerNorm → GELU MLP) and a spatial merger (``merge``
neighbouring patches concatenated and projected to the language model's hidden size) turn it into
the embeddings that replace the image placeholder tokens of the prompt.  Several images of one step
run as one ragged batch with ``cu_seqlens`` marking their patch ranges
(reference: src/vllm_torchtpu/runner/mm_encoder_manager.py, kernels/flash_attention/ — segment-id
flash attention for ViT encoders).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import ops
from .linear import seeded_normal


@dataclass
class VisionConfig:
    patch_dim: int = 588            # channels * patch * patch (* temporal patch)
    hidden_size: int = 256
    num_heads: int = 4
    depth: int = 2
    mlp_ratio: int = 4
    merge: int = 4                  # patches merged into one output token
    out_hidden_size: int = 256      # language model hidden size
    eps: float = 1e-6
    dtype: torch.dtype = torch.float32
    init_std: float = 0.02
    seed: int = 0


class VisionBlock:
    def __init__(self, name: str, cfg: VisionConfig, device):
        h, d, dev = cfg.hidden_size, cfg.dtype, device
        mk = lambda n, shape: seeded_normal(f"{name}.{n}", shape, cfg.init_std, d, dev, cfg.seed)
        self.cfg = cfg
        self.ln1_w, self.ln1_b = torch.ones(h, dtype=d, device=dev), torch.zeros(h, dtype=d, device=dev)
        self.ln2_w, self.ln2_b = torch.ones(h, dtype=d, device=dev), torch.zeros(h, dtype=d, device=dev)
        self.qkv_w, self.qkv_b = mk("attn.qkv", (3 * h, h)), torch.zeros(3 * h, dtype=d, device=dev)
        self.proj_w, self.proj_b = mk("attn.proj", (h, h)), torch.zeros(h, dtype=d, device=dev)
        self.fc1_w, self.fc1_b = mk("mlp.fc1", (cfg.mlp_ratio * h, h)), torch.zeros(cfg.mlp_ratio * h, dtype=d, device=dev)
        self.fc2_w, self.fc2_b = mk("mlp.fc2", (h, cfg.mlp_ratio * h)), torch.zeros(h, dtype=d, device=dev)

    def forward(self, x: torch.Tensor, cu_seqlens: list) -> torch.Tensor:
        c = self.cfg
        T, H = x.shape[0], c.num_heads
        D = c.hidden_size // H
        y = F.layer_norm(x, (c.hidden_size,), self.ln1_w, self.ln1_b, c.eps)
        qkv = ops.gemm(y, self.qkv_w, self.qkv_b).reshape(T, 3, H, D)
        o = encoder_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu_seqlens)
        x = x + ops.gemm(o.reshape(T, H * D), self.proj_w, self.proj_b)
        y = F.layer_norm(x, (c.hidden_size,), self.ln2_w, self.ln2_b, c.eps)
        return x + ops.gemm(F.gelu(ops.gemm(y, self.fc1_w, self.fc1_b)), self.fc2_w, self.fc2_b)


def encoder_attention(q, k, v, cu_seqlens):
    """The CUDA kernel for bf16 tensors with head_dim 64 / 128 on a GPU, the fp32 oracle otherwise."""
    if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128):
        return ops.cuda_ops().encoder_attention(q.contiguous(), k.contiguous(), v.contiguous(), cu_seqlens)
    from ..ops import reference
    return reference.encoder_attention(q, k, v, cu_seqlens)


class VisionEncoder:
    def __init__(self, cfg: VisionConfig, device="cpu", name: str = "visual"):
        self.cfg, self.device = cfg, device
        d = cfg.dtype
        mk = lambda n, shape: seeded_normal(f"{name}.{n}", shape, cfg.init_std, d, device, cfg.seed)
        self.patch_w = mk("patch_embed", (cfg.hidden_size, cfg.patch_dim))
        self.blocks = [VisionBlock(f"{name}.blocks.{i}", cfg, device) for i in range(cfg.depth)]
        self.ln_w = torch.ones(cfg.hidden_size, dtype=d, device=device)
        self.ln_b = torch.zeros(cfg.hidden_size, dtype=d, device=device)
        self.merge_w = mk("merger", (cfg.out_hidden_size, cfg.merge * cfg.hidden_size))

    def tokens_for(self, num_patches: int) -> int:
        return num_patches // self.cfg.merge

    def forward(self, patches: torch.Tensor, patch_counts: list) -> list:
        """``patches`` [sum(patch_counts), patch_dim] of several images; returns one [tokens, out_hidden]
        embedding matrix per image (patch counts are multiples of ``merge``)."""
        c = self.cfg
        assert all(n % c.merge == 0 for n in patch_counts), "patch count must be a multiple of the merge size"
        cu = [0]
        for n in patch_counts:
            cu.append(cu[-1] + int(n))
        x = ops.gemm(patches.to(c.dtype), self.patch_w, None)
        for blk in self.blocks:
            x = blk.forward(x, cu)
        x = F.layer_norm(x, (c.hidden_size,), self.ln_w, self.ln_b, c.eps)
        y = ops.gemm(x.reshape(-1, c.merge * c.hidden_size), self.merge_w, None)
        return [y[cu[i] // c.merge: cu[i + 1] // c.merge] for i in range(len(patch_counts))]
