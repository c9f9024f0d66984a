"""A Wan-style diffusion transformer on the package's kernels.

Per block: adaLN modulation from the timestep embedding (shift / scale / gate for the attention and the
MLP), self-attention over the latent tokens with q/k RMSNorm over all channels + 3-axis interleaved RoPE
(the fused kernel), cross-attention to the text embeddings, and a GELU(tanh) MLP.  Linear layers run through
``ops.gemm`` (the tcgen05 GEMM on a GPU), self-attention through ``omni.attention.diffusion_attention``
(reference: the model code lives in the external omni runtime; the device pieces it calls are
src/vllm_torchtpu/omni/attention.py, omni/rope.py, kernels/diffusion_attention/qk_norm_rope.py, and the
per-model fixes in omni/patches.py:149-340)."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import ops
from .attention import diffusion_attention
from .ops import qk_norm_rope
from .rope import rope_table_3d


@dataclass
class DiTConfig:
    in_channels: int = 16            # latent channels
    patch: tuple = (1, 2, 2)         # (frames, rows, columns) of latent cells per token
    hidden_size: int = 256
    num_heads: int = 4
    head_dim: int = 64
    ffn_dim: int = 1024
    num_layers: int = 2
    text_dim: int = 128
    freq_dim: int = 64               # sinusoidal timestep features
    eps: float = 1e-6
    rope_theta: float = 10000.0
    dtype: torch.dtype = torch.bfloat16
    seed: int = 0

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.patch[0] * self.patch[1] * self.patch[2]


def tiny_dit() -> DiTConfig:
    return DiTConfig()


def _linear(x, w, b=None):
    shape = x.shape[:-1]
    y = ops.gemm(x.reshape(-1, x.shape[-1]), w, b)
    return y.view(*shape, w.shape[0])


def _layer_norm(x, eps):
    """Affine-free LayerNorm in fp32 (the modulation supplies scale and shift)."""
    return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), eps=eps)


def timestep_features(t: torch.Tensor, dim: int) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    ang = t.float()[:, None] * freqs[None]
    return torch.cat([ang.cos(), ang.sin()], -1)


class DiTBlock:
    def __init__(self, cfg: DiTConfig, idx: int, make):
        C, F = cfg.hidden_size, cfg.ffn_dim
        inner = cfg.num_heads * cfg.head_dim
        n = f"blocks.{idx}"
        self.cfg = cfg
        self.qkv_w, self.qkv_b = make(f"{n}.attn1.qkv.weight", (3 * inner, C)), make(f"{n}.attn1.qkv.bias", (3 * inner,))
        self.norm_q, self.norm_k = make(f"{n}.attn1.norm_q.weight", (inner,), ones=True), \
            make(f"{n}.attn1.norm_k.weight", (inner,), ones=True)
        self.o_w, self.o_b = make(f"{n}.attn1.o.weight", (C, inner)), make(f"{n}.attn1.o.bias", (C,))
        self.xq_w = make(f"{n}.attn2.q.weight", (inner, C))
        self.xkv_w = make(f"{n}.attn2.kv.weight", (2 * inner, cfg.text_dim))
        self.xo_w, self.xo_b = make(f"{n}.attn2.o.weight", (C, inner)), make(f"{n}.attn2.o.bias", (C,))
        self.ff1_w, self.ff1_b = make(f"{n}.ffn.0.weight", (F, C)), make(f"{n}.ffn.0.bias", (F,))
        self.ff2_w, self.ff2_b = make(f"{n}.ffn.2.weight", (C, F)), make(f"{n}.ffn.2.bias", (C,))
        self.modulation = make(f"{n}.modulation", (6, C), std=C ** -0.5)

    def forward(self, x, temb6, text, cos, sin):
        """x [B, S, C]; temb6 [B, 6, C] fp32; text [B, L, text_dim]; cos / sin [S, D / 2]."""
        cfg = self.cfg
        B, S, C = x.shape
        H, D = cfg.num_heads, cfg.head_dim
        inner = H * D
        m = (self.modulation.float()[None] + temb6).unbind(1)       # shift, scale, gate x 2
        h = (_layer_norm(x, cfg.eps) * (1 + m[1][:, None]) + m[0][:, None]).to(x.dtype)
        qkv = _linear(h, self.qkv_w, self.qkv_b).view(B * S, 3 * inner)
        q, k = qk_norm_rope(qkv, self.norm_q, self.norm_k, cos.repeat(B, 1) if B > 1 else cos,
                            sin.repeat(B, 1) if B > 1 else sin, H, H, D, cfg.eps)
        v = qkv[:, 2 * inner:].reshape(B, S, H, D)
        a = diffusion_attention(q.view(B, S, H, D), k.view(B, S, H, D), v)
        x = (x.float() + m[2][:, None] * _linear(a.reshape(B, S, inner), self.o_w, self.o_b).float()).to(x.dtype)
        # cross-attention to the text: few keys, different length from the queries
        hq = _linear(_layer_norm(x, cfg.eps).to(x.dtype), self.xq_w).view(B, S, H, D)
        kv = _linear(text, self.xkv_w).view(B, text.shape[1], 2, H, D)
        a = diffusion_attention(hq, kv[:, :, 0], kv[:, :, 1])
        x = x + _linear(a.reshape(B, S, inner), self.xo_w, self.xo_b)
        h = (_layer_norm(x, cfg.eps) * (1 + m[4][:, None]) + m[3][:, None]).to(x.dtype)
        h = torch.nn.functional.gelu(_linear(h, self.ff1_w, self.ff1_b).float(), approximate="tanh").to(x.dtype)
        return (x.float() + m[5][:, None] * _linear(h, self.ff2_w, self.ff2_b).float()).to(x.dtype)


class DiffusionTransformer:
    """Velocity predictor v(x_t, t, text) over video / image latents [B, C, F, H, W]."""

    def __init__(self, cfg: DiTConfig, device="cuda", state_dict: dict = None):
        self.cfg, self.device = cfg, torch.device(device)
        self._missing = []

        def make(name, shape, std=0.02, ones=False):
            if state_dict is not None:
                if name not in state_dict:
                    self._missing.append(name)
                else:
                    t = state_dict[name]
                    if tuple(t.shape) != tuple(shape):
                        raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)}, expected {tuple(shape)}")
                    return t.to(device=self.device, dtype=cfg.dtype).contiguous()
            if ones:
                return torch.ones(shape, dtype=cfg.dtype, device=self.device)
            if len(shape) == 1:
                return torch.zeros(shape, dtype=cfg.dtype, device=self.device)
            import zlib
            g = torch.Generator().manual_seed((cfg.seed << 20) ^ zlib.crc32(name.encode()))
            return (torch.randn(shape, generator=g) * std).to(device=self.device, dtype=cfg.dtype)

        C = cfg.hidden_size
        self.patch_w, self.patch_b = make("patch_embedding.weight", (C, cfg.patch_dim)), make("patch_embedding.bias", (C,))
        self.t1_w, self.t1_b = make("time_embedding.0.weight", (C, cfg.freq_dim)), make("time_embedding.0.bias", (C,))
        self.t2_w, self.t2_b = make("time_embedding.2.weight", (C, C)), make("time_embedding.2.bias", (C,))
        self.tp_w, self.tp_b = make("time_projection.weight", (6 * C, C)), make("time_projection.bias", (6 * C,))
        self.blocks = [DiTBlock(cfg, i, make) for i in range(cfg.num_layers)]
        self.head_mod = make("head.modulation", (2, C), std=C ** -0.5)
        self.head_w, self.head_b = make("head.weight", (cfg.patch_dim, C)), make("head.bias", (cfg.patch_dim,))
        if self._missing:
            raise ValueError(f"checkpoint lacks {len(self._missing)} tensors, first: {self._missing[:4]}")
        self._rope = {}

    def state_dict(self) -> dict:
        out = {"patch_embedding.weight": self.patch_w, "patch_embedding.bias": self.patch_b,
               "time_embedding.0.weight": self.t1_w, "time_embedding.0.bias": self.t1_b,
               "time_embedding.2.weight": self.t2_w, "time_embedding.2.bias": self.t2_b,
               "time_projection.weight": self.tp_w, "time_projection.bias": self.tp_b,
               "head.modulation": self.head_mod, "head.weight": self.head_w, "head.bias": self.head_b}
        names = {"qkv_w": "attn1.qkv.weight", "qkv_b": "attn1.qkv.bias", "norm_q": "attn1.norm_q.weight",
                 "norm_k": "attn1.norm_k.weight", "o_w": "attn1.o.weight", "o_b": "attn1.o.bias",
                 "xq_w": "attn2.q.weight", "xkv_w": "attn2.kv.weight", "xo_w": "attn2.o.weight",
                 "xo_b": "attn2.o.bias", "ff1_w": "ffn.0.weight", "ff1_b": "ffn.0.bias", "ff2_w": "ffn.2.weight",
                 "ff2_b": "ffn.2.bias", "modulation": "modulation"}
        for i, b in enumerate(self.blocks):
            for attr, n in names.items():
                out[f"blocks.{i}.{n}"] = getattr(b, attr)
        return out

    # ---- latents <-> tokens -------------------------------------------------------
    def grid_of(self, latents) -> tuple:
        _, _, F, H, W = latents.shape
        pf, ph, pw = self.cfg.patch
        if F % pf or H % ph or W % pw:
            raise ValueError(f"latent grid {(F, H, W)} is not a multiple of the patch {self.cfg.patch}")
        return F // pf, H // ph, W // pw

    def patchify(self, latents):
        B, C, F, H, W = latents.shape
        pf, ph, pw = self.cfg.patch
        g = self.grid_of(latents)
        x = latents.view(B, C, g[0], pf, g[1], ph, g[2], pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
        return x.reshape(B, g[0] * g[1] * g[2], self.cfg.patch_dim)

    def unpatchify(self, tokens, grid):
        B = tokens.shape[0]
        pf, ph, pw = self.cfg.patch
        x = tokens.view(B, grid[0], grid[1], grid[2], self.cfg.in_channels, pf, ph, pw)
        return x.permute(0, 4, 1, 5, 2, 6, 3, 7).reshape(B, self.cfg.in_channels, grid[0] * pf, grid[1] * ph,
                                                         grid[2] * pw)

    def forward(self, latents: torch.Tensor, timestep: torch.Tensor, text: torch.Tensor) -> torch.Tensor:
        """latents [B, C, F, H, W], timestep [B], text [B, L, text_dim] -> velocity of the latents' shape."""
        cfg = self.cfg
        grid = self.grid_of(latents)
        if grid not in self._rope:
            self._rope[grid] = rope_table_3d(grid, cfg.head_dim, cfg.rope_theta, self.device)
        cos, sin = self._rope[grid]
        x = _linear(self.patchify(latents.to(cfg.dtype)), self.patch_w, self.patch_b)
        # a fresh fp32 timestep embedding per call: the modulation is sensitive to bf16 rounding of t
        te = timestep_features(timestep.to(self.device), cfg.freq_dim).to(cfg.dtype)
        te = _linear(torch.nn.functional.silu(_linear(te, self.t1_w, self.t1_b).float()).to(cfg.dtype),
                     self.t2_w, self.t2_b)
        temb6 = _linear(torch.nn.functional.silu(te.float()).to(cfg.dtype), self.tp_w, self.tp_b).float()
        temb6 = temb6.view(-1, 6, cfg.hidden_size)
        text = text.to(device=self.device, dtype=cfg.dtype)
        for blk in self.blocks:
            x = blk.forward(x, temb6, text, cos, sin)
        m = (self.head_mod.float()[None] + te.float()[:, None]).unbind(1)
        h = (_layer_norm(x, cfg.eps) * (1 + m[1][:, None]) + m[0][:, None]).to(cfg.dtype)
        return self.unpatchify(_linear(h, self.head_w, self.head_b), grid)
