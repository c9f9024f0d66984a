"""Kimi-Linear style hybrid decoder: Kimi Delta Attention (KDA) layers with every
``full_attention_interval``-th layer a softmax attention layer over the paged KV cache.

KDA layer (reference: src/vllm_torchtpu/layers/adapter/custom_ops/kda_attention_op.py:322-445 and
kernels/gdn/v3/compute_kda.py): fused q|k|v projection → causal short convolution + SiLU → q/k L2
normalisation → gated delta rule whose log-decay is per key channel (low-rank gate projection
``f_b(f_a(x))`` activated with ``A_log`` / ``dt_bias``, optionally floored at ``kda_gate_lower_bound``)
→ per-head RMSNorm times a sigmoid output gate (low-rank ``g_b(g_a(x))``) → row-parallel o_proj.
State per request and layer: the convolution window and a [H, dk, dv] fp32 matrix, both in pools
indexed by the request's batch slot.  Heads are sharded over TP.

The full-attention layers here are GQA layers; the reference pairs KDA with MLA layers in its
production configuration, which this package provides for the DeepSeek family only."""
from __future__ import annotations

import torch

from .. import ops
from ..config import ModelConfig
from ..layers.linear import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear, seeded_normal
from ..ops import gdn_reference as gref
from ..parallel.state import get_state
from .llama import LlamaDecoderLayer
from .qwen3_next import Qwen3NextDecoderLayer, Qwen3NextForCausalLM


class KimiDeltaAttention:
    def __init__(self, name: str, cfg: ModelConfig, device, quant):
        tp = get_state().tp.size
        self.name, self.cfg, self.device = name, cfg, device
        H_total = cfg.gdn_num_v_heads
        assert cfg.gdn_num_k_heads == H_total, "KDA has one key head per value head"
        self.H = H_total // tp
        self.dk, self.dv = cfg.gdn_head_k_dim, cfg.gdn_head_v_dim
        self.Hk = self.Hv = self.H
        self.K = cfg.gdn_conv_kernel
        self.rank = cfg.kda_gate_rank or cfg.gdn_head_k_dim
        self.lower_bound = cfg.kda_gate_lower_bound
        kw = dict(dtype=cfg.dtype, device=device, quant_config=quant)
        kd, vd = H_total * self.dk, H_total * self.dv
        self.in_qkv = ColumnParallelLinear(f"{name}.qkv_proj", cfg.hidden_size, [kd, kd, vd], **kw)
        self.f_a = ReplicatedLinear(f"{name}.f_a_proj", cfg.hidden_size, self.rank, **kw)
        self.f_b = ColumnParallelLinear(f"{name}.f_b_proj", self.rank, [kd], **kw)
        self.g_a = ReplicatedLinear(f"{name}.g_a_proj", cfg.hidden_size, self.rank, **kw)
        self.g_b = ColumnParallelLinear(f"{name}.g_b_proj", self.rank, [vd], **kw)
        self.b_proj = ColumnParallelLinear(f"{name}.b_proj", cfg.hidden_size, [H_total], **kw)
        self.out = RowParallelLinear(f"{name}.o_proj", vd, cfg.hidden_size, **kw)
        self.channels = 2 * self.H * self.dk + self.H * self.dv
        self.conv_w = None
        self.A_log = None
        self.dt_bias = None
        self.norm_w = torch.ones(self.dv, dtype=cfg.dtype, device=device)
        self.eps = cfg.rms_norm_eps

    def linears(self):
        return [self.in_qkv, self.f_a, self.f_b, self.g_a, self.g_b, self.b_proj, self.out]

    def init_dummy(self, std, seed):
        for l in self.linears():
            l.init_dummy(std, seed)
        d, dev = self.cfg.dtype, self.device
        self.conv_w = seeded_normal(f"{self.name}.conv1d", (self.channels, self.K), 0.2, d, dev, seed)
        self.A_log = seeded_normal(f"{self.name}.A_log", (self.H,), 0.5, torch.float32, dev, seed)
        self.dt_bias = seeded_normal(f"{self.name}.dt_bias", (self.H, self.dk), 0.5, torch.float32, dev, seed)

    def weight_bytes(self):
        n = sum(l.weight_bytes() for l in self.linears())
        return n + self.conv_w.numel() * self.conv_w.element_size()

    def state_shapes(self, max_reqs: int):
        return (max_reqs + 1, self.channels, self.K - 1), (max_reqs + 1, self.H, self.dk, self.dv)

    def recur(self, inputs, meta, cache):
        """The stateful part: short conv with its carried window + KDA recurrence over the rows ``meta``
        describes; advances the pools in place.  inputs = (mixed [T, C], a [T, H, dk], b [T, H])."""
        mixed, a, b = inputs
        conv_pool, rec_pool = cache
        T, H, dk, dv = mixed.shape[0], self.H, self.dk, self.dv
        if mixed.is_cuda:
            cu = ops.cuda_ops()
            y = cu.short_conv(mixed, meta, conv_pool, self.conv_w)
            q, k, v = y.split([H * dk, H * dk, H * dv], dim=-1)
            o = cu.kda_forward(q.reshape(T, H, dk), k.reshape(T, H, dk), v.reshape(T, H, dv), a, b, meta, rec_pool,
                               self.A_log, self.dt_bias, self.lower_bound)
        else:
            y = torch.zeros_like(mixed)
            qsl, sl, slots = meta.query_start_loc.tolist(), meta.seq_lens.tolist(), meta.state_slots.tolist()
            for r in range(meta.num_reqs):
                qs, qe = qsl[r], qsl[r + 1]
                if qe <= qs:
                    continue
                if sl[r] - (qe - qs) == 0:
                    conv_pool[slots[r]].zero_()
                y[qs:qe] = gref.causal_conv1d_update(mixed[qs:qe], conv_pool[slots[r]], self.conv_w)
            q, k, v = y.split([H * dk, H * dk, H * dv], dim=-1)
            o = gref.kda_forward(q.reshape(T, H, dk), k.reshape(T, H, dk), v.reshape(T, H, dv), a, b, meta, rec_pool,
                                 self.A_log, self.dt_bias, self.lower_bound)
        return o

    def forward(self, x, cache, meta):
        T, H, dk, dv = x.shape[0], self.H, self.dk, self.dv
        mixed = self.in_qkv(x)
        a = self.f_b(self.f_a(x)).reshape(T, H, dk)
        b = self.b_proj(x)
        gate = self.g_b(self.g_a(x)).reshape(T, H, dv)
        inputs = (mixed.contiguous(), a.contiguous(), b.contiguous())
        rb = getattr(meta, "state_rollback", None)
        if rb is not None:
            rb.capture(self, cache, inputs)        # verification step: rejected drafts are rolled back later
        o = self.recur(inputs, meta, cache)
        o = ops.rms_norm(o.reshape(T * H, dv), self.norm_w, self.eps).reshape(T, H, dv)
        o = (o.float() * torch.sigmoid(gate.float())).to(x.dtype)
        return self.out(o.reshape(T, H * dv))


class KimiLinearDecoderLayer(Qwen3NextDecoderLayer):
    def __init__(self, idx: int, cfg: ModelConfig, device, quant):
        self.full_attention = cfg.layer_is_full_attention(idx)
        if self.full_attention:
            LlamaDecoderLayer.__init__(self, idx, cfg, device, quant)
            if cfg.is_mla:
                # the published layout: latent attention in the full-attention layers (absorbed form, latent cache)
                from .deepseek_v3 import MLAAttention
                self.self_attn = MLAAttention(f"model.layers.{idx}.self_attn", cfg, device, quant)
            return
        name = f"model.layers.{idx}"
        self.idx = idx
        self.eps = cfg.rms_norm_eps
        self.input_ln = torch.ones(cfg.hidden_size, dtype=cfg.dtype, device=device)
        self.post_ln = torch.ones(cfg.hidden_size, dtype=cfg.dtype, device=device)
        self.self_attn = KimiDeltaAttention(f"{name}.self_attn", cfg, device, quant)
        self.mlp = self._make_ffn(name, cfg, device, quant)


class KimiLinearForCausalLM(Qwen3NextForCausalLM):
    layer_cls = KimiLinearDecoderLayer

    def init_dummy(self) -> None:
        super().init_dummy()
        if self.cfg.is_mla:
            for l in self.layers:
                if l.full_attention:
                    l.self_attn.init_dummy(self.cfg.init_std, self.cfg.seed)     # adds the absorbed kv_b matrices

    def weight_bytes(self) -> int:
        n = super().weight_bytes()
        if self.cfg.is_mla:
            for l in self.layers:
                if l.full_attention:
                    n += sum(t.numel() * t.element_size() for t in (l.self_attn.w_uk, l.self_attn.w_uv))
        return n

    def kv_cache_shape(self, num_blocks: int, block_size: int) -> tuple:
        if self.cfg.is_mla:
            return (num_blocks, block_size, self.cfg.kv_lora_rank + self.cfg.qk_rope_head_dim)
        return super().kv_cache_shape(num_blocks, block_size)

    def kv_bytes_per_block(self, block_size: int, kv_dtype: torch.dtype) -> int:
        if not self.cfg.is_mla:
            return super().kv_bytes_per_block(block_size, kv_dtype)
        n_full = sum(1 for l in self.layers if l.full_attention)
        return n_full * block_size * (self.cfg.kv_lora_rank + self.cfg.qk_rope_head_dim) * \
            torch.empty((), dtype=kv_dtype).element_size()
