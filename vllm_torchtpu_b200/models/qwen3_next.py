"""Hybrid Gated-DeltaNet decoder (Qwen3-Next / Qwen3.5 style): every ``full_attention_interval``-th
layer is softmax GQA attention over the paged KV cache, the others are Gated DeltaNet linear
attention whose state (a conv window and a [Hv, dk, dv] matrix per request) lives in per-layer
state pools indexed by the request's batch slot, not in scheduler blocks
(reference: src/vllm_torchtpu/layers/adapter/custom_ops/gdn_attention_op.py,
core/runner_slot_mamba.py:66-209 "GDN groups that take no scheduler blocks").

GDN layer: in_proj → [q|k|v] channels + z gate + (b, a) per value head → causal conv1d + SiLU →
gated delta rule → RMSNorm(o) * SiLU(z) → out_proj (row parallel).
Heads are sharded over TP (k heads and v heads alike)."""
from __future__ import annotations

import torch

from .. import ops
from ..config import ModelConfig
from ..layers.linear import ColumnParallelLinear, RowParallelLinear, seeded_normal
from ..ops import gdn_reference as gref
from ..parallel.state import get_state
from .llama import LlamaDecoderLayer, LlamaForCausalLM, LlamaMLP
from .qwen3_moe import MoEBlock


class GatedDeltaNet:
    def __init__(self, name: str, cfg: ModelConfig, device, quant):
        st = get_state()
        tp = st.tp.size
        self.name, self.cfg, self.device = name, cfg, device
        self.Hk, self.Hv = cfg.gdn_num_k_heads // tp, cfg.gdn_num_v_heads // tp
        self.dk, self.dv = cfg.gdn_head_k_dim, cfg.gdn_head_v_dim
        self.K = cfg.gdn_conv_kernel
        kw = dict(dtype=cfg.dtype, device=device, quant_config=quant)
        key_dim, val_dim = cfg.gdn_num_k_heads * self.dk, cfg.gdn_num_v_heads * self.dv
        self.in_qkvz = ColumnParallelLinear(f"{name}.in_proj_qkvz", cfg.hidden_size,
                                            [key_dim, key_dim, val_dim, val_dim], **kw)
        self.in_ba = ColumnParallelLinear(f"{name}.in_proj_ba", cfg.hidden_size,
                                          [cfg.gdn_num_v_heads, cfg.gdn_num_v_heads], **kw)
        self.out = RowParallelLinear(f"{name}.out_proj", val_dim, cfg.hidden_size, **kw)
        self.channels = 2 * self.Hk * self.dk + self.Hv * self.dv
        self.conv_w = None
        self.A_log = None
        self.dt_bias = None
        self.norm_w = torch.ones(self.dv, dtype=cfg.dtype, device=device)
        self.eps = cfg.rms_norm_eps

    def linears(self):
        return [self.in_qkvz, self.in_ba, self.out]

    def init_dummy(self, std, seed):
        for l in self.linears():
            l.init_dummy(std, seed)
        d, dev = self.cfg.dtype, self.device
        self.conv_w = seeded_normal(f"{self.name}.conv1d", (self.channels, self.K), 0.2, d, dev, seed)
        self.A_log = seeded_normal(f"{self.name}.A_log", (self.Hv,), 0.5, torch.float32, dev, seed)
        self.dt_bias = seeded_normal(f"{self.name}.dt_bias", (self.Hv,), 0.5, torch.float32, dev, seed)

    def weight_bytes(self):
        n = sum(l.weight_bytes() for l in self.linears())
        return n + self.conv_w.numel() * self.conv_w.element_size()

    def state_shapes(self, max_reqs: int):
        return (max_reqs + 1, self.channels, self.K - 1), (max_reqs + 1, self.Hv, self.dk, self.dv)

    def recur(self, inputs, meta, cache):
        """The stateful part: conv window + delta-rule recurrence over the rows ``meta`` describes; advances
        the pools in place.  inputs = (mixed [T, C], a [T, Hv], b [T, Hv])."""
        mixed, a, b = inputs
        conv_pool, rec_pool = cache
        if mixed.is_cuda:
            return ops.cuda_ops().gdn_forward(mixed, a, b, meta, conv_pool, rec_pool, self.conv_w, self.A_log,
                                              self.dt_bias, self.Hk, self.Hv, self.dk, self.dv)
        return gref.gdn_forward(mixed, a, b, None, meta, conv_pool, rec_pool, self.conv_w, self.A_log,
                                self.dt_bias, self.Hk, self.Hv, self.dk, self.dv)

    def forward(self, x, cache, meta):
        T = x.shape[0]
        qkvz = self.in_qkvz(x)
        kd, vd = self.Hk * self.dk, self.Hv * self.dv
        mixed, z = qkvz[:, :2 * kd + vd], qkvz[:, 2 * kd + vd:]
        ba = self.in_ba(x)
        b, a = ba[:, :self.Hv], ba[:, self.Hv:]
        inputs = (mixed.contiguous(), a.contiguous(), b.contiguous())
        rb = getattr(meta, "state_rollback", None)
        if rb is not None:
            rb.capture(self, cache, inputs)        # verification step: rejected drafts are rolled back later
        o = self.recur(inputs, meta, cache)
        o = ops.rms_norm(o.reshape(T * self.Hv, self.dv), self.norm_w, self.eps).reshape(T, self.Hv, self.dv)
        zf = z.reshape(T, self.Hv, self.dv).float()
        o = (o.float() * torch.nn.functional.silu(zf)).to(x.dtype)
        return self.out(o.reshape(T, self.Hv * self.dv))


class Qwen3NextDecoderLayer(LlamaDecoderLayer):
    def __init__(self, idx: int, cfg: ModelConfig, device, quant):
        self.full_attention = cfg.layer_is_full_attention(idx)
        if self.full_attention:
            super().__init__(idx, cfg, device, quant)
            return
        name = f"model.layers.{idx}"
        self.idx = idx
        self.eps = cfg.rms_norm_eps
        self.input_ln = torch.ones(cfg.hidden_size, dtype=cfg.dtype, device=device)
        self.post_ln = torch.ones(cfg.hidden_size, dtype=cfg.dtype, device=device)
        self.self_attn = GatedDeltaNet(f"{name}.linear_attn", cfg, device, quant)
        self.mlp = self._make_ffn(name, cfg, device, quant)

    def _make_ffn(self, name, cfg, device, quant):
        if cfg.layer_is_moe(self.idx):
            return MoEBlock(f"{name}.mlp", cfg, device, quant)
        return LlamaMLP(f"{name}.mlp", cfg, cfg.intermediate_size, device, quant)


class Qwen3NextForCausalLM(LlamaForCausalLM):
    layer_cls = Qwen3NextDecoderLayer

    def init_dummy(self) -> None:
        cfg = self.cfg
        std, seed = cfg.init_std, cfg.seed
        if self.pp_first or cfg.tie_word_embeddings:
            self.embed = seeded_normal("model.embed_tokens", (cfg.vocab_size, cfg.hidden_size), std, cfg.dtype,
                                       self.device, seed)
        if self.pp_last:
            self.lm_head = self._shard_vocab(seeded_normal("lm_head", (cfg.vocab_size, cfg.hidden_size), std,
                                                           cfg.dtype, self.device, seed))
        for l in self.layers:
            if l.full_attention:
                for lin in l.self_attn.linears():
                    lin.init_dummy(std, seed)
            else:
                l.self_attn.init_dummy(std, seed)
            l.mlp.init_dummy(std, seed)

    def weight_bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for t in (self.embed, self.lm_head) if t is not None)
        for l in self.layers:
            n += (sum(x.weight_bytes() for x in l.self_attn.linears()) if l.full_attention
                  else l.self_attn.weight_bytes())
            n += l.mlp.weight_bytes()
        return n

    def _attn_layer(self):
        return next(l for l in self.layers if l.full_attention).self_attn.attn

    def kv_cache_shape(self, num_blocks: int, block_size: int) -> tuple:
        a = self._attn_layer()
        return (num_blocks, 2, a.num_kv_heads, block_size, a.head_dim)

    def kv_bytes_per_block(self, block_size: int, kv_dtype: torch.dtype) -> int:
        a = self._attn_layer()
        n_full = sum(1 for l in self.layers if l.full_attention)
        return n_full * 2 * a.num_kv_heads * block_size * a.head_dim * torch.empty((), dtype=kv_dtype).element_size()

    def allocate_kv_caches(self, num_blocks: int, block_size: int, kv_dtype, device, max_reqs: int = 256):
        caches = []
        for l in self.layers:
            if l.full_attention:
                caches.append(torch.zeros(self.kv_cache_shape(num_blocks, block_size), dtype=kv_dtype, device=device))
            else:
                cs, rs = l.self_attn.state_shapes(max_reqs)
                caches.append((torch.zeros(cs, dtype=self.cfg.dtype, device=device),
                               torch.zeros(rs, dtype=torch.float32, device=device)))
        return caches
