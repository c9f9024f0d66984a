"""Qwen3-MoE family (Qwen3-30B-A3B, Qwen3-Coder): GQA attention with per-head q/k
RMSNorm, every FFN a routed mixture of experts (softmax router, top-k, renormalised).
Mixtral (no q/k norm, experts of `intermediate_size`) and Qwen2-MoE (attention bias,
one shared expert behind a sigmoid gate) are the same model with other configuration.

Under expert parallelism attention runs data-parallel (each rank holds all heads
and serves its own requests) and the experts are sharded over the EP group; the
MoE layer exchanges tokens with the fused dispatch/combine kernel."""
from __future__ import annotations

import torch

from ..layers.moe import FusedMoE
from ..layers.linear import seeded_normal
from .llama import LlamaDecoderLayer, LlamaForCausalLM, LlamaMLP


class MoEBlock:
    """Routed experts plus optional shared experts (dense MLP added to the routed output)."""

    def __init__(self, name, cfg, device, quant):
        self.experts = FusedMoE(f"{name}", cfg, device, quant)
        self.shared = None
        self.shared_gate = None                 # [hidden]: the shared expert's output times sigmoid(x . w)
        self.name, self.cfg, self.device = name, cfg, device
        if cfg.num_shared_experts > 0:
            size = cfg.shared_expert_intermediate_size or cfg.moe_intermediate_size * cfg.num_shared_experts
            self.shared = LlamaMLP(f"{name}.shared_experts", cfg, size, device, quant)
            if cfg.shared_expert_gate:
                self.shared_gate = torch.zeros(cfg.hidden_size, dtype=cfg.dtype, device=device)

    def linears(self):
        return [self.experts.gate] + (self.shared.linears() if self.shared else [])

    def init_dummy(self, std, seed):
        self.experts.init_dummy(std, seed)
        if self.shared:
            self.shared.init_dummy(std, seed)
        if self.shared_gate is not None:
            self.shared_gate = seeded_normal(f"{self.name}.shared_expert_gate", (self.cfg.hidden_size,), std,
                                             self.cfg.dtype, self.device, seed)

    def weight_bytes(self):
        return self.experts.weight_bytes() + (self.shared.weight_bytes() if self.shared else 0)

    def forward(self, x):
        y = self.experts.forward(x)
        if self.shared is not None:
            sh = self.shared.forward(x)
            if self.shared_gate is not None:
                y = torch.addcmul(y, torch.sigmoid(torch.mv(x, self.shared_gate).float()).to(x.dtype)[:, None], sh)
            else:
                y = y + sh
        return y


class Qwen3MoeDecoderLayer(LlamaDecoderLayer):
    def _make_ffn(self, name, cfg, device, quant):
        if cfg.layer_is_moe(self.idx):
            return MoEBlock(f"{name}.mlp", cfg, device, quant)
        return LlamaMLP(f"{name}.mlp", cfg, cfg.intermediate_size, device, quant)


class Qwen3MoeForCausalLM(LlamaForCausalLM):
    layer_cls = Qwen3MoeDecoderLayer
