"""Qwen3-MoE family (Qwen3-30B-A3B, Qwen3-Coder): GQA attention with per-head q/k
RMSNorm, every FFN a routed mixture of experts (softmax router, top-k, renormalised).

Under expert parallelism attention runs data-parallel (each rank holds all heads
and serves its own requests) and the experts are sharded over the EP group; the
MoE layer exchanges tokens with the fused dispatch/combine kernel."""
from __future__ import annotations

from ..layers.moe import FusedMoE
from .llama import LlamaDecoderLayer, LlamaForCausalLM, LlamaMLP


class MoEBlock:
    """Routed experts plus optional shared experts (dense MLP added to the routed output)."""

    def __init__(self, name, cfg, device, quant):
        self.experts = FusedMoE(f"{name}", cfg, device, quant)
        self.shared = None
        if cfg.num_shared_experts > 0:
            self.shared = LlamaMLP(f"{name}.shared_experts", cfg,
                                   cfg.moe_intermediate_size * cfg.num_shared_experts, device, quant)

    def linears(self):
        return [self.experts.gate] + (self.shared.linears() if self.shared else [])

    def init_dummy(self, std, seed):
        self.experts.init_dummy(std, seed)
        if self.shared:
            self.shared.init_dummy(std, seed)

    def weight_bytes(self):
        return self.experts.weight_bytes() + (self.shared.weight_bytes() if self.shared else 0)

    def forward(self, x):
        y = self.experts.forward(x)
        if self.shared is not None:
            y = y + self.shared.forward(x)
        return y


class Qwen3MoeDecoderLayer(LlamaDecoderLayer):
    def _make_ffn(self, name, cfg, device, quant):
        if cfg.layer_is_moe(self.idx):
            return MoEBlock(f"{name}.mlp", cfg, device, quant)
        return LlamaMLP(f"{name}.mlp", cfg, cfg.intermediate_size, device, quant)


class Qwen3MoeForCausalLM(LlamaForCausalLM):
    layer_cls = Qwen3MoeDecoderLayer
