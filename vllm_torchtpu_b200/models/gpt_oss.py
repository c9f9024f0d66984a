"""GPT-OSS family: GQA attention with per-head attention sinks and biases, sliding-window and full-attention
layers in alternation (``layer_types``), YaRN RoPE; every FFN a mixture of experts with a biased router (top-k on
the logits, softmax over the chosen ones), expert biases and the clamped OAI SwiGLU; experts in mxfp4 in the
published checkpoints (kept packed: W4A16 kernel).

The hidden size of the published models (2880) is not a multiple of the GEMM kernels' 128-row tile: the experts'
down projection is stored with zero rows up to the tile and its output is cut back.
(reference: src/vllm_torchtpu/layers/adapter/quantization/mxfp4.py:96-761 — the mxfp4 MoE method the reference
ships for this family; kernels/megablox/gmm_v2.py:30-38 swigluoai)"""
from __future__ import annotations

import torch

from ..layers.moe import FusedMoE
from .llama import LlamaDecoderLayer, LlamaForCausalLM


class GptOssMoEBlock:
    def __init__(self, name, cfg, device, quant):
        self.experts = FusedMoE(name, cfg, device, quant)
        self.shared = None
        self.shared_gate = None

    def linears(self):
        return [self.experts.gate]

    def init_dummy(self, std, seed):
        self.experts.init_dummy(std, seed)

    def weight_bytes(self):
        e = self.experts
        return e.weight_bytes() + sum(t.numel() * t.element_size() for t in (e.b13, e.b2) if t is not None)

    def forward(self, x):
        return self.experts.forward(x)


class GptOssDecoderLayer(LlamaDecoderLayer):
    def __init__(self, idx: int, cfg, device, quant):
        super().__init__(idx, cfg, device, quant)
        a = self.self_attn
        sliding = cfg.layer_sliding[idx % len(cfg.layer_sliding)] if cfg.layer_sliding else bool(cfg.sliding_window)
        a.attn.sliding_window = cfg.sliding_window if sliding else None
        # one learnable logit per query head that takes part in the softmax without a value
        self.sinks = torch.zeros(a.qkv.q_per_rank, dtype=torch.float32, device=device)
        a.attn.sinks = self.sinks
        self.q_heads = (a.qkv._r * a.qkv.q_per_rank, a.qkv.q_per_rank)     # this rank's slice of the heads

    def _make_ffn(self, name, cfg, device, quant):
        return GptOssMoEBlock(f"{name}.mlp", cfg, device, quant)

    def load_sinks(self, full: torch.Tensor) -> None:
        lo, n = self.q_heads
        self.sinks.copy_(full.float()[lo:lo + n].to(self.sinks.device))


class GptOssForCausalLM(LlamaForCausalLM):
    layer_cls = GptOssDecoderLayer

    def init_dummy(self) -> None:
        super().init_dummy()
        from ..layers.linear import seeded_normal
        for l in self.layers:
            l.sinks.copy_(seeded_normal(f"model.layers.{l.idx}.sinks", (self.cfg.num_q_heads,), 1.0, torch.float32,
                                        self.device, self.cfg.seed)[l.q_heads[0]:l.q_heads[0] + l.q_heads[1]])
            for lin in (l.self_attn.qkv, l.self_attn.o):
                if lin.bias is not None:
                    lin.bias = seeded_normal(lin.name + ".bias", (lin.bias.shape[0],), 0.05, lin.dtype, self.device,
                                             self.cfg.seed)
