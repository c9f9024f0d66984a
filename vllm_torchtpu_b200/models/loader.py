"""Hugging Face safetensors loader (and a matching exporter used by tests).

Checkpoint tensors are streamed file by file; q/k/v and gate/up pieces are buffered until their
fused parameter is complete, then handed to the layer's quantisation method, which shards for
this TP/EP rank and re-lays-out or re-quantises once
(reference flow: src/vllm_torchtpu/runner/tpu_runner.py:5999-6152 → vLLM loaders →
``process_weights_after_loading``, src/vllm_torchtpu/layers/adapter/quantization/fp8.py:1543-1675).
Block-scaled fp8 checkpoints carry ``<name>.weight_scale_inv`` next to ``<name>.weight``.
Under expert parallelism only the experts this rank owns are read
(reference: src/vllm_torchtpu/model_loader_patches.py:14-40).
"""
from __future__ import annotations

import glob
import json
import os
import re
from typing import Iterator, Optional

import torch

from ..logger import init_logger
from ..parallel.state import get_state

logger = init_logger(__name__)


def iter_safetensors(path: str) -> Iterator[tuple]:
    from safetensors import safe_open
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {path}")
    for f in files:
        with safe_open(f, framework="pt", device="cpu") as sf:
            for name in sf.keys():
                yield name, sf.get_tensor(name)


class _Pending:
    """Collects the pieces of a fused parameter."""

    def __init__(self, need: tuple):
        self.need = need
        self.parts: dict = {}

    def add(self, key, t):
        self.parts[key] = t
        return all(k in self.parts for k in self.need)

    def cat(self):
        return torch.cat([self.parts[k] for k in self.need], 0)


def _set_vec(dst: torch.Tensor, src: torch.Tensor) -> None:
    dst.copy_(src.to(device=dst.device, dtype=dst.dtype))


def load_safetensors(model, path: str) -> None:
    cfg = model.cfg
    st = get_state()
    lo, hi = model.layer_range
    layers = {lo + i: l for i, l in enumerate(model.layers)}
    pend: dict = {}
    scales: dict = {}
    seen = 0
    rx = re.compile(r"^model\.layers\.(\d+)\.(.+)$")

    def fused(key, need, part, tensor, target, suffix):
        p = pend.setdefault((key, suffix), _Pending(need))
        if p.add(part, tensor):
            if suffix == "weight":
                kw = {}
                sp = pend.get((key, "weight_scale_inv"))
                if sp is not None and all(k in sp.parts for k in need):
                    kw["scale_inv"] = sp.cat()
                target.load_weight(p.cat(), **kw)
            elif suffix == "bias":
                target.bias = target.shard_of(p.cat()[:, None])[:, 0].to(device=target.device,
                                                                         dtype=target.dtype).contiguous()

    for name, t in iter_safetensors(path):
        seen += 1
        if name == "model.embed_tokens.weight":
            if model.pp_first or cfg.tie_word_embeddings:
                model.embed = t.to(device=model.device, dtype=cfg.dtype)
                if cfg.tie_word_embeddings and model.pp_last:
                    model.lm_head = model._shard_vocab(model.embed)
            continue
        if name == "lm_head.weight":
            if model.pp_last:
                model.lm_head = model._shard_vocab(t.to(device=model.device, dtype=cfg.dtype))
            continue
        if name == "model.norm.weight":
            _set_vec(model.norm, t)
            continue
        m = rx.match(name)
        if not m:
            continue
        li, rest = int(m.group(1)), m.group(2)
        if li not in layers:
            continue
        layer = layers[li]
        a = layer.self_attn
        if rest == "input_layernorm.weight":
            _set_vec(layer.input_ln, t)
        elif rest == "post_attention_layernorm.weight":
            _set_vec(layer.post_ln, t)
        elif rest.startswith("self_attn."):
            sub = rest[len("self_attn."):]
            pm = re.match(r"^([qkv])_proj\.(weight|bias|weight_scale_inv)$", sub)
            if pm and hasattr(a, "qkv"):
                fused(("qkv", li), ("q", "k", "v"), pm.group(1), t, a.qkv, pm.group(2))
            elif sub == "o_proj.weight":
                a.o.load_weight(t, scale_inv=scales.pop((li, "o"), None)) if hasattr(a, "o") else None
            elif sub == "q_norm.weight" and a.q_norm_w is not None:
                _set_vec(a.q_norm_w, t)
            elif sub == "k_norm.weight" and a.k_norm_w is not None:
                _set_vec(a.k_norm_w, t)
            elif hasattr(a, "kv_a"):                      # MLA
                simple = {"q_a_proj.weight": "q_a", "q_b_proj.weight": "q_b", "q_proj.weight": "q_b",
                          "kv_a_proj_with_mqa.weight": "kv_a"}
                if sub in simple and getattr(a, simple[sub], None) is not None:
                    getattr(a, simple[sub]).load_weight(t)
                elif sub == "q_a_layernorm.weight":
                    _set_vec(a.q_a_ln, t)
                elif sub == "kv_a_layernorm.weight":
                    _set_vec(a.kv_a_ln, t)
                elif sub == "kv_b_proj.weight":
                    a.load_kv_b(t.to(device=model.device, dtype=cfg.dtype))
        elif rest.startswith("mlp."):
            sub = rest[len("mlp."):]
            mlp = layer.mlp
            pm = re.match(r"^(gate|up)_proj\.(weight|weight_scale_inv)$", sub)
            if pm and hasattr(mlp, "gate_up"):
                fused(("gu", li), ("gate", "up"), pm.group(1), t, mlp.gate_up, pm.group(2))
            elif sub == "down_proj.weight" and hasattr(mlp, "down"):
                mlp.down.load_weight(t)
            elif hasattr(mlp, "experts"):
                moe = mlp.experts
                if sub == "gate.weight":
                    moe.gate.load_weight(t)
                elif sub == "gate.e_score_correction_bias" and moe.score_bias is not None:
                    _set_vec(moe.score_bias, t)
                else:
                    em = re.match(r"^experts\.(\d+)\.(gate|up|down)_proj\.weight$", sub)
                    sm = re.match(r"^shared_experts?\.(gate|up|down)_proj\.weight$", sub)
                    if em:
                        e = int(em.group(1))
                        elo, ehi = moe.expert_range
                        if elo <= e < ehi:               # expert-parallel weight filter
                            p = pend.setdefault(("exp", li, e), _Pending(("gate", "up", "down")))
                            if p.add(em.group(2), t):
                                if moe.w13 is None:
                                    moe.method.alloc(moe)
                                I, r, n = moe.intermediate_size, moe.tp_rank, moe.tp_size
                                g = p.parts["gate"][r * I:(r + 1) * I] if n > 1 else p.parts["gate"]
                                u = p.parts["up"][r * I:(r + 1) * I] if n > 1 else p.parts["up"]
                                d = p.parts["down"][:, r * I:(r + 1) * I] if n > 1 else p.parts["down"]
                                moe.method.load_expert(moe, e - elo, g, u, d)
                                del pend[("exp", li, e)]
                    elif sm and mlp.shared is not None:
                        if sm.group(1) == "down":
                            mlp.shared.down.load_weight(t)
                        else:
                            fused(("sgu", li), ("gate", "up"), sm.group(1), t, mlp.shared.gate_up, "weight")
    logger.info("loaded %d tensors from %s on rank %d", seen, path, st.rank)


def save_hf_checkpoint(model, path: str, hf_config: Optional[dict] = None) -> None:
    """Write an unsharded single-rank dense/MoE model in Hugging Face layout (tests, export)."""
    from safetensors.torch import save_file
    cfg = model.cfg
    os.makedirs(path, exist_ok=True)
    out = {"model.embed_tokens.weight": model.embed, "model.norm.weight": model.norm, "lm_head.weight": model.lm_head}
    D = cfg.head_dim
    for i, l in enumerate(model.layers):
        pre = f"model.layers.{i}."
        out[pre + "input_layernorm.weight"] = l.input_ln
        out[pre + "post_attention_layernorm.weight"] = l.post_ln
        a = l.self_attn
        if hasattr(a, "qkv"):
            q, k, v = a.qkv.weight.split([cfg.num_q_heads * D, cfg.num_kv_heads * D, cfg.num_kv_heads * D], 0)
            out[pre + "self_attn.q_proj.weight"], out[pre + "self_attn.k_proj.weight"] = q, k
            out[pre + "self_attn.v_proj.weight"], out[pre + "self_attn.o_proj.weight"] = v, a.o.weight
            if a.q_norm_w is not None:
                out[pre + "self_attn.q_norm.weight"], out[pre + "self_attn.k_norm.weight"] = a.q_norm_w, a.k_norm_w
        mlp = l.mlp
        if hasattr(mlp, "gate_up"):
            I = mlp.gate_up.weight.shape[0] // 2
            out[pre + "mlp.gate_proj.weight"], out[pre + "mlp.up_proj.weight"] = mlp.gate_up.weight[:I], mlp.gate_up.weight[I:]
            out[pre + "mlp.down_proj.weight"] = mlp.down.weight
        else:
            moe = mlp.experts
            out[pre + "mlp.gate.weight"] = moe.gate.weight
            I = moe.intermediate_size
            for e in range(moe.num_local_experts):
                out[pre + f"mlp.experts.{e}.gate_proj.weight"] = moe.w13[e, :I]
                out[pre + f"mlp.experts.{e}.up_proj.weight"] = moe.w13[e, I:]
                out[pre + f"mlp.experts.{e}.down_proj.weight"] = moe.w2[e]
    save_file({k: v.detach().cpu().contiguous() for k, v in out.items()}, os.path.join(path, "model.safetensors"))
    if hf_config is not None:
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(hf_config, f)
