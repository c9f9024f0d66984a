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


def _fadvise(path: str, advice: int) -> None:
    """Page-cache hint for a whole file (no-op where the platform has none)."""
    if not hasattr(os, "posix_fadvise"):
        return
    try:
        fd = os.open(path, os.O_RDONLY)
        try:
            os.posix_fadvise(fd, 0, 0, advice)
        finally:
            os.close(fd)
    except OSError:
        pass


def iter_safetensors(path: str) -> Iterator[tuple]:
    """(name, tensor) of every tensor in a safetensors file or in the files of a directory.  While a file is
    parsed the kernel is asked to read the next one ahead (``B200_SAFETENSORS_PREFETCH``), and a consumed file
    can be dropped from the page cache so that a large checkpoint does not push the host out of memory
    (``B200_LOAD_EVICT_PAGE_CACHE``)
    (reference: src/vllm_torchtpu/model_loader_patches.py — prefetch load strategy, page-cache eviction)."""
    from safetensors import safe_open
    from .. import envs
    files = [path] if os.path.isfile(path) else sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {path}")
    prefetch, evict = envs.B200_SAFETENSORS_PREFETCH, envs.B200_LOAD_EVICT_PAGE_CACHE
    for i, f in enumerate(files):
        if prefetch and i + 1 < len(files):
            _fadvise(files[i + 1], getattr(os, "POSIX_FADV_WILLNEED", 3))
        with safe_open(f, framework="pt", device="cpu") as sf:
            for name in sf.keys():
                yield name, sf.get_tensor(name)
        if evict:
            _fadvise(f, getattr(os, "POSIX_FADV_DONTNEED", 4))


class _Collector:
    """Buffers the pieces of one parameter (the q/k/v or gate/up parts of a fused matrix, and for
    block-scaled fp8 checkpoints the ``weight_scale_inv`` grid of every part) until all of them have
    been read, in whatever order the files list them, then calls ``done(parts)`` once."""

    def __init__(self, need: set, done):
        self.need, self.done, self.parts = set(need), done, {}

    def add(self, key, tensor) -> bool:
        self.parts[key] = tensor
        if self.need.issubset(self.parts):
            self.done(self.parts)
            return True
        return False


def _set_vec(dst: torch.Tensor, src: torch.Tensor) -> None:
    dst.copy_(src.to(device=dst.device, dtype=dst.dtype))


def list_tensor_names(path: str) -> set:
    from safetensors import safe_open
    names = set()
    for f in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
        with safe_open(f, framework="pt", device="cpu") as sf:
            names.update(sf.keys())
    return names


_FP8_DTYPES = (torch.float8_e4m3fn, torch.float8_e5m2)


def load_safetensors(model, path: str) -> None:
    load_named_tensors(model, iter_safetensors(path), list_tensor_names(path), source=path)


_MIXTRAL_EXPERT = {"w1": "gate_proj", "w3": "up_proj", "w2": "down_proj"}


def canonical_name(name: str) -> str:
    """Checkpoint name → the Llama / Qwen-MoE naming the loader walks: Mixtral keeps its experts under
    ``block_sparse_moe`` with ``w1 / w3 / w2`` for gate / up / down."""
    if ".mlp.router." in name:                       # GPT-OSS names its router "router"
        name = name.replace(".mlp.router.", ".mlp.gate.")
    if ".block_sparse_moe." in name:
        name = name.replace(".block_sparse_moe.", ".mlp.")
        m = re.match(r"^(.*\.experts\.\d+\.)(w[123])(\..+)$", name)
        if m:
            name = m.group(1) + _MIXTRAL_EXPERT[m.group(2)] + m.group(3)
    return name


_OSS_EXPERT_TENSORS = ("gate_up_proj", "down_proj", "gate_up_proj_bias", "down_proj_bias", "gate_up_proj_blocks",
                       "gate_up_proj_scales", "down_proj_blocks", "down_proj_scales")


def _load_oss_experts(moe, parts: dict) -> None:
    """GPT-OSS expert stacks.  bf16: ``gate_up_proj`` [E, H, 2I] and ``down_proj`` [E, I, H] (input-major);
    mxfp4: ``*_blocks`` [E, rows, K / 32, 16] packed nibbles with ``*_scales`` [E, rows, K / 32].  Gate and up
    alternate along the 2I axis (gate at the even positions) in weights and biases alike."""
    from ..quantization.fp4 import Mxfp4MoEMethod, dequantize_mxfp4
    lo, hi = moe.expert_range
    if moe.w13 is None:
        moe.method.alloc(moe)
    packed = "gate_up_proj_blocks" in parts
    for e in range(lo, hi):
        if packed:
            gu_q = parts["gate_up_proj_blocks"][e].flatten(-2)            # [2I, H / 2]
            gu_s = parts["gate_up_proj_scales"][e]
            d_q = parts["down_proj_blocks"][e].flatten(-2)                # [H, I / 2]
            d_s = parts["down_proj_scales"][e]
            w13_q, w13_s = torch.cat([gu_q[0::2], gu_q[1::2]], 0), torch.cat([gu_s[0::2], gu_s[1::2]], 0)
            if isinstance(moe.method, Mxfp4MoEMethod) and moe.tp_size == 1:
                moe.method.load_packed_expert(moe, e - lo, w13_q.contiguous(), w13_s.contiguous(), d_q, d_s)
            else:
                w13 = dequantize_mxfp4(w13_q.contiguous(), w13_s.contiguous())
                I = w13.shape[0] // 2
                moe.method.load_expert(moe, e - lo, w13[:I], w13[I:], dequantize_mxfp4(d_q.contiguous(), d_s.contiguous()))
        else:
            gu = parts["gate_up_proj"][e].t()                             # [2I, H]
            moe.method.load_expert(moe, e - lo, gu[0::2], gu[1::2], parts["down_proj"][e].t())
        if "gate_up_proj_bias" in parts:
            b = parts["gate_up_proj_bias"][e]
            moe.load_expert_bias(e - lo, b[0::2], b[1::2], parts["down_proj_bias"][e])


def load_named_tensors(model, tensors, names: set, source: str = "memory") -> None:
    """Load checkpoint-named tensors (Hugging Face layout) from any iterator of (name, tensor): a directory
    of safetensors files, or tensors handed over in memory by a trainer (``LLMEngine.update_weights``).
    ``names`` is the set of all names the iterator will yield (fused parameters wait for their pieces)."""
    path = source
    cfg = model.cfg
    st = get_state()
    lo, hi = model.layer_range
    layers = {lo + i: l for i, l in enumerate(model.layers)}
    open_groups: dict = {}
    seen = 0
    rx = re.compile(r"^model\.layers\.(\d+)\.(.+)$")
    names = {canonical_name(n) for n in names}

    def submit(gid, ckpt_prefixes: dict, part: str, kind: str, tensor, done) -> None:
        """Piece ``kind`` ("weight" or "weight_scale_inv") of ``part`` of parameter group ``gid``;
        ``ckpt_prefixes`` maps every part to its checkpoint name so that the group knows which scale
        tensors the checkpoint holds.  ``done(parts)`` gets {(part, kind): tensor}."""
        g = open_groups.get(gid)
        if g is None:
            need = set()
            for pt, prefix in ckpt_prefixes.items():
                need.add((pt, "weight"))
                if prefix + ".weight_scale_inv" in names:
                    need.add((pt, "weight_scale_inv"))
            g = open_groups[gid] = _Collector(need, done)
        if g.add((part, kind), tensor):
            del open_groups[gid]

    def cat_parts(parts, order, kind):
        got = [parts.get((p, kind)) for p in order]
        if any(t is None for t in got):
            return None
        return torch.cat(got, 0) if len(got) > 1 else got[0]

    def load_linear(target, order, what):
        def done(parts):
            w = cat_parts(parts, order, "weight")
            s = cat_parts(parts, order, "weight_scale_inv")
            if w.dtype in _FP8_DTYPES and s is None:
                raise ValueError(f"{what}: the checkpoint holds fp8 weights without weight_scale_inv")
            bn = int(cfg.weight_block_size[0])
            if s is not None and any(parts[(p, "weight")].shape[0] % bn for p in order[:-1]):
                # the row blocks of the packed pieces do not line up with one grid: expand each piece
                from ..quantization.fp8 import dequantize_weight_block
                w = torch.cat([dequantize_weight_block(parts[(p, "weight")], parts[(p, "weight_scale_inv")].float(),
                                                       tuple(cfg.weight_block_size)) for p in order], 0)
                s = None
            target.load_weight(w, **({"scale_inv": s} if s is not None else {}))
        return done

    def linear_piece(gid, target, prefixes: dict, part, kind, t, what):
        submit(gid, prefixes, part, kind, t, load_linear(target, tuple(prefixes), what))

    for name, t in tensors:
        seen += 1
        name = canonical_name(name)
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
        pre = f"model.layers.{li}."
        if rest == "input_layernorm.weight":
            _set_vec(layer.input_ln, t)
        elif rest == "post_attention_layernorm.weight":
            _set_vec(layer.post_ln, t)
        elif rest.startswith("self_attn."):
            sub = rest[len("self_attn."):]
            ap = pre + "self_attn."
            pm = re.match(r"^([qkv])_proj\.(weight|bias|weight_scale_inv)$", sub)
            om = re.match(r"^o_proj\.(weight|weight_scale_inv)$", sub)
            mm = re.match(r"^(q_a_proj|q_b_proj|q_proj|kv_a_proj_with_mqa|kv_b_proj)\.(weight|weight_scale_inv)$", sub)
            if pm and hasattr(a, "qkv"):
                if pm.group(2) == "bias":
                    def bias_done(parts, target=a.qkv):
                        full = torch.cat([parts[(p, "weight")] for p in ("q", "k", "v")], 0)
                        target.bias = target.shard_of(full[:, None])[:, 0].to(
                            device=target.device, dtype=target.dtype).contiguous()
                    g = open_groups.setdefault(("qkv_bias", li), _Collector(
                        {(p, "weight") for p in ("q", "k", "v")}, bias_done))
                    if g.add((pm.group(1), "weight"), t):
                        del open_groups[("qkv_bias", li)]
                else:
                    linear_piece(("qkv", li), a.qkv, {p: f"{ap}{p}_proj" for p in ("q", "k", "v")},
                                 pm.group(1), pm.group(2), t, f"{ap}qkv_proj")
            elif sub == "qkv_proj.weight" and hasattr(a, "qkv"):
                a.qkv.load_weight(t)                     # Phi-3: q, k, v rows already stacked in this order
            elif om and hasattr(a, "o"):
                linear_piece(("o", li), a.o, {"o": ap + "o_proj"}, "o", om.group(1), t, ap + "o_proj")
            elif sub == "o_proj.bias" and hasattr(a, "o"):
                a.o.bias = t.to(device=a.o.device, dtype=a.o.dtype).contiguous()
            elif sub == "sinks" and hasattr(layer, "load_sinks"):
                layer.load_sinks(t)
            elif sub == "q_norm.weight" and a.q_norm_w is not None:
                _set_vec(a.q_norm_w, t)
            elif sub == "k_norm.weight" and a.k_norm_w is not None:
                _set_vec(a.k_norm_w, t)
            elif hasattr(a, "kv_a"):                      # MLA
                simple = {"q_a_proj": "q_a", "q_b_proj": "q_b", "q_proj": "q_b", "kv_a_proj_with_mqa": "kv_a"}
                if mm and mm.group(1) in simple and getattr(a, simple[mm.group(1)], None) is not None:
                    linear_piece((mm.group(1), li), getattr(a, simple[mm.group(1)]),
                                 {"w": ap + mm.group(1)}, "w", mm.group(2), t, ap + mm.group(1))
                elif mm and mm.group(1) == "kv_b_proj":
                    def kvb_done(parts, a=a):
                        w, s = parts[("w", "weight")], parts.get(("w", "weight_scale_inv"))
                        if w.dtype in _FP8_DTYPES:
                            if s is None:
                                raise ValueError("kv_b_proj: fp8 weights without weight_scale_inv")
                            from ..quantization.fp8 import dequantize_weight_block
                            w = dequantize_weight_block(w, s.float(), tuple(cfg.weight_block_size))
                        a.load_kv_b(w.to(device=model.device, dtype=cfg.dtype))
                    submit(("kv_b", li), {"w": ap + "kv_b_proj"}, "w", mm.group(2), t, kvb_done)
                elif sub == "q_a_layernorm.weight":
                    _set_vec(a.q_a_ln, t)
                elif sub == "kv_a_layernorm.weight":
                    _set_vec(a.kv_a_ln, t)
        elif rest.startswith("mlp."):
            sub = rest[len("mlp."):]
            mp = pre + "mlp."
            mlp = layer.mlp
            pm = re.match(r"^(gate|up)_proj\.(weight|weight_scale_inv)$", sub)
            dm = re.match(r"^down_proj\.(weight|weight_scale_inv)$", sub)
            if pm and hasattr(mlp, "gate_up"):
                linear_piece(("gu", li), mlp.gate_up, {p: f"{mp}{p}_proj" for p in ("gate", "up")},
                             pm.group(1), pm.group(2), t, mp + "gate_up_proj")
            elif sub == "gate_up_proj.weight" and hasattr(mlp, "gate_up"):
                mlp.gate_up.load_weight(t)               # Phi-3: gate rows then up rows
            elif dm and hasattr(mlp, "down"):
                linear_piece(("down", li), mlp.down, {"d": mp + "down_proj"}, "d", dm.group(1), t, mp + "down_proj")
            elif hasattr(mlp, "experts"):
                moe = mlp.experts
                if sub == "gate.weight":
                    moe.gate.load_weight(t)
                elif sub == "gate.bias":
                    moe.gate.bias = t.to(device=moe.gate.device, dtype=moe.gate.dtype).contiguous()
                elif sub.startswith("experts.") and sub[len("experts."):] in _OSS_EXPERT_TENSORS:
                    # GPT-OSS: one tensor per projection for the whole expert stack (bf16 or mxfp4 blocks + scales)
                    key = sub[len("experts."):]
                    g = open_groups.get(("oss", li))
                    if g is None:
                        need = {k for k in _OSS_EXPERT_TENSORS if f"{mp}experts.{k}" in names}
                        g = open_groups[("oss", li)] = _Collector(need, lambda parts, moe=moe: _load_oss_experts(moe, parts))
                    if g.add(key, t):
                        del open_groups[("oss", li)]
                elif sub == "gate.e_score_correction_bias" and moe.score_bias is not None:
                    _set_vec(moe.score_bias, t)
                elif sub == "shared_expert_gate.weight" and getattr(mlp, "shared_gate", None) is not None:
                    _set_vec(mlp.shared_gate, t.reshape(-1))
                else:
                    em = re.match(r"^experts\.(\d+)\.(gate|up|down)_proj\.(weight|weight_scale_inv)$", sub)
                    sm = re.match(r"^(shared_experts?)\.(gate|up|down)_proj\.(weight|weight_scale_inv)$", sub)
                    if em:
                        e = int(em.group(1))
                        elo, ehi = moe.expert_range
                        if elo <= e < ehi:               # expert-parallel weight filter
                            def exp_done(parts, moe=moe, e=e, elo=elo):
                                if moe.w13 is None:
                                    moe.method.alloc(moe)
                                moe.method.load_expert(
                                    moe, e - elo, parts[("gate", "weight")], parts[("up", "weight")],
                                    parts[("down", "weight")],
                                    scales=tuple(parts.get((p, "weight_scale_inv")) for p in ("gate", "up", "down")))
                            submit(("exp", li, e), {p: f"{mp}experts.{e}.{p}_proj" for p in ("gate", "up", "down")},
                                   em.group(2), em.group(3), t, exp_done)
                    elif sm and mlp.shared is not None:
                        sp = mp + sm.group(1) + "."
                        if sm.group(2) == "down":
                            linear_piece(("sdown", li), mlp.shared.down, {"d": sp + "down_proj"}, "d", sm.group(3), t,
                                         sp + "down_proj")
                        else:
                            linear_piece(("sgu", li), mlp.shared.gate_up,
                                         {p: f"{sp}{p}_proj" for p in ("gate", "up")}, sm.group(2), sm.group(3), t,
                                         sp + "gate_up_proj")
    if open_groups:
        missing = {str(k): sorted(map(str, g.need - set(g.parts))) for k, g in list(open_groups.items())[:4]}
        raise ValueError(f"checkpoint {path} is incomplete; missing pieces (first groups): {missing}")
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
            if a.qkv.bias is not None:
                for p_, b_ in zip("qkv", a.qkv.bias.split([cfg.num_q_heads * D, cfg.num_kv_heads * D,
                                                            cfg.num_kv_heads * D], 0)):
                    out[pre + f"self_attn.{p_}_proj.bias"] = b_
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
            if getattr(mlp, "shared", None) is not None:
                sw, sp_ = mlp.shared.gate_up.weight, pre + "mlp.shared_expert."
                out[sp_ + "gate_proj.weight"], out[sp_ + "up_proj.weight"] = sw[:sw.shape[0] // 2], sw[sw.shape[0] // 2:]
                out[sp_ + "down_proj.weight"] = mlp.shared.down.weight
                if mlp.shared_gate is not None:
                    out[pre + "mlp.shared_expert_gate.weight"] = mlp.shared_gate[None, :]
    save_file({k: v.detach().cpu().contiguous() for k, v in out.items()}, os.path.join(path, "model.safetensors"))
    if hf_config is not None:
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(hf_config, f)
