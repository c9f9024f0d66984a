"""Ahead-of-time export of a serving directory, its validator and its loader.

The directory is what a deployment ships instead of the training checkpoint: the weights in the
layout the engine loads, the model configuration, the static shape plan of the engine (token and
request buckets = the CUDA graphs that will be captured, block size, KV dtype) and a manifest with
the SHA-256 of every file, so that a serving host can verify it before it starts.

    serving_dir/
      metadata.json                  format version, model + engine configuration, buckets, manifest
      serving_checkpoint/config.json        Hugging Face style model configuration
      serving_checkpoint/model.safetensors  weights

An engine that was loaded from a checkpoint directory (any architecture, any number of ranks) is exported by
copying that checkpoint: rank 0 writes, the other ranks wait; the parallel plan of the exporting engine
(tensor / pipeline / data / expert / context parallel degrees) is recorded and is the default of the loader,
which shards at load time.  A random-init engine is written from its parameters (single rank, Llama and
Qwen-MoE families).

(reference: src/vllm_torchtpu/experimental/export/ — exporter to a serving directory with
``metadata.json``, per-bucket programs and ``serving_checkpoint/``, validator; the per-bucket compiled
programs of the reference have no counterpart here because decode buckets are CUDA graphs captured
at start-up, so the exported plan lists the buckets instead.)
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Optional

import torch

FORMAT_VERSION = 1
_ARCH_NAMES = {"llama": "LlamaForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM"}


def to_hf_config(mc) -> dict:
    """ModelConfig -> the Hugging Face ``config.json`` fields that ``ModelConfig.from_hf_dict`` reads."""
    if mc.architecture not in _ARCH_NAMES:
        raise ValueError(f"export supports {sorted(_ARCH_NAMES)}, not {mc.architecture!r}")
    arch = _ARCH_NAMES[mc.architecture]
    if mc.architecture == "llama" and mc.qk_norm:
        arch = "Qwen3ForCausalLM"
    d = {"architectures": [arch], "num_hidden_layers": mc.num_layers, "hidden_size": mc.hidden_size,
         "num_attention_heads": mc.num_q_heads, "num_key_value_heads": mc.num_kv_heads, "head_dim": mc.head_dim,
         "intermediate_size": mc.intermediate_size, "vocab_size": mc.vocab_size, "rms_norm_eps": mc.rms_norm_eps,
         "rope_theta": mc.rope_theta, "rope_scaling": mc.rope_scaling, "max_position_embeddings": mc.max_model_len,
         "tie_word_embeddings": mc.tie_word_embeddings, "torch_dtype": str(mc.dtype).replace("torch.", "")}
    if mc.architecture == "qwen3_moe":
        d.update(num_experts=mc.num_experts, num_experts_per_tok=mc.num_experts_per_tok,
                 moe_intermediate_size=mc.moe_intermediate_size, norm_topk_prob=mc.moe_renormalize)
    return d


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 22), b""):
            h.update(chunk)
    return h.hexdigest()


_CKPT_FILES = (".safetensors", ".json", ".model", ".txt", ".tiktoken", ".jinja")


def _copy_checkpoint(src: str, dst: str) -> None:
    import shutil
    for name in sorted(os.listdir(src)):
        p = os.path.join(src, name)
        if os.path.isfile(p) and name.endswith(_CKPT_FILES):
            shutil.copyfile(p, os.path.join(dst, name))


def export_serving_dir(llm, out_dir: str) -> dict:
    """Write the serving directory of a loaded engine; returns the metadata (on every rank)."""
    from .models.loader import save_hf_checkpoint
    from .parallel.state import get_state
    eng = llm.engine
    cfg = eng.cfg
    st = get_state()
    world = cfg.parallel.world_size
    src = getattr(cfg, "model_path", None)
    if world != 1 and not src:
        raise ValueError("a random-init engine is exported from a single rank; engines of several ranks are "
                         "exported from the checkpoint directory they were loaded from")
    ckpt = os.path.join(out_dir, "serving_checkpoint")
    if st.rank == 0 or world == 1:
        os.makedirs(ckpt, exist_ok=True)
        if src:
            _copy_checkpoint(src, ckpt)
        else:
            save_hf_checkpoint(eng.runner.model, ckpt, to_hf_config(cfg.model))
    if world > 1 and st.world.cpu_group is not None:
        import torch.distributed as dist
        dist.barrier(group=st.world.cpu_group)            # the files are complete before anybody hashes them
    manifest = {}
    for name in sorted(os.listdir(ckpt)):
        p = os.path.join(ckpt, name)
        manifest[f"serving_checkpoint/{name}"] = {"sha256": _sha256(p), "bytes": os.path.getsize(p)}
    meta = {
        "format_version": FORMAT_VERSION,
        "model": {"name": cfg.model.name, "architecture": cfg.model.architecture,
                  "dtype": str(cfg.model.dtype).replace("torch.", ""),
                  "weight_bytes": int(eng.runner.model.weight_bytes())},
        "engine": {"block_size": cfg.cache.block_size, "kv_cache_dtype": cfg.cache.kv_cache_dtype,
                   "max_num_seqs": cfg.scheduler.max_num_seqs,
                   "max_num_batched_tokens": cfg.scheduler.max_num_batched_tokens,
                   "max_model_len": cfg.model.max_model_len,
                   "enable_prefix_caching": cfg.cache.enable_prefix_caching},
        "parallel": {"tensor_parallel_size": cfg.parallel.tensor_parallel_size,
                     "pipeline_parallel_size": cfg.parallel.pipeline_parallel_size,
                     "data_parallel_size": cfg.parallel.data_parallel_size,
                     "enable_expert_parallel": bool(cfg.parallel.enable_expert_parallel),
                     "decode_context_parallel_size": cfg.parallel.decode_context_parallel_size,
                     "world_size": world},
        "plan": {"token_buckets": list(cfg.token_buckets), "request_buckets": list(cfg.request_buckets),
                 "decode_graphs": [[int(r), bool(g)] for (r, g) in sorted(eng.runner.graphs)]},
        "manifest": manifest,
    }
    if st.rank == 0 or world == 1:
        with open(os.path.join(out_dir, "metadata.json"), "w") as f:
            json.dump(meta, f, indent=1, sort_keys=True)
    if world > 1 and st.world.cpu_group is not None:
        import torch.distributed as dist
        dist.barrier(group=st.world.cpu_group)
    return meta


def validate_serving_dir(path: str, check_hashes: bool = True) -> list:
    """Problems found in a serving directory (empty list = valid)."""
    problems = []
    mp = os.path.join(path, "metadata.json")
    if not os.path.isfile(mp):
        return [f"{mp} is missing"]
    try:
        with open(mp) as f:
            meta = json.load(f)
    except ValueError as e:
        return [f"metadata.json is not JSON: {e}"]
    if meta.get("format_version") != FORMAT_VERSION:
        problems.append(f"format_version {meta.get('format_version')!r}, this build reads {FORMAT_VERSION}")
    for key in ("model", "engine", "plan", "manifest"):
        if key not in meta:
            problems.append(f"metadata.json lacks {key!r}")
    for rel, ent in (meta.get("manifest") or {}).items():
        p = os.path.join(path, rel)
        if not os.path.isfile(p):
            problems.append(f"{rel} is missing")
            continue
        if os.path.getsize(p) != ent.get("bytes"):
            problems.append(f"{rel}: {os.path.getsize(p)} bytes, manifest says {ent.get('bytes')}")
        elif check_hashes and _sha256(p) != ent.get("sha256"):
            problems.append(f"{rel}: SHA-256 differs from the manifest")
    plan = meta.get("plan") or {}
    for name in ("token_buckets", "request_buckets"):
        b = plan.get(name) or []
        if not b or b != sorted(b):
            problems.append(f"plan.{name} must be a non-empty ascending list")
    par = meta.get("parallel")
    if par is not None:
        prod = par.get("tensor_parallel_size", 1) * par.get("pipeline_parallel_size", 1) * \
            par.get("data_parallel_size", 1)
        if prod != par.get("world_size", prod):
            problems.append(f"parallel plan: tp x pp x dp = {prod}, world_size {par.get('world_size')}")
        cfg_path = os.path.join(path, "serving_checkpoint", "config.json")
        if os.path.isfile(cfg_path):
            try:
                with open(cfg_path) as f:
                    hf = json.load(f)
                if hf.get("num_hidden_layers", 1) < par.get("pipeline_parallel_size", 1):
                    problems.append("parallel plan: more pipeline stages than layers")
            except ValueError:
                problems.append("serving_checkpoint/config.json is not JSON")
    eng = meta.get("engine") or {}
    if plan.get("request_buckets") and eng.get("max_num_seqs", 0) > plan["request_buckets"][-1]:
        problems.append("max_num_seqs exceeds the largest request bucket")
    return problems


def load_serving_dir(path: str, device: Optional[str] = None, **overrides):
    """Validate the directory and start an engine with the exported configuration."""
    from .engine.llm import LLM
    problems = validate_serving_dir(path)
    if problems:
        raise ValueError("invalid serving directory: " + "; ".join(problems))
    with open(os.path.join(path, "metadata.json")) as f:
        meta = json.load(f)
    eng = meta["engine"]
    kw = dict(max_num_seqs=eng["max_num_seqs"], max_num_batched_tokens=eng["max_num_batched_tokens"],
              block_size=eng["block_size"], kv_cache_dtype=eng["kv_cache_dtype"],
              enable_prefix_caching=eng["enable_prefix_caching"], max_model_len=eng["max_model_len"],
              dtype=meta["model"]["dtype"])
    par = meta.get("parallel") or {}
    for key in ("tensor_parallel_size", "pipeline_parallel_size", "data_parallel_size", "enable_expert_parallel",
                "decode_context_parallel_size"):
        if key in par and par[key] not in (1, False):
            kw[key] = par[key]                          # the exporting engine's plan; overrides win
    kw.update(overrides)
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    return LLM(os.path.join(path, "serving_checkpoint"), device=device, **kw)
