"""``launch``: export once, then serve the exported artifact.

    python -m vllm_torchtpu_b200 launch <model> [serve flags] [--export-cache DIR] [--dry-run]

splits the ``serve`` command line in two.  The flags that shape the artifact (model, dtype, quantisation,
parallel degrees, shape limits, KV-cache layout) go to ``export``, which writes a serving directory (weights,
configuration, bucket plan, SHA-256 manifest) into a cache keyed by the model's identity, those flags and the
exporter's own source, so a second launch with the same key skips the export.  The other flags (HTTP front
end, scheduling policy, speculative / KV-transfer configuration, memory fraction) go to ``serve``, which is
started over the artifact and replaces this process.  Both commands are printed before they run.  With a
world size above one both are wrapped in ``torch.distributed.run`` on this host.
(reference: src/vllm_torchtpu/experimental/rust/launcher.py:1-98 - the same split in front of an external
serving binary; here the server of this package is the runtime, so there is no binary to fetch or verify)"""
from __future__ import annotations

import hashlib
import json
import os
import shlex
import subprocess
import sys

# dest names of `serve` flags that shape the artifact; everything else only affects the running server
EXPORT_DESTS = ("tensor_parallel_size", "pipeline_parallel_size", "data_parallel_size", "enable_expert_parallel",
                "prefill_context_parallel_size", "decode_context_parallel_size", "cp_kv_cache_interleave_size",
                "max_model_len", "max_num_seqs", "max_num_batched_tokens", "block_size", "scheduler_block_size",
                "kv_cache_dtype", "quantization", "enable_prefix_caching", "device", "seed")
# flags the export needs to build an engine but that do not change what it writes
EXPORT_PASS_ONLY = ("num_gpu_blocks_override", "enforce_eager")


def _flag(dest: str) -> str:
    return "--" + dest.replace("_", "-")


def _model_identity(model: str) -> dict:
    """What makes two ``model`` arguments the same artifact: a preset's name, or a checkpoint directory's
    path with the size and modification time of every file in it."""
    if os.path.isdir(model):
        files = {}
        for name in sorted(os.listdir(model)):
            st = os.stat(os.path.join(model, name))
            files[name] = [st.st_size, int(st.st_mtime)]
        return {"dir": os.path.abspath(model), "files": files}
    return {"name": model}


def _exporter_fingerprint() -> str:
    from .. import export
    with open(export.__file__, "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()[:16]


def split_args(a, parser) -> tuple:
    """(export flags, serve flags) as argv lists, from a parsed ``serve`` namespace.  Only flags that differ
    from the parser's defaults are emitted."""
    exp, srv = [], []
    for dest, val in sorted(vars(a).items()):
        if dest in ("cmd", "model", "export_cache", "dry_run") or val == parser.get_default(dest):
            continue
        if isinstance(val, bool):
            item = [_flag(dest)]
        elif isinstance(val, (dict, list)):
            item = [_flag(dest), json.dumps(val)]
        else:
            item = [_flag(dest), str(val)]
        if dest in EXPORT_DESTS:
            exp += item
            if dest in ("device", "seed") or "parallel" in dest or dest == "enable_expert_parallel":
                srv += item              # the server must start with the same world and on the same device
        elif dest in EXPORT_PASS_ONLY:
            exp += item
            srv += item
        else:
            srv += item
    return exp, srv


def artifact_dir(a, export_flags: list, cache_root: str) -> str:
    key = json.dumps({"model": _model_identity(a.model), "flags": export_flags,
                      "exporter": _exporter_fingerprint()}, sort_keys=True)
    name = os.path.basename(str(a.model).rstrip("/")) or "model"
    return os.path.join(cache_root, f"{name}-{hashlib.sha256(key.encode()).hexdigest()[:20]}")


def _wrap(world: int, argv: list) -> list:
    base = [sys.executable, "-m"]
    if world > 1:
        return base + ["torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                       "--master-port", os.environ.get("MASTER_PORT", "29511"), "-m", "vllm_torchtpu_b200"] + argv
    return base + ["vllm_torchtpu_b200"] + argv


def plan(a, parser) -> dict:
    cache_root = a.export_cache or os.path.join(os.path.expanduser("~"), ".cache", "vllm_torchtpu_b200", "exports")
    exp, srv = split_args(a, parser)
    out = artifact_dir(a, exp, cache_root)
    world = a.tensor_parallel_size * a.pipeline_parallel_size * a.data_parallel_size * \
        a.prefill_context_parallel_size
    return {"artifact": out, "world_size": world,
            "export": _wrap(world, ["export", a.model, "--output", out] + exp),
            "serve": _wrap(world, ["serve", out] + srv)}


def launch(a, parser) -> int:
    from ..export import validate_serving_dir
    p = plan(a, parser)
    have = os.path.exists(os.path.join(p["artifact"], "metadata.json")) and \
        not validate_serving_dir(p["artifact"], check_hashes=False)
    print("export:", "(cached) " if have else "", shlex.join(p["export"]), flush=True)
    print("serve: ", shlex.join(p["serve"]), flush=True)
    if a.dry_run:
        print(json.dumps(dict(p, cached=bool(have))))
        return 0
    if not have:
        os.makedirs(os.path.dirname(p["artifact"]), exist_ok=True)
        rc = subprocess.call(p["export"])
        if rc != 0:
            print(f"export failed with exit code {rc}", file=sys.stderr)
            return rc
    sys.stdout.flush()
    os.execv(p["serve"][0], p["serve"])
    return 0                                              # not reached
