"""Command line: ``python -m vllm_torchtpu_b200 serve <model> [flags]`` and ``... bench serve``.

Flag names follow the ``vllm serve`` surface the reference is driven with
(reference: docs/user_guide/parallelism.md:5-21, docs/user_guide/supported_models.md:58-77).
Under tensor or pipeline parallelism launch with ``torch.distributed.run``; rank 0 serves HTTP and
broadcasts the request stream, the other ranks follow it step by step."""
from __future__ import annotations

import argparse
import json
import os
import sys


def add_engine_args(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("model", help="preset name or a directory with config.json + safetensors")
    ap.add_argument("--tensor-parallel-size", "-tp", type=int, default=1)
    ap.add_argument("--pipeline-parallel-size", "-pp", type=int, default=1)
    ap.add_argument("--data-parallel-size", "-dp", type=int, default=1)
    ap.add_argument("--enable-expert-parallel", action="store_true")
    ap.add_argument("--prefill-context-parallel-size", type=int, default=1)
    ap.add_argument("--decode-context-parallel-size", type=int, default=1)
    ap.add_argument("--cp-kv-cache-interleave-size", type=int, default=1)
    ap.add_argument("--max-model-len", type=int, default=None)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--scheduler-block-size", type=int, default=0,
                    help="tokens per scheduler block (a multiple of --block-size, the kernels' page; 0: the same)")
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--num-gpu-blocks-override", type=int, default=None)
    ap.add_argument("--kv-cache-dtype", default="auto")
    ap.add_argument("--quantization", "-q", default=None)
    ap.add_argument("--enable-prefix-caching", action="store_true")
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--async-scheduling", action="store_true")
    ap.add_argument("--scheduler-cls", default="default")
    ap.add_argument("--speculative-config", type=json.loads, default=None)
    ap.add_argument("--kv-transfer-config", type=json.loads, default=None)
    ap.add_argument("--additional-config", type=json.loads, default=None)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--seed", type=int, default=0)


def make_llm(a):
    from ..engine.llm import LLM
    return LLM(a.model, tensor_parallel_size=a.tensor_parallel_size,
               pipeline_parallel_size=a.pipeline_parallel_size, data_parallel_size=a.data_parallel_size,
               enable_expert_parallel=a.enable_expert_parallel,
               prefill_context_parallel_size=a.prefill_context_parallel_size,
               decode_context_parallel_size=a.decode_context_parallel_size,
               cp_kv_cache_interleave_size=a.cp_kv_cache_interleave_size,
               scheduler_block_size=a.scheduler_block_size,
               max_model_len=a.max_model_len, max_num_seqs=a.max_num_seqs,
               max_num_batched_tokens=a.max_num_batched_tokens, block_size=a.block_size,
               gpu_memory_utilization=a.gpu_memory_utilization,
               num_gpu_blocks_override=a.num_gpu_blocks_override, kv_cache_dtype=a.kv_cache_dtype,
               quantization=a.quantization, enable_prefix_caching=a.enable_prefix_caching,
               enforce_eager=a.enforce_eager, async_scheduling=a.async_scheduling,
               scheduler_cls=a.scheduler_cls, speculative_config=a.speculative_config,
               kv_transfer_config=a.kv_transfer_config, additional_config=a.additional_config,
               device=a.device, seed=a.seed)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="vllm_torchtpu_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve", help="OpenAI-compatible server")
    add_engine_args(s)
    s.add_argument("--host", default="0.0.0.0")
    s.add_argument("--port", type=int, default=8000)
    s.add_argument("--served-model-name", default=None)
    ln = sub.add_parser("launch", help="export once (cached), then serve the exported artifact")
    add_engine_args(ln)
    ln.add_argument("--host", default="0.0.0.0")
    ln.add_argument("--port", type=int, default=8000)
    ln.add_argument("--served-model-name", default=None)
    ln.add_argument("--export-cache", default=None, help="directory the exported artifacts are cached in")
    ln.add_argument("--dry-run", action="store_true", help="print the export and serve commands and stop")
    p = sub.add_parser("proxy", help="prefill/decode disaggregation proxy")
    p.add_argument("--prefiller-hosts", nargs="+", default=["127.0.0.1"])
    p.add_argument("--prefiller-ports", nargs="+", type=int, default=[8100])
    p.add_argument("--decoder-hosts", nargs="+", default=["127.0.0.1"])
    p.add_argument("--decoder-ports", nargs="+", type=int, default=[8200])
    p.add_argument("--host", default="0.0.0.0")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--controller", default="", help="host:port of a KV controller: pick instances from its registry")
    c = sub.add_parser("controller", help="registry of prefill / decode engines (heartbeats, load-aware picks)")
    c.add_argument("--host", default="0.0.0.0")
    c.add_argument("--port", type=int, default=7600)
    c.add_argument("--ttl", type=float, default=10.0, help="seconds without a heartbeat before an engine is skipped")
    e = sub.add_parser("envs", help="list the environment knobs")
    x = sub.add_parser("export", help="write a serving directory (weights, configuration, shape plan, manifest)")
    add_engine_args(x)
    x.add_argument("--output", required=True)
    v = sub.add_parser("validate-export", help="check a serving directory against its manifest")
    v.add_argument("path")
    a = ap.parse_args(argv)

    from .. import env_validation
    from ..logger import init_logger
    log = init_logger(__name__)
    env_validation.report_unread(log)
    for err in env_validation.validate_values():
        log.error(err)
    if a.cmd == "envs":
        from .. import envs
        for name, var in sorted(envs.declared().items()):
            print(f"{name:40s} {var.type.__name__:6s} default={var.default!r}  {var.doc}")
        return 0
    if a.cmd == "launch":
        from .launcher import launch
        return launch(a, ln)
    if a.cmd == "validate-export":
        from ..export import validate_serving_dir
        problems = validate_serving_dir(a.path)
        for p in problems:
            print(p)
        print("valid" if not problems else f"{len(problems)} problem(s)")
        return 0 if not problems else 1
    if a.cmd == "export":
        from ..export import export_serving_dir
        meta = export_serving_dir(make_llm(a), a.output)
        print(json.dumps({"output": a.output, "files": sorted(meta["manifest"])}))
        return 0
    if a.cmd == "proxy":
        from ..kv_transfer.proxy import run_proxy
        run_proxy(a.prefiller_hosts, a.prefiller_ports, a.decoder_hosts, a.decoder_ports, a.host, a.port,
                  controller=a.controller)
        return
    if a.cmd == "controller":
        from ..kv_transfer.controller import run_controller
        run_controller(a.host, a.port, a.ttl)
        return 0
    if os.path.isfile(os.path.join(str(a.model), "metadata.json")) and \
            os.path.isdir(os.path.join(str(a.model), "serving_checkpoint")):
        # an exported artifact: checked against its manifest, its recorded plan gives the defaults and the
        # flags given on this command line override them
        from ..export import load_serving_dir
        given = {k: v for k, v in vars(a).items()
                 if k not in ("cmd", "model", "host", "port", "served_model_name", "device") and v != s.get_default(k)}
        llm = load_serving_dir(a.model, a.device, **given)
    else:
        llm = make_llm(a)
    rank = int(os.environ.get("RANK", "0"))
    name = a.served_model_name or llm.engine.cfg.model.name
    # several ranks: rank 0 takes the HTTP requests and broadcasts them step by step, the others follow
    synced = llm.engine.enable_request_sync()
    if rank == 0:
        from .openai_server import serve
        try:
            serve(llm.engine, name, llm.tokenizer, a.host, a.port)
        finally:
            llm.engine.stop_followers()
    elif synced:
        llm.engine.follow()
    if synced:
        from ..parallel.state import leave_process
        leave_process(0)
    return 0
