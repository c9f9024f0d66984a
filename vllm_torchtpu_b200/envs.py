"""Typed, lazy environment-variable registry.

Every knob the package reads is declared here once with a type, a default and
(optionally) a set of allowed values.  Values are parsed on first attribute
access (``envs.B200_FUSED_TP``) and cached; ``envs.reset()`` drops the cache
(tests).  Reading an undeclared name raises ``AttributeError``, so a typo in
code fails at the call site, and ``env_validation.report_unread`` flags typos in
the user's environment.

Same role as the reference's lazy registry of typed knobs
(reference: src/vllm_torchtpu/envs.py:22-240 and its ``environment_variables``
dict); the knobs themselves are the ones that make sense on NVLink/B200.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable, Optional, Sequence

_PREFIXES = ("B200_",)


@dataclass(frozen=True)
class EnvVar:
    name: str
    type: type
    default: Any
    doc: str
    choices: Optional[Sequence[Any]] = None
    parser: Optional[Callable[[str], Any]] = None


def _parse_bool(raw: str) -> bool:
    v = raw.strip().lower()
    if v in ("1", "true", "yes", "on"):
        return True
    if v in ("0", "false", "no", "off", ""):
        return False
    raise ValueError(f"not a boolean: {raw!r}")


def _parse_opt_int(raw: str) -> Optional[int]:
    raw = raw.strip()
    return None if raw == "" or raw.lower() == "none" else int(raw)


def _int_list(raw: str) -> list[int]:
    return [int(x) for x in raw.replace(";", ",").split(",") if x.strip()]


_REGISTRY: dict[str, EnvVar] = {}


def _decl(name, type_, default, doc, choices=None, parser=None):
    _REGISTRY[name] = EnvVar(name, type_, default, doc, choices, parser)


# --- logging / debug -------------------------------------------------------
_decl("B200_LOG_LEVEL", str, "INFO", "log level of the b200 logger",
      choices=("DEBUG", "INFO", "WARNING", "ERROR"))
_decl("B200_BOUNDS_CHECK", bool, False,
      "use kernels built with index range checks that record the bad index in a status word")
_decl("B200_KERNEL_LIB", str, "", "path of an alternative kernel .so (hot reload during development)")
_decl("B200_SPIN_LIMIT", int, 2_000_000,
      "iteration limit of every device-side flag wait before it reports TIMEOUT")
# --- execution ---------------------------------------------------------------
_decl("B200_CUDA_GRAPHS", bool, True, "capture decode steps per request bucket into CUDA graphs")
_decl("B200_GRAPH_TOKEN_BUCKETS", list, [], "extra token buckets to capture", parser=_int_list)
_decl("B200_TOKEN_BUCKET_EXTRA", list, [], "extra token paddings appended to the power-of-two set",
      parser=_int_list)
_decl("B200_TOKEN_BUCKET_LINEAR", int, 0, "if >0, add linear token buckets with this stride")
_decl("B200_MIN_NUM_SEQS", int, 8, "smallest request bucket")
_decl("B200_GEMM_IMPL", str, "tcgen05", "dense GEMM implementation",
      choices=("tcgen05", "cublas"))
_decl("B200_GEMM_2SM_MIN_T", int, 1024,
      "token count from which the dense and SwiGLU GEMMs run on the two-SM (cta_group::2) kernel; 0 = never")
_decl("B200_ATTN_PREFILL_IMPL", str, "tc", "prefill attention kernel: tcgen05 (head_dim 128) or legacy mma.sync",
      choices=("tc", "mma"))
_decl("B200_ATTN_SPLIT_KV", int, 0, "force the decode split-KV factor (0 = heuristic)")
_decl("B200_KV_SAVE_NAN_CHECK", bool, True, "screen KV blocks for NaN / Inf before they are stored or published")
_decl("B200_DECODE_MEGAKERNEL", bool, False,
      "decode-only steps of at most 64 requests of dense models run all layers in one persistent kernel "
      "(experimental: measured slower than the per-layer kernels, see profiles/decode_persistent_kernel_phases.md)")
_decl("B200_ASYNC_SCHEDULING", bool, True, "overlap host scheduling of step n+1 with device step n")
_decl("B200_NATIVE_HOST", bool, True, "use the C++ host runtime for block tables and input prep")
# --- tensor / expert parallel -------------------------------------------
_decl("B200_FUSED_TP", bool, True,
      "row-parallel GEMMs reduce across ranks inside the kernel over NVLink peer memory")
_decl("B200_TP_COMM", str, "p2p", "data plane of the fused TP kernels",
      choices=("p2p", "multimem", "nccl"))
_decl("B200_TP_ONE_SHOT_BYTES", int, 4 * 2**20,
      "fused TP all-reduce: push partials to every rank (one NVLink hop) while T*N*2*(world-1) is at most this")
_decl("B200_TP_DEFER_REDUCE", bool, True,
      "small row-parallel outputs are pushed to every rank and summed inside the following add+RMSNorm kernel")
_decl("B200_SYMM_HEAP_MB", int, 512, "size of the per-rank symmetric heap")
_decl("B200_BOUNDS_CHECK", bool, False,
      "load the attention kernels from the bounds-checked library (out-of-range block ids are counted)")
_decl("B200_DEVICE_SPEC_ACCEPT", bool, True, "speculative decoding: judge the drafts on the device")
_decl("B200_FP8_ROWS_MIN_TILES", int, 96,
      "fp8 block GEMM: use the token-major kernel from this many 128x256 output tiles (-1: never)")
_decl("B200_SAMPLE_CLUSTER", bool, True,
      "top-k / top-p sampling as a 4-CTA cluster per row (0: the one-CTA bisection kernel); read by the kernel library")
_decl("B200_FP8_ROWS_SKIP_PROMOTE", bool, False,
      "measurement aid of the token-major fp8 GEMM: skip the promotion (output undefined); read by the kernel library")
_decl("B200_SAFETENSORS_PREFETCH", bool, True, "checkpoint loading: ask the kernel to read the next file ahead")
_decl("B200_LOAD_EVICT_PAGE_CACHE", bool, False,
      "checkpoint loading: drop every consumed file from the page cache (large checkpoints on small hosts)")
_decl("B200_PCP_MIN_TOKENS", int, 512,
      "prefill context parallelism: shortest prefill chunk that is split over the ranks (shorter ones are replicated)")
_decl("B200_MOE_PIPELINE_CHUNKS", int, 0,
      "expert-parallel all-gather plane: split a step's tokens into this many chunks and overlap each chunk's "
      "collectives with its neighbours' expert GEMMs (0 / 1: off)")
_decl("B200_MOE_PIPELINE_MIN_CHUNK_TOKENS", int, 256, "pipelined MoE plane: fewest tokens per chunk worth a pipeline")
_decl("B200_MOE_ROUTING_SIM", str, "",
      "replace the router's choice: 'uniform' (round-robin, perfectly balanced) or 'hash' (hashed per token); "
      "for benchmarks with random-init routers")
_decl("B200_MOE_FUSED_EP", bool, True, "dispatch/combine inside the expert kernel over peer memory")
_decl("B200_MOE_EP_CAPACITY_FACTOR", float, 0.0,
      "fused EP plane: rows an owner can receive per call, as a multiple of call tokens * top_k; "
      "0 sizes for the worst case (every row of every rank routed to one owner), so nothing is ever dropped")
_decl("B200_MOE_EP_CALL_TOKENS", int, 2048, "fused EP plane: tokens per rank and call; longer steps make several calls")
_decl("B200_MOE_FUSED_EP_MIN_TOKENS", int, 0, "use the AG/RS path below this many tokens")
_decl("B200_MOE_SEQUENCE_PARALLEL", bool, False, "reduce-scatter after attention, all-gather before experts")
_decl("B200_MOE_TOPK_WEIGHTS_FLOAT32", bool, True, "keep routing weights in fp32")
_decl("B200_EXPERT_PLACEMENT", str, "linear", "expert→rank placement",
      choices=("linear", "round_robin", "static"))
_decl("B200_EXPERT_PLACEMENT_FILE", str, "", "JSON file with a static expert permutation")
_decl("B200_DP_SCHED_ENABLED", bool, False, "align prefill admission across DP ranks")
_decl("B200_DP_VOCAB_PARALLEL", bool, False, "shard embedding / lm_head over DP ranks")
_decl("B200_GREEDY_TOP_TOKENS", bool, True, "vocab-parallel argmax exchange instead of full logits gather")
# --- pipeline parallel -----------------------------------------------------
_decl("B200_PP_HANDOFF_DEPTH", int, 2, "send-queue depth of the PP hand-off")
_decl("B200_PP_MAX_POSTED_RECVS", int, 7, "posted receive cap of the PP hand-off")
_decl("B200_PP_LONE_PROMPT_CHUNKS", int, 0, "split a lone prompt into this many chunks (0 = stages)")
_decl("B200_PP_EQUAL_COST_CHUNKS", bool, True, "equal-cost rather than equal-size chunks")
_decl("B200_PP_CHUNK_SLACK", float, 0.1, "tolerated cost imbalance between chunks")
# --- context parallel ------------------------------------------------------
_decl("B200_DCP_LSE_MERGE_A2A", bool, False, "merge DCP partials by all-to-all instead of reduce-scatter")
_decl("B200_DCP_LSE_MERGE_A2A_MAX_TOKENS", int, 64, "token cap for the all-to-all merge")
_decl("B200_DCP_RS_OUT_FP32", bool, True, "reduce-scatter DCP outputs in fp32")
_decl("B200_PCP_KV_CHUNK_TOKENS", int, 65536, "tokens per KV workspace gather step")
_decl("B200_PCP_KV_WORKSPACE_TOKENS", int, 1048576, "KV workspace capacity in tokens")
# --- quantisation --------------------------------------------------------
_decl("B200_REQUANTIZE_BLOCK_SIZE", int, None, "re-quantise weights at load to this block size",
      parser=_parse_opt_int)
_decl("B200_REQUANTIZE_WEIGHT_DTYPE", str, "float8_e4m3fn", "target dtype of load-time requant")
_decl("B200_FP8_LINEAR_W8A16_MAX_ROWS", int, 0, "use weight-only fp8 below this many rows")
# --- sampling -------------------------------------------------------------
_decl("B200_SAMPLER_TOPK_CANDIDATES", int, 0, "candidate prefilter width of top-k/top-p (0 = off)")
# --- KV transfer / offload ---------------------------------------------------
_decl("B200_KV_TRANSFER_PORT", int, 9100, "base port of the KV data plane control socket")
_decl("B200_SIDE_CHANNEL_PORT", int, 9600, "base port of the connector handshake channel")
_decl("B200_P2P_WAIT_PULL_TIMEOUT", float, 120.0, "seconds a producer keeps blocks for a consumer")
_decl("B200_KV_STAGE_WAIT_TIMEOUT_SECS", float, 30.0, "seconds a consumer waits for a transfer stage")
_decl("B200_KV_IPC_KEY", str, "", "HMAC key of connector control messages (empty = random per job)")
_decl("B200_KV_TRANSPORT", str, "p2p", "KV data plane", choices=("p2p", "host"))
_decl("B200_OFFLOAD_DRAM_GB", float, 0.0, "pinned host memory of the KV offload store")
_decl("B200_OFFLOAD_DISK_DIR", str, "", "directory of the disk tier of the KV offload store")
_decl("B200_OFFLOAD_SAVE_RETRIES", int, 2, "retries of a failed offload save")
_decl("B200_OFFLOAD_WAIT_TIMEOUT_S", float, 30.0, "seconds to wait for an offload load")
# --- profiling -------------------------------------------------------------
_decl("B200_USE_PHASED_PROFILER", bool, False, "capture one trace per inference phase")
_decl("B200_PROFILE_DIR", str, "", "directory for profiler traces")
_decl("B200_STAGE_TIMING", bool, False, "record CUDA-event stage timers each step")
_decl("B200_CHECK_RECAPTURE", bool, False, "raise when a step needs a graph that was not captured at warm-up")
_decl("B200_ABORT_ON_PREEMPTION", bool, False, "finish a preempted request with an error instead of recomputing")
_decl("B200_SRPT_HOLD_BACK", int, 0, "SRPT scheduler: prefill hold-back budget")


_cache: dict[str, Any] = {}
_read: set[str] = set()


def declared() -> dict[str, EnvVar]:
    return dict(_REGISTRY)


def reset() -> None:
    _cache.clear()
    _read.clear()


def was_read(name: str) -> bool:
    return name in _read


def _parse(var: EnvVar, raw: str) -> Any:
    if var.parser is not None:
        val = var.parser(raw)
    elif var.type is bool:
        val = _parse_bool(raw)
    elif var.type in (int, float, str):
        val = var.type(raw)
    else:
        raise TypeError(f"{var.name}: no parser for {var.type}")
    if var.choices is not None:
        cmp = val.upper() if var.name == "B200_LOG_LEVEL" else val
        if cmp not in var.choices:
            raise ValueError(f"{var.name}={raw!r}: expected one of {list(var.choices)}")
    return val


def __getattr__(name: str) -> Any:
    var = _REGISTRY.get(name)
    if var is None:
        raise AttributeError(f"undeclared environment variable {name!r}")
    if name in _cache:
        return _cache[name]
    _read.add(name)
    raw = os.environ.get(name)
    val = var.default if raw is None else _parse(var, raw)
    _cache[name] = val
    return val


def known_prefixes() -> tuple[str, ...]:
    return _PREFIXES
