"""B200 platform: device facts, configuration rewriting and padding buckets.

Plays the role of the reference's ``TpuPlatform``
(reference: src/vllm_torchtpu/platforms/tpu_platform.py:454-1436): it names the
supported quantisation and KV-cache dtypes, validates requests, rewrites the
engine configuration before workers start, and derives the token / request
padding buckets.  Where the reference pre-compiles one XLA program per bucket,
this engine captures one CUDA graph per bucket, so the bucket sets below are
the graph-capture sets.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import envs
from .logger import init_logger

logger = init_logger(__name__)

HBM_BYTES_NOMINAL = 180 * 10**9
NUM_SMS = 148
L2_BYTES = 126 * 2**20


def next_pow2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def token_paddings(max_tokens: int, min_tokens: int = 16, extra=(), linear_stride: int = 0) -> list[int]:
    """Powers of two from ``min_tokens`` capped at ``max_tokens`` plus extras.

    Same policy as the reference's token bucket builder
    (reference: src/vllm_torchtpu/platforms/tpu_platform.py:1438-1554): the cap
    itself is always a bucket, extras and linear buckets are merged in.
    """
    out = set()
    n = max(1, min_tokens)
    while n < max_tokens:
        out.add(n)
        n *= 2
    out.add(max_tokens)
    for e in extra:
        if 0 < e <= max_tokens:
            out.add(int(e))
    if linear_stride > 0:
        out.update(range(linear_stride, max_tokens + 1, linear_stride))
    return sorted(out)


def request_paddings(max_num_seqs: int, min_num_seqs: Optional[int] = None) -> list[int]:
    """``min_num_seqs`` then powers of two up to ``max_num_seqs``
    (reference: src/vllm_torchtpu/runner/tpu_runner.py:9327-9342)."""
    lo = envs.B200_MIN_NUM_SEQS if min_num_seqs is None else min_num_seqs
    lo = min(lo, max_num_seqs)
    out = {lo, max_num_seqs}
    n = next_pow2(lo)
    while n < max_num_seqs:
        if n >= lo:
            out.add(n)
        n *= 2
    return sorted(out)


def pad_to_bucket(n: int, buckets: list[int]) -> int:
    for b in buckets:
        if n <= b:
            return b
    raise ValueError(f"{n} exceeds the largest bucket {buckets[-1]}")


@dataclass
class HbmBudget:
    """How the memory of one GPU is split (all in bytes)."""
    total: int
    weights: int
    activation_peak: int
    symmetric_heap: int
    connector_reserve: int
    graph_reserve: int
    utilization: float

    @property
    def kv_cache(self) -> int:
        usable = int(self.total * self.utilization)
        return max(0, usable - self.weights - self.activation_peak - self.symmetric_heap
                   - self.connector_reserve - self.graph_reserve)


class B200Platform:
    device_name = "cuda"
    device_type = "cuda"
    dist_backend = "nccl"
    cpu_dist_backend = "gloo"
    supported_quantization = ("fp8", "fp8_block", "online_fp8", "int8", "mxfp4", "nvfp4",
                              "compressed-tensors", "awq", "gptq")
    supported_kv_cache_dtypes = ("auto", "bfloat16", "fp8", "fp8_e4m3")
    supported_connectors = ("B200P2PConnector", "B200HostConnector", "B200MultiConnector",
                            "B200OffloadingConnector", "DecodeBenchConnector")
    supported_spec_methods = ("ngram", "suffix", "medusa", "eagle", "eagle3", "mtp", "dflash", "dspark")

    # ---- device facts ---------------------------------------------------
    @classmethod
    def is_available(cls) -> bool:
        return torch.cuda.is_available()

    @classmethod
    def check_device(cls, index: int = 0) -> tuple[int, int]:
        major, minor = torch.cuda.get_device_capability(index)
        if major != 10:
            raise RuntimeError(f"sm_100a kernels need a Blackwell B200 GPU, found sm_{major}{minor}")
        return major, minor

    @classmethod
    def total_memory(cls, index: int = 0) -> int:
        if torch.cuda.is_available():
            return torch.cuda.get_device_properties(index).total_memory
        return HBM_BYTES_NOMINAL

    @classmethod
    def fp8_dtype(cls) -> torch.dtype:
        return torch.float8_e4m3fn

    @classmethod
    def is_kv_cache_dtype_supported(cls, name: str) -> bool:
        return name in cls.supported_kv_cache_dtypes

    @classmethod
    def kv_cache_torch_dtype(cls, name: str, model_dtype: torch.dtype) -> torch.dtype:
        if name in ("auto",):
            return model_dtype
        if name == "bfloat16":
            return torch.bfloat16
        if name in ("fp8", "fp8_e4m3"):
            return torch.float8_e4m3fn
        raise ValueError(f"unsupported kv cache dtype {name}")

    # ---- requests ---------------------------------------------------------
    @classmethod
    def validate_request(cls, sampling_params) -> None:
        """Per-request seeds are rejected: all TP ranks draw from one per-replica
        generator so they agree on the sampled token
        (reference: src/vllm_torchtpu/platforms/tpu_platform.py:1391-1406)."""
        if getattr(sampling_params, "seed", None) is not None:
            raise ValueError("per-request seeds are not supported; set the engine seed instead")
        lp = getattr(sampling_params, "logprobs", None)
        if lp is not None and lp < 0:
            raise ValueError("full-vocabulary logprobs (-1) are not supported")

    # ---- configuration rewriting -----------------------------------------
    @classmethod
    def check_and_update_config(cls, cfg) -> None:
        m, p, c, s = cfg.model, cfg.parallel, cfg.cache, cfg.scheduler
        p.validate()
        if m.quantization is not None and m.quantization not in cls.supported_quantization:
            raise ValueError(f"quantization {m.quantization!r} is not supported on B200 "
                             f"(supported: {cls.supported_quantization})")
        kvd = c.kv_cache_dtype if c.kv_cache_dtype != "auto" else m.kv_cache_dtype
        if not cls.is_kv_cache_dtype_supported(kvd):
            raise ValueError(f"kv cache dtype {kvd!r} is not supported")
        c.kv_cache_dtype = kvd
        if kvd in ("fp8", "fp8_e4m3") and m.is_mla:
            raise ValueError("an fp8 KV cache is implemented for GQA attention only; the latent (MLA) cache "
                             "kernels read bf16")
        if c.block_size not in (16, 32, 64, 128, 256):
            raise ValueError("block_size must be one of 16/32/64/128/256")
        tp = p.tensor_parallel_size
        if not m.is_mla and m.num_kv_heads % tp and tp % m.num_kv_heads:
            raise ValueError(f"{m.num_kv_heads} kv heads cannot be sharded or replicated over tp={tp}")
        if c.scheduler_block_size:
            if c.scheduler_block_size % c.block_size:
                raise ValueError("scheduler_block_size must be a multiple of block_size (the kernels' page)")
            if p.decode_context_parallel_size > 1 or cfg.kv_transfer:
                raise ValueError("scheduler_block_size does not combine with decode context parallelism or "
                                 "KV transfer")
        dcp = p.decode_context_parallel_size
        if dcp > 1:
            # the ranks of a DCP group (consecutive TP ranks) must hold the same KV head: the cache of that
            # head is what gets dealt over them
            if m.is_mla:
                raise ValueError("decode context parallelism is implemented for GQA attention (the latent "
                                 "cache kernels have no position-sharded form)")
            if tp % (m.num_kv_heads * dcp):
                raise ValueError(f"decode_context_parallel_size={dcp} needs every KV head replicated over at "
                                 f"least {dcp} ranks: tp={tp} must be a multiple of kv heads x dcp = "
                                 f"{m.num_kv_heads * dcp}")
            if m.sliding_window or kvd in ("fp8", "fp8_e4m3"):
                raise ValueError("decode context parallelism: no sliding window, bf16 KV cache")
            if c.block_size % max(1, p.cp_kv_cache_interleave_size):
                raise ValueError("cp_kv_cache_interleave_size must divide block_size")
            if cfg.kv_transfer or cfg.speculative:
                raise ValueError("decode context parallelism does not combine with KV transfer or "
                                 "speculative decoding")
        if m.num_q_heads % tp:
            if m.is_mla or m.num_q_heads % m.num_kv_heads or m.architecture not in ("llama", "qwen3_moe"):
                raise ValueError(f"{m.num_q_heads} query heads do not divide over tp={tp}")
            # zero-pad the query heads of every KV group until they divide over the ranks; the padded
            # heads have zero q_proj rows and zero o_proj columns, so the function is unchanged
            g = m.num_q_heads // m.num_kv_heads
            gp = g
            while (m.num_kv_heads * gp) % tp:
                gp += 1
            m.num_q_heads_unpadded = m.num_q_heads
            m.num_q_heads = m.num_kv_heads * gp
            logger.info("query heads padded %d -> %d for tp=%d", m.num_q_heads_unpadded, m.num_q_heads, tp)
        if p.enable_expert_parallel and not m.is_moe:
            logger.warning("--enable-expert-parallel ignored: %s has no experts", m.name)
            p.enable_expert_parallel = False
        if p.enable_expert_parallel:
            ep = tp * p.data_parallel_size
            if m.num_experts % ep:
                raise ValueError(f"{m.num_experts} experts do not divide over ep={ep}")
        if p.pipeline_parallel_size > 1:
            from .parallel.pp import validate_pipeline_parallel_config
            validate_pipeline_parallel_config(cfg)
        if p.prefill_context_parallel_size > 1:
            from .parallel.pcp import PcpStaticSupportValidator
            PcpStaticSupportValidator(cfg).validate()
        s.max_num_batched_tokens = max(s.max_num_batched_tokens, 16)
        s.max_num_seqs = min(s.max_num_seqs, s.max_num_batched_tokens)
        if not s.enable_chunked_prefill and s.max_num_batched_tokens < m.max_model_len:
            raise ValueError("max_num_batched_tokens < max_model_len needs chunked prefill")
        if p.data_parallel_size > 1 and envs.B200_DP_SCHED_ENABLED and s.scheduler_cls == "default":
            s.scheduler_cls = "dp"
        if cfg.speculative:
            method = cfg.speculative.get("method")
            if method not in cls.supported_spec_methods:
                raise ValueError(f"speculative method {method!r} not in {cls.supported_spec_methods}")
            if m.is_hybrid_gdn and s.async_scheduling:
                # rejected drafts advance the recurrent state; it is rebuilt (snapshot + replay of the accepted
                # rows, runner/spec_boundary_state.py) when the host has the step's tokens, before the next launch
                logger.info("speculative decoding on a linear-attention hybrid: async scheduling switched off")
                s.async_scheduling = False
            if s.async_scheduling and method in ("ngram", "suffix"):
                raise ValueError("async scheduling is only supported with eagle-family drafters")
            if s.async_scheduling and method in ("mtp", "eagle", "eagle3", "dflash", "dspark"):
                # the draft layer catches up on a step's rows and drafts from its tokens before the next
                # step is scheduled
                logger.info("speculative method %s: async scheduling switched off", method)
                s.async_scheduling = False
            if method in ("mtp", "eagle", "eagle3", "dflash", "dspark") and p.decode_context_parallel_size > 1:
                raise ValueError("draft layers are not built for decode context parallelism")
        if cfg.kv_transfer:
            name = cfg.kv_transfer.get("kv_connector")
            if name not in cls.supported_connectors:
                raise ValueError(f"kv_connector {name!r} not in {cls.supported_connectors}")
        cfg.token_buckets = token_paddings(
            s.max_num_batched_tokens, 16,
            extra=list(envs.B200_TOKEN_BUCKET_EXTRA), linear_stride=envs.B200_TOKEN_BUCKET_LINEAR)
        cfg.request_buckets = request_paddings(s.max_num_seqs)
        cls.validate_token_budget(cfg)

    @classmethod
    def validate_token_budget(cls, cfg) -> None:
        if cfg.token_buckets[-1] < cfg.scheduler.max_num_batched_tokens:
            raise ValueError("largest token bucket is smaller than max_num_batched_tokens")

    # ---- memory ---------------------------------------------------------
    @classmethod
    def compute_hbm_budget(cls, cfg, weight_bytes: int, activation_peak: int,
                           total: Optional[int] = None) -> HbmBudget:
        world = cfg.parallel.tensor_parallel_size * cfg.parallel.data_parallel_size
        heap = envs.B200_SYMM_HEAP_MB * 2**20 if world > 1 else 0
        reserve = 0
        if cfg.kv_transfer:
            reserve = int(cfg.kv_transfer.get("kv_buffer_size", 256 * 2**20))
        graphs = 0 if cfg.enforce_eager else 512 * 2**20
        return HbmBudget(total or cls.total_memory(), weight_bytes, activation_peak, heap, reserve,
                         graphs, cfg.cache.gpu_memory_utilization)
