"""Engine configuration objects and the named model presets.

``ModelConfig`` holds architecture hyper-parameters (loadable from a Hugging
Face ``config.json``), ``ParallelConfig`` the TP/DP/PP/EP/PCP/DCP layout,
``CacheConfig`` the paged KV geometry, ``SchedulerConfig`` the batching limits.
``EngineConfig.finalize`` is where the platform rewrites the configuration the
way the reference's ``check_and_update_config`` does
(reference: src/vllm_torchtpu/platforms/tpu_platform.py:840-1295).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any, Optional

import torch

_DTYPES = {
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
}


def parse_dtype(d) -> torch.dtype:
    if isinstance(d, torch.dtype):
        return d
    return _DTYPES[str(d).replace("torch.", "")]


@dataclass
class ModelConfig:
    architecture: str = "llama"          # llama | qwen3_moe | deepseek_v3 | qwen3_next
    name: str = "tiny-llama"
    num_layers: int = 2
    hidden_size: int = 256
    num_q_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    intermediate_size: int = 512
    vocab_size: int = 1024
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: Optional[dict] = None
    rope_interleaved: bool = False       # False = neox half-rotation
    max_model_len: int = 2048
    dtype: torch.dtype = torch.bfloat16
    tie_word_embeddings: bool = False
    qk_norm: bool = False                # Qwen3 per-head RMSNorm on q and k
    attention_bias: bool = False         # Qwen2 qkv bias
    attention_out_bias: bool = False     # GPT-OSS: bias on the output projection too
    layer_sliding: tuple = ()            # per layer: sliding-window attention (True) or full attention; () = all alike
    moe_bias: bool = False               # router and expert biases (GPT-OSS)
    quant_ignored: tuple = ()            # substrings of layer names that stay unquantised besides lm_head / embed / router
    sliding_window: Optional[int] = None
    logit_softcap: Optional[float] = None
    attn_sinks: bool = False
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    hidden_act: str = "silu"                   # gated activation of the MLP / experts (ops.reference.parse_gated_act)
    num_shared_experts: int = 0
    shared_expert_intermediate_size: int = 0   # 0: moe_intermediate_size x num_shared_experts
    shared_expert_gate: bool = False           # shared expert output scaled by sigmoid(x . w) (Qwen2-MoE, Qwen3-Next)
    first_dense_layers: int = 0          # leading layers with a dense FFN
    moe_scoring: str = "softmax"         # softmax | sigmoid
    moe_renormalize: bool = True
    moe_routed_scaling: float = 1.0
    moe_n_group: int = 1
    moe_topk_group: int = 1
    moe_score_bias: bool = False
    # MLA
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    mla_use_nope: bool = False           # latent attention without rotary embeddings (Kimi-Linear: positions come from the KDA layers)
    # sparse MLA (DSA indexer)
    index_topk: int = 0
    index_n_heads: int = 0
    index_head_dim: int = 0
    # Gated DeltaNet hybrid (every `full_attention_interval`-th layer is softmax attention)
    full_attention_interval: int = 0
    num_q_heads_unpadded: int = 0        # checkpoint's query heads when num_q_heads was zero-padded for TP
    gdn_num_k_heads: int = 0
    gdn_num_v_heads: int = 0
    gdn_head_k_dim: int = 0
    gdn_head_v_dim: int = 0
    gdn_conv_kernel: int = 4
    kda_gate_rank: int = 0               # Kimi Delta Attention: rank of the gate projections (0 = head dim)
    kda_gate_lower_bound: Optional[float] = None   # floor of the per-channel log-decay (None = unbounded)
    # quantisation
    quantization: Optional[str] = None   # None | fp8 | fp8_block | int8 | mxfp4 | nvfp4 | online_fp8
    weight_block_size: tuple = (128, 128)
    kv_cache_dtype: str = "auto"         # auto | bfloat16 | fp8 | fp8_e4m3
    seed: int = 0
    init_std: float = 0.02

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    @property
    def is_hybrid_gdn(self) -> bool:
        return self.full_attention_interval > 0

    def layer_is_moe(self, i: int) -> bool:
        return self.is_moe and i >= self.first_dense_layers

    def layer_is_full_attention(self, i: int) -> bool:
        if not self.is_hybrid_gdn:
            return True
        return (i + 1) % self.full_attention_interval == 0

    @property
    def q_size(self) -> int:
        return self.num_q_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def num_params(self) -> int:
        h, L = self.hidden_size, self.num_layers
        n = 2 * self.vocab_size * h if not self.tie_word_embeddings else self.vocab_size * h
        for i in range(L):
            if self.is_mla:
                qk = self.qk_nope_head_dim + self.qk_rope_head_dim
                n += h * self.q_lora_rank + self.q_lora_rank * self.num_q_heads * qk if self.q_lora_rank else h * self.num_q_heads * qk
                n += h * (self.kv_lora_rank + self.qk_rope_head_dim)
                n += self.kv_lora_rank * self.num_q_heads * (self.qk_nope_head_dim + self.v_head_dim)
                n += self.num_q_heads * self.v_head_dim * h
            else:
                n += h * (self.q_size + 2 * self.kv_size) + self.q_size * h
            if self.layer_is_moe(i):
                n += self.num_experts * 3 * h * self.moe_intermediate_size + h * self.num_experts
                n += 3 * h * (self.shared_expert_intermediate_size
                              or self.num_shared_experts * self.moe_intermediate_size)
            else:
                n += 3 * h * self.intermediate_size
        return n

    @staticmethod
    def from_hf_dict(cfg: dict, name: str = "") -> "ModelConfig":
        """Map a Hugging Face ``config.json`` dictionary to ModelConfig."""
        arch = (cfg.get("architectures") or ["LlamaForCausalLM"])[0]
        mc = ModelConfig(name=name or cfg.get("_name_or_path", arch))
        mc.num_layers = cfg["num_hidden_layers"]
        mc.hidden_size = cfg["hidden_size"]
        mc.num_q_heads = cfg["num_attention_heads"]
        mc.num_kv_heads = cfg.get("num_key_value_heads", mc.num_q_heads)
        mc.head_dim = cfg.get("head_dim") or mc.hidden_size // mc.num_q_heads
        mc.intermediate_size = cfg.get("intermediate_size", 0)
        mc.vocab_size = cfg["vocab_size"]
        mc.rms_norm_eps = cfg.get("rms_norm_eps", 1e-6)
        mc.rope_theta = cfg.get("rope_theta", 10000.0)
        mc.rope_scaling = cfg.get("rope_scaling")
        mc.max_model_len = cfg.get("max_position_embeddings", 4096)
        mc.tie_word_embeddings = cfg.get("tie_word_embeddings", False)
        mc.dtype = parse_dtype(cfg.get("torch_dtype", "bfloat16"))
        mc.sliding_window = cfg.get("sliding_window") if cfg.get("use_sliding_window", True) else None
        act = cfg.get("hidden_act") or cfg.get("hidden_activation") or "silu"
        mc.hidden_act = {"silu": "silu", "swish": "silu", "gelu": "gelu", "gelu_new": "gelu_tanh",
                         "gelu_pytorch_tanh": "gelu_tanh", "gelu_tanh": "gelu_tanh"}.get(act, act)
        if cfg.get("swiglu_limit") and mc.hidden_act == "silu" and cfg.get("swiglu_oai", False):
            mc.hidden_act = f"swigluoai:1.702:{float(cfg['swiglu_limit'])}"
        if arch.startswith(("Llama", "Mistral", "Phi3")):
            mc.architecture = "llama"                   # Phi-3: fused qkv_proj / gate_up_proj in the checkpoint
        elif arch.startswith("Mixtral"):
            # Llama attention, every FFN a mixture of experts whose size is `intermediate_size`
            mc.architecture = "qwen3_moe"
            mc.num_experts = cfg["num_local_experts"]
            mc.num_experts_per_tok = cfg["num_experts_per_tok"]
            mc.moe_intermediate_size = cfg["intermediate_size"]
            mc.moe_renormalize = True
        elif arch.startswith("GptOss"):
            mc.architecture = "gpt_oss"
            mc.attention_bias = mc.attention_out_bias = bool(cfg.get("attention_bias", True))
            mc.num_experts = cfg["num_local_experts"]
            mc.num_experts_per_tok = cfg.get("num_experts_per_tok", cfg.get("experts_per_token", 4))
            mc.moe_intermediate_size = cfg["intermediate_size"]
            mc.moe_renormalize, mc.moe_scoring, mc.moe_bias = True, "softmax", True
            mc.hidden_act = f"swigluoai:1.702:{float(cfg.get('swiglu_limit', 7.0))}"
            types = cfg.get("layer_types") or ["sliding_attention", "full_attention"]
            mc.layer_sliding = tuple(t == "sliding_attention" for t in types)
            mc.sliding_window = cfg.get("sliding_window", 128)
            mc.quant_ignored = ("self_attn",)           # only the experts are mxfp4 in the published checkpoints
        elif arch.startswith("Qwen2Moe"):
            mc.architecture, mc.attention_bias = "qwen3_moe", True
            mc.num_experts = cfg["num_experts"]
            mc.num_experts_per_tok = cfg["num_experts_per_tok"]
            mc.moe_intermediate_size = cfg["moe_intermediate_size"]
            mc.moe_renormalize = cfg.get("norm_topk_prob", False)
            mc.shared_expert_intermediate_size = cfg.get("shared_expert_intermediate_size", 0)
            mc.num_shared_experts = 1 if mc.shared_expert_intermediate_size else 0
            mc.shared_expert_gate = mc.num_shared_experts > 0
            if cfg.get("decoder_sparse_step", 1) != 1:
                raise ValueError("Qwen2-MoE with decoder_sparse_step != 1 is not supported")
            dense_first = cfg.get("mlp_only_layers") or []
            if dense_first and dense_first == list(range(len(dense_first))):
                mc.first_dense_layers = len(dense_first)
        elif arch.startswith("Qwen2"):
            mc.architecture, mc.attention_bias = "llama", True
        elif arch.startswith("Qwen3Moe"):
            mc.architecture, mc.qk_norm = "qwen3_moe", True
            mc.num_experts = cfg["num_experts"]
            mc.num_experts_per_tok = cfg["num_experts_per_tok"]
            mc.moe_intermediate_size = cfg["moe_intermediate_size"]
            mc.moe_renormalize = cfg.get("norm_topk_prob", True)
            dense_first = cfg.get("mlp_only_layers") or []
            if dense_first and dense_first == list(range(len(dense_first))):
                mc.first_dense_layers = len(dense_first)        # leading layers with a plain MLP
        elif arch.startswith("Qwen3Next"):
            mc.architecture, mc.qk_norm = "qwen3_next", True
            mc.num_experts = cfg.get("num_experts", 0)
            mc.num_experts_per_tok = cfg.get("num_experts_per_tok", 0)
            mc.moe_intermediate_size = cfg.get("moe_intermediate_size", 0)
            mc.shared_expert_intermediate_size = cfg.get("shared_expert_intermediate_size", 0)
            mc.num_shared_experts = 1 if mc.shared_expert_intermediate_size else 0
            mc.shared_expert_gate = mc.num_shared_experts > 0
            mc.full_attention_interval = cfg.get("full_attention_interval", 4)
            mc.gdn_num_k_heads = cfg.get("linear_num_key_heads", 16)
            mc.gdn_num_v_heads = cfg.get("linear_num_value_heads", 32)
            mc.gdn_head_k_dim = cfg.get("linear_key_head_dim", 128)
            mc.gdn_head_v_dim = cfg.get("linear_value_head_dim", 128)
            mc.gdn_conv_kernel = cfg.get("linear_conv_kernel_dim", 4)
        elif arch.startswith("KimiLinear"):
            la = cfg.get("linear_attn_config") or {}
            mc.architecture = "kimi_linear"
            kda_layers = la.get("kda_layers") or []
            full_layers = la.get("full_attn_layers") or []
            mc.full_attention_interval = (full_layers[0] if full_layers else 4)
            mc.gdn_num_k_heads = mc.gdn_num_v_heads = la.get("num_heads", mc.num_q_heads)
            mc.gdn_head_k_dim = mc.gdn_head_v_dim = la.get("head_dim", 128)
            mc.gdn_conv_kernel = la.get("short_conv_kernel_size", 4)
            mc.kda_gate_rank = la.get("head_dim", 128)
            mc.num_experts = cfg.get("num_experts", 0)
            mc.num_experts_per_tok = cfg.get("num_experts_per_token", cfg.get("num_experts_per_tok", 0))
            mc.moe_intermediate_size = cfg.get("moe_intermediate_size", 0)
            mc.num_shared_experts = cfg.get("num_shared_experts", 0)
            del kda_layers
            if cfg.get("kv_lora_rank"):
                # the full-attention layers are multi-head latent attention (the published checkpoints)
                mc.q_lora_rank = cfg.get("q_lora_rank") or 0
                mc.kv_lora_rank = cfg["kv_lora_rank"]
                mc.qk_nope_head_dim = cfg["qk_nope_head_dim"]
                mc.qk_rope_head_dim = cfg["qk_rope_head_dim"]
                mc.v_head_dim = cfg["v_head_dim"]
                mc.mla_use_nope = bool(cfg.get("mla_use_nope", False))
                mc.rope_interleaved = True
        elif arch.startswith("Qwen3"):
            mc.architecture, mc.qk_norm = "llama", True
        elif arch.startswith(("DeepseekV3", "DeepseekV2", "DeepseekV32")):
            mc.architecture = "deepseek_v3"
            mc.num_experts = cfg.get("n_routed_experts", 0)
            mc.num_experts_per_tok = cfg.get("num_experts_per_tok", 0)
            mc.moe_intermediate_size = cfg.get("moe_intermediate_size", 0)
            mc.num_shared_experts = cfg.get("n_shared_experts", 0)
            mc.first_dense_layers = cfg.get("first_k_dense_replace", 0)
            mc.moe_scoring = cfg.get("scoring_func", "softmax")
            mc.moe_renormalize = cfg.get("norm_topk_prob", False)
            mc.moe_routed_scaling = cfg.get("routed_scaling_factor", 1.0)
            mc.moe_n_group = cfg.get("n_group", 1)
            mc.moe_topk_group = cfg.get("topk_group", 1)
            mc.moe_score_bias = cfg.get("topk_method", "") == "noaux_tc"
            mc.q_lora_rank = cfg.get("q_lora_rank") or 0
            mc.kv_lora_rank = cfg["kv_lora_rank"]
            mc.qk_nope_head_dim = cfg["qk_nope_head_dim"]
            mc.qk_rope_head_dim = cfg["qk_rope_head_dim"]
            mc.v_head_dim = cfg["v_head_dim"]
            mc.rope_interleaved = True
            mc.index_topk = cfg.get("index_topk", 0)
            mc.index_n_heads = cfg.get("index_n_heads", 0)
            mc.index_head_dim = cfg.get("index_head_dim", 0)
        else:
            raise ValueError(f"unsupported architecture {arch}")
        # features of real checkpoints that the kernels here do not cover are refused, not ignored
        prf = cfg.get("partial_rotary_factor", (cfg.get("rope_parameters") or {}).get("partial_rotary_factor", 1.0))
        if prf not in (None, 1, 1.0):
            raise ValueError(f"partial_rotary_factor {prf}: rotary embeddings over a part of the head are not built")
        if cfg.get("attn_output_gate"):
            raise ValueError("attn_output_gate (gated attention output) is not built")
        if not mc.is_mla and mc.head_dim not in (64, 128):
            raise ValueError(f"head_dim {mc.head_dim}: the attention kernels are built for 64 and 128")
        q = cfg.get("quantization_config")
        if q:
            method = q.get("quant_method")
            if method == "fp8":
                blk = q.get("weight_block_size")
                mc.quantization = "fp8_block" if blk else "fp8"
                if blk:
                    mc.weight_block_size = tuple(blk)
            elif method in ("mxfp4", "modelopt_fp4", "nvfp4", "compressed-tensors", "awq", "gptq"):
                mc.quantization = {"modelopt_fp4": "nvfp4"}.get(method, method)
        return mc

    @staticmethod
    def from_pretrained(path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            return ModelConfig.from_hf_dict(json.load(f), name=os.path.basename(path.rstrip("/")))


def _preset(**kw) -> ModelConfig:
    return ModelConfig(**kw)


def model_preset(name: str) -> ModelConfig:
    """Named architectures used by the benchmarks (random-init, no checkpoint)."""
    n = name.lower()
    if n in ("tiny-llama", "tiny"):
        return _preset(name="tiny-llama", dtype=torch.float32, max_model_len=256)
    if n in ("tiny-mqa",):
        # one KV head, replicated over tensor-parallel ranks: the shape decode context parallelism is for
        return _preset(name="tiny-mqa", dtype=torch.float32, num_kv_heads=1, max_model_len=256)
    if n in ("tiny-moe",):
        return _preset(name="tiny-moe", architecture="qwen3_moe", qk_norm=True, dtype=torch.float32,
                       num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128, max_model_len=256)
    if n in ("tiny-gpt-oss",):
        # GPT-OSS shape in small: sinks, alternating 8-token window / full attention, biases everywhere, OAI SwiGLU;
        # hidden 192 is not a multiple of 128 (like 2880), so the padded down projection is exercised
        return _preset(name="tiny-gpt-oss", architecture="gpt_oss", dtype=torch.float32, num_layers=4,
                       hidden_size=192, num_q_heads=4, num_kv_heads=2, head_dim=64, vocab_size=1024,
                       intermediate_size=128, max_model_len=256, num_experts=8, num_experts_per_tok=2,
                       moe_intermediate_size=128, moe_bias=True, attention_bias=True, attention_out_bias=True,
                       hidden_act="swigluoai:1.702:7.0", sliding_window=8, layer_sliding=(True, False),
                       rope_theta=150000.0,
                       rope_scaling={"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64,
                                     "beta_fast": 32.0, "beta_slow": 1.0, "truncate": False})
    if n in ("tiny-mla",):
        return _preset(name="tiny-mla", architecture="deepseek_v3", dtype=torch.float32, num_layers=3,
                       num_q_heads=4, num_kv_heads=4, head_dim=48, first_dense_layers=1,
                       num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                       num_shared_experts=1, moe_scoring="sigmoid", moe_score_bias=True,
                       moe_n_group=2, moe_topk_group=1, moe_routed_scaling=2.5,
                       q_lora_rank=96, kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16,
                       v_head_dim=32, rope_interleaved=True, max_model_len=256)
    if n in ("tiny-odd-heads",):
        return _preset(name="tiny-odd-heads", dtype=torch.float32, num_q_heads=3, num_kv_heads=1, head_dim=64,
                       hidden_size=256, max_model_len=256)
    if n in ("tiny-kda",):
        return _preset(name="tiny-kda", architecture="kimi_linear", dtype=torch.float32,
                       num_layers=4, full_attention_interval=4, gdn_num_k_heads=4, gdn_num_v_heads=4,
                       gdn_head_k_dim=32, gdn_head_v_dim=32, kda_gate_rank=16, max_model_len=256)
    if n in ("tiny-kda-mla",):
        # the Kimi-Linear layout: KDA layers with every fourth layer latent attention without rotary embeddings
        return _preset(name="tiny-kda-mla", architecture="kimi_linear", dtype=torch.float32,
                       num_layers=4, full_attention_interval=4, gdn_num_k_heads=4, gdn_num_v_heads=4,
                       gdn_head_k_dim=32, gdn_head_v_dim=32, kda_gate_rank=16, max_model_len=256,
                       kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                       rope_interleaved=True, mla_use_nope=True)
    if n in ("tiny-gdn",):
        return _preset(name="tiny-gdn", architecture="qwen3_next", qk_norm=True, dtype=torch.float32,
                       num_layers=4, full_attention_interval=2, gdn_num_k_heads=2, gdn_num_v_heads=4,
                       gdn_head_k_dim=32, gdn_head_v_dim=32, max_model_len=256)
    if n in ("llama-3.1-8b", "llama3.1-8b", "llama-8b"):
        return _preset(name="llama-3.1-8b", num_layers=32, hidden_size=4096, num_q_heads=32,
                       num_kv_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256,
                       rope_theta=500000.0, max_model_len=8192)
    if n in ("llama-3.1-70b", "llama-3.1-70b-fp8", "llama-70b"):
        return _preset(name="llama-3.1-70b-fp8", num_layers=80, hidden_size=8192, num_q_heads=64,
                       num_kv_heads=8, head_dim=128, intermediate_size=28672, vocab_size=128256,
                       rope_theta=500000.0, max_model_len=8192, quantization="fp8_block")
    if n in ("qwen3-30b-a3b", "qwen3-moe"):
        return _preset(name="qwen3-30b-a3b", architecture="qwen3_moe", num_layers=48, hidden_size=2048,
                       num_q_heads=32, num_kv_heads=4, head_dim=128, intermediate_size=6144,
                       vocab_size=151936, rope_theta=1000000.0, qk_norm=True, rms_norm_eps=1e-6,
                       num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
                       max_model_len=8192)
    if n in ("deepseek-v3", "deepseek-v3-fp8"):
        return _preset(name="deepseek-v3", architecture="deepseek_v3", num_layers=61, hidden_size=7168,
                       num_q_heads=128, num_kv_heads=128, head_dim=192, intermediate_size=18432,
                       vocab_size=129280, rms_norm_eps=1e-6, first_dense_layers=3,
                       num_experts=256, num_experts_per_tok=8, moe_intermediate_size=2048,
                       num_shared_experts=1, moe_scoring="sigmoid", moe_score_bias=True,
                       moe_n_group=8, moe_topk_group=4, moe_routed_scaling=2.5,
                       q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64,
                       v_head_dim=128, rope_interleaved=True, max_model_len=8192,
                       quantization="fp8_block")
    if n in ("qwen3-0.6b",):
        return _preset(name="qwen3-0.6b", num_layers=28, hidden_size=1024, num_q_heads=16,
                       num_kv_heads=8, head_dim=128, intermediate_size=3072, vocab_size=151936,
                       rope_theta=1000000.0, qk_norm=True, rms_norm_eps=1e-6, tie_word_embeddings=True,
                       max_model_len=8192)
    raise KeyError(f"unknown model preset {name!r}")


@dataclass
class ParallelConfig:
    tensor_parallel_size: int = 1
    data_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    enable_expert_parallel: bool = False
    prefill_context_parallel_size: int = 1
    decode_context_parallel_size: int = 1
    cp_kv_cache_interleave_size: int = 1
    # filled by the launcher
    rank: int = 0
    local_rank: int = 0
    world_size: int = 1
    backend: str = "nccl"

    @property
    def model_parallel_size(self) -> int:
        return (self.tensor_parallel_size * self.pipeline_parallel_size *
                self.prefill_context_parallel_size)

    def validate(self) -> None:
        want = self.model_parallel_size * self.data_parallel_size
        if self.world_size != want and self.world_size != 1:
            raise ValueError(f"world_size {self.world_size} != tp*pp*pcp*dp = {want}")
        if self.tensor_parallel_size % self.decode_context_parallel_size:
            raise ValueError("decode_context_parallel_size must divide tensor_parallel_size")


@dataclass
class CacheConfig:
    block_size: int = 16
    gpu_memory_utilization: float = 0.90
    num_gpu_blocks_override: Optional[int] = None
    kv_cache_memory_bytes: Optional[int] = None
    enable_prefix_caching: bool = False
    kv_cache_dtype: str = "auto"
    # tokens the scheduler counts per block; under decode context parallelism a block holds block_size
    # tokens on every rank of the DCP group, block_size * dcp in all (0: block_size)
    tokens_per_block: int = 0
    # tokens per scheduler block when it is a multiple of block_size (the kernels' page): a scheduler block
    # then owns that many consecutive kernel blocks of the pool (0: same as block_size)
    scheduler_block_size: int = 0

    @property
    def kernel_blocks_per_block(self) -> int:
        return max(1, self.scheduler_block_size // self.block_size) if self.scheduler_block_size else 1


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    enable_chunked_prefill: bool = True
    scheduler_cls: str = "default"       # default | dp | pp_chunk | prefix_aware | srpt
    async_scheduling: bool = False
    long_prefill_token_threshold: int = 0


@dataclass
class EngineConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    cache: CacheConfig = field(default_factory=CacheConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    device: str = "cuda"
    enforce_eager: bool = False
    load_format: str = "dummy"           # dummy (random init) | safetensors
    model_path: Optional[str] = None
    speculative: Optional[dict] = None
    kv_transfer: Optional[dict] = None
    lora: Optional[dict] = None
    additional: dict = field(default_factory=dict)
    # derived by the platform
    token_buckets: list = field(default_factory=list)
    request_buckets: list = field(default_factory=list)

    def finalize(self) -> "EngineConfig":
        from .platform import B200Platform
        B200Platform.check_and_update_config(self)
        return self

    def describe(self) -> dict[str, Any]:
        d = asdict(self)
        d["model"]["dtype"] = str(self.model.dtype)
        return d
