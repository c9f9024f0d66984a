"""Architecture name → model class."""
from __future__ import annotations

from ..config import ModelConfig


def get_model_class(cfg: ModelConfig):
    a = cfg.architecture
    if a == "llama":
        from .llama import LlamaForCausalLM
        return LlamaForCausalLM
    if a == "qwen3_moe":
        from .qwen3_moe import Qwen3MoeForCausalLM
        return Qwen3MoeForCausalLM
    if a == "gpt_oss":
        from .gpt_oss import GptOssForCausalLM
        return GptOssForCausalLM
    if a == "deepseek_v3":
        from .deepseek_v3 import DeepseekV3ForCausalLM
        return DeepseekV3ForCausalLM
    if a == "qwen3_next":
        from .qwen3_next import Qwen3NextForCausalLM
        return Qwen3NextForCausalLM
    if a == "kimi_linear":
        from .kimi_linear import KimiLinearForCausalLM
        return KimiLinearForCausalLM
    raise ValueError(f"no model class for architecture {a!r}")


def supported_architectures() -> list[str]:
    return ["llama", "qwen3_moe", "gpt_oss", "deepseek_v3", "qwen3_next", "kimi_linear"]
