"""Multi-LoRA serving: adapter registry with a fixed number of device slots, per-token adapter ids,
and batched shrink/expand (bgmv) on the wrapped linears.
(reference: src/vllm_torchtpu/lora/lora_manager.py, torch_punica_tpu.py, lora_ops.py:14-101)"""
from .manager import LoRAManager, LoRAAdapter  # noqa: F401
from .ops import bgmv_expand, bgmv_shrink, lora_apply  # noqa: F401
from . import wiring  # noqa: F401,E402
