"""Platform object for an external omni (diffusion / multimodal generation) runtime.

Only imported when that runtime is installed (``register_omni_b200_platform`` checks): it answers the
runtime's questions about the device and names the attention backend and profiler to use
(reference: src/vllm_torchtpu/omni/platform.py:30-229)."""
from __future__ import annotations

import torch

try:                                                    # the base class exists only with the runtime installed
    from vllm_omni.platforms.interface import OmniPlatform as _Base
except Exception:                                       # noqa: BLE001 - any import problem means "not installed"
    _Base = object


class OmniB200Platform(_Base):
    device_name = "cuda"
    device_type = "cuda"
    dispatch_key = "CUDA"
    dist_backend = "nccl"

    @classmethod
    def get_diffusion_attn_backend_cls(cls, selected_backend=None, head_size: int = 128) -> str:
        return "vllm_torchtpu_b200.omni.backend.B200DiffusionAttentionBackend"

    @classmethod
    def supports_torch_inductor(cls) -> bool:
        return False                                     # hand-written kernels and CUDA graphs, no tracing compiler

    @classmethod
    def supports_diffusion_dense_flash_attention(cls) -> bool:
        return True

    @classmethod
    def supports_float64(cls) -> bool:
        return True

    @classmethod
    def supports_cpu_offload(cls) -> bool:
        return True

    @classmethod
    def set_device(cls, device) -> None:
        torch.cuda.set_device(device)

    @classmethod
    def get_torch_device(cls, local_rank=None) -> torch.device:
        return torch.device("cuda", torch.cuda.current_device() if local_rank is None else local_rank)

    @classmethod
    def get_device_count(cls) -> int:
        return torch.cuda.device_count()

    @classmethod
    def get_device_version(cls):
        major, minor = torch.cuda.get_device_capability()
        return f"sm_{major}{minor}"

    @classmethod
    def synchronize(cls, device=None) -> None:
        torch.cuda.synchronize(device)

    @classmethod
    def empty_cache(cls) -> None:
        torch.cuda.empty_cache()

    @classmethod
    def get_device_total_memory(cls, device_id: int = 0) -> int:
        return torch.cuda.get_device_properties(device_id).total_memory

    @classmethod
    def get_free_memory(cls, device=None) -> int:
        return torch.cuda.mem_get_info(device)[0]

    @classmethod
    def max_memory_allocated(cls, device=None) -> int:
        return torch.cuda.max_memory_allocated(device)

    @classmethod
    def max_memory_reserved(cls, device=None) -> int:
        return torch.cuda.max_memory_reserved(device)

    @classmethod
    def reset_peak_memory_stats(cls, device=None) -> None:
        torch.cuda.reset_peak_memory_stats(device)
