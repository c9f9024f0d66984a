"""``B200VllmPlatform``: the vLLM ``Platform`` of this package.

On a machine with the NVIDIA driver the class extends vLLM's CUDA platform, so device queries, memory
accounting, dtype checks and the CUDA worker all stay vLLM's own; what changes is what the reference's
platform changes (reference: src/vllm_torchtpu/platforms/tpu_platform.py:454-1436): the attention
backend (this package's ragged paged attention), the device communicator (NVLink peer-memory
all-reduce for small tensors), the block size default, request validation and the quantisation
list.  Where the driver library cannot be loaded (build hosts) the class extends the abstract
``Platform`` so that plugin resolution and configuration checks can still be exercised."""
from __future__ import annotations

from typing import TYPE_CHECKING, Optional

from vllm.platforms.interface import Platform, PlatformEnum

from ..logger import init_logger

logger = init_logger(__name__)

try:                                                    # needs libcuda
    from vllm.platforms.cuda import CudaPlatform as _Base
    _HAVE_CUDA_BASE = True
except Exception:                                       # noqa: BLE001
    _Base = Platform
    _HAVE_CUDA_BASE = False

if TYPE_CHECKING:
    from vllm.config import VllmConfig

ATTENTION_BACKEND = "vllm_torchtpu_b200.vllm_plugin.attention.B200AttentionBackend"
COMMUNICATOR = "vllm_torchtpu_b200.vllm_plugin.communicator.B200Communicator"


class B200VllmPlatform(_Base):
    # the CUDA enum keeps vLLM's CUDA code paths (is_cuda() is True); the plugin protocol does not
    # require PlatformEnum.OOT
    _enum = PlatformEnum.CUDA
    device_name: str = "cuda"
    device_type: str = "cuda"
    dispatch_key: str = "CUDA"
    ray_device_key: str = "GPU"
    dist_backend: str = "nccl"
    device_control_env_var: str = "CUDA_VISIBLE_DEVICES"

    # ---- attention -------------------------------------------------------------------------
    @classmethod
    def get_attn_backend_cls(cls, selected_backend, attn_selector_config=None, *args, **kwargs) -> str:
        """This package's backend for decoder attention it covers (bf16, head size 64 / 128, no MLA);
        everything else keeps vLLM's choice."""
        cfg = attn_selector_config
        head_size = getattr(cfg, "head_size", None)
        use_mla = bool(getattr(cfg, "use_mla", False))
        dtype = getattr(cfg, "dtype", None)
        import torch
        ours = (not use_mla and head_size in (64, 128) and dtype in (None, torch.bfloat16)
                and not getattr(cfg, "use_sparse", False))
        name = getattr(selected_backend, "name", None)
        if name == "CUSTOM" or (selected_backend is None and ours):
            if not ours:
                raise ValueError("the b200 attention backend covers bf16 decoder attention with head size 64 or 128")
            logger.info("using the b200 ragged paged attention backend")
            return ATTENTION_BACKEND
        if _HAVE_CUDA_BASE:
            return super().get_attn_backend_cls(selected_backend, attn_selector_config, *args, **kwargs)
        raise ValueError(f"attention backend {name!r} needs the CUDA platform")

    @classmethod
    def get_device_communicator_cls(cls) -> str:
        return COMMUNICATOR

    # ---- configuration -----------------------------------------------------------------------
    @classmethod
    def check_and_update_config(cls, vllm_config: "VllmConfig") -> None:
        if _HAVE_CUDA_BASE:
            super().check_and_update_config(vllm_config)
        cache = getattr(vllm_config, "cache_config", None)
        if cache is not None and getattr(cache, "block_size", None) in (None, 0):
            cache.block_size = 16
        par = getattr(vllm_config, "parallel_config", None)
        if par is not None and getattr(par, "worker_cls", "auto") == "auto":
            par.worker_cls = "vllm.v1.worker.gpu_worker.Worker"
        model = getattr(vllm_config, "model_config", None)
        if model is not None:
            import torch
            if getattr(model, "dtype", torch.bfloat16) not in (torch.bfloat16, torch.float16, torch.float32):
                raise ValueError(f"unsupported model dtype {model.dtype}")

    @classmethod
    def validate_request(cls, *args, **kwargs) -> None:
        """Per-request seeds are refused, as on the reference platform (tpu_platform.py:1391-1406):
        the sampler draws its noise from one replica-wide generator so that TP ranks agree."""
        params = kwargs.get("params")
        if params is None:
            params = next((a for a in args if hasattr(a, "seed") and hasattr(a, "temperature")), None)
        if params is not None and getattr(params, "seed", None) is not None:
            raise ValueError("per-request seeds are not supported on this platform")

    @classmethod
    def is_kv_cache_dtype_supported(cls, kv_cache_dtype: str, model_config=None) -> bool:
        return kv_cache_dtype in ("auto", "bfloat16", "fp8", "fp8_e4m3")

    @classmethod
    def use_custom_allreduce(cls) -> bool:
        return False                 # the communicator below owns the peer-memory plane

    if not _HAVE_CUDA_BASE:
        @classmethod
        def get_device_name(cls, device_id: int = 0) -> str:
            return "NVIDIA B200"

        @classmethod
        def get_device_total_memory(cls, device_id: int = 0) -> int:
            return 180 * 2**30

        @classmethod
        def is_async_output_supported(cls, enforce_eager: Optional[bool]) -> bool:
            return True

        @classmethod
        def inference_mode(cls):
            import torch
            return torch.no_grad()
