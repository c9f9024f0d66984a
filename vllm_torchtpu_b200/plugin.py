"""Plugin entry points for hosts that run vLLM next to this package.

``register_b200_platform`` follows vLLM's out-of-tree platform protocol: it returns the dotted path of
the platform class when this machine has a Blackwell GPU and the kernel library is present, else
``None`` so that vLLM keeps looking (reference: src/vllm_torchtpu/platforms/__init__.py:56-61,
pyproject.toml entry points).  The engine in this package does not need vLLM; the hook only makes
the platform facts (buckets, supported quantisation and KV dtypes, request validation, HBM budget)
available to a vLLM process."""
from __future__ import annotations

import os
from typing import Optional

from .logger import init_logger

logger = init_logger(__name__)

PLATFORM_CLASS = "vllm_torchtpu_b200.platform.B200Platform"


def register_b200_platform() -> Optional[str]:
    try:
        import torch
    except Exception:                                   # noqa: BLE001
        return None
    if not torch.cuda.is_available():
        return None
    major, minor = torch.cuda.get_device_capability(0)
    if major != 10:
        logger.info("b200 platform plugin: compute capability %d.%d is not sm_100, not registering", major, minor)
        return None
    from .csrc import build
    if not os.path.exists(build.lib_path()):
        logger.warning("b200 platform plugin: %s is missing (python -m vllm_torchtpu_b200.csrc.build)",
                       build.lib_path())
        return None
    logger.info("b200 platform plugin: %s on %s", PLATFORM_CLASS, torch.cuda.get_device_name(0))
    return PLATFORM_CLASS


def register_models() -> list:
    """Architectures this package implements, for hosts that want the list."""
    from .models.registry import supported_architectures
    return supported_architectures()
