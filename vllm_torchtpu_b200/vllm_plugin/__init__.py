"""vLLM platform plugin: the pieces a vLLM process needs to run on this package's sm_100a kernels.

Two entry points, as in the reference (reference: pyproject.toml:117-127,
src/vllm_torchtpu/platforms/__init__.py:56-61, layers/__init__.py:17-25):

* ``vllm.platform_plugins`` -> :func:`register_platform` returns the dotted path of
  :class:`.platform.B200VllmPlatform` on a machine with a Blackwell GPU and the built kernel library;
* ``vllm.general_plugins`` -> :func:`register_general` registers the attention backend under
  ``AttentionBackendEnum.CUSTOM`` and the out-of-tree providers of RMSNorm and SiLU*mul.

Everything here programs against the vLLM that is installed next to this package; the native engine
(``vllm_torchtpu_b200.engine``) does not need vLLM and does not import this sub-package."""
from __future__ import annotations

import os
from typing import Optional

from ..logger import init_logger

logger = init_logger(__name__)

PLATFORM_CLASS = "vllm_torchtpu_b200.vllm_plugin.platform.B200VllmPlatform"
ATTENTION_BACKEND = "vllm_torchtpu_b200.vllm_plugin.attention.B200AttentionBackend"

_registered = False


def register_platform() -> Optional[str]:
    """Platform plugin hook.  ``B200_VLLM_PLUGIN_FORCE=1`` skips the hardware probe (tests)."""
    if os.environ.get("B200_VLLM_PLUGIN_FORCE", "") == "1":
        return PLATFORM_CLASS
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
    from ..csrc import build
    if not os.path.exists(build.lib_path()):
        logger.warning("b200 platform plugin: %s is missing (python -m vllm_torchtpu_b200.csrc.build)",
                       build.lib_path())
        return None
    logger.info("b200 platform plugin: %s on %s", PLATFORM_CLASS, torch.cuda.get_device_name(0))
    return PLATFORM_CLASS


def register_general() -> None:
    """General plugin hook: attention backend + custom-op providers.  Safe to call more than once and on
    machines without a GPU (the providers import the kernel library lazily)."""
    global _registered
    if _registered:
        return
    _registered = True
    try:
        from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend
        register_backend(AttentionBackendEnum.CUSTOM, ATTENTION_BACKEND)
    except Exception as e:                              # noqa: BLE001 - another vLLM layout: keep going
        logger.warning("b200 plugin: attention backend not registered: %r", e)
    try:
        from . import custom_ops
        custom_ops.register()
    except Exception as e:                              # noqa: BLE001
        logger.warning("b200 plugin: custom-op providers not registered: %r", e)
