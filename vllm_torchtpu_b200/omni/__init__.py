"""Diffusion / multimodal generation on B200.

The reference serves diffusion transformers (Wan, Flux, LTX-2, Qwen-Image) as a platform plugin of an
external omni runtime and contributes the device pieces: a dense non-causal flash attention, rotary
embeddings written for the device's layout, a fused q/k norm + RoPE kernel, patches and a profiler
(reference: src/vllm_torchtpu/omni/__init__.py, omni/platform.py:30-229).  Here the same device pieces
are native, and a small runtime of their own carries them, so that a diffusion transformer runs without
the external package:

* ``attention``   dense bidirectional attention on the tcgen05 prefill kernel, SDPA for masked / causal calls
* ``rope``        multi-axis (frame, row, column) rotary tables, interleaved rotation
* ``ops``         fused q/k RMSNorm + interleaved RoPE (``csrc/omni.cu``)
* ``dit``         a Wan-style diffusion transformer (adaLN modulation, self + cross attention, GELU MLP)
* ``scheduler``   flow-matching Euler steps with a shifted sigma schedule
* ``pipeline``    classifier-free guided sampling loop with per-step timing

``register_omni_b200_platform`` is the entry point an omni runtime looks up; it names the platform class
only when both CUDA and that runtime are present.
"""
from __future__ import annotations

from typing import Optional


def register_omni_b200_platform() -> Optional[str]:
    """Entry point of the ``vllm_omni.platform_plugins`` group
    (reference: src/vllm_torchtpu/omni/__init__.py:18-28)."""
    import importlib.util

    import torch
    if not torch.cuda.is_available() or importlib.util.find_spec("vllm_omni") is None:
        return None
    return "vllm_torchtpu_b200.omni.platform.OmniB200Platform"


__all__ = ["register_omni_b200_platform"]
