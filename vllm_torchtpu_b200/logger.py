"""Package logger.

One lazily configured ``logging`` hierarchy rooted at ``b200``; every module
asks for ``init_logger(__name__)``.  Mirrors the role of the reference's lazy
logger wrapper (reference: src/vllm_torchtpu/logger.py:17-35) without
depending on vLLM.
"""
from __future__ import annotations

import logging
import os
import sys

_ROOT = "b200"
_configured = False


def _configure() -> None:
    global _configured
    if _configured:
        return
    root = logging.getLogger(_ROOT)
    level = os.environ.get("B200_LOG_LEVEL", "INFO").upper()
    root.setLevel(getattr(logging, level, logging.INFO))
    if not root.handlers:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter(
            "%(levelname)s %(asctime)s [%(name)s] %(message)s", "%H:%M:%S"))
        root.addHandler(h)
    root.propagate = False
    _configured = True


def init_logger(name: str) -> logging.Logger:
    _configure()
    short = name.replace("vllm_torchtpu_b200", "").strip(".")
    return logging.getLogger(f"{_ROOT}.{short}" if short else _ROOT)
