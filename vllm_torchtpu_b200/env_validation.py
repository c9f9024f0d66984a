"""Report environment variables that look like ours but that nothing reads.

A user who exports ``B200_FUSED_TPP=0`` gets no error from a lazy registry; this
module finds such names (our prefix, not declared) and suggests the closest
declared knob.  Same purpose as the reference's unread-env report
(reference: src/vllm_torchtpu/env_validation.py:42-152).
"""
from __future__ import annotations

import difflib
import os
from dataclasses import dataclass
from typing import Mapping, Optional

from . import envs


@dataclass(frozen=True)
class UnknownEnv:
    name: str
    suggestion: Optional[str]

    def message(self) -> str:
        hint = f" (did you mean {self.suggestion}?)" if self.suggestion else ""
        return f"environment variable {self.name} is set but nothing reads it{hint}"


def find_unknown(environ: Optional[Mapping[str, str]] = None) -> list[UnknownEnv]:
    environ = os.environ if environ is None else environ
    declared = envs.declared()
    out = []
    for name in sorted(environ):
        if not name.startswith(envs.known_prefixes()) or name in declared:
            continue
        close = difflib.get_close_matches(name, declared, n=1, cutoff=0.75)
        out.append(UnknownEnv(name, close[0] if close else None))
    return out


def validate_values(environ: Optional[Mapping[str, str]] = None) -> list[str]:
    """Parse every declared variable that is set; return the error messages."""
    environ = os.environ if environ is None else environ
    errors = []
    for name, var in envs.declared().items():
        if name in environ:
            try:
                envs._parse(var, environ[name])
            except (ValueError, TypeError) as e:
                errors.append(str(e))
    return errors


def report_unread(logger=None, environ=None) -> list[UnknownEnv]:
    unknown = find_unknown(environ)
    if logger is not None:
        for u in unknown:
            logger.warning(u.message())
    return unknown
