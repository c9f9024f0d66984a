"""Structured decoding: per-request grammars produce a packed vocabulary bitmask each step, which a
device op applies to the logits rows before sampling
(reference: src/vllm_torchtpu/structured_decoding/structured_decoding_manager.py:32-474)."""
from .manager import (ChoiceGrammar, RegexGrammar, StructuredDecodingManager, apply_token_bitmask,  # noqa: F401
                      pack_bitmask)
