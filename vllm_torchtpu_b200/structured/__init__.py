"""Structured decoding: per-request grammars produce a packed vocabulary bitmask each step, which a
device op applies to the logits rows before sampling
(reference: src/vllm_torchtpu/structured_decoding/structured_decoding_manager.py:32-474)."""
from .manager import (ChoiceGrammar, RegexGrammar, StructuredDecodingManager, apply_token_bitmask,  # noqa: F401
                      pack_bitmask)


def vocab_strings_of(tokenizer, vocab_size: int) -> list:
    """Text of every token id, as the grammar matcher needs it.  Ids beyond the tokenizer's vocabulary (padding
    rows of the embedding) and ids the tokenizer cannot render get a string no grammar accepts."""
    n = min(vocab_size, len(tokenizer)) if hasattr(tokenizer, "__len__") else vocab_size
    try:
        out = list(tokenizer.batch_decode([[i] for i in range(n)]))
    except Exception:                                    # noqa: BLE001 - tokenizers without batch_decode
        out = []
        for i in range(n):
            try:
                out.append(tokenizer.decode([i]))
            except Exception:                            # noqa: BLE001
                out.append("\x00")
    out = [s if isinstance(s, str) and s else "\x00" for s in out]
    return out + ["\x00"] * (vocab_size - len(out))
