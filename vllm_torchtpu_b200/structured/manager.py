"""Grammars and the bitmask plumbing.

Two built-in grammar kinds (an external matcher such as xgrammar can be plugged in through the
same ``allowed_token_ids`` / ``accept`` interface):

* ``ChoiceGrammar``: the output must be one of several token-id sequences (a trie walk);
* ``RegexGrammar``: the decoded text must match a regular expression; a token is allowed when
  text + token can still be extended to a full match (``regex`` partial matching).

The mask is packed 32 tokens per int32 word, row per request, exactly the layout the device op
consumes, so the host→device copy is vocab/8 bytes per constrained request.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch


class ChoiceGrammar:
    def __init__(self, choices: Sequence[Sequence[int]], eos_token_id: Optional[int] = None):
        self.trie: dict = {}
        for seq in choices:
            node = self.trie
            for t in seq:
                node = node.setdefault(int(t), {})
            node[None] = True
        self.node = self.trie
        self.eos = eos_token_id
        self.finished = False

    def allowed_token_ids(self) -> list:
        if self.finished:
            return [self.eos] if self.eos is not None else []
        ids = [t for t in self.node if t is not None]
        if None in self.node and self.eos is not None:
            ids.append(self.eos)
        return ids

    def accept(self, token: int) -> bool:
        if token == self.eos and None in self.node:
            self.finished = True
            return True
        nxt = self.node.get(int(token))
        if nxt is None:
            return False
        self.node = nxt
        if list(nxt.keys()) == [None]:
            self.finished = True
        return True


class RegexGrammar:
    def __init__(self, pattern: str, vocab: Sequence[str], eos_token_id: Optional[int] = None):
        import regex
        self.rx = regex.compile(pattern)
        self.vocab = list(vocab)
        self.text = ""
        self.eos = eos_token_id
        self.finished = False

    def _ok(self, s: str) -> bool:
        m = self.rx.fullmatch(s, partial=True)
        return m is not None

    def allowed_token_ids(self) -> list:
        if self.finished:
            return [self.eos] if self.eos is not None else []
        ids = [i for i, tok in enumerate(self.vocab) if tok and self._ok(self.text + tok)]
        if self.eos is not None and self.rx.fullmatch(self.text) is not None:
            ids.append(self.eos)
        return ids

    def accept(self, token: int) -> bool:
        if token == self.eos:
            self.finished = self.rx.fullmatch(self.text) is not None
            return self.finished
        s = self.text + self.vocab[token]
        if not self._ok(s):
            return False
        self.text = s
        return True


def pack_bitmask(allowed_ids: Sequence[int], vocab_size: int) -> np.ndarray:
    words = np.zeros((vocab_size + 31) // 32, dtype=np.uint32)
    ids = np.asarray(list(allowed_ids), dtype=np.int64)
    ids = ids[(ids >= 0) & (ids < vocab_size)]
    np.bitwise_or.at(words, ids >> 5, (np.uint32(1) << (ids & 31).astype(np.uint32)))
    return words.view(np.int32)


def apply_token_bitmask(logits: torch.Tensor, bitmask: torch.Tensor, rows: Optional[torch.Tensor] = None):
    """logits [R, V]; bitmask [M, ceil(V/32)] int32; rows [M] = logits row of each mask row
    (None: row i ↔ mask i).  Disallowed tokens get -inf, in place."""
    V = logits.shape[1]
    if logits.is_cuda and logits.dtype in (torch.bfloat16, torch.float32) and logits.stride(-1) == 1:
        from ..ops import cuda_misc
        return cuda_misc.apply_token_bitmask(logits, bitmask, rows)
    bits = (bitmask.to(torch.int64)[:, :, None] >> torch.arange(32, device=bitmask.device)) & 1
    allow = bits.reshape(bitmask.shape[0], -1)[:, :V].bool()
    if rows is None:
        logits.masked_fill_(~allow, float("-inf"))
    else:
        sub = logits[rows.long()]
        sub.masked_fill_(~allow, float("-inf"))
        logits[rows.long()] = sub
    return logits


class StructuredDecodingManager:
    def __init__(self, vocab_size: int, vocab: Optional[Sequence[str]] = None, eos_token_id: Optional[int] = None):
        self.vocab_size, self.vocab, self.eos = vocab_size, vocab, eos_token_id
        self.grammars: dict = {}

    def add_request(self, request_id: str, spec: dict) -> None:
        if "choice" in spec:
            self.grammars[request_id] = ChoiceGrammar(spec["choice"], self.eos)
        elif "regex" in spec or "json" in spec or spec.get("json_object"):
            if self.vocab is None:
                raise ValueError("regex- and schema-constrained decoding need the tokenizer vocabulary")
            if "regex" in spec:
                pattern = spec["regex"]
            elif "json" in spec:
                from .json_schema import schema_to_regex
                pattern = schema_to_regex(spec["json"])
            else:
                from .json_schema import any_json_object_regex
                pattern = any_json_object_regex()
            self.grammars[request_id] = RegexGrammar(pattern, self.vocab, self.eos)
        else:
            raise ValueError(f"unsupported structured output spec: {sorted(spec)}")

    def remove_request(self, request_id: str) -> None:
        self.grammars.pop(request_id, None)

    def build_bitmask(self, request_ids: Sequence[str]):
        """(bitmask [M, words] int32 tensor, rows [M]) for the constrained requests of a step."""
        rows, masks = [], []
        for i, rid in enumerate(request_ids):
            g = self.grammars.get(rid)
            if g is not None:
                rows.append(i)
                masks.append(pack_bitmask(g.allowed_token_ids(), self.vocab_size))
        if not rows:
            return None, None
        return torch.from_numpy(np.stack(masks)), torch.tensor(rows, dtype=torch.int64)

    def accept_tokens(self, sampled: dict) -> None:
        for rid, toks in sampled.items():
            g = self.grammars.get(rid)
            if g is not None:
                for t in toks:
                    if not g.accept(int(t)):
                        raise RuntimeError(f"token {t} violates the grammar of request {rid}")
