"""Edits of the logits in front of the sampler: allowed tokens, logit bias, presence / frequency /
repetition penalties and min-p.

The order is the one of the upstream sampler: allowed tokens and the additive bias first, then the
penalties over the tokens seen so far, then min-p (which looks at the distribution after temperature).
Rows that ask for none of this are not touched; a step that has such a row runs eagerly (the edits are
index operations whose sizes change from step to step, so they are kept out of the captured graphs).

With asynchronous scheduling the newest token of a request is still on the device when the next step is
planned: the host passes the request's batch slot instead and the count of that token is added from the
device-resident last-token table, so the penalties see the complete history without a host round trip.
(reference: src/vllm_torchtpu/experimental/export/sampling.py:112-150 - repetition over prompt and output,
presence and frequency over the generated tokens only; its min-p input is ignored, here it is applied)
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass
class RowAdjust:
    row: int                                   # row of the logits matrix
    temperature: float = 0.0
    min_p: float = 0.0
    presence: float = 0.0
    frequency: float = 0.0
    repetition: float = 1.0
    bias: Optional[dict] = None
    allowed: Optional[list] = None
    prompt_ids: list = field(default_factory=list)     # only filled when repetition != 1
    output_ids: list = field(default_factory=list)     # only filled when a penalty is set
    inflight_slot: Optional[int] = None        # batch slot whose last token the host has not read yet

    @property
    def has_penalty(self) -> bool:
        return bool(self.presence or self.frequency or self.repetition != 1.0)


def plan_row(row: int, sp, prompt_ids, output_ids, inflight_slot=None) -> Optional[RowAdjust]:
    """The edits one sampling row needs, or None."""
    if not sp.has_logit_adjust:
        return None
    pen = sp.has_penalties
    return RowAdjust(row, float(sp.temperature), float(sp.min_p) if not sp.greedy else 0.0,
                     float(sp.presence_penalty), float(sp.frequency_penalty), float(sp.repetition_penalty),
                     dict(sp.logit_bias) if sp.logit_bias else None,
                     list(sp.allowed_token_ids) if sp.allowed_token_ids else None,
                     list(prompt_ids) if sp.repetition_penalty != 1.0 else [],
                     list(output_ids) if pen else [], inflight_slot if pen else None)


def _pairs(rows_local, id_lists, vocab):
    rr, tt = [], []
    for j, ids in zip(rows_local, id_lists):
        for t in ids:
            if 0 <= t < vocab:
                rr.append(j)
                tt.append(int(t))
    return rr, tt


def apply_logit_adjust(logits: torch.Tensor, rows: list, last_tokens: Optional[torch.Tensor] = None) -> None:
    """Edit ``logits`` [R, V] in place."""
    if not rows:
        return
    V, dev = logits.shape[-1], logits.device
    lt = lambda x: torch.tensor(x, dtype=torch.long, device=dev)            # noqa: E731
    for r in rows:
        if r.allowed:
            keep = torch.zeros(V, dtype=torch.bool, device=dev)
            keep[lt([t for t in r.allowed if 0 <= t < V])] = True
            logits[r.row].masked_fill_(~keep, float("-inf"))
    br, bt, bv = [], [], []
    for r in rows:
        for t, b in (r.bias or {}).items():
            if 0 <= t < V:
                br.append(r.row)
                bt.append(int(t))
                bv.append(float(b))
    if br:
        logits.index_put_((lt(br), lt(bt)), torch.tensor(bv, dtype=logits.dtype, device=dev), accumulate=True)
    pen = [r for r in rows if r.has_penalty]
    if pen:
        nr = len(pen)
        ridx = lt([r.row for r in pen])
        cnt = torch.zeros(nr, V, dtype=torch.float32, device=dev)
        rr, tt = _pairs(range(nr), [r.output_ids for r in pen], V)
        if rr:
            cnt.index_put_((lt(rr), lt(tt)), torch.ones(len(rr), device=dev), accumulate=True)
        infl = [(j, r.inflight_slot) for j, r in enumerate(pen) if r.inflight_slot is not None]
        if infl:
            if last_tokens is None:
                raise ValueError("a token in flight needs the device-resident last-token table")
            toks = last_tokens[lt([s for _, s in infl])].long().clamp_(0, V - 1)
            cnt.index_put_((lt([j for j, _ in infl]), toks), torch.ones(len(infl), device=dev), accumulate=True)
        seen = cnt > 0
        sub = logits[ridx].float()
        if any(r.repetition != 1.0 for r in pen):
            m = seen.clone()
            rr, tt = _pairs(range(nr), [r.prompt_ids for r in pen], V)
            if rr:
                m[lt(rr), lt(tt)] = True
            rp = torch.tensor([r.repetition for r in pen], dtype=torch.float32, device=dev)[:, None]
            sub = torch.where(m, torch.where(sub > 0, sub / rp, sub * rp), sub)
        fp = torch.tensor([r.frequency for r in pen], dtype=torch.float32, device=dev)[:, None]
        pp = torch.tensor([r.presence for r in pen], dtype=torch.float32, device=dev)[:, None]
        sub = sub - fp * cnt - pp * seen.float()
        logits[ridx] = sub.to(logits.dtype)
    mp = [r for r in rows if r.min_p > 0.0 and r.temperature > 0.0]
    if mp:
        ridx = lt([r.row for r in mp])
        sub = logits[ridx].float()
        # p_i < min_p * p_max  <=>  l_i < l_max + T * ln(min_p) for p = softmax(l / T)
        gap = torch.tensor([r.temperature * math.log(r.min_p) for r in mp], dtype=torch.float32, device=dev)[:, None]
        lim = sub.max(-1, keepdim=True).values + gap
        logits[ridx] = sub.masked_fill(sub < lim, float("-inf")).to(logits.dtype)
