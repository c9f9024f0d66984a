"""Rejection sampling for speculative decoding.

Greedy: a draft token is kept while it equals the target arg-max; the first mismatch is replaced
by the target token; if all k drafts are kept a bonus token is appended.
Random: draft token x_i (drawn from q_i) is kept with probability min(1, p_i(x_i) / q_i(x_i)); at
the first rejection a token is drawn from normalise(max(p_i - q_i, 0)); all kept -> bonus token
from p_{k}.  Deterministic drafters (n-gram) have one-hot q.
The functions below state the rule on the host (the CPU path and the oracle of the tests); on a GPU the
same rules run as kernels: ``ops.cuda.spec_accept`` (deterministic drafts, judged against the tokens the
target's sampler drew; the runner's verification steps use it) and ``ops.cuda.rejection_sample`` (sampled
drafts with their distributions).
(reference: src/vllm_torchtpu/layers/adapter/sample/rejection_sampler.py:35-686)"""
from __future__ import annotations

from typing import Optional

import torch


def greedy_accept(draft: list, target_argmax: list) -> list:
    """target_argmax has len(draft) + 1 entries (one per verified position + bonus)."""
    out = []
    for i, d in enumerate(draft):
        if d == target_argmax[i]:
            out.append(d)
        else:
            out.append(target_argmax[i])
            return out
    out.append(target_argmax[len(draft)])
    return out


def rejection_sample(draft: torch.Tensor, target_probs: torch.Tensor, draft_probs: Optional[torch.Tensor],
                     uniform: torch.Tensor, resample_uniform: torch.Tensor) -> list:
    """draft [k]; target_probs [k+1, V]; draft_probs [k, V] or None (one-hot); uniform [k] in (0,1);
    resample_uniform [k+1] picks the replacement / bonus token by inverse CDF."""
    k = draft.numel()
    out = []
    for i in range(k):
        x = int(draft[i])
        p = float(target_probs[i, x])
        q = 1.0 if draft_probs is None else float(draft_probs[i, x])
        if q > 0 and float(uniform[i]) <= min(1.0, p / q):
            out.append(x)
            continue
        resid = target_probs[i].clone()
        if draft_probs is None:
            resid[x] = max(0.0, p - 1.0)
        else:
            resid = (resid - draft_probs[i]).clamp_min(0)
        z = resid.sum()
        resid = resid / z if z > 0 else target_probs[i]
        out.append(_inverse_cdf(resid, float(resample_uniform[i])))
        return out
    out.append(_inverse_cdf(target_probs[k], float(resample_uniform[k])))
    return out


def _inverse_cdf(probs: torch.Tensor, u: float) -> int:
    c = probs.float().cumsum(0)
    idx = int(torch.searchsorted(c, torch.tensor(u * float(c[-1]), dtype=c.dtype, device=c.device)))
    return min(idx, probs.numel() - 1)
