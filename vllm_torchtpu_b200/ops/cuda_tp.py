"""Bindings used by the tensor-parallel sampling path."""
from __future__ import annotations

from ctypes import c_int

import torch

from . import count_launch
from . import cuda as _c


def argmax_pair(logits):
    R, V = logits.shape
    val = torch.empty(R, dtype=torch.float32, device=logits.device)
    idx = torch.empty(R, dtype=torch.int32, device=logits.device)
    _c._check(_c.lib().b200_argmax_pair(_c._p(logits), c_int(_c._logit_dtype(logits)), c_int(R), c_int(V),
                                        c_int(logits.stride(0)), _c._p(val), _c._p(idx), _c._stream()),
              "argmax_pair")
    count_launch()
    return val, idx


def select_best(vals, idx, shard_size: int):
    world, R = vals.shape
    out = torch.empty(R, dtype=torch.int32, device=vals.device)
    _c._check(_c.lib().b200_select_best(_c._p(vals), _c._p(idx), c_int(world), c_int(R), c_int(shard_size),
                                        _c._p(out), _c._stream()), "select_best")
    count_launch()
    return out


def greedy_top_tokens(local_logits, comm, shard_size: int):
    """Arg-max over a vocab-sharded logits matrix without gathering it."""
    val, idx = argmax_pair(local_logits)
    vals = comm.all_gather(val.unsqueeze(0), dim=0)
    idxs = comm.all_gather(idx.unsqueeze(0), dim=0)
    return select_best(vals.contiguous(), idxs.contiguous(), shard_size)
