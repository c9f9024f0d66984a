"""Input embedding and lm_head sharded over the data-parallel replicas.

With expert parallelism over data-parallel attention every replica is a full copy of the model outside its
MoE layers, so the embedding table and the lm_head are the largest replicated tensors (two 129 280 x 7168
bf16 matrices are 3.7 GB per GPU).  Here each replica keeps rows [r * Vs, (r + 1) * Vs) of both and the
replicas, which already run their steps in lockstep at one agreed number of token rows, exchange:

* embedding: all-gather the step's token ids, look up the rows this replica owns (zero elsewhere),
  reduce-scatter: every replica gets its own tokens' embeddings, each produced by the one owner;
* lm_head: all-gather the rows to project (every replica pads to the same agreed row count), project onto
  the local vocabulary shard, all-to-all: replica j receives every shard's logits for its own rows and
  concatenates them to full-vocabulary logits.

Sound only because the replicas step in lockstep (one embedding and one logits call per step on every
replica, placeholder steps included); features that call the lm_head a data-dependent number of times
(prompt logprobs, drafters) are refused in this mode.
(reference: src/vllm_torchtpu/layers/adapter/dp_vocab_parallel.py:14-324)"""
from __future__ import annotations

import torch

from .. import ops
from .communicator import DeviceCommunicator


class DpVocabParallel:
    def __init__(self, comm: DeviceCommunicator, vocab_size: int):
        self.comm = comm
        self.size, self.rank = comm.size, comm.rank
        self.vocab_size = vocab_size
        self.shard = -(-vocab_size // self.size)
        self.lo = self.rank * self.shard
        self.rows = None            # agreed number of lm_head rows of the current step (None: symmetric call)

    def shard_rows(self, full: torch.Tensor) -> torch.Tensor:
        """Rows of a [V, H] table this replica owns, zero-padded to the common shard size."""
        if full.shape[0] == self.shard and self.size * self.shard != full.shape[0]:
            return full                                              # sharded already
        if full.shape[0] != self.vocab_size:
            raise ValueError(f"expected a [{self.vocab_size}, H] table, got {tuple(full.shape)}")
        part = full[self.lo:self.lo + self.shard]
        if part.shape[0] < self.shard:
            part = torch.cat([part, part.new_zeros(self.shard - part.shape[0], full.shape[1])])
        return part.clone().contiguous()

    def embed(self, ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        """ids [T] (the same T on every replica) -> [T, H]."""
        every = self.comm.all_gather(ids.to(torch.int32), dim=0).long()
        local = every - self.lo
        mine = (local >= 0) & (local < self.shard)
        e = ops.embedding(local.clamp(0, self.shard - 1).to(ids.dtype), table)
        e = e * mine[:, None].to(e.dtype)
        return self.comm.reduce_scatter(e, dim=0).contiguous()

    def logits(self, rows: torch.Tensor, lm_shard: torch.Tensor) -> torch.Tensor:
        """rows [R, H] -> full-vocabulary logits [R, V]."""
        R = rows.shape[0]
        n = self.rows if self.rows is not None else R
        if R > n:
            raise RuntimeError(f"{R} logits rows exceed the {n} rows the replicas agreed on")
        if R < n:
            rows = torch.cat([rows, rows.new_zeros(n - R, rows.shape[1])])
        every = self.comm.all_gather(rows.contiguous(), dim=0)                       # [dp * n, H]
        part = ops.gemm(every, lm_shard)                                             # [dp * n, Vs]
        got = self.comm.all_to_all(part, split_dim=0, concat_dim=1)                  # [n, dp * Vs]
        return got[:R, :self.vocab_size].contiguous()
