"""Speculative decoding on linear-attention hybrids: undo the state advance of rejected drafts.

A verification step runs k + 1 rows per request through every layer.  Attention layers need no care (a
rejected row's K/V slot is rewritten when the position is decoded again), but a recurrent layer has folded
all k + 1 rows into its state by the time the host learns that only ``a`` of them count.  Instead of keeping
k + 1 copies of every state (the state of one Gated DeltaNet layer is 2 MB per request at Qwen3-Next sizes)
this keeps, per recurrent layer and only for the step's verifying requests,

* one snapshot of the states taken before the step, and
* the layer's own inputs at the verification rows (the projected q/k/v channels and gate inputs: a few KB
  per row),

and, once acceptance is known, restores the snapshot of the requests that rejected something and replays
their first ``a`` rows through the layer's stateful part alone (``layer.recur``): one extra launch of the
recurrence per layer instead of a second pass through the model.  Requests that accepted every draft keep
the state they have.
(reference: src/vllm_torchtpu/runner/spec_boundary_state.py — the reference keeps K + 1 boundary states per
request and picks one by the accepted count)"""
from __future__ import annotations

import numpy as np
import torch

from .attn_metadata import AttentionMetadata


class StateRollback:
    def __init__(self, req_index, slots, row_start, n_rows, pos0, device):
        """Verifying requests of a step: index in the step's request list, batch slot, first verification
        row, number of verification rows (k + 1) and the position of the first of them."""
        self.req_index = np.asarray(req_index, dtype=np.int64)
        self.slots = np.asarray(slots, dtype=np.int64)
        self.row_start = np.asarray(row_start, dtype=np.int64)
        self.n_rows = np.asarray(n_rows, dtype=np.int64)
        self.pos0 = np.asarray(pos0, dtype=np.int64)
        self.device = device
        rows = np.concatenate([s + np.arange(n) for s, n in zip(self.row_start, self.n_rows)])
        self.row_off = np.concatenate([[0], np.cumsum(self.n_rows)])[:-1]
        self._rows_t = torch.from_numpy(rows).to(device)
        self._slots_t = torch.from_numpy(self.slots).to(device)
        self.saved: list = []           # (layer, cache, snapshots, input rows)
        self.stats = {"snapshots": 0, "rolled_back": 0, "replayed_rows": 0}

    def capture(self, layer, cache, inputs) -> None:
        """Called by a recurrent layer in front of its stateful part."""
        snap = tuple(pool.index_select(0, self._slots_t) for pool in cache)
        rows = tuple(t.index_select(0, self._rows_t) for t in inputs)
        self.saved.append((layer, cache, snap, rows))
        self.stats["snapshots"] += 1

    def rollback(self, accepted) -> int:
        """``accepted[i]`` = rows of verifying request i that count (accepted drafts + the token sampled
        after them).  Returns the number of requests whose state was rebuilt."""
        accepted = np.minimum(np.asarray(accepted, dtype=np.int64), self.n_rows)
        need = np.nonzero(accepted < self.n_rows)[0]
        saved, self.saved = self.saved, []
        if not len(need) or not saved:
            return 0
        dev = self.device
        need_t = torch.from_numpy(need).to(dev)
        slots_t = self._slots_t.index_select(0, need_t)
        a = accepted[need]
        replay = np.nonzero(a > 0)[0]
        meta = sel_t = None
        if len(replay):
            ar = a[replay]
            qsl = np.zeros(len(replay) + 1, dtype=np.int64)
            np.cumsum(ar, out=qsl[1:])
            sel = np.concatenate([self.row_off[need[j]] + np.arange(a[j]) for j in replay])
            sel_t = torch.from_numpy(sel).to(dev)
            seq = self.pos0[need[replay]] + ar
            i32 = lambda x: torch.from_numpy(np.ascontiguousarray(x, dtype=np.int32)).to(dev)     # noqa: E731
            nd = int((ar == 1).sum()) if bool((np.sort(ar != 1) == (ar != 1)).all()) else 0
            meta = AttentionMetadata(
                positions=i32(np.concatenate([self.pos0[need[j]] + np.arange(a[j]) for j in replay])),
                slot_mapping=i32(np.full(int(qsl[-1]), -1)), block_tables=i32(np.zeros((len(replay), 1))),
                seq_lens=i32(seq), query_start_loc=i32(qsl), num_reqs=len(replay), num_tokens=int(qsl[-1]),
                num_decode_reqs=nd, max_query_len=int(ar.max()), max_seq_len=int(seq.max()),
                request_distribution=(nd, nd, len(replay)), state_slots=i32(self.slots[need[replay]]),
                seq_lens_cpu=torch.from_numpy(seq.astype(np.int32)),
                query_start_loc_cpu=torch.from_numpy(qsl.astype(np.int32)))
        for layer, cache, snap, rows in saved:
            for pool, s in zip(cache, snap):
                pool.index_copy_(0, slots_t, s.index_select(0, need_t))
            if meta is not None:
                layer.recur(tuple(t.index_select(0, sel_t).contiguous() for t in rows), meta, cache)
        self.stats["rolled_back"] += len(need)
        self.stats["replayed_rows"] += int(a.sum())
        return len(need)
