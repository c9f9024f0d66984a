"""Medusa drafter: K small heads on the target's last hidden state, head i guessing token t + i + 1.

A head is ``num_layers`` residual blocks ``x + SiLU(W x + b)`` followed by its own vocabulary projection
(the shape of published Medusa checkpoints: ``medusa_heads.<i>.<l>.linear.{weight,bias}`` and
``medusa_heads.<i>.<num_layers>.weight``; a checkpoint without the projection reuses the target's
``lm_head``).  All requests of a step are drafted together on the device: one GEMM per block and head on
this package's kernels, one arg-max per head, one copy of the [R, K] token matrix to the host.
Drafts are arg-max tokens, i.e. a one-hot draft distribution, which is what the verification step's
exact-match acceptance assumes.  Without ``model`` in the speculative config the heads are random and
accept next to nothing: that mode only exercises the runner paths.
(reference: src/vllm_torchtpu/spec_decode/ — the reference takes its Medusa heads from vLLM's
``medusa`` speculative method, docs/user_guide/speculative_decoding.md:5-16)"""
from __future__ import annotations

import re

import torch

from .. import ops
from ..layers.linear import seeded_normal


class MedusaProposer:
    def __init__(self, cfg, runner, k: int, path: str | None = None, num_layers: int = 1):
        self.num_speculative_tokens = k
        self.runner = runner
        runner.keep_hidden = True
        m = cfg.model
        self.dtype, self.device = m.dtype, runner.device
        self.blocks: list = []          # per head: [(W [H, H], b [H])]
        self.heads: list = []           # per head: vocabulary projection [V, H] or None (target's lm_head)
        self.last_hidden: dict = {}
        self.last_confidences: dict = {}
        self.stats = {"proposed": 0, "requests": 0}
        if path:
            self._load(path, k)
        else:
            for i in range(k):
                self.blocks.append([(seeded_normal(f"medusa.{i}.{l}.w", (m.hidden_size, m.hidden_size),
                                                   m.init_std, m.dtype, self.device),
                                     torch.zeros(m.hidden_size, dtype=m.dtype, device=self.device))
                                    for l in range(num_layers)])
                self.heads.append(None)

    def _load(self, path: str, k: int) -> None:
        from ..models.loader import iter_safetensors
        lin, proj = {}, {}
        pat_lin = re.compile(r"(?:medusa_heads|blocks)\.(\d+)\.(\d+)\.linear\.(weight|bias)$")
        pat_proj = re.compile(r"(?:medusa_heads\.(\d+)\.\d+|lm_heads\.(\d+))\.weight$")
        for name, t in iter_safetensors(path):
            mm = pat_lin.search(name)
            if mm:
                lin.setdefault(int(mm.group(1)), {}).setdefault(int(mm.group(2)), {})[mm.group(3)] = t
                continue
            mm = pat_proj.search(name)
            if mm:
                proj[int(mm.group(1) if mm.group(1) is not None else mm.group(2))] = t
        if not lin:
            raise ValueError(f"{path}: no Medusa head tensors (medusa_heads.<i>.<l>.linear.weight)")
        n = min(k, max(lin) + 1)
        self.num_speculative_tokens = n
        to = dict(device=self.device, dtype=self.dtype)
        for i in range(n):
            layers = []
            for l in sorted(lin.get(i, {})):
                w = lin[i][l]["weight"].to(**to).contiguous()
                b = lin[i][l].get("bias")
                layers.append((w, (b if b is not None else torch.zeros(w.shape[0])).to(**to).contiguous()))
            self.blocks.append(layers)
            self.heads.append(proj[i].to(**to).contiguous() if i in proj else None)

    # ---- runner hand-off ------------------------------------------------------------------------------
    def note_step(self, out, res, sampled: dict) -> None:
        """Keep, per request, the hidden state of the row that produced its last accepted token."""
        if res.hidden is None:
            return
        spec_k = res.extra.get("spec_k") if res.extra else None
        off = 0
        for i, rid in enumerate(res.req_ids):
            kk = int(spec_k[i]) if spec_k is not None else 0
            if rid in sampled and sampled[rid]:
                self.last_hidden[rid] = res.hidden[off + min(len(sampled[rid]), kk + 1) - 1]
            off += kk + 1
        for s in out.scheduled:
            if s.request.status.finished:
                self.last_hidden.pop(s.request.request_id, None)
                self.last_confidences.pop(s.request.request_id, None)

    def draft_tokens(self, hidden: torch.Tensor) -> torch.Tensor:
        """hidden [R, H] -> arg-max draft tokens [R, K] (device)."""
        lm_head = self.runner.model.lm_head
        cols = []
        for layers, head in zip(self.blocks, self.heads):
            x = hidden
            for w, b in layers:
                x = x + torch.nn.functional.silu(ops.gemm(x, w, b).to(x.dtype))
            logits = ops.gemm(x, head if head is not None else lm_head)
            cols.append(ops.cuda_ops().argmax(logits) if hidden.is_cuda
                        else logits.float().argmax(-1).to(torch.int32))
        return torch.stack(cols, 1)

    def propose(self, out, sampled: dict) -> dict:
        rids, rows, room = [], [], []
        for s in out.scheduled:
            rid = s.request.request_id
            h = self.last_hidden.get(rid)
            if h is None or rid not in sampled or s.request.status.finished:
                continue
            left = s.request.sampling_params.max_tokens - len(s.request.output_token_ids) - len(sampled[rid]) - 1
            if left <= 0:
                continue
            rids.append(rid)
            rows.append(h)
            room.append(min(self.num_speculative_tokens, left))
        if not rids:
            return {}
        toks = self.draft_tokens(torch.stack(rows).to(self.dtype)).cpu().tolist()
        self.stats["requests"] += len(rids)
        drafts = {}
        for rid, row, k in zip(rids, toks, room):
            drafts[rid] = [int(t) for t in row[:k]]
            self.stats["proposed"] += k
        return drafts
