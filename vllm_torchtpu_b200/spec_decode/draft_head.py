"""Draft-head proposer (EAGLE-3 / MTP family): a one-layer head fed with the target model's last
hidden state and the embedding of the token just sampled predicts the next k tokens
autoregressively.  With random-init weights (benchmarks) its acceptance rate is near zero; it
exists so the runner paths (hidden-state hand-off, k-token verification, rejection) are exercised.
(reference: src/vllm_torchtpu/spec_decode/eagle3.py, mtp_fused_loop.py)"""
from __future__ import annotations

import torch

from ..layers.linear import seeded_normal


class DraftHeadProposer:
    def __init__(self, cfg, runner, k: int, method: str):
        self.num_speculative_tokens = k
        self.method = method
        self.runner = runner
        runner.keep_hidden = True
        m = cfg.model
        dev = runner.device
        self.fc = seeded_normal(f"draft.{method}.fc", (m.hidden_size, 2 * m.hidden_size), m.init_std, m.dtype, dev)
        self.norm = torch.ones(m.hidden_size, dtype=m.dtype, device=dev)
        self.eps = m.rms_norm_eps
        self.last_hidden: dict = {}
        self.last_confidences: dict = {}      # request id -> the head's probability of each draft token

    def note_hidden(self, request_id: str, hidden_row: torch.Tensor) -> None:
        self.last_hidden[request_id] = hidden_row

    def note_step(self, out, res, sampled: dict) -> None:
        """Keep, per request, the hidden state of the row that produced its last accepted token: row
        ``offset + accepted - 1`` of a verification step (k + 1 rows per request), row i otherwise."""
        if res.hidden is None:
            return
        spec_k = res.extra.get("spec_k") if res.extra else None
        off = 0
        for i, rid in enumerate(res.req_ids):
            k = int(spec_k[i]) if spec_k is not None else 0
            if rid in sampled and sampled[rid]:
                row = off + min(len(sampled[rid]), k + 1) - 1
                self.last_hidden[rid] = res.hidden[row]
            off += k + 1
        for s in out.scheduled:
            if s.request.status.finished:
                self.last_hidden.pop(s.request.request_id, None)
                self.last_confidences.pop(s.request.request_id, None)

    def propose(self, out, sampled: dict) -> dict:
        from ..ops import reference as ref
        model = self.runner.model
        drafts = {}
        for s in out.scheduled:
            rid = s.request.request_id
            h = self.last_hidden.get(rid)
            if h is None or rid not in sampled or s.request.status.finished:
                continue
            room = s.request.sampling_params.max_tokens - len(s.request.output_token_ids) - len(sampled[rid]) - 1
            k = min(self.num_speculative_tokens, max(0, room))
            tok = sampled[rid][-1]
            toks, conf = [], []
            hf = h.float()
            for _ in range(k):
                e = model.embed[tok].float()
                hf = torch.cat([hf, e]) @ self.fc.float().t()
                hn = ref.rms_norm(hf[None].to(self.norm.dtype), self.norm, self.eps)[0].float()
                probs = torch.softmax(hn @ model.lm_head.float().t(), dim=-1)
                tok = int(probs.argmax())
                toks.append(tok)
                conf.append(float(probs[tok]))
            if toks:
                drafts[rid] = toks
                self.last_confidences[rid] = conf
        return drafts
