"""Parallel block drafting (DFlash family, and its semi-autoregressive DSpark variant).

The drafter is a small stack of transformer layers (the target's own layer class, each with one more KV
tensor behind the target's block tables) that proposes all k tokens in ONE forward pass:

* **context** — the inputs of three target layers are concatenated and projected (``fc``) to one feature row
  per token; every draft layer turns that row into a key and a value at the token's position (its own
  ``input_layernorm`` and k / v projection, RoPE at the position).  This runs once per engine step over the
  rows the target just processed (accepted rows only) and needs no attention: it is the "context KV computed
  from the target's hidden states".
* **block** — the just-sampled token (the anchor) and k mask tokens form a block at the next k + 1 positions.
  Every block row attends to all context positions and to ALL block rows (not causally): the block's keys and
  values are written into the look-ahead slots first and each row is then run as a one-row request over the
  whole length, so the existing paged kernels give the non-causal block for free.  Mask row j yields the draft
  for position anchor + j.

``dspark`` uses the same drafter in the layout where the anchor row already predicts the next token (k rows
instead of k + 1) and, when the checkpoint carries a Markov head (``markov_head.embed.weight`` [vocab, r] and
``markov_head.proj.weight`` [draft vocab, r]), re-scores the positions one after another with a bias from the
previously chosen draft token.

Checkpoint names: ``fc.weight`` [H, 3H], ``layers.<l>.*`` (decoder layers), ``norm.weight``, optional
``lm_head.weight`` (+ ``d2t``), optional ``embed_tokens.weight``; ``mask_token_id`` comes from the speculative
config (default: the last vocabulary id).  Drafts are arg-max tokens; without ``model`` the weights are random.
(reference: src/vllm_torchtpu/spec_decode/dflash.py, spec_decode/dspark.py:14-36)"""
from __future__ import annotations

import re
from types import SimpleNamespace

import numpy as np
import torch

from .. import ops
from ..layers.linear import seeded_normal
from ..runner.attn_metadata import AttentionMetadata


class DFlashProposer:
    extra_lookahead = 2            # the block reaches two positions past the verification rows' slots

    def __init__(self, cfg, runner, k: int, kind: str = "dflash", path: str | None = None,
                 num_layers: int = 1, mask_token_id: int | None = None):
        assert kind in ("dflash", "dspark")
        self.kind, self.num_speculative_tokens = kind, k
        self.runner, self.cfg = runner, cfg
        m = self.m = cfg.model
        self.device, self.dtype, self.eps = runner.device, m.dtype, m.rms_norm_eps
        if runner.dcp_size > 1 or m.is_hybrid_gdn or m.is_mla:
            raise ValueError("block drafting is built for GQA attention targets without context parallelism")
        model = runner.model
        if not hasattr(model, "aux_layers"):
            raise ValueError(f"block drafting needs auxiliary hidden states, which {type(model).__name__} lacks")
        L = m.num_layers
        model.aux_layers = tuple(sorted((min(2, L - 1), L // 2, max(0, L - 3))))
        runner.keep_hidden = True
        runner.keep_all_hidden = True
        self.block_size = runner.block_size
        self.mask_token_id = int(mask_token_id if mask_token_id is not None else m.vocab_size - 1)
        self.anchor_predicts = kind == "dspark"           # dspark layout: k rows, every row predicts the next token
        H = m.hidden_size
        self.layers = [model.layer_cls(L + i, m, self.device, None) for i in range(num_layers)]
        self.fc = torch.zeros(H, 3 * H, dtype=self.dtype, device=self.device)
        self.out_norm = torch.ones(H, dtype=self.dtype, device=self.device)
        self.embed = self.head = self.d2t = None
        self.markov_embed = self.markov_proj = None
        if path:
            self._load(path)
        else:
            std, seed = m.init_std, m.seed
            for i, lay in enumerate(self.layers):
                for part in (lay.self_attn, lay.mlp):
                    if hasattr(part, "init_dummy"):
                        part.init_dummy(std, seed)
                    else:
                        for lin in part.linears():
                            lin.init_dummy(std, seed)
            self.fc = seeded_normal(f"draft.{kind}.fc", (H, 3 * H), std, self.dtype, self.device, seed)
        self.kv_caches = [torch.zeros_like(runner.kv_caches[-1]) for _ in self.layers]
        self._res = None
        self.last_confidences: dict = {}
        self.stats = {"proposed": 0, "requests": 0, "context_rows": 0, "block_rows": 0, "passes": 0}
        self.log = None

    # ---- weights -------------------------------------------------------------------------------------------
    def _load(self, path: str) -> None:
        from ..models.loader import iter_safetensors, list_tensor_names, load_named_tensors
        L = self.m.num_layers
        to = dict(device=self.device, dtype=self.dtype)

        def rename(name: str):
            n = re.sub(r"^(model\.)?", "", name)
            mm = re.match(r"^layers\.(\d+)\.(.+)$", n)
            if mm and int(mm.group(1)) < len(self.layers):
                return f"model.layers.{L + int(mm.group(1))}.{mm.group(2)}"
            return n
        names = {rename(n) for n in list_tensor_names(path)}
        found = set()

        def stream():
            for raw, t in iter_safetensors(path):
                n = rename(raw)
                if n.startswith("model.layers."):
                    found.add(n)
                    yield n, t
                elif n == "fc.weight":
                    if tuple(t.shape) != tuple(self.fc.shape):
                        raise ValueError(f"{raw}: shape {tuple(t.shape)}, expected {tuple(self.fc.shape)}")
                    self.fc = t.to(**to).contiguous()
                elif n == "norm.weight":
                    self.out_norm.copy_(t.to(**to))
                elif n == "lm_head.weight":
                    self.head = t.to(**to).contiguous()
                elif n == "embed_tokens.weight":
                    self.embed = t.to(**to).contiguous()
                elif n == "d2t":
                    self.d2t = t.to(device=self.device, dtype=torch.int64)
                elif n == "markov_head.embed.weight":
                    self.markov_embed = t.to(**to).contiguous()
                elif n == "markov_head.proj.weight":
                    self.markov_proj = t.to(**to).contiguous()
        shim = SimpleNamespace(cfg=self.m, layer_range=(L, L + len(self.layers)), layers=self.layers,
                               device=self.device, pp_first=False, pp_last=False)
        load_named_tensors(shim, stream(), names, source=path)
        if not found:
            raise ValueError(f"{path}: no draft layer tensors (layers.<l>.*)")
        if self.head is not None and self.d2t is None and self.head.shape[0] != self.m.vocab_size:
            raise ValueError("a draft vocabulary smaller than the target's needs the d2t table")

    # ---- helpers ---------------------------------------------------------------------------------------------
    def _i32(self, a) -> torch.Tensor:
        return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(self.device)

    def _slots(self, batch_slots, pos):
        b, bs = self.runner.batch, self.block_size
        blk = b.block_table[batch_slots, pos // bs]
        return blk.astype(np.int64) * bs + pos % bs

    def _write_context(self, aux_rows: torch.Tensor, pos: np.ndarray, slot_map: np.ndarray) -> None:
        """Keys and values of the context rows for every draft layer (no attention)."""
        ctx = ops.gemm(aux_rows, self.fc).to(self.dtype)
        positions, slots = self._i32(pos), self._i32(slot_map)
        for lay, cache in zip(self.layers, self.kv_caches):
            a = lay.self_attn
            qkv = a.qkv(ops.rms_norm(ctx, lay.input_ln, self.eps))
            at = a.attn
            ops.rope_and_cache(qkv, positions, at.inv_freq, cache, slots, at.num_q_heads, at.num_kv_heads,
                               at.head_dim, at.rope_interleaved, at.q_norm_w, at.k_norm_w, at.eps, at.k_scale,
                               at.v_scale)

    def _block_meta(self, batch_slots, start, rows_per_req: int) -> AttentionMetadata:
        """Every block row as a one-row request over the whole length: context + the complete block."""
        b = self.runner.batch
        n = len(batch_slots)
        T = n * rows_per_req
        req = np.repeat(np.arange(n), rows_per_req)
        pos = start[req] + np.tile(np.arange(rows_per_req), n)
        seq = np.repeat(start + rows_per_req, rows_per_req)
        qsl = np.arange(T + 1, dtype=np.int64)
        tslots = batch_slots[req]
        return AttentionMetadata(
            positions=self._i32(pos), slot_mapping=self._i32(self._slots(tslots, pos)),
            block_tables=self._i32(b.block_table[tslots]), seq_lens=self._i32(seq), query_start_loc=self._i32(qsl),
            num_reqs=T, num_tokens=T, num_decode_reqs=T, max_query_len=1, max_seq_len=int(seq.max()),
            logits_indices=self._i32(np.arange(T)), request_distribution=(T, T, T), state_slots=self._i32(tslots),
            seq_lens_cpu=torch.from_numpy(seq.astype(np.int32)), query_start_loc_cpu=torch.from_numpy(qsl.astype(np.int32)))

    def _logits(self, g: torch.Tensor) -> torch.Tensor:
        h = ops.rms_norm(g, self.out_norm, self.eps)
        lg = ops.gemm(h, self.head) if self.head is not None else self.runner.model.compute_logits(h)
        return lg.float()

    # ---- engine hand-off ---------------------------------------------------------------------------------------
    def note_step(self, out, res, sampled: dict) -> None:
        self._res = res

    def propose(self, out, sampled: dict) -> dict:
        res, self._res = self._res, None
        if res is None or res.hidden_all is None or res.rows is None:
            return {}
        by_id = {s.request.request_id: s.request for s in out.scheduled}
        qsl, slots_all, pos0_all = res.rows["qsl"], res.rows["slots"], res.rows["pos0"]
        k = self.num_speculative_tokens
        ctx_rows, ctx_pos, ctx_slot, drafting = [], [], [], []
        for i, rid in enumerate(res.req_ids):
            req = by_id.get(rid)
            if req is None:
                continue
            new = list(sampled.get(rid) or [])
            seq_len = len(req.all_token_ids) + len(new)
            n_i, p0, bslot = int(qsl[i + 1] - qsl[i]), int(pos0_all[i]), int(slots_all[i])
            # rows whose token belongs to the sequence: everything but rejected drafts
            valid = min(n_i, seq_len - 1 - p0) if new else n_i
            if valid > 0:
                pos = p0 + np.arange(valid)
                ctx_rows.append(qsl[i] + np.arange(valid))
                ctx_pos.append(pos)
                ctx_slot.append(self._slots(np.full(valid, bslot), pos))
            if new and not req.status.finished:
                left = req.sampling_params.max_tokens - len(req.output_token_ids) - len(new) - 1
                want = max(0, min(k, left, self.m.max_model_len - seq_len - 2))
                if want > 0:
                    drafting.append((req, bslot, seq_len, int(new[-1]), want))
        dev = self.device
        if ctx_rows:
            rows = np.concatenate(ctx_rows)
            aux = res.hidden_all.index_select(0, torch.from_numpy(rows).to(dev)).to(self.dtype)
            self._write_context(aux, np.concatenate(ctx_pos), np.concatenate(ctx_slot))
            self.stats["context_rows"] += len(rows)
        if not drafting:
            return {}
        # ---- one block pass for all drafting requests
        rpr = k if self.anchor_predicts else k + 1
        n = len(drafting)
        bslots = np.array([d[1] for d in drafting], dtype=np.int64)
        start = np.array([d[2] - 1 for d in drafting], dtype=np.int64)          # position of the anchor token
        ids = np.full((n, rpr), self.mask_token_id, dtype=np.int32)
        ids[:, 0] = [d[3] for d in drafting]
        meta = self._block_meta(bslots, start, rpr)
        hidden = ops.embedding(torch.from_numpy(ids.reshape(-1)).to(dev),
                               self.embed if self.embed is not None else self.runner.model.embed)
        residual = None
        for lay, cache in zip(self.layers, self.kv_caches):
            hidden, residual = lay.forward(hidden, residual, cache, meta)
        g = ops.materialize(hidden) + residual
        logits = self._logits(g).view(n, rpr, -1)
        if not self.anchor_predicts:
            logits = logits[:, 1:]                                              # mask rows only
        self.stats["block_rows"] += n * rpr
        self.stats["passes"] += 1
        tok, conf = self._pick(logits)
        tok_h, conf_h = tok.cpu().tolist(), conf.cpu().tolist()
        drafts, confs = {}, {}
        for (req, _, seq_len, _, want), tr, cr in zip(drafting, tok_h, conf_h):
            drafts[req.request_id] = [int(t) for t in tr[:want]]
            confs[req.request_id] = [float(c) for c in cr[:want]]
            if self.log is not None:
                self.log.append((req.request_id, seq_len, tuple(drafts[req.request_id])))
        self.last_confidences = confs
        self.stats["requests"] += n
        self.stats["proposed"] += sum(len(d) for d in drafts.values())
        return drafts

    def _pick(self, logits: torch.Tensor):
        """[n, k, V_draft] -> (target token ids [n, k], probabilities); the Markov head, when present, re-scores
        position j with a bias from the token chosen at position j - 1."""
        n, k, _ = logits.shape
        if self.markov_embed is None or self.markov_proj is None:
            tok = logits.argmax(-1)
            conf = torch.softmax(logits, -1).gather(2, tok[..., None])[..., 0]
        else:
            toks, confs, prev = [], [], None
            for j in range(k):
                lj = logits[:, j]
                if prev is not None:
                    lj = lj + (self.markov_embed[prev].float() @ self.markov_proj.float().t())
                t = lj.argmax(-1)
                confs.append(torch.softmax(lj, -1).gather(1, t[:, None])[:, 0])
                toks.append(t)
                prev = t + self.d2t[t] if self.d2t is not None else t
            tok, conf = torch.stack(toks, 1), torch.stack(confs, 1)
        if self.d2t is not None:
            tok = tok + self.d2t[tok]
        return tok.to(torch.int32), conf
