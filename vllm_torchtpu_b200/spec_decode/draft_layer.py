"""Drafters that are one transformer layer with attention and a KV cache of their own: DeepSeek-style
MTP modules, EAGLE-1/2 heads and EAGLE-3 heads.

The draft layer is built from the target model's own layer class (so an MTP module of an MLA + MoE model
is an MLA + MoE layer, sharded over tensor-parallel ranks like the target's) and gets one more KV tensor
of the target's shape, addressed through the target's block tables: draft position p lives in the slot of
target position p.  Row p of the drafter reads the target's hidden state of position p together with the
embedding of token p + 1 and predicts token p + 2.

Every engine step has two phases:

1. *catch-up* — one variable-length pass over all rows of the target step whose next token is known
   (prompt chunks, accepted verification rows; rejected rows are left out and their slots are simply
   rewritten later).  It writes the drafter's K/V for those positions; the last row of every sampling
   request yields draft 1.
2. *look-ahead* — k − 1 single-row passes that feed the drafter its own output state and previous draft;
   they write into the look-ahead slots the scheduler reserved for the verification step.

Forms (``speculative_config["method"]``):

* ``mtp``   : ``x = eh_proj([enorm(e); hnorm(h)])`` → layer → ``shared_head.head(shared_head.norm(.))``
  (checkpoint names ``model.layers.<L>.{enorm,hnorm,eh_proj,shared_head.*,self_attn.*,mlp.*}`` with L the
  target's layer count);
* ``eagle`` : ``x = fc([e; h])`` → layer without input norm → the target's ``lm_head``
  (``fc.weight``, ``layers.0.*``);
* ``eagle3``: ``g = fc([h_low; h_mid; h_high])`` from three target layers, attention over
  ``[input_layernorm(e); hidden_norm(g)]`` (2·hidden wide), own norm and a reduced draft vocabulary mapped
  back with ``d2t`` (``fc.weight``, ``midlayer.*``, ``norm.weight``, ``lm_head.weight``, ``d2t``).

Drafts are arg-max tokens.  Without ``model`` in the speculative config the weights are random (the
paths run, next to nothing is accepted).
(reference: src/vllm_torchtpu/spec_decode/eagle3.py, spec_decode/mtp_fused_loop.py,
docs/user_guide/speculative_decoding.md:5-16)"""
from __future__ import annotations

import re
from types import SimpleNamespace

import numpy as np
import torch

from .. import ops
from ..layers.linear import seeded_normal
from ..runner.attn_metadata import AttentionMetadata


class DraftLayerProposer:
    def __init__(self, cfg, runner, k: int, kind: str, path: str | None = None):
        assert kind in ("mtp", "eagle", "eagle3")
        self.kind, self.num_speculative_tokens = kind, k
        self.runner, self.cfg = runner, cfg
        m = cfg.model
        self.m = m
        self.device, self.dtype = runner.device, m.dtype
        if runner.dcp_size > 1:
            raise ValueError("draft layers are not built for decode context parallelism")
        model = runner.model
        runner.keep_hidden = True
        runner.keep_all_hidden = True
        self.block_size = runner.block_size
        L = m.num_layers
        if kind == "eagle3":
            # inputs of a low, a middle and a high layer (a layer may repeat in models of fewer than 6 layers)
            aux = tuple(sorted((min(2, L - 1), L // 2, max(0, L - 3))))
            if not hasattr(model, "aux_layers"):
                raise ValueError(f"eagle3 needs auxiliary hidden states, which {type(model).__name__} does not expose")
            model.aux_layers = aux
            self.n_aux = 3
        quant = None
        if kind == "mtp" and m.quantization:
            from ..quantization import QuantConfig
            quant = QuantConfig(m.quantization, m.weight_block_size, ignored_layers=("lm_head", "embed", "gate."))
        self.layer_idx = L                  # checkpoint index of the module (model.layers.<L>.*)
        # on a linear-attention hybrid the module is a full-attention layer: build it at the index of the
        # target's last full-attention layer and give it a cache of that layer's shape
        self.build_idx = L
        if m.is_hybrid_gdn:
            self.build_idx = max(i for i in range(L) if m.layer_is_full_attention(i))
        self.layer = model.layer_cls(self.build_idx, m, self.device, quant)
        H = m.hidden_size
        one = lambda: torch.ones(H, dtype=self.dtype, device=self.device)      # noqa: E731
        self.eps = m.rms_norm_eps
        self.embed = None                   # own embedding table, else the target's
        self.head = None                    # own vocabulary projection, else the target's lm_head
        self.d2t = None                     # eagle3: draft id -> target id offset
        self.fc_bias = None
        if kind == "mtp":
            self.enorm, self.hnorm, self.out_norm = one(), one(), one()
            self.fc = torch.zeros(H, 2 * H, dtype=self.dtype, device=self.device)
        elif kind == "eagle":
            self.fc = torch.zeros(H, 2 * H, dtype=self.dtype, device=self.device)
        else:
            self.fc = torch.zeros(H, self.n_aux * H, dtype=self.dtype, device=self.device)
            self.hidden_norm, self.out_norm = one(), one()
            from ..models.llama import QKVParallelLinear
            a = self.layer.self_attn
            a.qkv = QKVParallelLinear(f"model.layers.{L}.self_attn.qkv_proj", 2 * H, m.num_q_heads, m.num_kv_heads,
                                      m.head_dim, unpadded_q=m.num_q_heads_unpadded, bias=m.attention_bias,
                                      dtype=m.dtype, device=self.device, quant_config=None)
        par = cfg.parallel
        if (par.data_parallel_size > 1 and par.enable_expert_parallel and hasattr(self.layer.mlp, "experts")):
            # the replicas draft at different times and with different row counts, but an expert-parallel
            # layer needs every rank of the group in each of its collectives
            raise ValueError("a draft layer with expert-parallel experts under data-parallel attention is not "
                             "built (its passes would have to run in lockstep over the replicas)")
        if path:
            self._load(path)
        else:
            self._init_random()
        # one more KV tensor, addressed by the target's block tables
        def blank(c):
            return torch.zeros_like(c) if torch.is_tensor(c) else type(c)(blank(x) for x in c)
        # the draft layer has the shape of the target layer it was modelled on
        self.kv_cache = blank(runner.kv_caches[self.build_idx - model.layer_range[0]] if m.is_hybrid_gdn
                              else runner.kv_caches[-1])
        self._res = None
        self.last_confidences: dict = {}
        self.stats = {"proposed": 0, "requests": 0, "catch_up_rows": 0, "passes": 0}
        self.log = None                     # tests: list of (request id, sequence length, drafts)

    # ---- weights -------------------------------------------------------------------------------------
    def _init_random(self) -> None:
        std, seed = self.m.init_std, self.m.seed
        for part in (self.layer.self_attn, self.layer.mlp):
            if hasattr(part, "init_dummy"):             # MLA attention (absorbed kv_b), MLP and MoE blocks
                part.init_dummy(std, seed)
            else:
                for lin in part.linears():
                    lin.init_dummy(std, seed)
        self.fc = seeded_normal(f"draft.{self.kind}.fc", tuple(self.fc.shape), std, self.dtype, self.device, seed)

    def _load(self, path: str) -> None:
        """Read a drafter checkpoint; layer tensors are renamed to ``model.layers.<L>.*`` and go through the
        package's checkpoint loader (fused q/k/v and gate/up, tensor-parallel shards, fp8 scales)."""
        from ..models.loader import iter_safetensors, list_tensor_names, load_named_tensors
        L = self.layer_idx
        pre = f"model.layers.{L}."
        to = dict(device=self.device, dtype=self.dtype)

        def rename(name: str):
            if self.kind == "mtp":
                return name if name.startswith(pre) else None
            n = re.sub(r"^(model\.)?", "", name)
            n = re.sub(r"^(layers\.0|midlayer)\.", pre, n)
            return n

        own = {"enorm.weight": "enorm", "hnorm.weight": "hnorm", "shared_head.norm.weight": "out_norm",
               "hidden_norm.weight": "hidden_norm"}
        layer_names, found = set(), set()
        for raw in list_tensor_names(path):
            n = rename(raw)
            if n and n.startswith(pre):
                layer_names.add(n)

        def stream():
            for raw, t in iter_safetensors(path):
                n = rename(raw)
                if n is None:
                    continue
                tail = n[len(pre):] if n.startswith(pre) else n
                if tail in own and hasattr(self, own[tail]):
                    getattr(self, own[tail]).copy_(t.to(**to))
                elif tail in ("eh_proj.weight", "fc.weight"):
                    if tuple(t.shape) != tuple(self.fc.shape):
                        raise ValueError(f"{raw}: shape {tuple(t.shape)}, expected {tuple(self.fc.shape)}")
                    self.fc = t.to(**to).contiguous()
                elif tail == "fc.bias":
                    self.fc_bias = t.to(**to).contiguous()
                elif tail in ("shared_head.head.weight", "lm_head.weight"):
                    self.head = t.to(**to).contiguous()
                elif tail == "norm.weight" and self.kind == "eagle3":
                    self.out_norm.copy_(t.to(**to))
                elif tail == "embed_tokens.weight":
                    self.embed = t.to(**to).contiguous()
                elif tail == "d2t":
                    self.d2t = t.to(device=self.device, dtype=torch.int64)
                elif n.startswith(pre):
                    found.add(n)
                    yield n, t
                continue
        shim = SimpleNamespace(cfg=self.m, layer_range=(L, L + 1), layers=[self.layer], device=self.device,
                               pp_first=False, pp_last=False)
        load_named_tensors(shim, stream(), layer_names, source=path)
        if not found:
            raise ValueError(f"{path}: no draft layer tensors found for method {self.kind!r}")
        if self.head is not None and self.d2t is None and self.head.shape[0] != self.m.vocab_size:
            raise ValueError("a draft vocabulary smaller than the target's needs the d2t table")

    # ---- one pass of the draft layer --------------------------------------------------------------------
    def _embed(self, ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(ids, self.embed if self.embed is not None else self.runner.model.embed)

    def _forward(self, ids: torch.Tensor, h_in: torch.Tensor, meta, first: bool) -> torch.Tensor:
        """ids [T], h_in [T, H] (eagle3 catch-up: [T, n_aux·H]) -> the layer's output state g [T, H]."""
        e = self._embed(ids)
        lay = self.layer
        if self.kind == "mtp":
            x = ops.gemm(torch.cat([ops.rms_norm(e, self.enorm, self.eps),
                                    ops.rms_norm(h_in, self.hnorm, self.eps)], -1), self.fc)
            hid, res = lay.forward(x.to(self.dtype), None, self.kv_cache, meta)
            return ops.materialize(hid) + res
        if self.kind == "eagle":
            x = ops.gemm(torch.cat([e, h_in], -1), self.fc, self.fc_bias).to(self.dtype)
            a = lay.self_attn.forward(x, self.kv_cache, meta)
            hn, res = ops.fused_add_rms_norm(a, x, lay.post_ln, self.eps)
            return ops.materialize(lay.mlp.forward(hn)) + res
        g = ops.gemm(h_in, self.fc).to(self.dtype) if first else h_in
        x = torch.cat([ops.rms_norm(e, lay.input_ln, self.eps), ops.rms_norm(g, self.hidden_norm, self.eps)], -1)
        a = lay.self_attn.forward(x, self.kv_cache, meta)
        hn, res = ops.fused_add_rms_norm(a, g, lay.post_ln, self.eps)
        return ops.materialize(lay.mlp.forward(hn)) + res

    def _tokens(self, g: torch.Tensor):
        """Output state rows -> (arg-max target token ids [R] on the host, their probabilities)."""
        model = self.runner.model
        if self.kind == "eagle":
            h = g
        else:
            h = ops.rms_norm(g, self.out_norm, self.eps)
        logits = ops.gemm(h, self.head) if self.head is not None else model.compute_logits(h)
        lf = logits.float()
        tok = lf.argmax(-1)
        conf = torch.softmax(lf, -1).gather(1, tok[:, None])[:, 0]
        if self.d2t is not None:
            tok = tok + self.d2t[tok]
        return tok.to(torch.int32), conf

    def _meta(self, slots, pos0, nrows) -> AttentionMetadata:
        """Metadata of a pass: request i runs ``nrows[i]`` rows from position ``pos0[i]``; requests with one
        row must come first."""
        b, bs, dev = self.runner.batch, self.block_size, self.device
        n = len(slots)
        qsl = np.zeros(n + 1, dtype=np.int64)
        np.cumsum(nrows, out=qsl[1:])
        T = int(qsl[-1])
        req_idx = np.repeat(np.arange(n), nrows)
        pos = pos0[req_idx] + (np.arange(T) - qsl[req_idx])
        tslots = slots[req_idx]
        blk = b.block_table[tslots, pos // bs]
        slot_map = blk.astype(np.int64) * bs + pos % bs
        seq = pos0 + nrows
        i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(dev)     # noqa: E731
        nd = int((nrows == 1).sum())
        assert bool((nrows[:nd] == 1).all()), "one-row requests come first"
        return AttentionMetadata(
            positions=i32(pos), slot_mapping=i32(slot_map), block_tables=i32(b.block_table[slots]),
            seq_lens=i32(seq), query_start_loc=i32(qsl), num_reqs=n, num_tokens=T, num_decode_reqs=nd,
            max_query_len=int(nrows.max()), max_seq_len=int(seq.max()), logits_indices=i32(qsl[1:] - 1),
            request_distribution=(nd, nd, n), state_slots=i32(slots),
            seq_lens_cpu=torch.from_numpy(seq.astype(np.int32)), query_start_loc_cpu=torch.from_numpy(qsl.astype(np.int32)))

    # ---- engine hand-off ---------------------------------------------------------------------------------
    def note_step(self, out, res, sampled: dict) -> None:
        self._res = res

    def propose(self, out, sampled: dict) -> dict:
        res, self._res = self._res, None
        if res is None or res.hidden_all is None or res.rows is None:
            return {}
        by_id = {s.request.request_id: s.request for s in out.scheduled}
        qsl, slots_all, pos0_all = res.rows["qsl"], res.rows["slots"], res.rows["pos0"]
        ent = []        # (one-row flag, request index, request, valid rows, sequence, drafts wanted)
        for i, rid in enumerate(res.req_ids):
            req = by_id.get(rid)
            if req is None:
                continue
            new = list(sampled.get(rid) or [])
            seq = list(req.all_token_ids) + new
            n_i, p0 = int(qsl[i + 1] - qsl[i]), int(pos0_all[i])
            valid = min(n_i, len(seq) - 1 - p0)
            if valid <= 0:
                continue
            want = 0
            if new and not req.status.finished:
                left = req.sampling_params.max_tokens - len(req.output_token_ids) - len(new) - 1
                want = max(0, min(self.num_speculative_tokens, left, self.m.max_model_len - len(seq) - 1))
            ent.append((valid != 1, i, req, valid, seq, want))
        if not ent:
            return {}
        ent.sort(key=lambda t: (t[0], t[1]))
        idx = np.array([t[1] for t in ent])
        nrows = np.array([t[3] for t in ent], dtype=np.int64)
        slots, pos0 = slots_all[idx].astype(np.int64), pos0_all[idx].astype(np.int64)
        meta = self._meta(slots, pos0, nrows)
        rows = np.concatenate([qsl[i] + np.arange(v) for _, i, _, v, _, _ in ent])
        toks = np.concatenate([np.asarray(seq[int(p) + 1:int(p) + 1 + v], dtype=np.int32)
                               for (_, _, _, v, seq, _), p in zip(ent, pos0)])
        dev = self.device
        h_rows = res.hidden_all.index_select(0, torch.from_numpy(rows).to(dev))
        g = self._forward(torch.from_numpy(toks).to(dev), h_rows.to(self.dtype), meta, first=True)
        self.stats["catch_up_rows"] += len(rows)
        self.stats["passes"] += 1
        last = np.cumsum(nrows) - 1
        active = [j for j, t in enumerate(ent) if t[5] > 0]
        if not active:
            return {}
        g_last = g.index_select(0, torch.from_numpy(last[active]).to(dev))
        tok, conf = self._tokens(g_last)
        tok_h, conf_h = tok.cpu().tolist(), conf.cpu().tolist()
        drafts = {ent[j][2].request_id: [int(t)] for j, t in zip(active, tok_h)}
        confs = {ent[j][2].request_id: [float(c)] for j, c in zip(active, conf_h)}
        # look-ahead passes: the drafter reads its own state and its previous draft
        step = 1
        cur = list(range(len(active)))          # indices into `active` still drafting
        while True:
            cur_next = [c for c in cur if ent[active[c]][5] > step]
            if not cur_next:
                break
            sel = torch.tensor([cur.index(c) for c in cur_next], device=dev)
            g_last, tok = g_last.index_select(0, sel), tok.index_select(0, sel)
            cur = cur_next
            js = [active[c] for c in cur]
            p = np.array([len(ent[j][4]) - 2 + step for j in js], dtype=np.int64)
            meta = self._meta(slots[js], p, np.ones(len(js), dtype=np.int64))
            g_last = self._forward(tok, g_last, meta, first=False)
            tok, conf = self._tokens(g_last)
            for j, t, c in zip(js, tok.cpu().tolist(), conf.cpu().tolist()):
                drafts[ent[j][2].request_id].append(int(t))
                confs[ent[j][2].request_id].append(float(c))
            step += 1
            self.stats["passes"] += 1
        self.last_confidences = confs
        self.stats["requests"] += len(drafts)
        self.stats["proposed"] += sum(len(d) for d in drafts.values())
        if self.log is not None:
            for j in active:
                rid = ent[j][2].request_id
                self.log.append((rid, len(ent[j][4]), tuple(drafts[rid])))
        return drafts
