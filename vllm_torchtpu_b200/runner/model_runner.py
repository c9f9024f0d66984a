"""Model runner: turns a SchedulerOutput into one device step.

Responsibilities (the reference's runner has the same ones,
reference: src/vllm_torchtpu/runner/tpu_runner.py:4287-4776, 5440-5998):
persistent batch bookkeeping, input preparation with the batch ordered
``[decode][prefill/mixed]``, padding of every device-side shape to a bucket,
the forward pass, logits for the sampling rows, sampling, and an asynchronous
copy of the sampled tokens back to the host.  Where the reference pre-compiles
one XLA program per token bucket (``capture_model``, tpu_runner.py:7496), this
runner captures one CUDA graph per decode request bucket and runs prefill/mixed
steps eagerly (they are long enough to hide launch latency).

Sampled tokens also stay on the device in ``last_tokens[batch_slot]`` so the next
step can be launched before the host has read them (async scheduling): input
rows whose token the host does not know yet carry ``token_src = batch_slot`` and
the embedding kernel reads the id from ``last_tokens``.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from .. import envs, ops
from ..config import EngineConfig
from ..logger import init_logger
from ..models.registry import get_model_class
from ..parallel.state import get_state
from ..platform import B200Platform, pad_to_bucket
from .attn_metadata import AttentionMetadata
from .input_batch import InputBatch, StepBuffers

logger = init_logger(__name__)


DEVICE_STATUS_NAMES = {1: "a GEMM consumer waited for a TMA stage", 2: "a TMA producer waited for a free stage",
                       3: "an epilogue waited for its accumulator", 4: "an MMA issuer waited for a free accumulator",
                       5: "a kernel waited for a flag of a peer GPU or of another CTA",
                       6: "an index was out of range, or a receive buffer of the expert-parallel plane overflowed",
                       7: "a kernel waited for its copies in flight"}


class DeviceWaitTimeout(RuntimeError):
    """A bounded wait inside a kernel gave up (the kernel returned early and left this status code):
    the step's results are not valid."""

    def __init__(self, code: int):
        self.code = code
        super().__init__(f"device status {code}: {DEVICE_STATUS_NAMES.get(code, 'unknown code')}; "
                         "the step did not complete")


@dataclass
class StepResult:
    """Handle on a launched step; ``get()`` waits for the token copy."""
    req_ids: list
    samples: list                   # bool per request
    tokens_host: Optional[torch.Tensor]
    event: Optional[object]
    num_reqs: int
    d2h_bytes: int = 0
    extra: dict = field(default_factory=dict)
    lp: Optional[dict] = None       # sample / prompt logprob tensors of the step (device or host)
    hidden: Optional[torch.Tensor] = None   # final-norm hidden state of every sampled row (draft heads)
    hidden_all: Optional[torch.Tensor] = None   # ... of every row of the step (drafters with their own KV cache)
    rows: Optional[dict] = None     # row layout of the step: query_start_loc, first position, batch slot per request
    status_host: Optional[torch.Tensor] = None   # copy of the device status word taken after the step

    def take_logprobs(self):
        """After ``get()``: ({request_id: entry}, {request_id: [entry per prompt position]}).  An entry is
        {"token_id", "logprob", "rank", "top": [(token_id, logprob), ...]}."""
        if not self.lp:
            return None, None

        def entries(tok, pack, k):
            tok_lp, top_lp, top_id, rank = (t.cpu().tolist() for t in pack)
            return [{"token_id": int(t), "logprob": float(lp), "rank": int(r),
                     "top": [(int(i), float(v)) for i, v in zip(ids[:k], vals[:k])]}
                    for t, lp, vals, ids, r in zip(tok, tok_lp, top_lp, top_id, rank)]
        sample, prompt = {}, {}
        if self.lp.get("sample") is not None:
            rows, ks, pack = self.lp["sample"]
            toks = self.tokens_host[: self.num_reqs].tolist()
            ent = entries([toks[i] for i in rows], pack, max(ks))
            for i, k, e in zip(rows, ks, ent):
                e["top"] = e["top"][:k]
                sample[self.req_ids[i]] = e
        for rid, targets, k, pack in self.lp.get("prompt", []):
            prompt[rid] = entries(targets, pack, k)
        return sample, prompt

    def get(self) -> dict:
        if self.event is not None:
            self.event.synchronize()
        if self.status_host is not None:
            code = int(self.status_host[0])
            if code:
                raise DeviceWaitTimeout(code)
        if self.tokens_host is None:
            return {}
        if not self.extra:
            toks = self.tokens_host[: self.num_reqs].tolist()
            return {rid: [t] for rid, t, s in zip(self.req_ids, toks, self.samples) if s}
        # speculative verification: request i owns spec_k[i] + 1 consecutive rows of target tokens;
        # a draft is kept while it equals the target's token at its position
        from ..sample.rejection_sampler import greedy_accept
        spec_k, drafts, stats = self.extra["spec_k"], self.extra["drafts"], self.extra["stats"]
        kmax = self.extra.get("device_accept")
        if kmax is not None:
            # the acceptance ran on the device: counts [R] followed by tokens [R, kmax + 1]
            n = self.num_reqs
            flat = self.tokens_host[: n * (kmax + 2)].tolist()
            out = {}
            for i, (rid, k, s) in enumerate(zip(self.req_ids, spec_k.tolist(), self.samples)):
                if s:
                    base = n + i * (kmax + 1)
                    acc = flat[base:base + flat[i]]
                    out[rid] = acc
                    stats["spec_accepted"] = stats.get("spec_accepted", 0) + len(acc) - 1
                    stats["spec_drafted"] = stats.get("spec_drafted", 0) + k
            return out
        rows = self.tokens_host[: int(spec_k.sum()) + self.num_reqs].tolist()
        out, off = {}, 0
        for rid, k, d, s in zip(self.req_ids, spec_k.tolist(), drafts, self.samples):
            tgt = rows[off:off + k + 1]
            off += k + 1
            if s:
                acc = greedy_accept(d, tgt)
                out[rid] = acc
                stats["spec_accepted"] = stats.get("spec_accepted", 0) + len(acc) - 1
                stats["spec_drafted"] = stats.get("spec_drafted", 0) + k
        return out


class ModelRunner:
    def __init__(self, cfg: EngineConfig, device: Optional[str] = None):
        self.cfg = cfg
        self.device = torch.device(device or cfg.device)
        self.is_cuda = self.device.type == "cuda"
        self.mcfg = cfg.model
        self.block_size = cfg.cache.block_size
        st0 = get_state()
        self.dcp_size, self.dcp_rank = st0.dcp.size, st0.dcp.rank_in_group
        self.dcp_interleave = max(1, cfg.parallel.cp_kv_cache_interleave_size)
        self.max_reqs = cfg.scheduler.max_num_seqs
        self.max_tokens = cfg.scheduler.max_num_batched_tokens
        self.batch = InputBatch(self.max_reqs, self.mcfg.max_model_len, self.block_size,
                                cfg.cache.kernel_blocks_per_block)
        self.model = None
        self.kv_caches: list = []
        self.num_blocks = 0
        self.graphs: dict = {}
        self.graph_pool = None
        self.launch_counter = 0          # kernels launched by this runner (bench accounting)
        self.kernels_per_graph: dict = {}
        self.stats = {"steps": 0, "graph_steps": 0, "eager_steps": 0, "h2d_bytes": 0, "d2h_bytes": 0}
        self._gen = torch.Generator(device=self.device)
        self._gen.manual_seed(self.mcfg.seed + 1234)
        self._stage_timers = None
        self.structured = None           # StructuredDecodingManager when a request asks for it
        self._step_bitmask = None
        self.timing_events = None        # (start event, end event, decode-only?, tokens) per step when enabled
        self._step_extras = None         # logprob / min_tokens work of the current step (see _plan_extras)
        self.keep_hidden = False         # a draft head wants the hidden state of the sampled rows
        self.mm_manager = None           # multimodal encoder manager (runner/mm_encoder.py)
        self._mm_plan = None             # (request id, first prompt token, first row, rows) of this step
        self._last_h = None
        self.keep_all_hidden = False     # a draft layer with attention wants the hidden state of every row
        self._last_h_all = None
        self.extra_kv_layers = 0         # KV layers a drafter allocates beside the model's (HBM budget)
        self._pool_plan = None           # pooling requests of the current step: (id, row lo, row hi, mode, last chunk)
        self._pool_acc: dict = {}        # request id -> [sum or last row, count]
        if envs.B200_STAGE_TIMING and self.is_cuda:
            from ..tracing.stage_timing import RunnerStageTiming
            self._stage_timers = RunnerStageTiming()

    # ------------------------------------------------------------------ setup
    def load_model(self) -> None:
        t0 = time.time()
        cls = get_model_class(self.mcfg)
        st = get_state()
        layer_range = None
        if st.pp.size > 1:
            from ..parallel.pp import partition_layers
            layer_range = partition_layers(self.mcfg.num_layers, st.pp.size)[st.pp.rank_in_group]
        self.model = cls(self.mcfg, self.device, layer_range=layer_range)
        if self.cfg.load_format == "dummy" or not self.cfg.model_path:
            self.model.init_dummy()
        else:
            from ..models.loader import load_safetensors
            load_safetensors(self.model, self.cfg.model_path)
        if self.is_cuda and st.tp.size > 1:
            from ..parallel.communicator import ensure_tp_heap
            ensure_tp_heap(self.max_tokens, self.mcfg.hidden_size)
        if self.is_cuda and st.expert_parallel and st.ep.size > 1 and getattr(self.mcfg, "num_experts", 0):
            from ..parallel.communicator import ensure_ep_heap
            # tokens are identical on the ranks of a TP group: each of them dispatches one slice
            # longer steps go through the plane in several calls, which bounds the receive buffers
            per_rank = min(-(-self.max_tokens // st.tp.size), envs.B200_MOE_EP_CALL_TOKENS)
            ensure_ep_heap(per_rank, self.mcfg.num_experts_per_tok, self.mcfg.hidden_size,
                           self.mcfg.moe_intermediate_size, self.mcfg.num_experts)
        if (self.cfg.additional or {}).get("dp_vocab_parallel"):
            self._enable_dp_vocab()
        logger.info("model %s loaded: %.2f GB weights on this rank in %.1fs", self.mcfg.name,
                    self.model.weight_bytes() / 1e9, time.time() - t0)

    def _enable_dp_vocab(self) -> None:
        """Shard the embedding table and the lm_head over the data-parallel replicas (opt-in through
        ``additional_config={"dp_vocab_parallel": true}``)."""
        st = get_state()
        if not (st.dp.size > 1 and st.expert_parallel):
            raise ValueError("dp_vocab_parallel needs data-parallel replicas coupled by expert parallelism "
                             "(they step in lockstep, which the exchanges rely on)")
        if st.tp.size > 1 or st.pp.size > 1 or self.dcp_size > 1:
            raise ValueError("dp_vocab_parallel is built for replicas of one GPU (no TP / PP / DCP inside a replica)")
        if self.cfg.speculative:
            raise ValueError("dp_vocab_parallel and speculative decoding are exclusive (drafters call the lm_head a "
                             "data-dependent number of times)")
        from ..parallel.communicator import DeviceCommunicator
        from ..parallel.dp_vocab import DpVocabParallel
        self.model.enable_dp_vocab(DpVocabParallel(DeviceCommunicator(st.dp, None), self.mcfg.vocab_size))

    def _alloc_step_buffers(self) -> None:
        mb = self.batch.max_blocks
        self.bufs_prefill = StepBuffers(self.max_tokens, self.max_reqs, mb, self.device)
        self.bufs_decode = StepBuffers(self.max_reqs, self.max_reqs, mb, self.device)
        self.last_tokens = torch.zeros(self.max_reqs, dtype=torch.int32, device=self.device)
        self._spec_k_dev = torch.zeros(self.max_reqs, dtype=torch.int32, device=self.device)
        self.tokens_host = [torch.zeros(self.max_reqs * 9, dtype=torch.int32, pin_memory=self.is_cuda)
                            for _ in range(4)]
        self.status_host = [torch.zeros(1, dtype=torch.int32, pin_memory=self.is_cuda) for _ in range(4)]
        if self.is_cuda:
            from ..ops import cuda as _cuda
            self.status_dev = _cuda.Workspace.get(self.device).status[:1]   # code written by bounded device waits
        else:
            self.status_dev = torch.zeros(1, dtype=torch.int32)
        self._tok_ring = 0

    def determine_num_blocks(self) -> int:
        c = self.cfg.cache
        if c.num_gpu_blocks_override:
            return c.num_gpu_blocks_override
        kv_dtype = B200Platform.kv_cache_torch_dtype(c.kv_cache_dtype, self.mcfg.dtype)
        per_block = self.model.kv_bytes_per_block(self.block_size, kv_dtype)
        if self.extra_kv_layers:
            per_block += self.extra_kv_layers * per_block // max(1, len(self.model.layers))
        if c.kv_cache_memory_bytes:
            return max(2, c.kv_cache_memory_bytes // per_block)
        if not self.is_cuda:
            need = self.max_reqs * self.batch.max_blocks
            return min(need, 4096) + 1
        # peak activation of a full-size step, measured with an eager dummy run
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        self.init_kv_cache(2)
        self._dummy_run(self.max_tokens, min(self.max_reqs, max(1, self.max_tokens // 128)))
        torch.cuda.synchronize()
        peak = torch.cuda.max_memory_allocated() - base
        self.kv_caches = []
        torch.cuda.empty_cache()
        budget = B200Platform.compute_hbm_budget(self.cfg, self.model.weight_bytes(), peak)
        free, total = torch.cuda.mem_get_info()
        kv_bytes = min(budget.kv_cache, int(free * 0.95) - peak)
        n = max(2, kv_bytes // per_block)
        logger.info("HBM: total %.1f GB, weights %.1f GB, activation peak %.2f GB -> KV %.1f GB = %d blocks",
                    total / 1e9, self.model.weight_bytes() / 1e9, peak / 1e9, kv_bytes / 1e9, n)
        return int(n)

    def init_kv_cache(self, num_blocks: int) -> None:
        self.num_blocks = num_blocks
        kv_dtype = B200Platform.kv_cache_torch_dtype(self.cfg.cache.kv_cache_dtype, self.mcfg.dtype)
        self.kv_caches = self.model.allocate_kv_caches(num_blocks, self.block_size, kv_dtype, self.device,
                                                       self.max_reqs) \
            if hasattr(self.model, "allocate_kv_caches") else [
                torch.zeros(self.model.kv_cache_shape(num_blocks, self.block_size), dtype=kv_dtype,
                            device=self.device) for _ in self.model.layers]
        if not hasattr(self, "bufs_prefill"):
            self._alloc_step_buffers()
        if self.is_cuda and hasattr(self.model, "setup_decode_fusion"):
            self.model.setup_decode_fusion(self.kv_caches)
            if self.model.decode_mega is None:
                logger.info("persistent decode kernel not used: %s", self.model.decode_mega_reason)

    # ------------------------------------------------------------ input prep
    def _update_batch(self, out) -> None:
        for rid in out.finished_ids:
            self.batch.remove(rid)
        for rid in out.preempted_ids:
            self.batch.remove(rid)
        for s in out.scheduled:
            if s.is_new or s.request.request_id not in self.batch.slot_of:
                self.batch.add(s.request, s.request.block_ids)
            else:
                self.batch.append_blocks(self.batch.slot_of[s.request.request_id], s.new_block_ids)

    def _prepare_inputs(self, out, pad_tokens_to: int = 0):
        scheds = out.scheduled
        n = len(scheds)
        b = self.batch
        is_dec = [s.num_new_tokens == 1 and s.start > 0 for s in scheds]
        order = [i for i in range(n) if is_dec[i]] + [i for i in range(n) if not is_dec[i]]
        scheds = [scheds[i] for i in order]
        num_decode = sum(is_dec)
        slots = np.fromiter((b.slot_of[s.request.request_id] for s in scheds), dtype=np.int64, count=n)
        num_new = np.fromiter((s.num_new_tokens for s in scheds), dtype=np.int64, count=n)
        starts = np.fromiter((s.start for s in scheds), dtype=np.int64, count=n)
        T = int(num_new.sum())
        decode_only = num_decode == n
        bufs = self.bufs_decode if decode_only else self.bufs_prefill
        if decode_only and not self.cfg.enforce_eager and self.is_cuda:
            R_pad = pad_to_bucket(n, self.cfg.request_buckets)
            T_pad = R_pad
        else:
            R_pad, T_pad = n, T
        if pad_tokens_to > T_pad:
            # lockstep with other replicas: more rows than this rank needs (padded rows: no request)
            if decode_only and T_pad == R_pad and pad_tokens_to in self.cfg.request_buckets and self.is_cuda \
                    and not self.cfg.enforce_eager:
                R_pad = T_pad = pad_tokens_to           # still a captured decode bucket
            else:
                T_pad = pad_tokens_to
                if decode_only:
                    bufs = self.bufs_prefill            # the decode buffers hold one row per request
        qsl = np.zeros(n + 1, dtype=np.int64)
        np.cumsum(num_new, out=qsl[1:])
        if decode_only:
            req_idx = np.arange(n)
            pos = starts
        else:
            req_idx = np.repeat(np.arange(n), num_new)
            pos = starts[req_idx] + (np.arange(T) - qsl[req_idx])
        tslots = slots[req_idx]
        spec_k = np.fromiter((len(s.spec_token_ids) for s in scheds), dtype=np.int64, count=n)
        has_spec = bool(spec_k.any())
        if has_spec:
            # draft tokens are staged behind the known tokens of their row (not counted as known)
            for i, s in enumerate(scheds):
                if s.spec_token_ids:
                    nk = int(b.num_known[slots[i]])
                    b.token_ids[slots[i], nk:nk + len(s.spec_token_ids)] = s.spec_token_ids
            known = pos < (b.num_known[tslots] + spec_k[req_idx])
            rows = np.concatenate([np.arange(qsl[i + 1] - 1 - spec_k[i], qsl[i + 1]) for i in range(n)])
            row_req = np.repeat(np.arange(n), spec_k + 1)
        else:
            known = pos < b.num_known[tslots]
            rows, row_req = qsl[1:] - 1, np.arange(n)
        L = len(rows)
        L_pad = L if has_spec else R_pad
        rslots = slots[row_req]
        ids = b.token_ids[tslots, np.minimum(pos, b.token_ids.shape[1] - 1)]
        seq_lens_np = starts + num_new
        if self.dcp_size > 1:
            # the cache is dealt over the DCP ranks by position in runs of `il`: a token is written only by
            # its owner, at its index among the owner's tokens; the scheduler's blocks hold block_size * dcp
            # tokens, block_size of them on every rank, so the block index carries over
            c, d, il = self.dcp_size, self.dcp_rank, self.dcp_interleave
            local = (pos // (il * c)) * il + pos % il
            blk = b.block_table[tslots, local // self.block_size]
            slot_map = np.where((pos // il) % c == d,
                                blk.astype(np.int64) * self.block_size + local % self.block_size, -1)
            full, rem = np.divmod(seq_lens_np, il * c)
            local_lens = full * il + np.clip(rem - d * il, 0, il)
        else:
            blk = b.block_table[tslots, pos // self.block_size]
            slot_map = blk.astype(np.int64) * self.block_size + pos % self.block_size
            local_lens = seq_lens_np

        hv = bufs.host_view
        v = hv("input_ids", T_pad); v[:T] = ids; v[T:] = 0
        v = hv("positions", T_pad); v[:T] = pos; v[T:] = 0
        v = hv("slot_mapping", T_pad); v[:T] = slot_map; v[T:] = -1
        v = hv("token_src", T_pad); v[:T] = np.where(known, -1, tslots); v[T:] = -1
        v = hv("query_start_loc", R_pad + 1); v[:n + 1] = qsl; v[n + 1:] = T
        v = hv("seq_lens", R_pad); v[:n] = local_lens; v[n:] = 0
        v = hv("global_seq_lens", R_pad); v[:n] = seq_lens_np; v[n:] = 0
        v = hv("logits_indices", L_pad); v[:L] = rows; v[L:] = 0
        v = hv("top_k", L_pad); v[:L] = b.top_k[rslots]; v[L:] = 0
        v = hv("batch_slots", R_pad); v[:n] = slots; v[n:] = -1
        v = hv("temperature", L_pad, np.float32); v[:L] = b.temperature[rslots]; v[L:] = 0
        v = hv("top_p", L_pad, np.float32); v[:L] = b.top_p[rslots]; v[L:] = 1
        hv("rng_step").view(np.int64)[0] = self.stats["steps"]
        hv("num_valid")[0] = T
        bufs.np_bt[:n] = b.block_table[slots]
        if R_pad > n:
            bufs.np_bt[n:R_pad] = 0
        all_greedy = bool((b.temperature[slots] <= 1e-5).all())
        seq_lens_np = local_lens
        return dict(scheds=scheds, n=n, T=T, R_pad=R_pad, T_pad=T_pad, num_decode=num_decode,
                    decode_only=decode_only, bufs=bufs, all_greedy=all_greedy,
                    max_q=int(num_new.max()) if n else 0, max_seq=int(seq_lens_np.max()) if n else 0,
                    seq_lens_np=seq_lens_np, qsl_np=qsl, L=L, L_pad=L_pad, has_spec=has_spec,
                    row_req=row_req, spec_k=spec_k)

    def _make_meta(self, p) -> AttentionMetadata:
        bufs, R, T = p["bufs"], p["R_pad"], p["T_pad"]
        dv = bufs.dev_view
        return AttentionMetadata(
            positions=dv("positions", T), slot_mapping=dv("slot_mapping", T),
            block_tables=bufs.dev_bt[:R], seq_lens=dv("seq_lens", R),
            query_start_loc=dv("query_start_loc", R + 1), num_reqs=p["n"], num_tokens=p["T"],
            num_decode_reqs=p["num_decode"], max_query_len=p["max_q"], max_seq_len=p["max_seq"],
            logits_indices=dv("logits_indices", p.get("L_pad", R)),
            request_distribution=(p["num_decode"], p["num_decode"], p["n"]),
            padded_num_reqs=R, padded_num_tokens=T, state_slots=dv("batch_slots", R),
            seq_lens_cpu=torch.from_numpy(p["seq_lens_np"]), query_start_loc_cpu=torch.from_numpy(p["qsl_np"]),
            dcp_size=self.dcp_size, dcp_rank=self.dcp_rank, dcp_interleave=self.dcp_interleave,
            global_seq_lens=dv("global_seq_lens", R) if self.dcp_size > 1 else None)

    # --------------------------------------------------------------- forward
    def _forward_and_sample(self, bufs, meta, T, R, all_greedy: bool, L=None):
        """Everything that runs on the device for one step (also the captured region).
        ``L`` = number of sampled rows when it differs from the request count (spec-verify steps)."""
        if not self.mcfg.is_moe:
            return self._forward_and_sample_inner(bufs, meta, T, R, all_greedy, L)
        # rows behind the real tokens (bucket or lockstep padding) take no expert: the routing reads the
        # step's count of real rows from this device word
        from ..layers.moe import set_step_valid_tokens
        set_step_valid_tokens(bufs.dev_view("num_valid", 1))
        try:
            return self._forward_and_sample_inner(bufs, meta, T, R, all_greedy, L)
        finally:
            set_step_valid_tokens(None)

    def _forward_and_sample_inner(self, bufs, meta, T, R, all_greedy: bool, L=None):
        dv = bufs.dev_view
        n_req_pad, verify = R, L is not None
        R = L if verify else R
        ids = dv("input_ids", T)
        st = get_state()
        if st.pp.size > 1:
            return self._forward_and_sample_pp(bufs, meta, T, R, n_req_pad, all_greedy, verify)
        hidden0 = self._embed(ids, dv("token_src", T))
        if self._mm_plan and hidden0 is not None:
            # image / video embeddings replace the placeholder-token rows of the prompt
            for rid, start, row0, nrows in self._mm_plan:
                self.mm_manager.merge_into(hidden0, rid, start, row0, nrows)
        hidden, residual = self.model.forward(ids, meta, self.kv_caches, hidden=hidden0)
        if self._pool_plan:
            self._pool(hidden, residual)
        ex = self._step_extras
        if ex is not None and ex["prompt"]:
            self._prompt_logprobs(hidden, residual, ex)
        rows = self._select_rows(hidden, residual, meta.logits_indices)
        h = self.model.finalize(*rows)
        if getattr(meta, "pcp", None) is not None:
            from ..parallel.communicator import get_pcp_comm
            from .pcp_step import broadcast_sample_rows
            h = broadcast_sample_rows(meta.pcp, h, get_pcp_comm())
        if self.keep_hidden:
            self._last_h = h
        if self.keep_all_hidden:
            aux = getattr(self.model, "aux_hidden", None)
            self._last_h_all = torch.cat(aux, -1) if aux else self.model.finalize(hidden, residual)
        st = get_state()
        if (self.is_cuda and all_greedy and st.tp.size > 1 and envs.B200_GREEDY_TOP_TOKENS
                and self.model.vocab_shard is not None and ex is None):
            # vocab-parallel arg-max: exchange (value, index) pairs instead of gathering the logits
            from ..ops import cuda_tp
            from ..parallel.communicator import get_tp_comm
            local = self.model.local_logits(h)
            tokens = cuda_tp.greedy_top_tokens(local, get_tp_comm(), self.model.vocab_shard)
            if not verify:
                self._store_last_tokens(tokens, dv("batch_slots", n_req_pad))
            return tokens, local
        logits = self.model.compute_logits(h)
        if self._step_bitmask is not None:
            # structured decoding: tokens the grammars forbid get -inf before sampling
            from ..structured import apply_token_bitmask
            bm, rows = self._step_bitmask
            apply_token_bitmask(logits, bm.to(logits.device), rows.to(logits.device))
        if ex is not None and ex["mask_rows"]:
            # min_tokens: end-of-sequence and stop tokens cannot be sampled yet
            # (reference: src/vllm_torchtpu/runner/min_tokens.py)
            r_i = torch.tensor(ex["mask_rows"], dtype=torch.long, device=logits.device)
            t_i = torch.tensor(ex["mask_ids"], dtype=torch.long, device=logits.device)
            logits[r_i, t_i] = float("-inf")
        if ex is not None and ex["adjust"]:
            from .logit_adjust import apply_logit_adjust
            apply_logit_adjust(logits, ex["adjust"], self.last_tokens)
        if self.is_cuda:
            # noise comes from Philox inside the kernel, keyed by (seed, step counter in device memory)
            tokens = ops.cuda_ops().sample(logits, dv("temperature", R, torch.float32), dv("top_k", R),
                                           dv("top_p", R, torch.float32), None, all_greedy,
                                           seed=self.mcfg.seed, step_tensor=dv("rng_step").view(torch.int64))
        else:
            uniform = None
            if not all_greedy:
                uniform = torch.rand(logits.shape, generator=self._gen, dtype=torch.float32)
            tokens = ops.sample(logits, dv("temperature", R, torch.float32), dv("top_k", R),
                                dv("top_p", R, torch.float32), uniform, all_greedy).to(torch.int32)
        if not verify:
            self._store_last_tokens(tokens, dv("batch_slots", n_req_pad))
        if ex is not None and ex["lp_rows"]:
            idx = torch.tensor(ex["lp_rows"], dtype=torch.long, device=logits.device)
            ex["out"]["sample"] = (ex["lp_rows"], ex["lp_ks"],
                                   self._gather_logprobs(logits[idx], tokens[idx], max(1, max(ex["lp_ks"]))))
        return tokens, logits

    def _gather_logprobs(self, logits, token_ids, k: int):
        if self.is_cuda:
            return ops.cuda_ops().gather_logprobs(logits.contiguous(), token_ids.contiguous(), k)
        from ..ops import reference
        return reference.gather_logprobs(logits, token_ids.long(), k)

    def _prompt_logprobs(self, hidden, residual, ex, chunk: int = 1024) -> None:
        """Log-probability of every prompt token given its prefix, for the prompt rows of this step, in
        row chunks so that the [rows, vocab] logits stay bounded
        (reference: src/vllm_torchtpu/runner/prompt_logprobs.py)."""
        for rid, lo, hi, targets, k in ex["prompt"]:
            packs = []
            for a in range(lo, hi, chunk):
                b = min(hi, a + chunk)
                idx = torch.arange(a, b, dtype=torch.int32, device=hidden.device)
                h = self.model.finalize(*self._select_rows(hidden, residual, idx))
                logits = self.model.compute_logits(h)
                tg = torch.tensor(targets[a - lo:b - lo], dtype=torch.int32, device=hidden.device)
                packs.append(self._gather_logprobs(logits, tg, max(1, k)))
            pack = tuple(torch.cat([p[j] for p in packs]) for j in range(4))
            ex["out"].setdefault("prompt", []).append((rid, targets, k, pack))

    def _plan_extras(self, p):
        """Per-step work outside the plain sample: logprobs of the sampled tokens, the min_tokens mask,
        logit edits (penalties, bias, allowed tokens, min-p) and prompt logprobs.  Steps that need any of it
        run eagerly."""
        if p.get("has_spec") or get_state().pp.size > 1:
            return None
        lp_rows, lp_ks, mask_rows, mask_ids, prompt, adjust = [], [], [], [], [], []
        qsl = p["qsl_np"]
        for i, s in enumerate(p["scheds"]):
            req = s.request
            sp = req.sampling_params
            if s.samples:
                if sp.logprobs is not None:
                    lp_rows.append(i)
                    lp_ks.append(int(sp.logprobs))
                # tokens produced before this step's sample (placeholders count steps still in flight,
                # this one included)
                n_out = len(req.output_token_ids) + max(0, req.num_output_placeholders - 1)
                if sp.min_tokens and n_out < sp.min_tokens:
                    ids = list(sp.stop_token_ids)
                    if req.eos_token_id is not None and not sp.ignore_eos:
                        ids.append(req.eos_token_id)
                    for t in ids:
                        if 0 <= t < self.mcfg.vocab_size:
                            mask_rows.append(i)
                            mask_ids.append(int(t))
                if sp.has_logit_adjust:
                    from .logit_adjust import plan_row
                    # a token sampled by a step whose result the host has not read yet is counted from
                    # the device-resident last-token table
                    inflight = self.batch.slot_of.get(req.request_id) if req.num_output_placeholders > 1 else None
                    adjust.append(plan_row(i, sp, req.prompt_token_ids, req.output_token_ids, inflight))
            if sp.prompt_logprobs is not None and s.start < req.num_prompt_tokens:
                lo = int(qsl[i])
                n_rows = min(int(qsl[i + 1]) - lo, req.num_prompt_tokens - s.start)
                targets = list(req.prompt_token_ids[s.start + 1: s.start + n_rows + 1])
                if targets:
                    prompt.append((req.request_id, lo, lo + len(targets), targets, int(sp.prompt_logprobs)))
        if not (lp_rows or mask_rows or prompt or adjust):
            return None
        return {"lp_rows": lp_rows, "lp_ks": lp_ks, "mask_rows": mask_rows, "mask_ids": mask_ids,
                "prompt": prompt, "adjust": adjust, "out": {}}

    def _pp_handoff(self):
        if getattr(self, "_pp", None) is None:
            from ..parallel.pp import NcclTransport, PPHandoff
            st = get_state()
            self._pp = PPHandoff(NcclTransport(), prev_rank=None if st.pp.is_first else st.pp.prev_rank,
                                 next_rank=None if st.pp.is_last else st.pp.next_rank,
                                 hidden_size=self.mcfg.hidden_size, dtype=self.mcfg.dtype, device=self.device,
                                 my_rank=st.rank)
        return self._pp

    def _forward_and_sample_pp(self, bufs, meta, T, R, n_req_pad, all_greedy, verify):
        """One step on one pipeline stage.  Every stage schedules the same batch (the schedulers run in
        lockstep); a stage receives hidden + residual as one tensor from its predecessor, runs its
        layers and hands the sum on; the last stage samples and broadcasts the tokens to the others
        (reference: src/vllm_torchtpu/distributed/pp_buffered.py:14-85, runner/tpu_runner.py:8953-9034)."""
        import torch.distributed as dist
        dv = bufs.dev_view
        st = get_state()
        pp = self._pp_handoff()
        ids = dv("input_ids", T)
        if st.pp.is_first:
            hidden, residual = self._embed(ids, dv("token_src", T)), None
        else:
            hidden, residual, _ = pp.start_forward(T)
        hidden, residual = self.model.forward(ids, meta, self.kv_caches, hidden=hidden, residual=residual)
        last_global = st.pp.ranks[-1]
        if st.pp.is_last:
            rows = self._select_rows(hidden, residual, meta.logits_indices)
            h = self.model.finalize(*rows)
            logits = self.model.compute_logits(h)
            if self._step_bitmask is not None:
                from ..structured import apply_token_bitmask
                bm, brows = self._step_bitmask
                apply_token_bitmask(logits, bm.to(logits.device), brows.to(logits.device))
            uniform = None
            if not all_greedy and not self.is_cuda:
                uniform = torch.rand(logits.shape, generator=self._gen, dtype=torch.float32)
            if self.is_cuda:
                tokens = ops.cuda_ops().sample(logits, dv("temperature", R, torch.float32), dv("top_k", R),
                                               dv("top_p", R, torch.float32), None, all_greedy,
                                               seed=self.mcfg.seed, step_tensor=dv("rng_step").view(torch.int64))
            else:
                tokens = ops.sample(logits, dv("temperature", R, torch.float32), dv("top_k", R),
                                    dv("top_p", R, torch.float32), uniform, all_greedy).to(torch.int32)
            pp.end_forward(hidden, residual)           # counts the transfer; nothing is sent
        else:
            pp.end_forward(hidden, residual)
            tokens = torch.empty(R, dtype=torch.int32, device=self.device)
            logits = None
        tokens = tokens.contiguous()
        dist.broadcast(tokens, src=last_global, group=st.pp.device_group)
        if not verify:
            self._store_last_tokens(tokens, dv("batch_slots", n_req_pad))
        return tokens, logits

    def _pool(self, hidden, residual) -> None:
        """Embedding requests: the final-norm hidden states of the prompt rows of this step are summed
        (mean pooling, accumulated over prefill chunks) or the last row is kept (static shapes: the
        whole step is normalised once; reference: src/vllm_torchtpu/runner/tpu_pooling.py)."""
        hn = self.model.finalize(hidden, residual).float()
        for rid, lo, hi, mode, last_chunk in self._pool_plan:
            acc = self._pool_acc.setdefault(rid, [None, 0])
            if mode == "mean":
                part = hn[lo:hi].sum(0)
                acc[0] = part if acc[0] is None else acc[0] + part
                acc[1] += hi - lo
            elif mode == "max":
                part = hn[lo:hi].max(0).values
                acc[0], acc[1] = (part if acc[0] is None else torch.maximum(acc[0], part)), 1
            elif mode == "cls":
                if acc[0] is None:                   # the first row of the first chunk
                    acc[0], acc[1] = hn[lo].clone(), 1
            elif mode == "all":
                # one vector per prompt token (token classification / late-interaction retrieval)
                acc[0] = hn[lo:hi].clone() if acc[0] is None else torch.cat([acc[0], hn[lo:hi]], 0)
                acc[1] = 1
            elif last_chunk:
                acc[0], acc[1] = hn[hi - 1].clone(), 1
        self._pool_plan = None

    def take_pooled(self, rid: str):
        acc = self._pool_acc.pop(rid, None)
        if acc is None or acc[0] is None:
            return None
        return (acc[0] / max(1, acc[1])).cpu().tolist()

    def _embed(self, ids, token_src):
        if self.model.embed is None:
            return None
        dpv = getattr(self.model, "dp_vocab", None)
        if dpv is not None:
            # the table is sharded over the replicas: resolve the on-device token feedback first, then exchange
            use_last = token_src >= 0
            real = torch.where(use_last, self.last_tokens[token_src.clamp_min(0).long()], ids)
            return dpv.embed(real, self.model.embed)
        if self.is_cuda:
            return ops.cuda_ops().embedding(ids, self.model.embed, token_src, self.last_tokens)
        use_last = token_src >= 0
        real = torch.where(use_last, self.last_tokens[token_src.clamp_min(0).long()], ids)
        return ops.embedding(real, self.model.embed)

    def _select_rows(self, hidden, residual, idx):
        if self.is_cuda:
            return ops.cuda_ops().gather_rows(hidden, residual, idx)
        i = idx.long()
        return hidden[i], (residual[i] if residual is not None else None)

    def _store_last_tokens(self, tokens, batch_slots):
        if self.is_cuda:
            ops.cuda_ops().scatter_tokens(tokens, batch_slots, self.last_tokens)
        else:
            valid = batch_slots >= 0
            self.last_tokens[batch_slots[valid].long()] = tokens[valid]

    def step_shape(self, out) -> tuple:
        """(padded token rows, 1 if the step cannot use a decode graph) of a scheduled step, for the
        data-parallel lockstep agreement."""
        scheds = out.scheduled
        if not scheds:
            return 0, 0
        T = sum(s.num_new_tokens for s in scheds)
        decode_only = all(s.num_new_tokens == 1 and s.start > 0 for s in scheds)
        if decode_only and not self.cfg.enforce_eager and self.is_cuda:
            return pad_to_bucket(len(scheds), self.cfg.request_buckets), 0
        return T, 0 if decode_only else 1

    def logits_rows(self, out) -> int:
        """Rows this step hands to the lm_head before any lockstep padding (for the replicas' agreement when
        the vocabulary is sharded over them)."""
        n = len(out.scheduled)
        if not n:
            return 1                                   # a placeholder step projects one row
        decode_only = all(s.num_new_tokens == 1 and s.start > 0 for s in out.scheduled)
        if decode_only and not self.cfg.enforce_eager and self.is_cuda:
            return pad_to_bucket(n, self.cfg.request_buckets)
        return n

    def execute_dummy_batch(self, T: int) -> None:
        """A step without requests for a replica that must take part in the group's collectives:
        one placeholder request (no KV writes, output ignored) padded to ``T`` rows
        (reference: src/vllm_torchtpu/worker/tpu_worker.py:696-713)."""
        bufs = self.bufs_prefill
        per = max(1, min(T, self.mcfg.max_model_len, self.block_size * self.batch.max_blocks))
        hv = bufs.host_view
        hv("input_ids", T)[:] = 0
        v = hv("positions", T); v[:] = 0; v[:per] = np.arange(per)
        hv("slot_mapping", T)[:] = -1
        hv("token_src", T)[:] = -1
        hv("query_start_loc", 2)[:] = [0, per]
        hv("seq_lens", 1)[:] = per
        hv("logits_indices", 1)[:] = per - 1
        hv("top_k", 1)[:] = 0
        hv("batch_slots", 1)[:] = -1
        hv("temperature", 1, np.float32)[:] = 0
        hv("top_p", 1, np.float32)[:] = 1
        bufs.np_bt[:1] = 0
        hv("num_valid")[0] = 0                     # every row of a placeholder step is padding: no expert work
        bufs.upload(1)
        p = dict(bufs=bufs, n=1, T=per, R_pad=1, T_pad=T, num_decode=0, max_q=per, max_seq=per,
                 seq_lens_np=np.full(1, per, dtype=np.int64), qsl_np=np.array([0, per], dtype=np.int64))
        self._forward_and_sample(bufs, self._make_meta(p), T, 1, True)

    def execute_model(self, out, pad_tokens_to: int = 0) -> StepResult:
        """``pad_tokens_to`` > 0 pads the step to at least that many token rows (data-parallel lockstep);
        a negative value additionally forces the eager path for this step."""
        if not out.scheduled:
            self._update_batch(out)
            return StepResult([], [], None, None, 0)
        self._update_batch(out)
        self._pcp_plan = None
        st_ = get_state()
        if st_.pcp.size > 1:
            # long prefill chunks are cut into pieces and this rank computes two of them (runner/pcp_step.py)
            from types import SimpleNamespace
            from .pcp_step import bind_rows, split_step
            mm = self.mm_manager.items if self.mm_manager is not None else {}
            local, self._pcp_plan = split_step(out.scheduled, st_.pcp.size, st_.pcp.rank_in_group,
                                               envs.B200_PCP_MIN_TOKENS, self.batch.slot_of, self.batch.block_table,
                                               self.block_size, self.device, has_mm=lambda rid: rid in mm)
            if self._pcp_plan is not None:
                if pad_tokens_to:
                    raise RuntimeError("prefill context parallelism and data-parallel lockstep are exclusive")
                out = SimpleNamespace(scheduled=local)
        p = self._prepare_inputs(out, pad_tokens_to=abs(pad_tokens_to))
        if pad_tokens_to < 0:
            p["decode_only"] = False
        bufs, n, R, T = p["bufs"], p["n"], p["R_pad"], p["T_pad"]
        if self._pcp_plan is not None:
            bind_rows(self._pcp_plan, p["scheds"], self.device)
            # a piece that ends no chunk stores no token (its slot belongs to the piece that does)
            bufs.host_view("batch_slots", R)[self._pcp_plan.mute_rows] = -1
            self.stats["pcp_split_steps"] = self.stats.get("pcp_split_steps", 0) + 1
        self.stats["h2d_bytes"] += bufs.upload(R)
        meta = self._make_meta(p)
        meta.pcp = self._pcp_plan
        self._pending_rollback = None
        if p.get("has_spec") and self.mcfg.is_hybrid_gdn:
            # recurrent layers fold all k + 1 rows into their state: keep what it takes to undo rejected ones
            from .spec_boundary_state import StateRollback
            k_, qsl_ = p["spec_k"], p["qsl_np"]
            idx_ = np.nonzero(k_ > 0)[0]
            start_ = qsl_[idx_ + 1] - 1 - k_[idx_]
            rb = StateRollback(idx_, bufs.host_view("batch_slots", n)[idx_], start_, k_[idx_] + 1,
                               bufs.host_view("positions", p["T"])[start_], self.device)
            meta.state_rollback = rb
            self._pending_rollback = (rb, [p["scheds"][int(i)].request.request_id for i in idx_])
        self.stats["steps"] += 1
        ev0 = None
        if self.timing_events is not None and self.is_cuda:
            ev0 = torch.cuda.Event(enable_timing=True)
            ev0.record()
        lora_idx = None
        if getattr(self, "lora_manager", None) is not None:
            names = [s.request.sampling_params.lora_name for s in p["scheds"]]
            lora_idx = self.lora_manager.token_indices(names, [s.num_new_tokens for s in p["scheds"]])
            if lora_idx is not None and lora_idx.numel() < T:
                pad = torch.full((T - lora_idx.numel(),), -1, dtype=lora_idx.dtype, device=lora_idx.device)
                lora_idx = torch.cat([lora_idx, pad])
            from ..lora import wiring
            wiring.set_step(lora_idx)
        self._pool_plan = None
        if any(s.request.sampling_params.pooling for s in p["scheds"]):
            plan, qsl_np = [], p["qsl_np"]
            for i, s in enumerate(p["scheds"]):
                mode = s.request.sampling_params.pooling
                if mode and s.start < s.request.num_prompt_tokens:
                    last = s.start + s.num_new_tokens >= s.request.num_prompt_tokens
                    plan.append((s.request.request_id, int(qsl_np[i]), int(qsl_np[i + 1]), mode, last))
            self._pool_plan = plan or None
        self._step_bitmask = None
        if self.structured is not None and self.structured.grammars:
            bm, rows = self.structured.build_bitmask([s.request.request_id for s in p["scheds"]])
            if bm is not None:
                self._step_bitmask = (bm, rows)
        self._step_extras = self._plan_extras(p)
        self._mm_plan = None
        if self.mm_manager is not None and self.mm_manager.items:
            qsl_np = p["qsl_np"]
            self._mm_plan = [(s.request.request_id, s.start, int(qsl_np[i]), int(qsl_np[i + 1] - qsl_np[i]))
                             for i, s in enumerate(p["scheds"])
                             if s.request.request_id in self.mm_manager.items
                             and s.start < s.request.num_prompt_tokens] or None
        use_graph = (self.is_cuda and p["decode_only"] and not self.cfg.enforce_eager
                     and p["T_pad"] == p["R_pad"] and envs.B200_CUDA_GRAPHS and self._step_bitmask is None and lora_idx is None
                     and self._step_extras is None and not self.keep_hidden and self.dcp_size == 1
                     and getattr(self.model, "dp_vocab", None) is None
                     and get_state().pp.size == 1)          # pipeline stages hand off through host threads
        if use_graph:
            key = (R, p["all_greedy"])
            g = self.graphs.get(key)
            if g is None:
                if envs.B200_CHECK_RECAPTURE and self.graphs:
                    raise RuntimeError(f"decode bucket {key} was not captured at warm-up")
                g = self._capture(key, bufs, meta, T, R, p["all_greedy"])
            g["graph"].replay()
            tokens = g["tokens"]
            self.stats["graph_steps"] += 1
            self.launch_counter += g["launches"]
        else:
            from ..ops import launch_count
            c0 = launch_count()
            tokens, _ = self._forward_and_sample(bufs, meta, T, R, p["all_greedy"],
                                                 L=p["L_pad"] if p.get("has_spec") else None)
            self.launch_counter += launch_count() - c0
            self.stats["eager_steps"] += 1
        if ev0 is not None:
            ev1 = torch.cuda.Event(enable_timing=True)
            ev1.record()
            self.timing_events.append((ev0, ev1, bool(p["decode_only"]), int(p["T"])))   # T = token rows of the step
        host = self.tokens_host[self._tok_ring]
        st_host = self.status_host[self._tok_ring]
        self._tok_ring = (self._tok_ring + 1) % len(self.tokens_host)
        ev = None
        rows = p["L_pad"] if p.get("has_spec") else R
        device_accept = None
        if p.get("has_spec") and self.is_cuda and envs.B200_DEVICE_SPEC_ACCEPT:
            kmax = int(p["spec_k"].max())
            if 0 < kmax <= 7:
                # drafts are judged where the target tokens are: the host reads counts and accepted tokens
                k_dev = self._spec_k_dev[:n]
                k_dev.copy_(torch.from_numpy(np.ascontiguousarray(p["spec_k"], dtype=np.int32)), non_blocking=True)
                acc, cnt = ops.cuda_ops().spec_accept(tokens, bufs.dev_view("input_ids"), meta.query_start_loc, k_dev, n,
                                                      kmax)
                tokens = torch.cat([cnt, acc.flatten()])
                rows = n * (kmax + 2)
                device_accept = kmax
        if self.is_cuda:
            host[:rows].copy_(tokens[:rows], non_blocking=True)
            # the status word of the bounded device waits travels with the tokens: a kernel that gave
            # up turns into an exception when the host reads this step's result
            st_host.copy_(self.status_dev, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        else:
            host[:rows] = tokens[:rows]
            st_host.copy_(self.status_dev)
        self.stats["d2h_bytes"] += rows * 4 + 4
        res = StepResult([s.request.request_id for s in p["scheds"]], [s.samples for s in p["scheds"]],
                         host, ev, n, rows * 4 + 4, status_host=st_host)
        if self.keep_hidden:
            res.hidden, self._last_h = self._last_h, None
        if self.keep_all_hidden:
            res.hidden_all, self._last_h_all = self._last_h_all, None
            n_ = p["n"]
            slots_ = p["bufs"].host_view("batch_slots", n_).copy()
            res.rows = {"qsl": p["qsl_np"][:n_ + 1].copy(), "slots": slots_,
                        "pos0": p["bufs"].host_view("positions", p["T"])[p["qsl_np"][:n_]].copy()}
        if self._step_extras is not None:
            res.lp = self._step_extras["out"]
            self._step_extras = None
        if p.get("has_spec"):
            res.extra = {"spec_k": p["spec_k"], "drafts": [list(s.spec_token_ids) for s in p["scheds"]],
                         "stats": self.stats}
            if device_accept is not None:
                res.extra["device_accept"] = device_accept
        return res

    def note_sampled(self, result: dict) -> None:
        """Host learnt the tokens of a finished step: extend the persistent rows; on a hybrid, rebuild the
        recurrent state of requests that rejected drafts."""
        pend, self._pending_rollback = getattr(self, "_pending_rollback", None), None
        if pend is not None:
            rb, rids = pend
            n_back = rb.rollback([len(result.get(rid) or ()) for rid in rids])
            self.stats["state_rollbacks"] = self.stats.get("state_rollbacks", 0) + n_back
        for rid, toks in result.items():
            slot = self.batch.slot_of.get(rid)
            if slot is not None:
                for t in toks:
                    self.batch.append_token(slot, t)

    # ------------------------------------------------------------ CUDA graphs
    def _capture(self, key, bufs, meta, T, R, all_greedy):
        from ..ops import launch_count
        logger.debug("capturing decode graph for bucket %s", key)
        # warm-up on a side stream so lazy initialisation does not end up in the graph
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._forward_and_sample(bufs, meta, T, R, all_greedy)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        c0 = launch_count()
        with torch.cuda.graph(g, pool=self.graph_pool):
            tokens, _ = self._forward_and_sample(bufs, meta, T, R, all_greedy)
        if self.graph_pool is None:
            self.graph_pool = g.pool()
        entry = {"graph": g, "tokens": tokens, "launches": launch_count() - c0}
        self.graphs[key] = entry
        return entry

    def capture_model(self) -> None:
        """Capture every decode request bucket (greedy variant) ahead of serving."""
        if not (self.is_cuda and envs.B200_CUDA_GRAPHS) or self.cfg.enforce_eager or get_state().pp.size > 1:
            return
        t0 = time.time()
        for R in reversed(self.cfg.request_buckets):
            self._dummy_decode(R, capture=True)
        torch.cuda.synchronize()
        logger.info("captured %d decode graphs in %.1fs", len(self.graphs), time.time() - t0)

    def _dummy_decode(self, R: int, capture: bool = False) -> None:
        bufs = self.bufs_decode
        hv = bufs.host_view
        hv("input_ids", R)[:] = 0
        hv("positions", R)[:] = 0
        hv("slot_mapping", R)[:] = -1
        hv("token_src", R)[:] = -1
        hv("query_start_loc", R + 1)[:] = np.arange(R + 1)
        hv("seq_lens", R)[:] = 1
        hv("logits_indices", R)[:] = np.arange(R)
        hv("top_k", R)[:] = 0
        hv("batch_slots", R)[:] = -1
        hv("temperature", R, np.float32)[:] = 0
        hv("top_p", R, np.float32)[:] = 1
        bufs.np_bt[:R] = 0
        hv("num_valid")[0] = R
        bufs.upload(R)
        p = dict(bufs=bufs, n=R, T=R, R_pad=R, T_pad=R, num_decode=R, max_q=1, max_seq=1,
                 seq_lens_np=np.ones(R, dtype=np.int64), qsl_np=np.arange(R + 1, dtype=np.int64))
        meta = self._make_meta(p)
        if capture:
            self._capture((R, True), bufs, meta, R, R, True)
        else:
            self._forward_and_sample(bufs, meta, R, R, True)

    def _dummy_run(self, T: int, R: int) -> None:
        """Eager full-size prefill-shaped step for memory profiling / warm-up."""
        if not hasattr(self, "bufs_prefill"):
            self._alloc_step_buffers()
        bufs = self.bufs_prefill
        R = max(1, min(R, self.max_reqs))
        per = max(1, T // R)
        per = min(per, self.mcfg.max_model_len)
        T = per * R
        hv = bufs.host_view
        hv("input_ids", T)[:] = 0
        hv("positions", T)[:] = np.tile(np.arange(per), R)
        hv("slot_mapping", T)[:] = -1
        hv("token_src", T)[:] = -1
        qsl = np.arange(R + 1, dtype=np.int64) * per
        hv("query_start_loc", R + 1)[:] = qsl
        hv("seq_lens", R)[:] = per
        hv("logits_indices", R)[:] = qsl[1:] - 1
        hv("top_k", R)[:] = 0
        hv("batch_slots", R)[:] = -1
        hv("temperature", R, np.float32)[:] = 0
        hv("top_p", R, np.float32)[:] = 1
        bufs.np_bt[:R] = 0
        hv("num_valid")[0] = T
        bufs.upload(R)
        p = dict(bufs=bufs, n=R, T=T, R_pad=R, T_pad=T, num_decode=0, max_q=per, max_seq=per,
                 seq_lens_np=np.full(R, per, dtype=np.int64), qsl_np=qsl)
        self._forward_and_sample(bufs, self._make_meta(p), T, R, True)
