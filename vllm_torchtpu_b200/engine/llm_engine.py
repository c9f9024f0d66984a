"""Engine core: scheduler + model runner + the step loop.

One engine drives one model replica (all TP/PP ranks of that replica run this
same loop in lockstep: the scheduler is deterministic, so every rank derives
the same SchedulerOutput from the same request stream).  Offline, every rank is
handed the same prompts.  Behind a server only the replica's first rank sees
HTTP requests: it broadcasts, once per step, the requests added and aborted since
the previous step, and the other ranks follow (``enable_request_sync`` /
``follow``); this plays the part of the reference's executor, which broadcasts
every scheduler output to its workers
(reference: src/vllm_torchtpu/executors/tpu_multiproc_executor.py:29-61).
With async scheduling the loop keeps one step in flight: step n+1 is scheduled
and launched while step n's tokens travel back to the host.
"""
from __future__ import annotations

import time
from collections import deque
from typing import Optional

import torch

from .. import envs
from ..config import EngineConfig
from ..logger import init_logger
from ..parallel.state import get_state, init_distributed
from ..platform import B200Platform
from ..runner.model_runner import ModelRunner
from ..sampling_params import SamplingParams
from .request import Request
from .scheduler import Scheduler

logger = init_logger(__name__)


class ReplicaRequestSync:
    """Request stream of one replica, leader to followers: one object broadcast on the CPU (gloo)
    group per engine step carrying the operations to apply before that step."""

    def __init__(self, group):
        self.group = group
        self.is_leader = group.rank_in_group == 0
        self.pending: list = []
        self.stopped = False
        self.last_exchange = time.monotonic()

    def exchange(self, step: bool, stop: bool = False) -> dict:
        import torch.distributed as dist
        box = [None]
        if self.is_leader:
            box[0] = {"ops": self.pending, "step": step, "stop": stop}
            self.pending = []
        dist.broadcast_object_list(box, src=self.group.ranks[0], group=self.group.cpu_group)
        self.last_exchange = time.monotonic()
        return box[0]


def make_scheduler(cfg: EngineConfig, num_blocks: int, connector=None, num_spec_tokens: int = 0):
    name = cfg.scheduler.scheduler_cls
    kw = dict(connector=connector, num_spec_tokens=num_spec_tokens,
              sliding_window=cfg.model.sliding_window,
              abort_on_preemption=bool(cfg.additional.get("abort_on_preemption",
                                                          envs.B200_ABORT_ON_PREEMPTION)))
    if name == "default":
        return Scheduler(cfg.scheduler, cfg.cache, num_blocks, **kw)
    from ..schedulers import get_scheduler_class
    return get_scheduler_class(name)(cfg.scheduler, cfg.cache, num_blocks, **kw)


class LLMEngine:
    def __init__(self, cfg: EngineConfig, *, init_dist: bool = True):
        self.cfg = cfg.finalize() if not cfg.token_buckets else cfg
        if init_dist:
            init_distributed(cfg.parallel, backend=None if cfg.device == "cuda" else "gloo")
        st = get_state()
        dev = cfg.device
        if dev == "cuda":
            dev = f"cuda:{st.local_rank}"
            torch.cuda.set_device(st.local_rank)
        self.runner = ModelRunner(self.cfg, dev)
        self.runner.load_model()
        if cfg.speculative:
            from ..spec_decode import DRAFT_LAYER_METHODS
            if cfg.speculative.get("method") in DRAFT_LAYER_METHODS:
                self.runner.extra_kv_layers = int(cfg.speculative.get("num_hidden_layers", 1)) \
                    if cfg.speculative.get("method") in ("dflash", "dspark") else 1        # the draft layer's KV tensor counts in the HBM budget
        num_blocks = self.runner.determine_num_blocks()
        if st.world_size > 1 and st.world.cpu_group is not None:
            # the ranks of a pipeline stage must agree within a tolerance; everyone adopts the minimum
            from .kv_block_agreement import agree_over_group
            num_blocks = agree_over_group(num_blocks, st.rank, st.pp.rank_in_group, st.world.cpu_group)
        self.runner.init_kv_cache(num_blocks)
        # the scheduler counts its own (possibly larger) blocks: each owns m consecutive kernel blocks
        num_blocks //= cfg.cache.kernel_blocks_per_block
        self.connector = None
        if cfg.kv_transfer:
            from ..kv_transfer.factory import create_connector
            self.connector = create_connector(cfg, self.runner)
        self.spec = None
        num_spec = 0
        if cfg.speculative:
            from ..spec_decode import create_proposer
            self.spec = create_proposer(cfg, self.runner)
            num_spec = self.spec.num_speculative_tokens
        self.adaptive = None
        if cfg.speculative and cfg.speculative.get("enable_adaptive_verification"):
            from ..spec_decode.adaptive_verification import (AdaptiveVerificationManager, StepCostTable,
                                                             validate_adaptive_verification_config)
            validate_adaptive_verification_config(cfg)
            samples = cfg.speculative.get("step_cost_samples") or self._profile_step_costs()
            self.adaptive = AdaptiveVerificationManager(StepCostTable(samples), num_spec)
        self.scheduler = make_scheduler(self.cfg, num_blocks,
                                        self.connector.scheduler if self.connector else None, num_spec)
        if self.connector is not None and getattr(self.connector, "controller", None) is not None:
            sch = self.scheduler
            self.connector.load_fn = lambda: {"running": len(sch.running), "waiting": len(sch.waiting),
                                              "free_blocks": sch.kv.pool.num_free_blocks}
        if self.spec is not None and num_spec:
            self.scheduler.lookahead_extra = int(getattr(self.spec, "extra_lookahead", 0))
        self.runner.capture_model()
        # Data-parallel replicas coupled by expert parallelism run their steps in lockstep: the MoE
        # collectives of a step need every rank, with equal padded row counts on the gather plane
        # (reference: src/vllm_torchtpu/runner/tpu_runner.py:4132-4180, worker/tpu_worker.py:696-713).
        self._dp_lockstep = st.dp.size > 1 and st.expert_parallel
        self._dp_group_busy = True
        self._inflight: deque = deque()
        self._next_id = 0
        self.eos_token_id: Optional[int] = None
        self.step_count = 0
        self._sync: Optional[ReplicaRequestSync] = None
        self._applying = False

    # ---- request stream of a multi-rank replica behind a server ---------------------------------
    def enable_request_sync(self) -> bool:
        """Call on every rank before serving.  From then on requests are given to the first rank only
        (``add_request`` / ``abort_request`` / the LoRA calls queue there) and reach the other ranks,
        which run ``follow()``, with the next step."""
        st = get_state()
        if st.world_size == 1:
            return False
        if st.dp.size > 1:
            raise NotImplementedError("one server per data-parallel replica: request sync covers TP x PP ranks")
        self._sync = ReplicaRequestSync(st.world)
        return True

    def _queue_op(self, op: tuple) -> bool:
        if self._sync is not None and self._sync.is_leader and not self._applying:
            self._sync.pending.append(op)
            return True
        return False

    def _sync_point(self, step: bool, stop: bool = False) -> dict:
        msg = self._sync.exchange(step, stop)
        self._applying = True
        try:
            for op in msg["ops"]:
                kind = op[0]
                try:
                    if kind == "add":
                        self.add_request(*op[1], **op[2])
                    elif kind == "abort":
                        self.abort_request(op[1])
                    elif kind == "call":
                        getattr(self, op[1])(*op[2])
                except Exception as e:      # noqa: BLE001 - the leader validated the same operation
                    logger.error("request operation %s failed on rank %d: %r", kind, get_state().rank, e)
        finally:
            self._applying = False
        return msg

    def idle_tick(self, every_s: float = 2.0) -> None:
        """Leader, while idle: keep the followers' blocking receive from timing out."""
        if self._sync is not None and self._sync.is_leader and not self._sync.stopped and \
                time.monotonic() - self._sync.last_exchange > every_s:
            self._sync_point(step=False)

    def stop_followers(self) -> None:
        if self._sync is not None and self._sync.is_leader and not self._sync.stopped:
            self._sync.stopped = True
            self._sync_point(step=False, stop=True)

    def follow(self) -> None:
        """Ranks other than the replica's first: apply what the leader broadcasts and step with it."""
        assert self._sync is not None and not self._sync.is_leader
        while True:
            msg = self._sync_point(step=False)
            if msg["stop"]:
                return
            if msg["step"]:
                self._step_inner()

    # ---- requests ---------------------------------------------------------------
    def add_request(self, prompt_token_ids: list, sampling_params: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, kv_transfer_params: Optional[dict] = None,
                    mm_items: Optional[list] = None, priority: int = 0) -> str:
        """``mm_items``: [(patches [num_patches, patch_dim], prompt_offset), ...] — images or video chunks
        whose embeddings replace the placeholder tokens starting at ``prompt_offset`` (needs
        ``enable_vision`` first)."""
        sp = sampling_params or SamplingParams()
        B200Platform.validate_request(sp)
        if len(prompt_token_ids) + sp.max_tokens > self.cfg.model.max_model_len:
            raise ValueError(f"prompt ({len(prompt_token_ids)}) + max_tokens ({sp.max_tokens}) exceeds "
                             f"max_model_len ({self.cfg.model.max_model_len})")
        if not prompt_token_ids:
            raise ValueError("empty prompt")
        sp.verify()
        if sp.prompt_logprobs is not None and getattr(self.runner.model, "dp_vocab", None) is not None:
            raise ValueError("prompt_logprobs are not available with dp_vocab_parallel (the lm_head exchange runs "
                             "once per step on every replica)")
        if sp.has_logit_adjust and (self.cfg.speculative or self.cfg.parallel.pipeline_parallel_size > 1):
            # verification rows and pipeline stages sample without the per-step logit edits
            raise ValueError("penalties, logit_bias, allowed_token_ids and min_p are not supported together with "
                             "speculative decoding or pipeline parallelism")
        rid = request_id or f"req-{self._next_id}"
        self._next_id += 1
        if self._queue_op(("add", (list(prompt_token_ids), sp), dict(request_id=rid, mm_items=mm_items,
                                                                      kv_transfer_params=kv_transfer_params,
                                                                      priority=priority))):
            return rid          # applied on every rank, this one included, at the next step
        if sp.structured:
            if self.runner.structured is None:
                from ..structured import StructuredDecodingManager
                self.runner.structured = StructuredDecodingManager(self.cfg.model.vocab_size,
                                                                   getattr(self, "vocab_strings", None),
                                                                   self.eos_token_id)
            self.runner.structured.add_request(rid, sp.structured)
        if mm_items:
            if self.runner.mm_manager is None:
                raise ValueError("multimodal items need a vision encoder: call enable_vision first")
            from ..runner.mm_encoder import MMItem
            items = [MMItem(rid, i, p, int(off)) for i, (p, off) in enumerate(mm_items)]
            self.runner.mm_manager.add_request(rid, items)
            for it in items:
                if it.prompt_offset + it.num_tokens > len(prompt_token_ids):
                    self.runner.mm_manager.remove_request(rid)
                    raise ValueError("a multimodal item's placeholder range runs past the prompt")
        self.scheduler.add_request(Request(rid, list(prompt_token_ids), sp, self.eos_token_id,
                                           kv_transfer_params=kv_transfer_params, priority=int(priority)))
        return rid

    def enable_vision(self, vision_cfg, max_patches_per_batch: int = 8192):
        """Attach a vision encoder whose output width is the model's hidden size.  Prefix caching is
        keyed by token ids only, so requests with multimodal items must not share cached blocks."""
        from ..layers.vision import VisionEncoder
        from ..runner.mm_encoder import MMEncoderManager
        if vision_cfg.out_hidden_size != self.cfg.model.hidden_size:
            raise ValueError("vision out_hidden_size must equal the model's hidden size")
        if self.cfg.cache.enable_prefix_caching:
            raise ValueError("multimodal requests need enable_prefix_caching=False")
        enc = VisionEncoder(vision_cfg, self.runner.device)
        self.runner.mm_manager = MMEncoderManager(enc, max_patches_per_batch)
        return self.runner.mm_manager

    # ---- LoRA adapters (reference: src/vllm_torchtpu/worker/tpu_worker.py:898-908) -----------------
    def _lora(self):
        if getattr(self, "lora_manager", None) is None:
            from ..lora import LoRAManager, wiring
            add = self.cfg.additional or {}
            self.lora_manager = LoRAManager(int(add.get("max_loras", 4)), int(add.get("max_lora_rank", 64)),
                                            dtype=self.cfg.model.dtype, device=self.runner.device)
            wiring.attach(self.runner.model, self.lora_manager)
            self.runner.lora_manager = self.lora_manager
        return self.lora_manager

    # ---- weights and kernels at run time -------------------------------------------------------------
    def update_weights(self, named_tensors) -> int:
        """Replace model weights in place from checkpoint-named tensors (a dict or an iterable of
        (name, tensor) in Hugging Face layout, unsharded: every rank takes its shard), e.g. after a
        trainer's optimizer step.  Partial updates are allowed as long as fused parameters come complete
        (q, k and v together; gate and up together).  Cached prefixes are dropped: they were computed with
        the old weights.  Call between steps, with no request in flight.
        (reference: src/vllm_torchtpu/worker/tpu_worker.py sync_weights)"""
        if self.scheduler.has_unfinished() or self._inflight:
            raise RuntimeError("update_weights needs an idle engine")
        items = list(named_tensors.items()) if isinstance(named_tensors, dict) else list(named_tensors)
        from ..models.loader import load_named_tensors
        load_named_tensors(self.runner.model, iter(items), {n for n, _ in items}, source="update_weights")
        if getattr(self.runner.model, "dp_vocab", None) is not None:
            self.runner.model.enable_dp_vocab(self.runner.model.dp_vocab)      # a replaced table is sharded again
        self.scheduler.kv.pool.reset_prefix_cache()
        mega = getattr(self.runner.model, "decode_mega", None)
        if mega is not None:
            self.runner.model.setup_decode_fusion(self.runner)      # descriptors point at the old tensors
        if self.runner.graphs:
            # captured graphs hold the addresses of the replaced tensors
            self.runner.graphs.clear()
            self.runner.capture_model()
        return len(items)

    def reload_kernels(self, path: Optional[str] = None) -> str:
        """Load the kernel library again (after a rebuild, or from ``path``) and re-capture the decode graphs:
        kernels can be iterated on without restarting the server.
        (reference: src/vllm_torchtpu/worker/tpu_worker.py:862 reload_kernels)"""
        if self.scheduler.has_unfinished() or self._inflight:
            raise RuntimeError("reload_kernels needs an idle engine")
        from ..ops import cuda
        loaded = cuda.reload_lib(path)
        if self.runner.graphs:
            self.runner.graphs.clear()
            self.runner.capture_model()
        return loaded

    def add_lora(self, name: str, rank: int, alpha: float, weights: dict) -> bool:
        """weights: {"model.layers.N.self_attn.q_proj": (A [r, in], B [out, r]), ...}."""
        from ..lora import LoRAAdapter
        if self._queue_op(("call", "add_lora", (name, rank, alpha, weights))):
            return True
        return self._lora().add_adapter(LoRAAdapter(name, rank, alpha, weights))

    def remove_lora(self, name: str) -> bool:
        if self._queue_op(("call", "remove_lora", (name,))):
            return True
        return self._lora().remove_adapter(name)

    def pin_lora(self, name: str) -> bool:
        if self._queue_op(("call", "pin_lora", (name,))):
            return True
        return self._lora().pin_adapter(name)

    def list_loras(self) -> list:
        return self._lora().list_adapters()

    def _profile_step_costs(self) -> list:
        """(rows, ms) of placeholder steps of a few sizes, for the adaptive verification cost table."""
        import time
        import torch
        out = []
        cap = max(8, min(self.cfg.scheduler.max_num_batched_tokens, 512))
        for rows in sorted({8, 32, 64, 128, 256, cap}):
            if rows > cap:
                continue
            times = []
            for _ in range(3):
                if self.runner.is_cuda:
                    torch.cuda.synchronize()
                t0 = time.perf_counter()
                self.runner.execute_dummy_batch(rows)
                if self.runner.is_cuda:
                    torch.cuda.synchronize()
                times.append((time.perf_counter() - t0) * 1e3)
            out.append((rows, sorted(times)[1]))
        return out

    def abort_request(self, request_id: str) -> None:
        if self._queue_op(("abort", request_id)):
            return
        self.scheduler.abort_request(request_id)

    def has_unfinished(self) -> bool:
        if self._sync is not None and self._sync.pending:
            return True
        if self._dp_lockstep:
            # Replicas coupled by expert parallelism must call step() the same number of times (every
            # step holds a host all-reduce and the MoE collectives), so the loop condition is the flag
            # they agreed on in the last step; a replica without requests keeps stepping (placeholder
            # batches) while any other has work.  Launches left in flight when the group goes idle hold
            # no requests; drain() retires them without a collective.
            return self._dp_group_busy or self.scheduler.has_unfinished()
        return self.scheduler.has_unfinished() or bool(self._inflight)

    # ---- stepping ---------------------------------------------------------------
    def _launch(self):
        out = self.scheduler.schedule()
        pad_to = 0
        if self._dp_lockstep:
            from ..parallel.communicator import DeviceCommunicator
            st = get_state()
            t_pad, eager = self.runner.step_shape(out)
            busy = 1 if (out.scheduled or self.scheduler.has_unfinished()
                         or any(o.scheduled for o, _ in self._inflight)) else 0
            throttled = hasattr(self.scheduler, "throttle_prefills")
            pending = self.scheduler.pending_prefill_tokens() if throttled else 0
            dpv = getattr(self.runner.model, "dp_vocab", None)
            rows = self.runner.logits_rows(out) if dpv is not None else 0
            agreed = DeviceCommunicator(st.dp, None).cpu_all_reduce_max([t_pad, eager, busy, pending, rows])
            if dpv is not None:
                # every replica pads its lm_head rows to one count that follows from the agreed values alone: a
                # decode step padded up to an agreed request bucket projects that many rows
                dpv.rows = max(agreed[4], agreed[0] if agreed[0] in self.cfg.request_buckets else 0)
            self._dp_group_busy = bool(agreed[2])
            if throttled:
                # replicas admit prefills in the same steps, so that one replica's long prefill does
                # not stretch the decode steps of the others more often than necessary
                # (reference: src/vllm_torchtpu/core/tpu_scheduler.py:22-57)
                self.scheduler.throttle_prefills([agreed[3]])
            if not self._dp_group_busy:
                return out, self.runner.execute_model(out)           # nothing anywhere: empty result
            if not out.scheduled:
                self.runner.execute_dummy_batch(max(1, agreed[0]))
                return out, self.runner.execute_model(out)
            pad_to = agreed[0]
            if agreed[1]:
                pad_to = -agreed[0]           # some replica runs a prefill: everybody runs this step eagerly
        if self.connector is not None:
            self.connector.worker.start_load_kv(out.kv_connector_metadata)
        res = self.runner.execute_model(out, pad_tokens_to=pad_to)
        if self.connector is not None:
            self.connector.worker.save_kv(out.kv_connector_metadata)
        return out, res

    def _retire(self, out, res) -> list:
        try:
            sampled = res.get()
        except Exception as e:          # noqa: BLE001 - a device wait timed out: fail this step's requests
            from ..runner.model_runner import DeviceWaitTimeout
            if not isinstance(e, DeviceWaitTimeout) or get_state().world_size > 1:
                # with several ranks the failure is not symmetric (one rank's wait gave up): failing
                # requests locally would let the ranks' schedules diverge, so the process ends and the
                # launcher takes the group down
                raise
            return self._fail_step(out, e)
        self.runner.note_sampled(sampled)
        if self.runner.structured is not None:
            self.runner.structured.accept_tokens(sampled)
        spec_next = None
        if self.spec is not None and sampled:
            if hasattr(self.spec, "note_step"):
                self.spec.note_step(out, res, sampled)
            spec_next = self.spec.propose(out, sampled)
            if self.adaptive is not None and spec_next:
                # verify only the draft prefixes that are worth their rows in the next step
                spec_next = self.adaptive.trim(spec_next, getattr(self.spec, "last_confidences", {}),
                                               base_rows=len(self.scheduler.running))
        sample_lp, prompt_lp = res.take_logprobs()
        if prompt_lp:
            by_id = {s.request.request_id: s.request for s in out.scheduled}
            for rid, ents in prompt_lp.items():
                req = by_id.get(rid)
                if req is not None:
                    if not req.prompt_logprobs:
                        req.prompt_logprobs = [None]          # the first prompt token has no prefix
                    req.prompt_logprobs.extend(ents)
        finished = self.scheduler.update_from_output(out, sampled, spec_next, logprobs=sample_lp)
        for r in finished:
            if r.sampling_params.pooling:
                r.pooled = self.runner.take_pooled(r.request_id)
            if self.runner.mm_manager is not None:
                self.runner.mm_manager.remove_request(r.request_id)
        if self.runner.structured is not None:
            for r in finished:
                self.runner.structured.remove_request(r.request_id)
        if self.connector is not None:
            if finished:
                # requests that just finished may have blocks to publish or store: do it now rather
                # than at the next schedule(), which may never come
                self.connector.worker.save_kv(self.connector.scheduler.build_connector_meta(None))
            for rid in self.connector.worker.get_finished_sending():
                self.scheduler.free_delayed(rid)
        return finished

    def _fail_step(self, out, err) -> list:
        """The device reported that a bounded wait gave up during this step: its requests end with an
        error (their KV content is not trustworthy), the status word is cleared and serving continues
        (reference: src/vllm_torchtpu/distributed/pp_buffered.py:354-369 — helper-thread errors are
        re-raised on the worker; here the failing unit is the step)."""
        from ..engine.request import RequestStatus
        logger.error("step failed: %s", err)
        self.runner.status_dev.zero_()
        mega = getattr(self.runner.model, "decode_mega", None)
        if mega is not None:
            mega.reset()                 # the persistent kernel left its barrier words mid-step
        self.device_errors = getattr(self, "device_errors", 0) + 1
        failed = []
        for s in out.scheduled:
            req = s.request
            if req.status.finished:
                continue
            req.error = f"device_wait_timeout: {err}"
            self.scheduler._finish(req, RequestStatus.FINISHED_ERROR)
            failed.append(req)
        self.runner.note_sampled({})
        return failed

    def step(self) -> list:
        """Advance the engine; returns requests that finished."""
        if self._sync is not None:
            self._sync_point(step=True)
        return self._step_inner()

    def _step_inner(self) -> list:
        self.step_count += 1
        if not self.scheduler.async_mode:
            out, res = self._launch()
            return self._retire(out, res)
        finished = []
        if self._dp_lockstep:
            # one launch (and one agreement) per step on every replica; all but the newest launch are
            # retired, and a launch without requests right away
            self._inflight.append(self._launch())
            while len(self._inflight) > 1:
                finished += self._retire(*self._inflight.popleft())
            if self._inflight and not self._inflight[-1][0].scheduled:
                finished += self._retire(*self._inflight.popleft())
            return finished
        if self.scheduler.has_unfinished():
            self._inflight.append(self._launch())
        if len(self._inflight) > 1 or (self._inflight and not self.scheduler.has_unfinished()):
            out, res = self._inflight.popleft()
            finished = self._retire(out, res)
        elif self._inflight and not self._inflight[-1][0].scheduled:
            out, res = self._inflight.popleft()
            finished = self._retire(out, res)
        return finished

    def drain(self) -> list:
        finished = []
        while self._inflight:
            out, res = self._inflight.popleft()
            finished += self._retire(out, res)
        return finished

    def run_until_done(self) -> list:
        done = []
        idle = 0
        if self._dp_lockstep:
            self._dp_group_busy = True          # step at least once: another replica may have requests
        while self.has_unfinished():
            f = self.step()
            done += f
            idle = 0 if f or self._inflight else idle + 1
            if idle > 10000:
                raise RuntimeError("engine made no progress for 10000 steps")
        return done
