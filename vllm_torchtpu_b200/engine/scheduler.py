"""Continuous-batching scheduler with chunked prefill, prefix caching,
preemption, speculative tokens, KV-connector hooks and one-step-ahead (async)
scheduling.

Each ``schedule()`` hands every running request the tokens it still has to
compute (one for a decoding request, a chunk for a prefilling one) inside a
token budget, then admits waiting requests.  ``num_computed_tokens`` is
advanced at schedule time, so the next step can be scheduled before the device
has produced this step's tokens; the not-yet-known tokens are counted as
placeholders.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Optional

from ..logger import init_logger
from .block_manager import KVCacheManager
from .request import Request, RequestStatus

logger = init_logger(__name__)


@dataclass
class ScheduledRequest:
    request: Request
    num_new_tokens: int
    start: int                      # num_computed_tokens before this step
    is_new: bool = False            # first time in the runner's persistent batch (or resumed)
    samples: bool = True            # produces a token this step
    num_spec_tokens: int = 0
    new_block_ids: list = field(default_factory=list)
    spec_token_ids: list = field(default_factory=list)


@dataclass
class SchedulerOutput:
    step_id: int
    scheduled: list
    finished_ids: list
    preempted_ids: list
    total_num_tokens: int
    kv_connector_metadata: object = None

    @property
    def num_reqs(self) -> int:
        return len(self.scheduled)

    @property
    def is_decode_only(self) -> bool:
        return all(s.num_new_tokens == 1 and s.start > 0 for s in self.scheduled)


class Scheduler:
    def __init__(self, scheduler_config, cache_config, num_blocks: int, *, connector=None,
                 num_spec_tokens: int = 0, sliding_window=None, abort_on_preemption: bool = False):
        self.cfg = scheduler_config
        tokens_per_block = getattr(cache_config, "tokens_per_block", 0) or cache_config.block_size
        self.kv = KVCacheManager(num_blocks, tokens_per_block, cache_config.enable_prefix_caching, sliding_window)
        self.block_size = tokens_per_block
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.requests: dict[str, Request] = {}
        self.finished_since_last: list[str] = []
        self.connector = connector
        self.num_spec_tokens = num_spec_tokens
        self.lookahead_extra = 0            # slots a drafter writes beyond the verification rows
        self.abort_on_preemption = abort_on_preemption
        self.step_id = 0
        self.async_mode = scheduler_config.async_scheduling
        self.stats = {"preemptions": 0, "prefix_hit_tokens": 0, "prefix_query_tokens": 0, "scheduled_tokens": 0}
        self._in_batch: set[str] = set()
        self._delayed_blocks: dict = {}

    # ---- admission ---------------------------------------------------------
    def add_request(self, req: Request) -> None:
        if req.request_id in self.requests:
            raise ValueError(f"duplicate request id {req.request_id}")
        req.sampling_params.verify()
        self.requests[req.request_id] = req
        self.waiting.append(req)

    def abort_request(self, request_id: str) -> None:
        req = self.requests.get(request_id)
        if req is None or req.status.finished:
            return
        self._finish(req, RequestStatus.FINISHED_ABORTED)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    @property
    def num_unfinished(self) -> int:
        return len(self.waiting) + len(self.running)

    # ---- policy hooks (subclasses override) --------------------------------
    def _select_waiting(self) -> Optional[Request]:
        """Next waiting request to try; default FCFS."""
        return self.waiting[0] if self.waiting else None

    def _may_admit_prefill(self, req: Request, budget: int) -> bool:
        return True

    # ---- main ---------------------------------------------------------------
    def schedule(self) -> SchedulerOutput:
        budget = self.cfg.max_num_batched_tokens
        scheduled: list[ScheduledRequest] = []
        preempted: list[str] = []
        threshold = self.cfg.long_prefill_token_threshold

        # 1. running requests
        i = 0
        while i < len(self.running) and budget > 0:
            req = self.running[i]
            want = (req.num_tokens_with_placeholders + len(req.spec_token_ids)
                    - req.num_computed_tokens)
            if want <= 0 or (req.num_output_placeholders and len(req.output_token_ids)
                             + req.num_output_placeholders >= req.sampling_params.max_tokens):
                i += 1                  # its last token is still in flight
                continue
            n = min(want, budget)
            if threshold and n > threshold:
                n = threshold
            if not self.cfg.enable_chunked_prefill and n < want:
                i += 1
                continue
            new_blocks = None
            while True:
                new_blocks = self.kv.allocate_slots(req, n, lookahead=self.num_spec_tokens + self.lookahead_extra)
                if new_blocks is not None:
                    break
                victim = self._pick_victim(req)
                if victim is None:
                    break
                self._preempt(victim)
                preempted.append(victim.request_id)
                if victim is req:
                    break
                scheduled = [s for s in scheduled if s.request is not victim]
            if new_blocks is None or req.status is not RequestStatus.RUNNING:
                if req.status is RequestStatus.RUNNING:
                    i += 1
                continue
            scheduled.append(self._make_sched(req, n, new_blocks))
            budget -= n
            i += 1

        # 2. waiting requests
        if not preempted:
            skipped: list[Request] = []
            while self.waiting and budget > 0 and len(self.running) < self.cfg.max_num_seqs:
                req = self._select_waiting()
                if req is None:
                    break
                if req.status is RequestStatus.WAITING_FOR_REMOTE_KVS:
                    if self.connector is not None and self.connector.is_load_done(req):
                        req.status = RequestStatus.WAITING
                    else:
                        self.waiting.remove(req)
                        skipped.append(req)
                        continue
                if not self._may_admit_prefill(req, budget):
                    break
                cached_blocks, num_cached = ([], 0)
                if req.num_computed_tokens == 0 and not req.block_ids:
                    cached_blocks, num_cached = self.kv.get_computed_blocks(req)
                    ext = 0
                    load_async = False
                    if self.connector is not None:
                        ext, load_async = self.connector.get_num_new_matched_tokens(req, num_cached)
                    req.num_computed_tokens = num_cached
                    if ext > 0:
                        blocks = self.kv.allocate_slots(req, ext, cached_blocks)
                        if blocks is None:
                            req.num_computed_tokens = 0
                            self.connector.request_not_admitted(req)
                            break
                        self.connector.update_state_after_alloc(req, req.block_ids, ext)
                        req.num_computed_tokens = num_cached + ext
                        cached_blocks = []
                        if load_async:
                            req.status = RequestStatus.WAITING_FOR_REMOTE_KVS
                            self.waiting.remove(req)
                            skipped.append(req)
                            continue
                want = req.num_tokens - req.num_computed_tokens
                if want <= 0:
                    # whole prompt came from the connector: recompute the last token for logits
                    req.num_computed_tokens = req.num_tokens - 1
                    want = 1
                n = min(want, budget)
                if threshold and n > threshold:
                    n = threshold
                if n < want and not self.cfg.enable_chunked_prefill:
                    break
                new_blocks = self.kv.allocate_slots(req, n, cached_blocks or None,
                                                    lookahead=self.num_spec_tokens + self.lookahead_extra)
                if new_blocks is None:
                    if not req.block_ids:
                        req.num_computed_tokens = 0
                    break
                self.waiting.remove(req)
                req.num_cached_tokens = max(req.num_cached_tokens, req.num_computed_tokens)
                self.stats["prefix_hit_tokens"] += num_cached
                if req.scheduled_time is None:
                    req.scheduled_time = time.monotonic()
                    self.stats["prefix_query_tokens"] += req.num_prompt_tokens
                req.status = RequestStatus.RUNNING
                self.running.append(req)
                scheduled.append(self._make_sched(req, n, list(req.block_ids)))
                budget -= n
            for r in reversed(skipped):
                self.waiting.appendleft(r)

        total = sum(s.num_new_tokens for s in scheduled)
        self.stats["scheduled_tokens"] += total
        out = SchedulerOutput(self.step_id, scheduled, self.finished_since_last, preempted, total)
        self.finished_since_last = []
        self.step_id += 1
        if self.connector is not None:
            out.kv_connector_metadata = self.connector.build_connector_meta(out)
        self._update_after_schedule(out)
        return out

    def _make_sched(self, req: Request, n: int, new_blocks: list) -> ScheduledRequest:
        start = req.num_computed_tokens
        end = start + n
        n_spec = 0
        if req.spec_token_ids and end > req.num_tokens_with_placeholders:
            n_spec = end - req.num_tokens_with_placeholders
        samples = end >= req.num_tokens_with_placeholders
        is_new = req.request_id not in self._in_batch
        self._in_batch.add(req.request_id)
        return ScheduledRequest(req, n, start, is_new, samples, n_spec, new_blocks,
                                list(req.spec_token_ids[:n_spec]))

    def _update_after_schedule(self, out: SchedulerOutput) -> None:
        for s in out.scheduled:
            req = s.request
            req.num_computed_tokens = s.start + s.num_new_tokens
            if self.async_mode and s.samples:
                req.num_output_placeholders += 1
            if s.num_spec_tokens:
                req.spec_token_ids = []

    # ---- preemption ----------------------------------------------------------
    def _pick_victim(self, needy: Request) -> Optional[Request]:
        if not self.running:
            return None
        victim = max(self.running, key=lambda r: (r.priority, r.arrival_time))
        return victim

    def _preempt(self, req: Request) -> None:
        self.stats["preemptions"] += 1
        self.running.remove(req)
        self.kv.free(req)
        self._in_batch.discard(req.request_id)
        if self.abort_on_preemption:
            # decode-side capacity preemption is a terminal, client-visible error
            # (reference: src/vllm_torchtpu/core/abort_on_preemption.py:14-27)
            req.error = "kv_cache_preempted"
            req.status = RequestStatus.FINISHED_ERROR
            req.finish_time = time.monotonic()
            self.finished_since_last.append(req.request_id)
            return
        req.status = RequestStatus.PREEMPTED
        req.num_computed_tokens = 0
        req.num_output_placeholders = 0
        req.spec_token_ids = []
        req.num_preemptions += 1
        req.status = RequestStatus.WAITING
        self.waiting.appendleft(req)

    # ---- results ---------------------------------------------------------------
    def update_from_output(self, out: SchedulerOutput, sampled: dict, spec_next: Optional[dict] = None,
                           logprobs: Optional[dict] = None) -> list[Request]:
        """``sampled[request_id]`` = list of accepted new tokens for that request
        (length 1 normally, up to k+1 after speculative verification)."""
        finished = []
        for s in out.scheduled:
            req = s.request
            if req.status.finished:
                continue
            if req.status is not RequestStatus.RUNNING:
                continue            # preempted after it was scheduled
            toks = sampled.get(req.request_id)
            if self.async_mode and s.samples:
                req.num_output_placeholders = max(0, req.num_output_placeholders - 1)
            if s.samples and toks:
                if s.num_spec_tokens:
                    rejected = s.num_spec_tokens + 1 - len(toks)
                    req.num_computed_tokens -= rejected
                now = time.monotonic()
                for t in toks:
                    req.output_token_ids.append(int(t))
                    if req.first_token_time is None:
                        req.first_token_time = now
                    if logprobs and req.request_id in logprobs:
                        req.logprobs.append(logprobs[req.request_id])
                    if req.check_stop():
                        break
            self.kv.cache_blocks(req, min(req.num_computed_tokens, req.num_tokens))
            if req.status.finished:
                self._finish(req, req.status)
                finished.append(req)
            elif spec_next and req.request_id in spec_next:
                req.spec_token_ids = list(spec_next[req.request_id])
        return finished

    def _finish(self, req: Request, status: RequestStatus) -> None:
        req.status = status
        req.finish_time = time.monotonic()
        if req in self.running:
            self.running.remove(req)
        elif req in self.waiting:
            self.waiting.remove(req)
        delay_free = False
        if self.connector is not None:
            delay_free, params = self.connector.request_finished(req, req.block_ids)
            if params:
                req.kv_transfer_params = params
        if not delay_free:
            self.kv.free(req)
        else:
            # the connector still needs the blocks; they are released by free_delayed()
            self._delayed_blocks[req.request_id] = req.block_ids
            req.block_ids = []
        self._in_batch.discard(req.request_id)
        self.finished_since_last.append(req.request_id)

    def free_delayed(self, request_id: str) -> None:
        """Called when a connector has finished sending a finished request's blocks."""
        blocks = self._delayed_blocks.pop(request_id, None)
        if blocks:
            self.kv.pool.release(blocks)
