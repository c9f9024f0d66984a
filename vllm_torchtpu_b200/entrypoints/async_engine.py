"""Asynchronous front of the engine: a background thread runs the step loop, callers
submit requests and await token streams.  The serving API and the proxy use it."""
from __future__ import annotations

import asyncio
import queue
import threading
import time
from dataclasses import dataclass
from typing import AsyncIterator, Optional

from ..engine.llm_engine import LLMEngine
from ..logger import init_logger
from ..sampling_params import SamplingParams

logger = init_logger(__name__)


@dataclass
class StreamItem:
    request_id: str
    new_token_ids: list
    finished: bool
    finish_reason: Optional[str] = None
    kv_transfer_params: Optional[dict] = None
    error: Optional[str] = None
    num_prompt_tokens: int = 0
    num_cached_tokens: int = 0
    logprobs: Optional[list] = None          # entries of new_token_ids when the request asked for them
    prompt_logprobs: Optional[list] = None   # with the final item
    pooled: Optional[list] = None            # embedding of a pooling request, with the final item


def _settle(fut, res, exc) -> None:
    if fut.cancelled():
        return
    if exc is not None:
        fut.set_exception(exc)
    else:
        fut.set_result(res)


class AsyncEngine:
    def __init__(self, engine: LLMEngine):
        self.engine = engine
        self._inbox: "queue.Queue" = queue.Queue()
        self._streams: dict = {}
        self._sent: dict = {}
        self._stop = False
        self._loop: Optional[asyncio.AbstractEventLoop] = None
        self.metrics = {"requests": 0, "output_tokens": 0, "prompt_tokens": 0, "steps": 0,
                        "ttft_sum": 0.0, "ttft_n": 0}
        from .metrics import ServingMetrics
        self.serving_metrics = ServingMetrics(engine.cfg.model.name)
        self._thread = threading.Thread(target=self._run, name="EngineLoop", daemon=True)
        self._thread.start()

    # ---- engine thread -------------------------------------------------------------
    def _run(self):
        eng = self.engine
        while not self._stop:
            try:
                while True:
                    kind, payload = self._inbox.get_nowait()
                    if kind == "add":
                        rid, toks, sp, kvp, mm, prio = payload
                        try:
                            eng.add_request(toks, sp, request_id=rid, kv_transfer_params=kvp, mm_items=mm,
                                            priority=prio)
                        except Exception as e:       # noqa: BLE001 - reported to the caller
                            self._emit(StreamItem(rid, [], True, "error", error=str(e)))
                    elif kind == "abort":
                        eng.abort_request(payload)
                    elif kind == "call":
                        # engine-thread work on behalf of a route (adapter loading): no step is in
                        # progress while it runs
                        fn, fut, loop = payload
                        try:
                            res, exc = fn(eng), None
                        except Exception as e:       # noqa: BLE001 - handed to the awaiting route
                            res, exc = None, e
                        loop.call_soon_threadsafe(_settle, fut, res, exc)
            except queue.Empty:
                pass
            if not eng.has_unfinished():
                eng.idle_tick()
                time.sleep(0.001)
                continue
            finished = eng.step()
            self.metrics["steps"] += 1
            for rid in list(self._streams):
                req = eng.scheduler.requests.get(rid)
                if req is None:
                    continue
                sent = self._sent.get(rid, 0)
                new = req.output_token_ids[sent:]
                done = req.status.finished
                if new or done:
                    self._sent[rid] = sent + len(new)
                    if sent == 0 and new and req.first_token_time:
                        self.metrics["ttft_sum"] += req.first_token_time - req.arrival_time
                        self.metrics["ttft_n"] += 1
                    self.metrics["output_tokens"] += len(new)
                    lps = req.logprobs[sent:sent + len(new)] if req.logprobs else None
                    self._emit(StreamItem(rid, list(new), done, req.status.value if done else None,
                                          req.kv_transfer_params if done else None, req.error,
                                          req.num_prompt_tokens, req.num_cached_tokens, lps,
                                          (req.prompt_logprobs or None) if done else None,
                                          getattr(req, "pooled", None) if done else None))
                    if done:
                        self.serving_metrics.observe_finished(req)
                        eng.scheduler.requests.pop(rid, None)
            del finished

    def _emit(self, item: StreamItem):
        q = self._streams.get(item.request_id)
        if q is None:
            return
        if self._loop is not None:
            self._loop.call_soon_threadsafe(q.put_nowait, item)
        if item.finished:
            self._streams.pop(item.request_id, None)
            self._sent.pop(item.request_id, None)

    # ---- caller side -----------------------------------------------------------------
    async def call(self, fn):
        """Run ``fn(engine)`` on the engine thread, between steps, and return its result."""
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        self._inbox.put(("call", (fn, fut, loop)))
        return await fut

    async def generate(self, request_id: str, prompt_token_ids: list, sp: SamplingParams,
                       kv_transfer_params: Optional[dict] = None,
                       mm_items: Optional[list] = None, priority: int = 0) -> AsyncIterator[StreamItem]:
        self._loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        self._streams[request_id] = q
        self.metrics["requests"] += 1
        self.metrics["prompt_tokens"] += len(prompt_token_ids)
        self._inbox.put(("add", (request_id, list(prompt_token_ids), sp, kv_transfer_params, mm_items, int(priority))))
        try:
            while True:
                item = await q.get()
                yield item
                if item.finished:
                    return
        finally:
            if request_id in self._streams:
                self._inbox.put(("abort", request_id))
                self._streams.pop(request_id, None)

    def shutdown(self):
        self._stop = True
        self._thread.join(timeout=2.0)
        self.engine.stop_followers()
