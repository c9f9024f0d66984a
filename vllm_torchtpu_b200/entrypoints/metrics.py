"""Serving metrics in the Prometheus text format.

Counters, gauges and histograms of the request life cycle (queue time, time to first token, time per output
token, end-to-end latency, tokens per request), the KV cache and prefix cache, preemptions and speculative
decoding.  Every series is exported under two names: ``b200_*`` and the ``vllm:*`` name dashboards written for
vLLM look for (the reference is scraped through vLLM's own metrics; reference:
docs/user_guide/supported_models.md "Profiling & observability").  No dependency: the text format is written
directly.
"""
from __future__ import annotations

import threading

LATENCY_BUCKETS = (0.001, 0.005, 0.01, 0.02, 0.04, 0.06, 0.08, 0.1, 0.25, 0.5, 0.75, 1.0, 2.5, 5.0, 7.5, 10.0,
                   20.0, 40.0, 80.0, 160.0, 640.0, 2560.0)
TOKEN_LATENCY_BUCKETS = (0.001, 0.0025, 0.005, 0.0075, 0.01, 0.015, 0.02, 0.025, 0.03, 0.04, 0.05, 0.075, 0.1,
                         0.15, 0.2, 0.3, 0.4, 0.5, 0.75, 1.0, 2.5, 5.0, 10.0)
COUNT_BUCKETS = (1, 2, 5, 10, 20, 50, 100, 200, 500, 1000, 2000, 5000, 10000, 20000, 50000, 100000)


class Histogram:
    def __init__(self, buckets):
        self.buckets = tuple(buckets)
        self.counts = [0] * (len(self.buckets) + 1)
        self.sum = 0.0
        self.n = 0

    def observe(self, v: float) -> None:
        self.sum += v
        self.n += 1
        for i, b in enumerate(self.buckets):
            if v <= b:
                self.counts[i] += 1
                return
        self.counts[-1] += 1

    def lines(self, name: str, labels: str) -> list:
        out, cum = [], 0
        sep = "," if labels else ""
        for b, c in zip(self.buckets, self.counts):
            cum += c
            out.append(f'{name}_bucket{{{labels}{sep}le="{b}"}} {cum}')
        out.append(f'{name}_bucket{{{labels}{sep}le="+Inf"}} {self.n}')
        tail = f"{{{labels}}}" if labels else ""
        out.append(f"{name}_sum{tail} {self.sum:.6f}")
        out.append(f"{name}_count{tail} {self.n}")
        return out


# series name (without prefix) -> (type, help text, vLLM name or None)
_SERIES = {
    "num_requests_running": ("gauge", "requests in the running set", "vllm:num_requests_running"),
    "num_requests_waiting": ("gauge", "requests waiting for admission", "vllm:num_requests_waiting"),
    "kv_cache_usage": ("gauge", "fraction of KV-cache blocks in use", "vllm:kv_cache_usage_perc"),
    "requests_total": ("counter", "requests received", None),
    "request_success_total": ("counter", "finished requests by reason", "vllm:request_success_total"),
    "prompt_tokens_total": ("counter", "prompt tokens received", "vllm:prompt_tokens_total"),
    "generation_tokens_total": ("counter", "tokens generated", "vllm:generation_tokens_total"),
    "engine_steps_total": ("counter", "engine steps", None),
    "preemptions_total": ("counter", "requests preempted", "vllm:num_preemptions_total"),
    "prefix_cache_queries_total": ("counter", "prompt tokens looked up in the prefix cache",
                                   "vllm:prefix_cache_queries_total"),
    "prefix_cache_hits_total": ("counter", "prompt tokens served from the prefix cache", "vllm:prefix_cache_hits_total"),
    "prefix_cache_hit_tokens_total": ("counter", "prompt tokens served from the prefix cache", None),
    "spec_decode_num_draft_tokens_total": ("counter", "draft tokens verified", "vllm:spec_decode_num_draft_tokens_total"),
    "spec_decode_num_accepted_tokens_total": ("counter", "draft tokens accepted",
                                              "vllm:spec_decode_num_accepted_tokens_total"),
    "time_to_first_token_seconds": ("histogram", "arrival to first token", "vllm:time_to_first_token_seconds"),
    "time_per_output_token_seconds": ("histogram", "mean time between output tokens of a request",
                                      "vllm:time_per_output_token_seconds"),
    "e2e_request_latency_seconds": ("histogram", "arrival to finish", "vllm:e2e_request_latency_seconds"),
    "request_queue_time_seconds": ("histogram", "arrival to first admission", "vllm:request_queue_time_seconds"),
    "request_prompt_tokens": ("histogram", "prompt tokens per request", "vllm:request_prompt_tokens"),
    "request_generation_tokens": ("histogram", "generated tokens per request", "vllm:request_generation_tokens"),
}


class ServingMetrics:
    def __init__(self, model_name: str = ""):
        self.model_name = model_name
        self._lock = threading.Lock()
        self.finished_by_reason: dict = {}
        self.hist = {"time_to_first_token_seconds": Histogram(LATENCY_BUCKETS),
                     "time_per_output_token_seconds": Histogram(TOKEN_LATENCY_BUCKETS),
                     "e2e_request_latency_seconds": Histogram(LATENCY_BUCKETS),
                     "request_queue_time_seconds": Histogram(LATENCY_BUCKETS),
                     "request_prompt_tokens": Histogram(COUNT_BUCKETS),
                     "request_generation_tokens": Histogram(COUNT_BUCKETS)}

    def observe_finished(self, req) -> None:
        """Called once per request when it leaves the engine (engine thread)."""
        with self._lock:
            reason = req.status.value
            self.finished_by_reason[reason] = self.finished_by_reason.get(reason, 0) + 1
            n_out = len(req.output_token_ids)
            self.hist["request_prompt_tokens"].observe(req.num_prompt_tokens)
            self.hist["request_generation_tokens"].observe(n_out)
            if req.scheduled_time is not None:
                self.hist["request_queue_time_seconds"].observe(max(0.0, req.scheduled_time - req.arrival_time))
            if req.first_token_time is not None:
                self.hist["time_to_first_token_seconds"].observe(max(0.0, req.first_token_time - req.arrival_time))
            if req.finish_time is not None:
                self.hist["e2e_request_latency_seconds"].observe(max(0.0, req.finish_time - req.arrival_time))
                if req.first_token_time is not None and n_out > 1:
                    self.hist["time_per_output_token_seconds"].observe(
                        max(0.0, req.finish_time - req.first_token_time) / (n_out - 1))

    def render(self, counters: dict, engine) -> str:
        """``counters``: the async engine's request / token / step counts."""
        sch = engine.scheduler
        rstats = getattr(getattr(engine, "runner", None), "stats", None) or {}
        values = {
            "num_requests_running": len(sch.running), "num_requests_waiting": len(sch.waiting),
            "kv_cache_usage": round(sch.kv.pool.usage, 6),
            "requests_total": counters.get("requests", 0), "prompt_tokens_total": counters.get("prompt_tokens", 0),
            "generation_tokens_total": counters.get("output_tokens", 0),
            "engine_steps_total": counters.get("steps", 0), "preemptions_total": sch.stats["preemptions"],
            "prefix_cache_queries_total": sch.stats.get("prefix_query_tokens", 0),
            "prefix_cache_hits_total": sch.stats["prefix_hit_tokens"],
            "prefix_cache_hit_tokens_total": sch.stats["prefix_hit_tokens"],
            "spec_decode_num_draft_tokens_total": int(rstats.get("spec_drafted", 0)),
            "spec_decode_num_accepted_tokens_total": int(rstats.get("spec_accepted", 0)),
        }
        label = f'model_name="{self.model_name}"'
        out = []
        with self._lock:
            for base, (kind, doc, compat) in _SERIES.items():
                for name, labels in ((f"b200_{base}", ""), (compat, label)):
                    if name is None:
                        continue
                    out.append(f"# HELP {name} {doc}")
                    out.append(f"# TYPE {name} {kind}")
                    if kind == "histogram":
                        out += self.hist[base].lines(name, labels)
                    elif base == "request_success_total":
                        sep = "," if labels else ""
                        for reason, n in sorted(self.finished_by_reason.items()):
                            out.append(f'{name}{{{labels}{sep}finished_reason="{reason}"}} {n}')
                    else:
                        out.append(f"{name}{{{labels}}} {values[base]}" if labels else f"{name} {values[base]}")
        out += self._connector_lines(getattr(engine, "connector", None), label)
        return "\n".join(out) + "\n"

    @staticmethod
    def _connector_lines(connector, label: str) -> list:
        """KV-transfer and offload statistics of the engine's connector(s), when there is one."""
        if connector is None:
            return []
        halves = []
        for part in [connector] + list(getattr(connector, "connectors", []) or []):
            halves += [getattr(part, "scheduler", None), getattr(part, "worker", None)]
        for side in ("scheduler", "worker"):
            halves += list(getattr(getattr(connector, side, None), "parts", []) or [])     # multi connector
        out, seen = [], set()
        for h in halves:
            st = getattr(h, "stats", None)
            if st is None:
                st = getattr(getattr(h, "s", None), "stats", None)      # state shared by the two P2P halves
            if st is None or id(st) in seen:
                continue
            seen.add(id(st))
            if isinstance(st, dict) and "external_hits" in st:
                for base, key in (("external_prefix_cache_queries_total", "external_queries"),
                                  ("external_prefix_cache_hits_total", "external_hits")):
                    out += [f"# TYPE b200_{base} counter", f"b200_{base} {st[key]}",
                            f"# TYPE vllm:{base} counter", f"vllm:{base}{{{label}}} {st[key]}"]
            elif hasattr(st, "snapshot"):
                s = st.snapshot()
                out += ["# TYPE b200_kv_loads_total counter",
                        f'b200_kv_loads_total{{result="ok"}} {s["loads_ok"]}',
                        f'b200_kv_loads_total{{result="failed"}} {s["loads_failed"]}',
                        "# TYPE b200_kv_blocks_total counter",
                        f'b200_kv_blocks_total{{direction="in"}} {s["blocks_loaded"]}',
                        f'b200_kv_blocks_total{{direction="out"}} {s["blocks_sent"]}',
                        "# TYPE b200_kv_sends_total counter",
                        f'b200_kv_sends_total{{result="pulled"}} {s["sends_pulled"]}',
                        f'b200_kv_sends_total{{result="expired"}} {s["sends_expired"]}',
                        "# TYPE b200_kv_load_seconds_p50 gauge", f'b200_kv_load_seconds_p50 {s["load_p50_s"]:.6f}']
        return out
