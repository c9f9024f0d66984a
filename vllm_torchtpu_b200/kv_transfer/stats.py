"""Connector statistics, optionally exported as Prometheus metrics
(reference: src/vllm_torchtpu/distributed/kv_transfer/tpu_connector_stats.py:14-489)."""
from __future__ import annotations

import threading
from dataclasses import dataclass, field


@dataclass
class KVConnectorStats:
    loads_ok: int = 0
    loads_failed: int = 0
    blocks_loaded: int = 0
    sends_pulled: int = 0
    sends_expired: int = 0
    blocks_sent: int = 0
    load_seconds: list = field(default_factory=list)
    _lock: threading.Lock = field(default_factory=threading.Lock, repr=False)

    def record_load(self, blocks: int, seconds: float, ok: bool) -> None:
        with self._lock:
            if ok:
                self.loads_ok += 1
                self.blocks_loaded += blocks
            else:
                self.loads_failed += 1
            self.load_seconds.append(seconds)
            if len(self.load_seconds) > 4096:
                del self.load_seconds[:2048]

    def record_send(self, blocks: int, expired: bool) -> None:
        with self._lock:
            if expired:
                self.sends_expired += 1
            else:
                self.sends_pulled += 1
                self.blocks_sent += blocks

    def snapshot(self) -> dict:
        with self._lock:
            ls = sorted(self.load_seconds)
            p50 = ls[len(ls) // 2] if ls else 0.0
            return {"loads_ok": self.loads_ok, "loads_failed": self.loads_failed,
                    "blocks_loaded": self.blocks_loaded, "sends_pulled": self.sends_pulled,
                    "sends_expired": self.sends_expired, "blocks_sent": self.blocks_sent,
                    "load_p50_s": p50}


class KVConnectorPromMetrics:
    """Counter / Gauge / Histogram view of ``KVConnectorStats`` (prometheus_client is optional)."""

    def __init__(self, registry=None, prefix: str = "b200_kv"):
        from prometheus_client import Counter, Gauge, Histogram
        kw = {"registry": registry} if registry is not None else {}
        self.loads = Counter(f"{prefix}_loads_total", "KV loads", ["result"], **kw)
        self.blocks = Counter(f"{prefix}_blocks_total", "KV blocks moved", ["direction"], **kw)
        self.pending = Gauge(f"{prefix}_pending_sends", "blocks kept for remote decoders", **kw)
        self.latency = Histogram(f"{prefix}_load_seconds", "KV load latency", **kw)
        self._last = KVConnectorStats().snapshot()

    def observe(self, stats: KVConnectorStats, pending_sends: int = 0) -> None:
        s = stats.snapshot()
        self.loads.labels("ok").inc(s["loads_ok"] - self._last["loads_ok"])
        self.loads.labels("failed").inc(s["loads_failed"] - self._last["loads_failed"])
        self.blocks.labels("in").inc(s["blocks_loaded"] - self._last["blocks_loaded"])
        self.blocks.labels("out").inc(s["blocks_sent"] - self._last["blocks_sent"])
        self.pending.set(pending_sends)
        if s["load_p50_s"]:
            self.latency.observe(s["load_p50_s"])
        self._last = s
