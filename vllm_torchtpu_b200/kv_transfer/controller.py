"""Controller of a disaggregated deployment: the registry the engines report to and the proxy picks from.

Engines register with their role (prefill / decode / both), HTTP endpoint, KV side-channel address, engine id,
tensor-parallel degree and block geometry, and then send heartbeats with their load (running and waiting
requests, free KV blocks).  The proxy asks for an instance of a role; the controller answers with the least
loaded one that is alive (heartbeat inside the time-to-live) and not marked unreachable.  A consumer whose pull
from a producer failed on the transport reports the producer; the controller stops handing it out until it
sends its next heartbeat.  All messages travel over the signed TCP side channel of the connectors.

The role of the reference's controller RPC server and of its source-unreachable marking
(reference: examples/disagg/run_raiden_controller.py:17-42,
src/vllm_torchtpu/distributed/kv_transfer/tpu_connector.py:1508-2615)."""
from __future__ import annotations

import threading
import time
from dataclasses import asdict, dataclass, field
from typing import Optional

from ..logger import init_logger
from .transport import TcpChannel

logger = init_logger(__name__)


@dataclass
class EngineRecord:
    engine_id: str
    role: str                       # "prefill" | "decode" | "both"
    http_url: str = ""
    kv_host: str = "127.0.0.1"
    kv_port: int = 0
    tp: int = 1
    model: str = ""
    geometry: Optional[dict] = None
    load: dict = field(default_factory=dict)        # running, waiting, free_blocks
    last_seen: float = 0.0
    unreachable_since: float = 0.0
    picks: int = 0

    def score(self) -> float:
        """Lower is better: queued work first, then occupancy."""
        l = self.load
        return 4.0 * l.get("waiting", 0) + l.get("running", 0) - 1e-6 * l.get("free_blocks", 0)


class KVController:
    def __init__(self, host: str = "127.0.0.1", port: int = 0, ttl_s: float = 10.0, clock=time.monotonic):
        self.ttl_s, self.clock = ttl_s, clock
        self.lock = threading.Lock()
        self.engines: dict = {}
        self.stats = {"registered": 0, "picks": 0, "unreachable_reports": 0, "expired": 0}
        self.channel = TcpChannel(host, port, self.handle)

    def address(self):
        return self.channel.address()

    def close(self):
        self.channel.close()

    # ---- message handler (side-channel threads) -------------------------------------------------------------
    def handle(self, msg: dict) -> dict:
        op = msg.get("op")
        fn = getattr(self, "_op_" + str(op).lower(), None)
        if fn is None:
            return {"ok": False, "error": f"unknown op {op!r}"}
        with self.lock:
            return fn(msg)

    def _alive(self, e: EngineRecord) -> bool:
        return self.clock() - e.last_seen <= self.ttl_s and not e.unreachable_since

    def _op_register(self, m):
        known = {f for f in EngineRecord.__dataclass_fields__}
        rec = EngineRecord(**{k: v for k, v in m.get("engine", {}).items() if k in known})
        if not rec.engine_id or rec.role not in ("prefill", "decode", "both"):
            return {"ok": False, "error": "engine_id and role (prefill | decode | both) are required"}
        rec.last_seen = self.clock()
        self.engines[rec.engine_id] = rec
        self.stats["registered"] += 1
        return {"ok": True, "ttl_s": self.ttl_s}

    def _op_heartbeat(self, m):
        e = self.engines.get(m.get("engine_id"))
        if e is None:
            return {"ok": False, "error": "not registered"}          # the engine registers again
        e.last_seen = self.clock()
        e.load = dict(m.get("load") or {})
        e.unreachable_since = 0.0                                    # it answers: reachable again
        return {"ok": True}

    def _op_deregister(self, m):
        return {"ok": self.engines.pop(m.get("engine_id"), None) is not None}

    def _op_unreachable(self, m):
        e = self.engines.get(m.get("engine_id"))
        self.stats["unreachable_reports"] += 1
        if e is not None and not e.unreachable_since:
            e.unreachable_since = self.clock()
            logger.warning("engine %s reported unreachable by %s", e.engine_id, m.get("reporter"))
        return {"ok": e is not None}

    def _op_list(self, m):
        role = m.get("role")
        out = []
        for e in self.engines.values():
            if role and e.role not in (role, "both"):
                continue
            d = asdict(e)
            d["alive"] = self._alive(e)
            out.append(d)
        return {"ok": True, "engines": out}

    def _op_pick(self, m):
        role, model = m.get("role"), m.get("model")
        exclude = set(m.get("exclude") or ())
        now = self.clock()
        for eid in [k for k, e in self.engines.items() if now - e.last_seen > 6 * self.ttl_s]:
            del self.engines[eid]                                    # long gone
            self.stats["expired"] += 1
        cands = [e for e in self.engines.values()
                 if e.role in (role, "both") and self._alive(e) and e.engine_id not in exclude
                 and (not model or not e.model or e.model == model)]
        if not cands:
            return {"ok": False, "error": f"no live {role} engine"}
        best = min(cands, key=lambda e: (e.score(), e.picks))
        best.picks += 1
        best.load["waiting"] = best.load.get("waiting", 0) + 1       # counted until its next heartbeat says otherwise
        self.stats["picks"] += 1
        return {"ok": True, "engine": asdict(best)}


class ControllerClient:
    """Engine side (register + heartbeats from a daemon thread) and proxy side (pick / report)."""

    def __init__(self, address, timeout_s: float = 2.0):
        self.address, self.timeout_s = tuple(address), timeout_s
        self._stop = threading.Event()
        self._thread = None

    def _call(self, msg: dict) -> dict:
        import socket
        from .base import sign_message, verify_message
        from .transport import _recv_frame, _send_frame
        with socket.create_connection(self.address, timeout=self.timeout_s) as s:
            s.settimeout(self.timeout_s)
            _send_frame(s, sign_message(msg))
            return verify_message(_recv_frame(s))

    def register(self, **engine) -> dict:
        self._engine = dict(engine)
        return self._call({"op": "REGISTER", "engine": engine})

    def heartbeat(self, engine_id: str, load: dict) -> dict:
        r = self._call({"op": "HEARTBEAT", "engine_id": engine_id, "load": load})
        if not r.get("ok") and r.get("error") == "not registered" and getattr(self, "_engine", None):
            self._call({"op": "REGISTER", "engine": self._engine})   # the controller restarted
            r = self._call({"op": "HEARTBEAT", "engine_id": engine_id, "load": load})
        return r

    def start_heartbeats(self, engine_id: str, load_fn, period_s: float = 2.0) -> None:
        def loop():
            while not self._stop.wait(period_s):
                try:
                    self.heartbeat(engine_id, load_fn())
                except (OSError, TimeoutError, ConnectionError, PermissionError) as e:
                    logger.warning("controller heartbeat failed: %r", e)
        self._thread = threading.Thread(target=loop, name="KV:Heartbeat", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()

    def pick(self, role: str, model: str = "", exclude=()) -> Optional[dict]:
        r = self._call({"op": "PICK", "role": role, "model": model, "exclude": list(exclude)})
        return r.get("engine") if r.get("ok") else None

    def report_unreachable(self, engine_id: str, reporter: str = "") -> None:
        self._call({"op": "UNREACHABLE", "engine_id": engine_id, "reporter": reporter})

    def list(self, role: str = "") -> list:
        return self._call({"op": "LIST", "role": role}).get("engines", [])

    def deregister(self, engine_id: str) -> None:
        self._call({"op": "DEREGISTER", "engine_id": engine_id})


def run_controller(host: str = "0.0.0.0", port: int = 7600, ttl_s: float = 10.0) -> None:
    c = KVController(host, port, ttl_s)
    logger.info("KV controller listening on %s:%d", *c.address())
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        c.close()
