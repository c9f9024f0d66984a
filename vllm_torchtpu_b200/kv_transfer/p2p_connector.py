"""Disaggregated prefill/decode connector over NVLink peer memory.

Protocol (request level, same contract as the reference's connectors,
reference: src/vllm_torchtpu/distributed/kv_transfer/zmq_shm_base.py:16-40,
tpu_connector.py:1331, docs/user_guide/disaggregated_serving.md:62-147):

  1. the proxy sends the prompt to a PREFILL engine with ``max_tokens=1``;
  2. when that request finishes, the producer keeps its KV blocks and answers with
     ``kv_transfer_params = {uuid, remote_engine_id, remote_block_ids, remote_host, remote_port,
     num_tokens}``;
  3. the proxy sends the request, with those params, to a DECODE engine;
  4. the consumer's scheduler counts the remote tokens as externally computed, allocates local
     blocks and parks the request in WAITING_FOR_REMOTE_KVS;
  5. the consumer's worker maps the producer's pool (once per engine pair), pulls the blocks
     GPU→GPU with one kernel, then tells the producer ``PULLED uuid``;
  6. the producer frees the blocks; blocks nobody pulled are freed after
     ``B200_P2P_WAIT_PULL_TIMEOUT`` seconds;
  7. a failed pull marks the request's blocks as load errors; by policy the request is
     recomputed locally (``recompute``) or finished with an error (``fail``).

Engines of several tensor-parallel ranks: every rank runs both halves over its own pool, rank r under the
engine id ``<engine_id>/r<r>`` and on port ``port + r``; transfer ids are derived from the request id, so
all ranks of the producer name a transfer alike and rank 0's ``kv_transfer_params`` speak for all.  Producer
and consumer may differ in degree: ``kv_transfer_params["remote_geometry"]`` carries the producer's block
layout, each consumer rank works out which head ranges to fetch from which producer ranks
(``reshard.plan_pull``) and a producer rank frees a transfer when every consumer rank that reads from it has
acknowledged (``reshard.readers_of``).
"""
from __future__ import annotations

import hashlib
import threading
import uuid as uuidlib
from typing import Optional

from .. import envs
from ..logger import init_logger
from .base import (ConnectorMetadata, Connector, KVConnectorRole, LoadMeta, SchedulerConnectorBase, SendMeta,
                   WorkerConnectorBase, now)
from .stats import KVConnectorStats
from .reshard import KVGeometry, plan_pull, readers_of, same_layout
from .transport import InProcessChannel, IpcTransport, LocalTransport, TcpChannel, TransferError

logger = init_logger(__name__)


class _Shared:
    """State both halves see (they live in one process)."""

    def __init__(self, engine_id: str, role: str, block_size: int, policy: str, geometry: KVGeometry = None,
                 base_engine_id: str = None):
        self.engine_id, self.role, self.block_size, self.policy = engine_id, role, block_size, policy
        self.geometry = geometry                 # this rank's block layout (None: single-rank, equal layouts)
        self.base_engine_id = base_engine_id or engine_id      # engine id without the rank suffix
        self.acks: dict = {}                     # uuid -> consumer ranks that acknowledged (producer)
        self.lock = threading.Lock()
        self.pending_sends: dict = {}        # uuid -> SendMeta (producer)
        self.pulled: set = set()             # uuids the consumer reported as taken
        self.loads: dict = {}                # request_id -> LoadMeta (consumer)
        self.load_done: set = set()
        self.load_failed: dict = {}          # request_id -> reason
        self.error_blocks: set = set()
        self.address = None
        self.stats = KVConnectorStats()


class P2PSchedulerHalf(SchedulerConnectorBase):
    def __init__(self, shared: _Shared):
        self.s = shared
        self._new_loads: list = []
        self._new_sends: list = []

    # ---- consumer ---------------------------------------------------------------
    def get_num_new_matched_tokens(self, request, num_cached: int):
        p = request.kv_transfer_params
        if not p or self.s.role == KVConnectorRole.PRODUCER or not p.get("remote_block_ids"):
            return 0, False
        if request.request_id in self.s.load_failed:
            return 0, False                      # recompute locally after a failed pull
        n_remote = min(int(p["num_tokens"]), request.num_prompt_tokens)
        ext = n_remote - 1 - num_cached           # the last prompt token is recomputed for its logits
        return (ext, True) if ext > 0 else (0, False)

    def update_state_after_alloc(self, request, block_ids: list, num_external: int) -> None:
        p = request.kv_transfer_params
        bs = self.s.block_size
        first = (request.num_computed_tokens) // bs           # blocks already held by the local prefix cache
        need = -(-(request.num_computed_tokens + num_external) // bs)
        remote = list(p["remote_block_ids"])[first:need]
        local = list(block_ids)[first:need]
        lm = LoadMeta(request.request_id, p["uuid"], p["remote_engine_id"], remote, local, num_external,
                      p.get("remote_host", "127.0.0.1"), p.get("remote_port", 0),
                      remote_geometry=p.get("remote_geometry"))
        with self.s.lock:
            self.s.loads[request.request_id] = lm
        self._new_loads.append(lm)

    def is_load_done(self, request) -> bool:
        rid = request.request_id
        with self.s.lock:
            if rid in self.s.load_failed:
                if self.s.policy == "fail":
                    request.error = f"kv_load_failed: {self.s.load_failed[rid]}"
                # recompute: give the blocks back to be filled locally
                request.num_computed_tokens = request.num_cached_tokens
                self.s.loads.pop(rid, None)
                return True
            if rid in self.s.load_done:
                self.s.load_done.discard(rid)
                self.s.loads.pop(rid, None)
                return True
        return False

    # ---- producer ---------------------------------------------------------------
    def request_finished(self, request, block_ids: list):
        if self.s.role == KVConnectorRole.CONSUMER or request.error or not block_ids:
            return False, None
        p = request.kv_transfer_params or {}
        if self.s.role == KVConnectorRole.BOTH and not p.get("do_remote_decode", False):
            return False, None
        # the same id on every rank of this engine (the ranks schedule alike)
        uid = hashlib.sha1(f"{self.s.base_engine_id}:{request.request_id}:{request.num_computed_tokens}"
                           .encode()).hexdigest()[:32]
        sm = SendMeta(request.request_id, uid, list(block_ids), request.num_computed_tokens,
                      now() + envs.B200_P2P_WAIT_PULL_TIMEOUT)
        with self.s.lock:
            self.s.pending_sends[uid] = sm
        self._new_sends.append(sm)
        host, port = (self.s.address or ("127.0.0.1", 0))[:2]
        g = self.s.geometry
        if g is not None and isinstance(port, int):
            port -= g.rank                       # the port of rank 0; rank r listens on port + r
        params = {"uuid": uid, "remote_engine_id": self.s.base_engine_id, "remote_block_ids": list(block_ids),
                  "remote_host": host, "remote_port": port, "num_tokens": request.num_computed_tokens}
        if g is not None:
            params["remote_geometry"] = g.to_dict()
        return True, params

    def build_connector_meta(self, scheduler_output) -> ConnectorMetadata:
        m = ConnectorMetadata(self._new_sends, self._new_loads, [])
        self._new_sends, self._new_loads = [], []
        return m


class P2PWorkerHalf(WorkerConnectorBase):
    def __init__(self, shared: _Shared, transport, channel_factory):
        self.s = shared
        self.transport = transport
        self.channel = channel_factory(self._handle)
        self.s.address = self.channel.address()
        self._opened: set = set()
        self._recv_done: list = []

    # ---- control plane (runs on the side-channel thread) -------------------------
    def _handle(self, msg: dict) -> dict:
        op = msg.get("op")
        if op == "HELLO":
            return {"ok": True, "pool": self.transport.export()}
        if op == "PULLED":
            with self.s.lock:
                if msg["uuid"] in self.s.pending_sends:
                    g, cg = self.s.geometry, msg.get("consumer_geometry")
                    if g is None or not cg:
                        self.s.pulled.add(msg["uuid"])
                    else:
                        # free when every consumer rank that reads from this rank has reported
                        c = KVGeometry.from_dict(cg)
                        got = self.s.acks.setdefault(msg["uuid"], set())
                        got.add(c.rank)
                        if got >= set(readers_of(g, c.tp, c)):
                            self.s.pulled.add(msg["uuid"])
                            del self.s.acks[msg["uuid"]]
            return {"ok": True}
        if op == "PING":
            return {"ok": True, "engine_id": self.s.engine_id}
        return {"ok": False, "error": f"unknown op {op!r}"}

    # ---- consumer -----------------------------------------------------------------
    def start_load_kv(self, meta: Optional[ConnectorMetadata]) -> None:
        if meta is None:
            return
        for lm in meta.loads:
            t0 = now()
            try:
                for engine, addr, span in self._sources(lm):
                    if engine not in self._opened:
                        hello = self.channel.request(addr, {"op": "HELLO"}, envs.B200_KV_STAGE_WAIT_TIMEOUT_SECS)
                        if not hello.get("ok"):
                            raise TransferError(hello.get("error", "handshake refused"))
                        self.transport.open_remote(hello["pool"])
                        self._opened.add(engine)
                    if span is None:
                        self.transport.pull(engine, lm.remote_block_ids, lm.local_block_ids)
                    else:
                        self.transport.pull(engine, lm.remote_block_ids, lm.local_block_ids, span)
                    ack = {"op": "PULLED", "uuid": lm.uuid}
                    if self.s.geometry is not None and lm.remote_geometry:
                        ack["consumer_geometry"] = self.s.geometry.to_dict()
                    try:
                        self.channel.request(addr, ack, 5.0)
                    except (OSError, TimeoutError, ConnectionError) as e:
                        # data is here; the producer will free the blocks when its timer expires
                        logger.warning("could not acknowledge pull of %s: %r", lm.uuid, e)
                with self.s.lock:
                    self.s.load_done.add(lm.request_id)
                self._recv_done.append(lm.request_id)
                self.s.stats.record_load(len(lm.local_block_ids), now() - t0, ok=True)
            except (TransferError, OSError, TimeoutError, ConnectionError, PermissionError) as e:
                logger.warning("KV load of request %s failed: %r", lm.request_id, e)
                ctl = getattr(self, "controller", None)
                if ctl is not None and isinstance(e, (OSError, TimeoutError, ConnectionError)):
                    try:                               # the source does not answer: keep others away from it
                        ctl.report_unreachable(lm.remote_engine, reporter=self.s.engine_id)
                    except (OSError, TimeoutError, ConnectionError):
                        pass
                with self.s.lock:
                    self.s.load_failed[lm.request_id] = repr(e)
                    self.s.error_blocks.update(lm.local_block_ids)
                self.s.stats.record_load(len(lm.local_block_ids), now() - t0, ok=False)

    def _sources(self, lm: LoadMeta) -> list:
        """[(engine id, control address, Span or None)] this rank fetches a transfer from."""
        inproc = isinstance(self.channel, InProcessChannel)
        g, rg = self.s.geometry, lm.remote_geometry
        if g is None or not rg:
            addr = ("inproc", lm.remote_engine) if inproc else (lm.remote_host, lm.remote_port)
            return [(lm.remote_engine, addr, None)]
        prod = KVGeometry.from_dict(rg)
        out = []
        for pr, span in plan_pull(g, prod):
            engine = rank_engine_id(lm.remote_engine, pr, prod.tp)
            addr = ("inproc", engine) if inproc else (lm.remote_host, lm.remote_port + pr)
            peer = KVGeometry(prod.tp, pr, prod.num_kv_heads, prod.head_bytes, prod.block_bytes)
            out.append((engine, addr, None if same_layout(g, peer) else span))
        return out

    def get_finished_recving(self) -> list:
        out, self._recv_done = self._recv_done, []
        return out

    def get_block_ids_with_load_errors(self) -> set:
        with self.s.lock:
            out, self.s.error_blocks = self.s.error_blocks, set()
        return out

    # ---- producer -----------------------------------------------------------------
    def get_finished_sending(self) -> list:
        done = []
        t = now()
        with self.s.lock:
            for uid, sm in list(self.s.pending_sends.items()):
                if uid in self.s.pulled:
                    self.s.pulled.discard(uid)
                    done.append(sm.request_id)
                    del self.s.pending_sends[uid]
                    self.s.stats.record_send(len(sm.block_ids), expired=False)
                elif t > sm.expires_at:
                    logger.warning("nobody pulled the KV of %s within the timeout; freeing", sm.request_id)
                    done.append(sm.request_id)
                    del self.s.pending_sends[uid]
                    self.s.stats.record_send(len(sm.block_ids), expired=True)
        return done

    def close(self):
        self.channel.close()


def rank_engine_id(engine_id: str, rank: int, tp: int) -> str:
    return engine_id if tp <= 1 else f"{engine_id}/r{rank}"


def create_p2p_connector(cfg, runner, *, transport=None, channel_factory=None) -> Connector:
    from ..parallel.state import get_state
    kt = cfg.kv_transfer or {}
    role = kt.get("kv_role", KVConnectorRole.BOTH)
    tp = get_state().tp
    if tp.size > 1 and not kt.get("engine_id"):
        raise ValueError("kv_transfer with tensor parallelism needs an explicit engine_id (the same on every rank)")
    base_id = kt.get("engine_id") or f"engine-{uuidlib.uuid4().hex[:8]}"
    engine_id = rank_engine_id(base_id, tp.rank_in_group, tp.size)
    extra = kt.get("kv_connector_extra_config", {})
    policy = kt.get("kv_load_failure_policy", "recompute")
    geometry = None
    first = runner.kv_caches[0] if runner.kv_caches else None
    if first is not None and hasattr(first, "dim"):
        geometry = KVGeometry.of_cache(first, tp.size, tp.rank_in_group, cfg.model.num_kv_heads)
    shared = _Shared(engine_id, role, cfg.cache.block_size, policy, geometry, base_id)
    if transport is None:
        kind = extra.get("transport", "ipc" if str(runner.device).startswith("cuda") else "local")
        transport = IpcTransport(engine_id) if kind == "ipc" else LocalTransport(engine_id)
    transport.register_pool(runner.kv_caches)
    if channel_factory is None:
        if extra.get("channel", "tcp") == "inproc":
            channel_factory = lambda h: InProcessChannel(engine_id, h)
        else:
            host = extra.get("host", "127.0.0.1")
            port = int(extra.get("port", 0))
            if tp.size > 1:
                if not port:
                    raise ValueError("kv_transfer with tensor parallelism needs a fixed port (rank r listens on port + r)")
                port += tp.rank_in_group
            channel_factory = lambda h: TcpChannel(host, port, h)
    worker = P2PWorkerHalf(shared, transport, channel_factory)
    sched = P2PSchedulerHalf(shared)
    c = Connector(sched, worker)
    c.shared = shared
    c.controller = None
    ctl_addr = extra.get("controller")
    if ctl_addr and tp.rank_in_group == 0:
        # rank 0 speaks for the engine: register with the controller and report load with every heartbeat
        # (the engine replaces `load_fn` with its scheduler's counts)
        from .controller import ControllerClient
        h, pt = (ctl_addr.rsplit(":", 1) if isinstance(ctl_addr, str) else ctl_addr)
        client = ControllerClient((h, int(pt)))
        role_name = {KVConnectorRole.PRODUCER: "prefill", KVConnectorRole.CONSUMER: "decode"}.get(role, "both")
        kv_host, kv_port = (shared.address or ("127.0.0.1", 0))[:2]
        c.load_fn = lambda: {"running": len(shared.loads), "waiting": 0, "pending_sends": len(shared.pending_sends)}
        try:
            client.register(engine_id=base_id, role=role_name, http_url=extra.get("http_url", ""),
                            kv_host=str(kv_host), kv_port=int(kv_port) if isinstance(kv_port, int) else 0,
                            tp=tp.size, model=cfg.model.name, geometry=geometry.to_dict() if geometry else None)
            client.start_heartbeats(base_id, lambda: c.load_fn(), float(extra.get("heartbeat_s", 2.0)))
            c.controller = client
            worker.controller = client
        except (OSError, TimeoutError, ConnectionError) as e:
            logger.warning("KV controller %s not reachable: %r", ctl_addr, e)
    return c
