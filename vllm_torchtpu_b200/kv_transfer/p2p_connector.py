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
"""
from __future__ import annotations

import threading
import uuid as uuidlib
from typing import Optional

from .. import envs
from ..logger import init_logger
from .base import (ConnectorMetadata, Connector, KVConnectorRole, LoadMeta, SchedulerConnectorBase, SendMeta,
                   WorkerConnectorBase, now)
from .stats import KVConnectorStats
from .transport import InProcessChannel, IpcTransport, LocalTransport, TcpChannel, TransferError

logger = init_logger(__name__)


class _Shared:
    """State both halves see (they live in one process)."""

    def __init__(self, engine_id: str, role: str, block_size: int, policy: str):
        self.engine_id, self.role, self.block_size, self.policy = engine_id, role, block_size, policy
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
                      p.get("remote_host", "127.0.0.1"), p.get("remote_port", 0))
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
        uid = uuidlib.uuid4().hex
        sm = SendMeta(request.request_id, uid, list(block_ids), request.num_computed_tokens,
                      now() + envs.B200_P2P_WAIT_PULL_TIMEOUT)
        with self.s.lock:
            self.s.pending_sends[uid] = sm
        self._new_sends.append(sm)
        host, port = (self.s.address or ("127.0.0.1", 0))[:2]
        return True, {"uuid": uid, "remote_engine_id": self.s.engine_id, "remote_block_ids": list(block_ids),
                      "remote_host": host, "remote_port": port, "num_tokens": request.num_computed_tokens}

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
                    self.s.pulled.add(msg["uuid"])
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
                addr = self._address_of(lm)
                if lm.remote_engine not in self._opened:
                    hello = self.channel.request(addr, {"op": "HELLO"}, envs.B200_KV_STAGE_WAIT_TIMEOUT_SECS)
                    if not hello.get("ok"):
                        raise TransferError(hello.get("error", "handshake refused"))
                    self.transport.open_remote(hello["pool"])
                    self._opened.add(lm.remote_engine)
                self.transport.pull(lm.remote_engine, lm.remote_block_ids, lm.local_block_ids)
                try:
                    self.channel.request(addr, {"op": "PULLED", "uuid": lm.uuid}, 5.0)
                except (OSError, TimeoutError, ConnectionError) as e:
                    # data is here; the producer will free the blocks when its timer expires
                    logger.warning("could not acknowledge pull of %s: %r", lm.uuid, e)
                with self.s.lock:
                    self.s.load_done.add(lm.request_id)
                self._recv_done.append(lm.request_id)
                self.s.stats.record_load(len(lm.local_block_ids), now() - t0, ok=True)
            except (TransferError, OSError, TimeoutError, ConnectionError, PermissionError) as e:
                logger.warning("KV load of request %s failed: %r", lm.request_id, e)
                with self.s.lock:
                    self.s.load_failed[lm.request_id] = repr(e)
                    self.s.error_blocks.update(lm.local_block_ids)
                self.s.stats.record_load(len(lm.local_block_ids), now() - t0, ok=False)

    def _address_of(self, lm: LoadMeta):
        if isinstance(self.channel, InProcessChannel):
            return ("inproc", lm.remote_engine)
        return (lm.remote_host, lm.remote_port)

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


def create_p2p_connector(cfg, runner, *, transport=None, channel_factory=None) -> Connector:
    kt = cfg.kv_transfer or {}
    role = kt.get("kv_role", KVConnectorRole.BOTH)
    engine_id = kt.get("engine_id") or f"engine-{uuidlib.uuid4().hex[:8]}"
    extra = kt.get("kv_connector_extra_config", {})
    policy = kt.get("kv_load_failure_policy", "recompute")
    shared = _Shared(engine_id, role, cfg.cache.block_size, policy)
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
            channel_factory = lambda h: TcpChannel(host, port, h)
    worker = P2PWorkerHalf(shared, transport, channel_factory)
    sched = P2PSchedulerHalf(shared)
    c = Connector(sched, worker)
    c.shared = shared
    return c
