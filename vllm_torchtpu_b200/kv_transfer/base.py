"""KV connector interfaces and wire metadata.

A connector has a scheduler half (decides how many prompt tokens come from outside,
tracks which blocks must outlive their request) and a worker half (moves the blocks).
The split and the call points are the ones of the reference's connectors
(reference: src/vllm_torchtpu/distributed/kv_transfer/tpu_connector.py:771-1060, 1077-1506):

scheduler half
  get_num_new_matched_tokens(request, num_locally_cached) -> (external_tokens, load_is_async)
  update_state_after_alloc(request, block_ids, external_tokens)
  build_connector_meta(scheduler_output) -> ConnectorMetadata (travels to the worker with the step)
  request_finished(request, block_ids) -> (delay_free, kv_transfer_params | None)
  is_load_done(request) -> bool

worker half
  start_load_kv(meta)            begin asynchronous loads for requests admitted this step
  save_kv(meta)                  make this step's finished prefill blocks available / store them
  get_finished_sending() -> ids  requests whose blocks the remote side has taken (free them now)
  get_finished_recving() -> ids  requests whose blocks have landed
  get_block_ids_with_load_errors()
"""
from __future__ import annotations

import hashlib
import hmac
import json
import os
import time
from dataclasses import dataclass, field
from typing import Optional


@dataclass
class SendMeta:
    request_id: str
    uuid: str
    block_ids: list
    num_tokens: int
    expires_at: float


@dataclass
class LoadMeta:
    request_id: str
    uuid: str
    remote_engine: str
    remote_block_ids: list
    local_block_ids: list
    num_tokens: int
    remote_host: str = "127.0.0.1"
    remote_port: int = 0
    remote_geometry: Optional[dict] = None      # the producer's block layout when degrees may differ


@dataclass
class ConnectorMetadata:
    sends: list = field(default_factory=list)
    loads: list = field(default_factory=list)
    frees: list = field(default_factory=list)          # uuids whose producer-side blocks may be released


class KVConnectorRole:
    PRODUCER = "kv_producer"
    CONSUMER = "kv_consumer"
    BOTH = "kv_both"


class SchedulerConnectorBase:
    def get_num_new_matched_tokens(self, request, num_cached: int):
        return 0, False

    def request_not_admitted(self, request) -> None:
        """Called when ``get_num_new_matched_tokens`` reported matches but the request could not be
        given its blocks in this step; connectors release what the query reserved."""

    def update_state_after_alloc(self, request, block_ids: list, num_external: int) -> None:
        pass

    def build_connector_meta(self, scheduler_output) -> ConnectorMetadata:
        return ConnectorMetadata()

    def request_finished(self, request, block_ids: list):
        return False, None

    def is_load_done(self, request) -> bool:
        return True


class WorkerConnectorBase:
    def start_load_kv(self, meta: Optional[ConnectorMetadata]) -> None:
        pass

    def save_kv(self, meta: Optional[ConnectorMetadata]) -> None:
        pass

    def get_finished_sending(self) -> list:
        return []

    def get_finished_recving(self) -> list:
        return []

    def get_block_ids_with_load_errors(self) -> set:
        return set()


class Connector:
    """Pair of halves; in this engine both live in the rank process."""

    def __init__(self, scheduler: SchedulerConnectorBase, worker: WorkerConnectorBase):
        self.scheduler = scheduler
        self.worker = worker


# ---- signed control messages -------------------------------------------------------
def ipc_key() -> bytes:
    from .. import envs
    k = envs.B200_KV_IPC_KEY
    if k:
        return k.encode()
    k = os.environ.get("_B200_KV_IPC_KEY_RUNTIME")
    if not k:
        k = hashlib.sha256(os.urandom(32)).hexdigest()
        os.environ["_B200_KV_IPC_KEY_RUNTIME"] = k
    return k.encode()


def sign_message(obj: dict, key: Optional[bytes] = None) -> bytes:
    """JSON body + HMAC-SHA256 tag; control messages between engines are authenticated
    (reference: src/vllm_torchtpu/distributed/kv_transfer/zmq_shm_base.py:80-123 signs its pickles)."""
    body = json.dumps(obj, sort_keys=True).encode()
    tag = hmac.new(key or ipc_key(), body, hashlib.sha256).hexdigest().encode()
    return tag + b"." + body


def verify_message(raw: bytes, key: Optional[bytes] = None) -> dict:
    tag, _, body = raw.partition(b".")
    want = hmac.new(key or ipc_key(), body, hashlib.sha256).hexdigest().encode()
    if not hmac.compare_digest(tag, want):
        raise PermissionError("KV control message failed authentication")
    return json.loads(body)


def now() -> float:
    return time.monotonic()
