"""Several connectors at once (disaggregation + offload): loads are taken from the first
connector that reports a hit, saves and notifications go to all of them
(reference: src/vllm_torchtpu/distributed/kv_transfer/tpu_multi_connector.py:24-96)."""
from __future__ import annotations

import copy

from .base import Connector, ConnectorMetadata, SchedulerConnectorBase, WorkerConnectorBase


class _MultiSched(SchedulerConnectorBase):
    def __init__(self, parts):
        self.parts = parts
        self._owner: dict = {}

    def get_num_new_matched_tokens(self, request, num_cached):
        for i, p in enumerate(self.parts):
            n, is_async = p.get_num_new_matched_tokens(request, num_cached)
            if n > 0:
                self._owner[request.request_id] = i
                return n, is_async
        return 0, False

    def request_not_admitted(self, request):
        i = self._owner.pop(request.request_id, None)
        if i is not None:
            self.parts[i].request_not_admitted(request)

    def update_state_after_alloc(self, request, block_ids, num_external):
        i = self._owner.get(request.request_id)
        if i is not None:
            self.parts[i].update_state_after_alloc(request, block_ids, num_external)

    def build_connector_meta(self, out):
        return [p.build_connector_meta(out) for p in self.parts]

    def request_finished(self, request, block_ids):
        delay, params = False, None
        for p in self.parts:
            d, pr = p.request_finished(request, block_ids)
            delay |= d
            params = params or pr
        self._owner.pop(request.request_id, None)
        return delay, params

    def is_load_done(self, request):
        i = self._owner.get(request.request_id)
        return True if i is None else self.parts[i].is_load_done(request)


class _MultiWorker(WorkerConnectorBase):
    def __init__(self, parts):
        self.parts = parts

    def start_load_kv(self, meta):
        for p, m in zip(self.parts, meta or [None] * len(self.parts)):
            p.start_load_kv(m)

    def save_kv(self, meta):
        for p, m in zip(self.parts, meta or [None] * len(self.parts)):
            p.save_kv(m)

    def get_finished_sending(self):
        return [r for p in self.parts for r in p.get_finished_sending()]

    def get_finished_recving(self):
        return [r for p in self.parts for r in p.get_finished_recving()]

    def get_block_ids_with_load_errors(self):
        out = set()
        for p in self.parts:
            out |= p.get_block_ids_with_load_errors()
        return out


def create_multi_connector(cfg, runner, **kw) -> Connector:
    from .factory import create_connector
    subs = []
    for sub in cfg.kv_transfer["kv_connector_extra_config"]["connectors"]:
        c2 = copy.copy(cfg)
        c2.kv_transfer = sub
        subs.append(create_connector(c2, runner, **kw))
    c = Connector(_MultiSched([s.scheduler for s in subs]), _MultiWorker([s.worker for s in subs]))
    c.parts = subs
    return c
