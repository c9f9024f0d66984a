"""DecodeBenchConnector: pretends every prompt's KV already arrived, so a decode instance can be
benchmarked without a prefill instance (the blocks keep whatever the pool holds)."""
from __future__ import annotations

from .base import Connector, SchedulerConnectorBase, WorkerConnectorBase


class _Sched(SchedulerConnectorBase):
    def get_num_new_matched_tokens(self, request, num_cached: int):
        ext = request.num_prompt_tokens - 1 - num_cached
        return (ext, False) if ext > 0 else (0, False)


def create_decode_bench_connector(cfg, runner) -> Connector:
    return Connector(_Sched(), WorkerConnectorBase())
