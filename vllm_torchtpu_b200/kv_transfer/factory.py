"""Connector factory keyed by the ``kv_connector`` name of ``--kv-transfer-config``
(the reference registers its connectors with vLLM's KVConnectorFactory and whitelists them in the
platform, reference: src/vllm_torchtpu/platforms/tpu_platform.py:443-451,1270-1295)."""
from __future__ import annotations

from .base import Connector


def create_connector(cfg, runner, **kw) -> Connector:
    name = (cfg.kv_transfer or {}).get("kv_connector")
    if name in ("B200P2PConnector", "B200HostConnector"):
        from .p2p_connector import create_p2p_connector
        if name == "B200HostConnector" and kw.get("transport") is None:
            # same protocol, blocks handed over through this process's address space instead of CUDA IPC
            # (producer and consumer engines in one process, or pools that live in host memory)
            from .transport import LocalTransport
            engine_id = (cfg.kv_transfer or {}).get("engine_id")
            if engine_id:
                kw["transport"] = LocalTransport(engine_id)
            else:
                cfg.kv_transfer.setdefault("kv_connector_extra_config", {}).setdefault("transport", "local")
        return create_p2p_connector(cfg, runner, **kw)
    if name == "B200OffloadingConnector":
        from .offload import create_offloading_connector
        return create_offloading_connector(cfg, runner, **kw)
    if name == "B200MultiConnector":
        from .multi import create_multi_connector
        return create_multi_connector(cfg, runner, **kw)
    if name == "DecodeBenchConnector":
        from .decode_bench import create_decode_bench_connector
        return create_decode_bench_connector(cfg, runner)
    raise ValueError(f"unknown kv_connector {name!r}")
