#!/bin/bash
# One prefill engine (GPU 0) and one decode engine (GPU 1) behind a proxy on one host, registered with a
# controller.  Usage: run_disagg_single_host.sh MODEL
set -euo pipefail
MODEL=${1:?model path or preset}
PY=${PYTHON:-python}
$PY -m vllm_torchtpu_b200 controller --host 127.0.0.1 --port 7600 &
CTL=$!
sleep 1
CUDA_VISIBLE_DEVICES=0 $PY -m vllm_torchtpu_b200 serve "$MODEL" --port 8100 --kv-transfer-config \
  '{"kv_connector": "B200P2PConnector", "kv_role": "kv_producer", "engine_id": "P0",
    "kv_connector_extra_config": {"port": 9100, "controller": "127.0.0.1:7600", "http_url": "http://127.0.0.1:8100"}}' &
PRE=$!
CUDA_VISIBLE_DEVICES=1 $PY -m vllm_torchtpu_b200 serve "$MODEL" --port 8200 --kv-transfer-config \
  '{"kv_connector": "B200P2PConnector", "kv_role": "kv_consumer", "engine_id": "D0",
    "kv_connector_extra_config": {"port": 9200, "controller": "127.0.0.1:7600", "http_url": "http://127.0.0.1:8200"}}' &
DEC=$!
trap 'kill $CTL $PRE $DEC 2>/dev/null || true' EXIT
$PY -m vllm_torchtpu_b200 proxy --controller 127.0.0.1:7600 --port 8000
