"""Multi-GPU tests: each spawns one process per GPU with torch.distributed.run on 127.0.0.1.
Skipped on machines with fewer than 2 GPUs."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(script, nproc, *args, env=None, timeout=240):
    e = dict(os.environ)
    e.update({"NCCL_NVLS_ENABLE": "0", "B200_SPIN_LIMIT": "300000"})
    e.update(env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(HERE, "workers", script), *args]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e)


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_fused_gemm_all_reduce_matches_nccl(nproc):
    _need(nproc)
    r = _run("tp_fused_worker.py", nproc)
    assert "TP_FUSED_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def _tokens(r):
    for line in r.stdout.splitlines():
        if line.startswith("RESULT "):
            return json.loads(line[7:])
    raise AssertionError(r.stdout[-3000:] + r.stderr[-3000:])


def test_tp2_engine_fused_plane_equals_nccl_plane():
    _need(2)
    fused = _tokens(_run("tp_engine_worker.py", 2))
    nccl = _tokens(_run("tp_engine_worker.py", 2, env={"B200_TP_COMM": "nccl"}))
    assert fused["status"] == 0
    # both planes sum bf16 partials in fp32 in rank order, so the tokens agree
    same = sum(a == b for a, b in zip(fused["tokens"], nccl["tokens"]))
    assert same >= 3, (fused, nccl)


@pytest.mark.parametrize("nproc", [2, 4])
def test_fused_expert_parallel_plane_matches_dense_moe(nproc):
    _need(nproc)
    r = _run("ep_fused_worker.py", nproc)
    assert "EP_FUSED_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_tp2_moe_engine_fused_ep_plane_equals_gather_plane():
    _need(2)
    fused = _tokens(_run("tp_engine_worker.py", 2, "--moe"))
    gathered = _tokens(_run("tp_engine_worker.py", 2, "--moe", env={"B200_MOE_FUSED_EP": "0"}))
    assert fused["status"] == 0 and gathered["status"] == 0
    same = sum(a == b for a, b in zip(fused["tokens"], gathered["tokens"]))
    assert same >= 3, (fused, gathered)


def test_ipc_transport_pulls_blocks_gpu_to_gpu():
    """Data plane of disaggregated prefill / decode: the consumer process maps the producer's pool
    (CUDA IPC) and one kernel copies the listed blocks of every layer over NVLink."""
    _need(2)
    r = _run("ipc_pull_worker.py", 2)
    assert "IPC_PULL_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
