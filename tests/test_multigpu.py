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


def _max_lp_gap(a, b):
    return max(abs(x - y) for ra, rb in zip(a, b) for x, y in zip(ra, rb))


def _assert_same_distribution(x, y):
    """Two planes of the same model: the log-probability of every prompt token (prefill logits of all
    positions) and of the sampled tokens up to the first differing token (decode logits) agree."""
    assert x["status"] == 0 and y["status"] == 0
    assert _max_lp_gap(x["prompt_lp"], y["prompt_lp"]) < 0.08, _max_lp_gap(x["prompt_lp"], y["prompt_lp"])
    for ta, tb, la, lb in zip(x["tokens"], y["tokens"], x["sample_lp"], y["sample_lp"]):
        n = next((i for i, (p, q) in enumerate(zip(ta, tb)) if p != q), len(ta))
        assert n >= 1, (ta, tb)                     # the first sampled token comes from the prefill
        assert max(abs(p - q) for p, q in zip(la[:n], lb[:n])) < 0.08
    assert sum(a == b for a, b in zip(x["tokens"], y["tokens"])) >= 3, (x["tokens"], y["tokens"])


def test_tp2_engine_fused_plane_matches_nccl_plane_in_log_probabilities():
    _need(2)
    fused = _tokens(_run("tp_engine_worker.py", 2, "--lp"))
    nccl = _tokens(_run("tp_engine_worker.py", 2, "--lp", env={"B200_TP_COMM": "nccl"}))
    _assert_same_distribution(fused, nccl)


def test_tp2_engine_graph_decode_matches_single_gpu():
    _need(2)
    one = _tokens(_run("tp_engine_worker.py", 1))
    two = _tokens(_run("tp_engine_worker.py", 2))
    assert one["status"] == 0 and two["status"] == 0
    assert sum(a == b for a, b in zip(one["tokens"], two["tokens"])) >= 3, (one, two)


def test_tp2_persistent_decode_kernel_matches_per_layer_kernels():
    """The persistent decode kernel with its push plane between two GPUs against the per-layer path."""
    _need(2)
    mega = _tokens(_run("tp_engine_worker.py", 2, env={"B200_DECODE_MEGAKERNEL": "1"}))
    base = _tokens(_run("tp_engine_worker.py", 2))
    assert mega["persistent_decode"] and not base["persistent_decode"]
    assert mega["status"] == 0 and base["status"] == 0
    assert sum(a == b for a, b in zip(mega["tokens"], base["tokens"])) >= 3, (mega, base)
    assert all(a[:3] == b[:3] for a, b in zip(mega["tokens"], base["tokens"])), (mega, base)


def test_pp2_engine_on_gpus_matches_single_gpu():
    _need(2)
    one = _tokens(_run("tp_engine_worker.py", 1))
    pp = _tokens(_run("tp_engine_worker.py", 2, "--pp"))
    assert pp["status"] == 0
    assert sum(a == b for a, b in zip(one["tokens"], pp["tokens"])) >= 3, (one, pp)


def test_tp2_decode_context_parallel_on_gpus_matches_single_gpu_in_log_probabilities():
    """KV cache sharded by position over two GPUs: all-gathered query heads attend the local share
    (position-aware causal mask in the prefill kernel), partial results merged by their log-sum-exp."""
    _need(2)
    one = _tokens(_run("tp_engine_worker.py", 1, "--mqa", "--lp"))
    dcp = _tokens(_run("tp_engine_worker.py", 2, "--dcp", "--lp"))
    _assert_same_distribution(one, dcp)


def test_dp2_expert_parallel_lockstep_on_gpus():
    """Two replicas with their own requests, experts sharded over both GPUs, steps in lockstep."""
    _need(2)
    one = _tokens(_run("tp_engine_worker.py", 1, "--moe"))
    dp = _tokens(_run("tp_engine_worker.py", 2, "--moe", "--dpep"))
    assert dp["status"] == 0
    assert sum(a == b for a, b in zip(one["tokens"], dp["tokens"])) >= 3, (one, dp)


def test_tp2_server_requests_reach_both_gpus():
    _need(2)
    r = _run("serve_sync_worker.py", 2, "cuda")
    served = _tokens(r)["tokens"]
    assert len(served) == 3 and all(len(t) == 8 for t in served)


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
