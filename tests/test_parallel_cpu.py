"""Multi-rank engine paths on CPU (gloo, two processes): tensor, pipeline and expert parallelism
must generate the tokens of the single-process engine."""
import json
import os
import socket
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(nproc, *args, timeout=240, script="cpu_parallel_worker.py"):
    worker = os.path.join(HERE, "workers", script)
    if nproc == 1:
        cmd = [sys.executable, worker, *args]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), worker, *args]
    env = dict(os.environ)
    env.update({"OMP_NUM_THREADS": "2", "CUDA_VISIBLE_DEVICES": ""})
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    for line in r.stdout.splitlines():
        if line.startswith("RESULT "):
            return json.loads(line[7:])["tokens"]
    raise AssertionError(r.stdout[-2000:] + r.stderr[-3000:])


@pytest.fixture(scope="module")
def single():
    return _run(1, "tp", "tiny-llama")


def test_tp2_matches_single_process(single):
    assert _run(2, "tp", "tiny-llama") == single


def test_pp2_matches_single_process(single):
    assert _run(2, "pp", "tiny-llama") == single


def test_pp2_async_scheduling_matches_single_process(single):
    assert _run(2, "pp", "tiny-llama", "--async") == single


@pytest.mark.parametrize("flags", [(), ("--il2",)])
def test_tp2_decode_context_parallel_matches_single_process(flags):
    """The KV cache of every sequence dealt over two ranks by position (chunked prefill of a 70-token
    prompt in 64-token steps included): same tokens as one process with the whole cache."""
    assert _run(2, "dcp", "tiny-mqa", *flags) == _run(1, "tp", "tiny-mqa")


def test_ep2_moe_matches_single_process():
    assert _run(2, "ep", "tiny-moe") == _run(1, "tp", "tiny-moe")


def test_dp2_with_expert_parallel_lockstep_matches_single_process():
    """Two replicas with different (and different numbers of) requests, experts sharded over both:
    steps run in lockstep with padded rows, an idle replica runs placeholder batches."""
    assert _run(2, "dpep", "tiny-moe") == _run(1, "tp", "tiny-moe")


def test_dp2_with_expert_parallel_and_async_scheduling_terminates_together():
    """One step in flight per replica: the replicas still agree on when the group is idle, so nobody is
    left alone in a collective."""
    one = _run(1, "tp", "tiny-moe")
    assert _run(2, "dpep", "tiny-moe", "--async") == one
    # the benchmark's closed-loop client (requests added while others are in flight, two serves)
    assert _run(2, "dpep", "tiny-moe", "--async", "--closed-loop") == one


def test_prefill_context_parallel_in_the_engine_matches_single_process(single):
    """Prefill chunks cut into head-tail pieces over two ranks (a 23-token prompt in one chunk, a 70-token one in
    chunks of 64 + 6, the short prompt and all decode steps replicated): every rank's cache is completed from the
    gathered keys / values and all ranks sample the tokens of the single-process engine."""
    assert _run(2, "pcp", "tiny-llama") == single
    assert _run(2, "pcp", "tiny-llama", "--async") == single
    # two PCP ranks of two tensor-parallel ranks each
    assert _run(4, "pcp", "tiny-llama", "--tp2", timeout=400) == single


def test_pipelined_moe_plane_matches_single_process():
    """The expert-parallel all-gather plane in token chunks whose collectives are started ahead of / finished
    behind the neighbouring chunks' expert GEMMs: same tokens, under TP-coupled EP and under DP lockstep."""
    one = _run(1, "tp", "tiny-moe")
    assert _run(2, "ep", "tiny-moe", "--moe-pipeline") == one
    assert _run(2, "dpep", "tiny-moe", "--moe-pipeline") == one


def test_dp2_vocab_sharded_over_the_replicas_matches_single_process():
    """Embedding table and lm_head sharded over the two replicas: ids are gathered and embeddings
    reduce-scattered, hidden rows gathered (padded to the agreed row count) and logits exchanged by all-to-all;
    uneven request counts, a replica that runs placeholder steps, and async scheduling."""
    one = _run(1, "tp", "tiny-moe")
    assert _run(2, "dpep", "tiny-moe", "--dp-vocab") == one
    assert _run(2, "dpep", "tiny-moe", "--dp-vocab", "--async", "--closed-loop") == one


def test_tp2_lora_matches_single_process(single):
    """Adapters sharded like the base weights (B rows of column-parallel targets, A columns of row-parallel
    targets with the partial update added before the all-reduce) reproduce the one-process tokens."""
    one = _run(1, "tplora", "tiny-llama")
    assert _run(2, "tplora", "tiny-llama") == one
    assert one[1] == single[1] and one[0] != single[0]          # request 1 runs without the adapter


def test_tp2_pads_query_heads_that_do_not_divide():
    """3 query heads on 2 ranks: every KV group is zero-padded to 4 heads (q_proj rows and o_proj columns),
    the KV head is replicated, and the tokens equal the one-process run."""
    assert _run(2, "tp", "tiny-odd-heads") == _run(1, "tp", "tiny-odd-heads")


@pytest.mark.parametrize("flags", [(), ("--async",)])
def test_tp2_server_requests_reach_every_rank(single, flags):
    """HTTP requests arrive at rank 0 only; it broadcasts them step by step and the follower rank runs
    the same steps, so the completions equal the one-process tokens."""
    assert _run(2, "cpu", *flags, script="serve_sync_worker.py") == single


def test_export_from_a_tensor_parallel_engine(tmp_path):
    """A TP2 engine loaded from a checkpoint exports its serving directory (rank 0 copies the checkpoint, the
    plan records the degrees); the directory validates and a single-rank engine loaded from it repeats the tokens."""
    import numpy as np
    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.engine.llm import LLM
    from vllm_torchtpu_b200.export import load_serving_dir, validate_serving_dir
    from vllm_torchtpu_b200.models.loader import save_hf_checkpoint
    donor = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    ckpt = str(tmp_path / "ckpt")
    hf = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4,
          "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 512, "vocab_size": 1024,
          "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 256, "torch_dtype": "float32"}
    save_hf_checkpoint(donor.engine.runner.model, ckpt, hf)
    out = str(tmp_path / "serving")
    toks = _run(2, "tp", ckpt, "--export", out)
    assert validate_serving_dir(out) == []
    meta = json.load(open(os.path.join(out, "metadata.json")))
    assert meta["parallel"]["tensor_parallel_size"] == 2 and meta["parallel"]["world_size"] == 2
    assert "serving_checkpoint/model.safetensors" in meta["manifest"]
    llm = load_serving_dir(out, device="cpu", init_dist=False, tensor_parallel_size=1)
    rng = np.random.RandomState(0)
    prompts = [rng.randint(0, 1024, size=n).tolist() for n in (5, 23, 70)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    assert [o.outputs[0].token_ids for o in llm.generate(prompts, sp)] == toks
    meta["parallel"]["world_size"] = 3
    json.dump(meta, open(os.path.join(out, "metadata.json"), "w"))
    assert any("parallel plan" in p for p in validate_serving_dir(out))


def test_dp_vocab_exchange_with_an_uneven_vocabulary():
    """Three replicas as threads over an in-memory communicator, a vocabulary that does not divide by three,
    different row counts padded to an agreed one: embeddings and logits equal the unsharded computation."""
    import threading

    import torch

    from vllm_torchtpu_b200.parallel.dp_vocab import DpVocabParallel
    n, V, H, T = 3, 10, 8, 5
    shared, bar = [None] * n, threading.Barrier(n)

    class ThreadComm:
        def __init__(self, rank):
            self.size, self.rank = n, rank

        def _swap(self, x):
            shared[self.rank] = x
            bar.wait()
            got = list(shared)
            bar.wait()
            return got

        def all_gather(self, x, dim=0):
            return torch.cat(self._swap(x), dim)

        def reduce_scatter(self, x, dim=0):
            tot = sum(self._swap(x))
            k = tot.shape[0] // n
            return tot[self.rank * k:(self.rank + 1) * k].clone()

        def all_to_all(self, x, split_dim=0, concat_dim=0):
            got = self._swap(x.chunk(n, dim=split_dim))
            return torch.cat([got[src][self.rank] for src in range(n)], dim=concat_dim)

    g = torch.Generator().manual_seed(0)
    table, head = torch.randn(V, H, generator=g), torch.randn(V, H, generator=g)
    ids = [torch.randint(0, V, (T,), generator=g) for _ in range(n)]
    rows = [torch.randn(r + 1, H, generator=g) for r in range(n)]          # 1, 2 and 3 rows
    out, errs = [None] * n, []

    def work(r):
        try:
            dv = DpVocabParallel(ThreadComm(r), V)
            t, h = dv.shard_rows(table), dv.shard_rows(head)
            assert t.shape == (4, H) and dv.shard_rows(t) is t              # padded shard; idempotent
            dv.rows = 4
            out[r] = (dv.embed(ids[r], t), dv.logits(rows[r], h))
            dv.rows = 2
            if r == 2:
                try:
                    dv.logits(rows[r], h)
                    errs.append("more rows than agreed were accepted")
                except RuntimeError:
                    pass
        except Exception as e:                       # noqa: BLE001 - reported by the main thread
            errs.append(repr(e))
            bar.abort()
    ts = [threading.Thread(target=work, args=(r,)) for r in range(n)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert not errs, errs
    for r in range(n):
        torch.testing.assert_close(out[r][0], table[ids[r]])
        torch.testing.assert_close(out[r][1], rows[r] @ head.T, rtol=1e-5, atol=1e-5)
        assert out[r][1].shape == (r + 1, V)
