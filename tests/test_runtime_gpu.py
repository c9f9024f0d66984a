"""Runtime-side kernels on one GPU: a bounded device wait that runs out (status word, no hang), the
paged-KV block mover with its range check and NaN screen, the KV write of the vLLM backend."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a GPU", allow_module_level=True)

from vllm_torchtpu_b200.kv_transfer.transport import PoolInfo, TransferError, copy_blocks, nan_blocks  # noqa: E402
from vllm_torchtpu_b200.ops import cuda, cuda_misc  # noqa: E402

DEV = "cuda"


def test_flag_wait_runs_out_and_reports_status_without_hanging():
    """The consumer of the push plane waits for tile flags of an epoch nobody raises: the wait gives up
    after its iteration limit, the kernel returns, the status word reads 'waited for a flag' and the
    context keeps working."""
    T, N, world, max_tiles = 4, 1024, 2, 64
    recv = torch.zeros(world * T * N, dtype=torch.bfloat16, device=DEV)
    flags = torch.zeros(world * max_tiles, dtype=torch.int32, device=DEV)          # never raised
    ctrl = torch.tensor([1, 0, 0, 0], dtype=torch.int32, device=DEV)               # producers "completed" epoch 1
    residual = torch.ones(T, N, dtype=torch.bfloat16, device=DEV)
    weight = torch.ones(N, dtype=torch.bfloat16, device=DEV)
    y = torch.full((T, N), 7.0, dtype=torch.bfloat16, device=DEV)
    ws = cuda.Workspace.get(torch.device(DEV))
    assert cuda.check_status() == 0
    stride = (T * N * 2 + 255) // 256 * 256
    cuda._check(cuda.lib().b200_reduce_pushed_rms_norm(
        cuda._p(recv), ctypes.c_ulonglong(stride), cuda._p(flags), ctypes.c_int(max_tiles), cuda._p(ctrl),
        cuda._p(residual), cuda._p(weight), cuda._p(y), ctypes.c_int(T), ctypes.c_int(N), ctypes.c_int(world),
        ctypes.c_float(1e-5), cuda._p(ws.status), ctypes.c_uint(2000), cuda._stream()), "reduce_pushed_rms_norm")
    torch.cuda.synchronize()                       # returns: the wait was bounded
    assert cuda.check_status() == 5                # ST_TIMEOUT_FLAG, and the word is cleared by the read
    assert torch.equal(y, torch.full_like(y, 7.0)) # rows whose flags never came are left untouched
    # the context is intact: the next launch works and reports no status
    x = torch.randn(T, N, device=DEV).bfloat16()
    out = cuda.rms_norm(x, weight, 1e-5)
    want = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)
    assert (out.float() - want).abs().max() < 2e-2 and cuda.check_status() == 0


def _pools(nb_src=12, nb_dst=9, layers=3, shape=(2, 2, 16, 64)):
    g = torch.Generator(device=DEV).manual_seed(0)
    src = [torch.randn((nb_src,) + shape, device=DEV, generator=g).bfloat16() for _ in range(layers)]
    dst = [torch.zeros((nb_dst,) + shape, dtype=torch.bfloat16, device=DEV) for _ in range(layers)]
    return src, dst


def test_block_copy_between_pools_and_pinned_host():
    src, dst = _pools()
    s_ids, d_ids = [3, 0, 11, 7], [1, 8, 2, 5]
    copy_blocks(PoolInfo("a", src), PoolInfo("b", dst), s_ids, d_ids)
    torch.cuda.synchronize()
    for a, b in zip(src, dst):
        assert torch.equal(b[d_ids], a[s_ids])
        untouched = [i for i in range(b.shape[0]) if i not in d_ids]
        assert int(b[untouched].abs().sum()) == 0
    # device -> pinned host slab -> another device pool (the offload tier's two directions)
    host = [torch.zeros((6,) + tuple(src[0].shape[1:]), dtype=torch.bfloat16, pin_memory=True) for _ in src]
    copy_blocks(PoolInfo("a", src), PoolInfo("h", host), [2, 4], [5, 0])
    torch.cuda.synchronize()
    assert all(torch.equal(h[[5, 0]], a[[2, 4]].cpu()) for a, h in zip(src, host))
    back = [torch.zeros_like(d) for d in dst]
    copy_blocks(PoolInfo("h", host), PoolInfo("c", back), [5, 0], [3, 4])
    torch.cuda.synchronize()
    assert all(torch.equal(b[[3, 4]], a[[2, 4]]) for a, b in zip(src, back))
    with pytest.raises(TransferError):
        copy_blocks(PoolInfo("a", src), PoolInfo("b", dst), [12], [0])
    assert cuda.check_status() == 0


@pytest.mark.parametrize("H,tp_p,tp_c", [(8, 4, 2), (8, 2, 4), (2, 4, 1), (4, 1, 2)])
def test_head_range_spans_move_between_pools_of_different_tp_degree(H, tp_p, tp_c):
    """The span copy kernel assembles a consumer rank's blocks from the producer ranks that hold its heads."""
    from vllm_torchtpu_b200.kv_transfer.reshard import KVGeometry, plan_pull
    from vllm_torchtpu_b200.kv_transfer.transport import copy_block_spans
    g = torch.Generator(device=DEV).manual_seed(0)
    N, bs, D, L = 10, 16, 128, 3
    full = [torch.randn((N, 2, H, bs, D), device=DEV, generator=g).bfloat16() for _ in range(L)]

    def rank_pool(tp, rank):
        h = max(1, H // tp)
        lo = (rank // max(1, tp // H)) * h
        return [t[:, :, lo:lo + h].contiguous() for t in full]
    prod = [PoolInfo(f"p{r}", rank_pool(tp_p, r)) for r in range(tp_p)]
    src_ids, dst_ids = [4, 1, 9, 3], [0, 5, 2, 7]
    for cr in range(tp_c):
        want = rank_pool(tp_c, cr)
        dst = PoolInfo("c", [torch.zeros_like(t) for t in want])
        plan = plan_pull(KVGeometry.of_cache(dst.layers[0], tp_c, cr, H),
                         KVGeometry.of_cache(prod[0].layers[0], tp_p, 0, H))
        for pr, span in plan:
            copy_block_spans(prod[pr], dst, src_ids, dst_ids, span)
        torch.cuda.synchronize()
        for got, w in zip(dst.layers, want):
            assert torch.equal(got[dst_ids], w[src_ids])
            untouched = [i for i in range(N) if i not in dst_ids]
            assert int(got[untouched].abs().sum()) == 0
    assert cuda.check_status() == 0


def test_nan_screen_flags_exactly_the_poisoned_blocks():
    src, _ = _pools()
    assert nan_blocks(PoolInfo("a", src), [0, 1, 2, 3]) == []
    src[1][2, 0, 1, 3, 5] = float("nan")
    src[2][9, 1, 0, 0, 0] = float("inf")
    assert nan_blocks(PoolInfo("a", src), [0, 2, 5, 9, 11]) == [2, 9]
    cpu = [t.cpu() for t in src]
    assert nan_blocks(PoolInfo("cpu", cpu), [0, 2, 5, 9, 11]) == [2, 9]


@pytest.mark.parametrize("slot_dtype", [torch.int32, torch.int64])
def test_kv_write_into_paged_cache(slot_dtype):
    T, Hkv, D, bs, nb = 37, 2, 128, 16, 9
    g = torch.Generator(device=DEV).manual_seed(2)
    qkv = torch.randn(T, (4 + 2 * Hkv) * D, device=DEV, generator=g).bfloat16()       # k / v are strided views
    k = qkv[:, 4 * D:(4 + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (4 + Hkv) * D:].view(T, Hkv, D)
    cache = torch.zeros(nb, 2, Hkv, bs, D, dtype=torch.bfloat16, device=DEV)
    slots = torch.randperm(nb * bs, device=DEV)[:T].to(slot_dtype)
    slots[5] = -1
    cuda_misc.kv_write(k, v, cache, slots)
    torch.cuda.synchronize()
    want = torch.zeros_like(cache)
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            want[s // bs, 0, :, s % bs] = k[t]
            want[s // bs, 1, :, s % bs] = v[t]
    assert torch.equal(cache, want)


def test_vocab_parallel_argmax_exchange():
    """Every rank reduces its vocabulary shard to (value, index) pairs; the pairs of all ranks pick the
    global arg-max (first index on ties).  The shards of a 4-rank layout are emulated on one GPU."""
    from vllm_torchtpu_b200.ops import cuda_tp
    R, V, world = 9, 4096, 4
    g = torch.Generator(device=DEV).manual_seed(4)
    logits = torch.randn(R, V, device=DEV, generator=g).bfloat16()
    logits[3, 100] = logits[3, 3000] = 9.0            # a tie across shards
    shard = V // world
    vals, idxs = zip(*[cuda_tp.argmax_pair(logits[:, r * shard:(r + 1) * shard]) for r in range(world)])
    got = cuda_tp.select_best(torch.stack(vals).contiguous(), torch.stack(idxs).contiguous(), shard)
    want = logits.float().argmax(-1)
    assert torch.equal(got.long(), want) and int(got[3]) == 100


def test_bounds_checked_attention_library_counts_bad_block_ids():
    """The attention kernels built with -DB200_BOUNDS_CHECK: clean tables count nothing, an id outside the
    pool is clamped and counted (a child process, since the library is chosen when it is first loaded)."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    r = subprocess.run([sys.executable, os.path.join(here, "workers", "bounds_check_worker.py")],
                       capture_output=True, text=True, timeout=240)
    assert "BOUNDS_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_kernel_library_can_be_reloaded_between_requests():
    """reload_kernels maps the library again under a fresh name, re-captures the decode graphs, and the engine
    keeps generating the same tokens."""
    import torch

    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.config import ModelConfig
    from vllm_torchtpu_b200.engine.llm import LLM
    from vllm_torchtpu_b200.ops import cuda
    cfg = ModelConfig(name="t", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=2048, max_model_len=256, dtype=torch.bfloat16)
    llm = LLM(cfg, device="cuda", max_num_seqs=4, max_num_batched_tokens=128, num_gpu_blocks_override=128,
              init_dist=False)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    before = [o.outputs[0].token_ids for o in llm.generate([[1, 2, 3, 4, 5]], sp)]
    again = [o.outputs[0].token_ids for o in llm.generate([[1, 2, 3, 4, 5]], sp)]
    assert again == before                                   # the engine is deterministic across calls
    old = cuda.lib()
    llm.engine.reload_kernels()
    assert cuda.lib() is not old
    after = [o.outputs[0].token_ids for o in llm.generate([[1, 2, 3, 4, 5]], sp)]
    assert after == before and cuda.check_status() == 0
