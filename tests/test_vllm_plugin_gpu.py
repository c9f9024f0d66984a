"""The vLLM plugin on a GPU: the attention backend against the oracle through vLLM's own metadata
classes, and ``vllm.LLM`` end to end against the native engine on the same checkpoint."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
vllm = pytest.importorskip("vllm")

if not torch.cuda.is_available():
    pytest.skip("needs a GPU", allow_module_level=True)

HERE = os.path.dirname(os.path.abspath(__file__))


def test_backend_forward_matches_oracle_through_vllm_metadata():
    from types import SimpleNamespace
    from vllm.v1.attention.backend import CommonAttentionMetadata
    from vllm_torchtpu_b200.ops import reference as ref
    from vllm_torchtpu_b200.vllm_plugin.attention import B200AttentionBackend
    dev = "cuda"
    Hq, Hkv, D, bs = 8, 2, 128, 16
    q_lens, ctx = [1, 1, 1, 37, 90], [200, 17, 64, 0, 31]          # decodes first, then prefills
    R, T = len(q_lens), sum(q_lens)
    seq = [c + q for c, q in zip(ctx, q_lens)]
    nblk = [-(-s // bs) for s in seq]
    nb = sum(nblk) + 1
    g = torch.Generator(device=dev).manual_seed(0)
    cache = (torch.randn(nb, 2, Hkv, bs, D, device=dev, generator=g) * 0.5).bfloat16()
    bt = torch.zeros(R, max(nblk), dtype=torch.int32)
    off = 1
    for r in range(R):
        bt[r, :nblk[r]] = torch.arange(off, off + nblk[r], dtype=torch.int32)
        off += nblk[r]
    qsl = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    slots = torch.cat([bt[r, (ctx[r] + torch.arange(q_lens[r])) // bs].long() * bs + (ctx[r] + torch.arange(q_lens[r])) % bs
                       for r in range(R)])
    q = (torch.randn(T, Hq * D, device=dev, generator=g)).bfloat16()
    k = (torch.randn(T, Hkv * D, device=dev, generator=g) * 0.5).bfloat16()
    v = (torch.randn(T, Hkv * D, device=dev, generator=g) * 0.5).bfloat16()
    common = CommonAttentionMetadata(
        query_start_loc=qsl.to(dev), query_start_loc_cpu=qsl, seq_lens=torch.tensor(seq, dtype=torch.int32, device=dev),
        num_reqs=R, num_actual_tokens=T, max_query_len=max(q_lens), max_seq_len=max(seq),
        block_table_tensor=bt.to(dev), slot_mapping=slots.to(dev))
    builder = B200AttentionBackend.get_builder_cls()(SimpleNamespace(block_size=bs), ["l0"], None, torch.device(dev))
    meta = builder.build(0, common)
    assert meta.native.num_decode_reqs == 3
    impl = B200AttentionBackend.get_impl_cls()(Hq, D, D ** -0.5, Hkv)
    out = torch.empty(T, Hq * D, dtype=torch.bfloat16, device=dev)
    got_cache = cache.clone()
    impl.forward(None, q, k, v, got_cache, meta, out)
    # oracle: write K / V, then ragged paged attention on the CPU restatement
    want_cache = cache.clone().float().cpu()
    kc, vc = k.float().cpu().view(T, Hkv, D), v.float().cpu().view(T, Hkv, D)
    for t, s in enumerate(slots.tolist()):
        want_cache[s // bs, 0, :, s % bs] = kc[t]
        want_cache[s // bs, 1, :, s % bs] = vc[t]
    assert torch.equal(got_cache.float().cpu(), want_cache)
    want = ref.paged_attention(q.float().cpu().view(T, Hq, D), want_cache, bt, torch.tensor(seq, dtype=torch.int32), qsl,
                               D ** -0.5, num_reqs=R)
    err = (out.float().cpu().view(T, Hq, D) - want.float()).abs().max()
    assert err < 3e-2, float(err)


def test_vllm_llm_generates_through_the_plugin():
    env = dict(os.environ)
    env.update({"VLLM_LOGGING_LEVEL": "WARNING", "TOKENIZERS_PARALLELISM": "false"})
    r = subprocess.run([sys.executable, os.path.join(HERE, "workers", "vllm_plugin_worker.py")], capture_output=True,
                       text=True, timeout=420, env=env)
    line = next((l for l in r.stdout.splitlines() if l.startswith("RESULT ")), None)
    assert line is not None, r.stdout[-2000:] + r.stderr[-4000:]
    res = json.loads(line[7:])
    assert res["platform"] == "B200VllmPlatform"
    assert res["backend"].endswith("B200AttentionBackend")
    assert res["b200_launches"] > 0                      # this package's kernels ran inside the vLLM process
    same = sum(a == b for a, b in zip(res["want"], res["got"]))
    # vLLM's linear layers are library GEMMs and the random-init logits are nearly flat: one arg-max
    # may flip, after which that sequence diverges; a semantic error would change every sequence
    assert same >= 2, res
