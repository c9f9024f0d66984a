"""CUDA kernels vs the plain-PyTorch fp32 statements of the same ops."""
import math

import pytest
import torch

from vllm_torchtpu_b200.ops import reference as ref
from vllm_torchtpu_b200.runner.attn_metadata import AttentionMetadata

pytestmark = pytest.mark.gpu
DEV = "cuda"


def cu():
    from vllm_torchtpu_b200.ops import cuda
    return cuda


def _close(a, b, rtol=2e-2, atol=2e-2):
    torch.testing.assert_close(a.float(), b.float(), rtol=rtol, atol=atol)


@pytest.mark.parametrize("T,H", [(1, 256), (7, 4096), (64, 8192), (33, 1000 * 8)])
def test_rms_norm(T, H):
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(T, H, device=DEV, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device=DEV, generator=g)).bfloat16()
    _close(cu().rms_norm(x, w, 1e-5), ref.rms_norm(x, w, 1e-5), 1e-2, 1e-2)
    r = torch.randn(T, H, device=DEV, generator=g).bfloat16()
    want_y, want_r = ref.fused_add_rms_norm(x, r.clone(), w, 1e-5)
    got_y, got_r = cu().fused_add_rms_norm(x, r, w, 1e-5)
    assert torch.equal(got_r, want_r)
    _close(got_y, want_y, 1e-2, 1e-2)


def test_silu_and_mul():
    x = torch.randn(77, 2 * 1536, device=DEV).bfloat16()
    _close(cu().silu_and_mul(x), ref.silu_and_mul(x), 1e-2, 1e-2)


def test_embedding_and_rows():
    table = torch.randn(1000, 512, device=DEV).bfloat16()
    ids = torch.randint(0, 1000, (50,), device=DEV, dtype=torch.int32)
    src = torch.full((50,), -1, device=DEV, dtype=torch.int32)
    last = torch.randint(0, 1000, (8,), device=DEV, dtype=torch.int32)
    src[3], src[10] = 2, 7
    want_ids = ids.clone()
    want_ids[3], want_ids[10] = last[2], last[7]
    assert torch.equal(cu().embedding(ids, table, src, last), table[want_ids.long()])
    idx = torch.tensor([4, 0, 49], device=DEV, dtype=torch.int32)
    h, r = cu().gather_rows(table[:50].contiguous(), table[50:100].contiguous(), idx)
    assert torch.equal(h, table[:50][idx.long()]) and torch.equal(r, table[50:100][idx.long()])
    toks = torch.tensor([11, 22, 33], device=DEV, dtype=torch.int32)
    slots = torch.tensor([5, -1, 0], device=DEV, dtype=torch.int32)
    cu().scatter_tokens(toks, slots, last)
    assert last[5] == 11 and last[0] == 33


@pytest.mark.parametrize("D,interleaved,qk_norm", [(128, False, False), (128, False, True), (64, True, False)])
def test_rope_and_cache(D, interleaved, qk_norm):
    T, Hq, Hkv, bs, nb = 37, 8, 2, 16, 12
    g = torch.Generator(device=DEV).manual_seed(1)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=DEV, generator=g).bfloat16()
    pos = torch.randint(0, 5000, (T,), device=DEV, dtype=torch.int32)
    inv = ref.rope_inv_freq(D, 500000.0).to(DEV)
    slots = torch.randperm(nb * bs, device=DEV)[:T].to(torch.int32)
    slots[5] = -1
    qn = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16() if qk_norm else None
    kn = (1 + 0.1 * torch.randn(D, device=DEV)).bfloat16() if qk_norm else None
    c1 = torch.zeros(nb, 2, Hkv, bs, D, device=DEV, dtype=torch.bfloat16)
    c2 = c1.clone()
    q1 = cu().rope_and_cache(qkv, pos, inv, c1, slots, Hq, Hkv, D, interleaved, qn, kn, 1e-6)
    q2 = ref.rope_and_cache(qkv, pos, inv, c2, slots, Hq, Hkv, D, interleaved, qn, kn, 1e-6)
    _close(q1, q2, 2e-2, 2e-2)
    _close(c1, c2, 2e-2, 2e-2)


def _attn_case(q_lens, ctx_lens, Hq, Hkv, D, bs=16, window=None, softcap=None, sinks=False, num_decode=0,
               kv_fp8=False):
    g = torch.Generator(device=DEV).manual_seed(2)
    R = len(q_lens)
    seq = [q + c for q, c in zip(q_lens, ctx_lens)]
    maxb = max(-(-s // bs) for s in seq) + 1
    nb = sum(-(-s // bs) for s in seq) + 2
    cache = (torch.randn(nb, 2, Hkv, bs, D, device=DEV, generator=g) * 0.5).bfloat16()
    k_scale, v_scale = 1.0, 1.0
    if kv_fp8:
        # e4m3 cache with per-tensor scales: the oracle dequantises the same bytes in fp32
        k_scale, v_scale = 0.02, 0.03
        cache = torch.stack([cache[:, 0].float() / k_scale, cache[:, 1].float() / v_scale],
                            1).to(torch.float8_e4m3fn)
    perm = (torch.randperm(nb - 1, device=DEV) + 1).to(torch.int32)
    bt = torch.zeros(R, maxb, dtype=torch.int32, device=DEV)
    off = 0
    for r, s in enumerate(seq):
        n = -(-s // bs)
        bt[r, :n] = perm[off:off + n]
        off += n
    T = sum(q_lens)
    q = torch.randn(T, Hq, D, device=DEV, generator=g).bfloat16()
    qsl = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    sl = torch.tensor(seq, dtype=torch.int32, device=DEV)
    meta = AttentionMetadata(positions=None, slot_mapping=None, block_tables=bt, seq_lens=sl,
                             query_start_loc=qsl, num_reqs=R, num_tokens=T, num_decode_reqs=num_decode,
                             max_query_len=max(q_lens), max_seq_len=max(seq),
                             padded_num_reqs=R, padded_num_tokens=T,
                             query_start_loc_cpu=qsl.cpu().long(), seq_lens_cpu=sl.cpu().long())
    sk = torch.randn(Hq, device=DEV) if sinks else None
    scale = D ** -0.5
    got, got_lse = cu().paged_attention(q, cache, meta, scale, sliding_window=window, softcap=softcap,
                                        sinks=sk, k_scale=k_scale, v_scale=v_scale, return_lse=True)
    want, want_lse = ref.paged_attention(q, cache, bt, sl, qsl, scale, num_reqs=R, sliding_window=window,
                                         softcap=softcap, sinks=sk, k_scale=k_scale, v_scale=v_scale,
                                         return_lse=True)
    _close(got, want, 2e-2, 2e-2)
    fin = torch.isfinite(want_lse)
    _close(got_lse[fin], want_lse[fin], 1e-2, 1e-2)


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (8, 1, 128), (4, 2, 64)])
def test_attention_decode(Hq, Hkv, D):
    ctx = [0, 15, 16, 100, 1023, 2500, 7]
    _attn_case([1] * len(ctx), ctx, Hq, Hkv, D, num_decode=len(ctx))


def test_attention_decode_many_splits(monkeypatch):
    monkeypatch.setenv("B200_ATTN_SPLIT_KV", "5")
    from vllm_torchtpu_b200 import envs
    envs.reset()
    _attn_case([1, 1, 1], [3000, 1, 77], 16, 4, 128, num_decode=3)


def test_attention_spec_verify_rows():
    # q_len 3 with 4 heads per kv head = 12 rows in the 16-row decode tile
    _attn_case([3, 3, 1], [50, 700, 9], 8, 2, 128, num_decode=3)


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (4, 2, 64)])
def test_attention_prefill_and_mixed(Hq, Hkv, D):
    _attn_case([1, 1, 200, 64, 65, 1, 333], [40, 900, 0, 128, 37, 0, 1000], Hq, Hkv, D, num_decode=2)


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (4, 2, 64)])
def test_attention_fp8_kv_cache(Hq, Hkv, D):
    ctx = [0, 15, 16, 100, 1023, 2500, 7]
    _attn_case([1] * len(ctx), ctx, Hq, Hkv, D, num_decode=len(ctx), kv_fp8=True)
    _attn_case([1, 1, 200, 64, 65, 1, 333], [40, 900, 0, 128, 37, 0, 1000], Hq, Hkv, D, num_decode=2,
               kv_fp8=True)
    _attn_case([1, 130, 17], [500, 300, 0], Hq, Hkv, D, window=128, sinks=True, num_decode=1, kv_fp8=True)


def test_attention_window_softcap_sinks():
    _attn_case([1, 130, 17], [500, 300, 0], 8, 2, 128, window=128, num_decode=1)
    _attn_case([1, 130], [500, 300], 8, 2, 128, softcap=30.0, num_decode=1)
    _attn_case([1, 130], [500, 300], 8, 2, 128, sinks=True, num_decode=1)


def test_argmax_and_sampling():
    R, V = 9, 128256
    g = torch.Generator(device=DEV).manual_seed(3)
    logits = (torch.randn(R, V, device=DEV, generator=g) * 3).bfloat16()
    assert torch.equal(cu().argmax(logits).long(), logits.float().argmax(-1))
    temp = torch.tensor([0.0, 0.7, 1.0, 1.3, 0.5, 1.0, 1.0, 0.9, 2.0], device=DEV)
    top_k = torch.tensor([0, 50, 0, 5, 1, 0, 1000, 20, 0], device=DEV, dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 0.9, 0.8, 1.0, 0.5, 0.95, 1.0, 1.0], device=DEV)
    u = cu().philox_uniform(R, V, 7, 3, DEV)
    assert 0.45 < float(u.mean()) < 0.55 and float(u.min()) > 0 and float(u.max()) < 1
    got = cu().sample(logits, temp, top_k, top_p, uniform=u)
    want = ref.sample(logits, temp, top_k, top_p, uniform=u)
    assert torch.equal(got.long(), want)
    step = torch.tensor([3], dtype=torch.int64, device=DEV)
    got2 = cu().sample(logits, temp, top_k, top_p, uniform=None, seed=7, step_tensor=step)
    assert torch.equal(got2, got)


def test_sampling_cluster_kernel_on_an_odd_vocabulary():
    """Rows of odd length start on odd element offsets (two-byte loads instead of pairs) and the last CTA of
    the cluster holds a ragged tail."""
    R, V = 6, 50001
    g = torch.Generator(device=DEV).manual_seed(5)
    logits = (torch.randn(R, V, device=DEV, generator=g) * 2.5).bfloat16()
    temp = torch.tensor([0.8, 0.0, 1.0, 1.2, 0.6, 1.0], device=DEV)
    top_k = torch.tensor([40, 0, 0, 3, 0, 2000], device=DEV, dtype=torch.int32)
    top_p = torch.tensor([0.9, 1.0, 0.7, 1.0, 1.0, 0.99], device=DEV)
    u = cu().philox_uniform(R, V, 11, 1, DEV)
    got = cu().sample(logits, temp, top_k, top_p, uniform=u)
    want = ref.sample(logits, temp, top_k, top_p, uniform=u)
    assert torch.equal(got.long(), want)


def test_logprobs():
    R, V = 5, 32000
    logits = torch.randn(R, V, device=DEV).bfloat16()
    tok = torch.randint(0, V, (R,), device=DEV)
    a = cu().gather_logprobs(logits, tok, 5)
    b = ref.gather_logprobs(logits, tok, 5)
    _close(a[0], b[0], 1e-3, 1e-3)
    _close(a[1], b[1], 1e-3, 1e-3)
    # bf16 logits tie often: ids may differ among equal values, the values they point at may not
    lf = logits.float()
    assert torch.equal(lf.gather(1, a[2].long()), lf.gather(1, b[2]))
    assert torch.equal(a[3].long(), b[3])


@pytest.mark.parametrize("Hq,Hkv,D", [(16, 16, 64), (8, 2, 128)])
def test_encoder_attention_bidirectional(Hq, Hkv, D):
    """Non-causal varlen attention (vision encoder): every token sees its whole sequence."""
    g = torch.Generator(device=DEV).manual_seed(5)
    lens = [1, 63, 64, 200, 577]
    offs = [0]
    for n in lens:
        offs.append(offs[-1] + n)
    T = offs[-1]
    q = torch.randn(T, Hq, D, device=DEV, generator=g).bfloat16()
    k = torch.randn(T, Hkv, D, device=DEV, generator=g).bfloat16()
    v = torch.randn(T, Hkv, D, device=DEV, generator=g).bfloat16()
    got = cu().encoder_attention(q, k, v, offs)
    want = ref.encoder_attention(q, k, v, offs)
    _close(got, want, 2e-2, 2e-2)


@pytest.mark.parametrize("spec", ["silu", "gelu", "gelu_tanh", "swigluoai", "swigluoai:1.5:2", "silu_clamp:3",
                                  "situ:3:none", "situ:3:2"])
def test_gated_activation_kernels(spec):
    from vllm_torchtpu_b200.ops import cuda
    from vllm_torchtpu_b200.ops import reference as ref
    g = torch.Generator(device=DEV).manual_seed(0)
    x = (torch.randn(37, 2 * 1032, device=DEV, generator=g) * 4).bfloat16()
    got = cuda.gated_act_and_mul(x, spec)
    want = ref.gated_act_and_mul(x.float(), spec)
    torch.testing.assert_close(got.float(), want, rtol=2e-2, atol=2e-2)


def test_moe_experts_with_oai_swiglu_on_the_device():
    from vllm_torchtpu_b200.ops import cuda
    from vllm_torchtpu_b200.ops import reference as ref
    g = torch.Generator(device=DEV).manual_seed(1)
    T, H, I, E, k = 50, 256, 128, 8, 2
    x = torch.randn(T, H, device=DEV, generator=g).bfloat16()
    w13 = (torch.randn(E, 2 * I, H, device=DEV, generator=g) * 0.08).bfloat16()
    w2 = (torch.randn(E, H, I, device=DEV, generator=g) * 0.08).bfloat16()
    logits = torch.randn(T, E, device=DEV, generator=g)
    wt, ids = torch.topk(torch.softmax(logits, -1), k, -1)
    ids, wt = ids.int().contiguous(), wt.float().contiguous()
    got = cuda.moe_experts(x, w13, w2, ids, wt, 0, act="swigluoai")
    want = ref.moe_experts(x, w13, w2, ids, wt, 0, act="swigluoai")
    err = (got.float() - want.float()).abs().max().item()
    assert err <= 3e-2 * want.float().abs().max().item() + 2e-2, err
    assert cuda.check_status() == 0
