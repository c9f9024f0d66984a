"""MLA latent-cache attention kernel (dense and top-k sparse) and cache write vs the fp32 statements."""
import pytest
import torch

from vllm_torchtpu_b200.ops import reference as ref
from vllm_torchtpu_b200.runner.attn_metadata import AttentionMetadata

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(q_lens, ctx_lens, H, L, R, bs=16, topk=None, seed=0):
    from vllm_torchtpu_b200.ops import cuda
    g = torch.Generator(device=DEV).manual_seed(seed)
    Dq = L + R
    n = len(q_lens)
    seq = [q + c for q, c in zip(q_lens, ctx_lens)]
    maxb = max(-(-s // bs) for s in seq) + 1
    nb = sum(-(-s // bs) for s in seq) + 2
    cache = (torch.randn(nb, bs, Dq, device=DEV, generator=g) * 0.5).bfloat16()
    perm = (torch.randperm(nb - 1, device=DEV, generator=g) + 1).to(torch.int32)
    bt = torch.zeros(n, maxb, dtype=torch.int32, device=DEV)
    off = 0
    for r, s in enumerate(seq):
        k = -(-s // bs)
        bt[r, :k] = perm[off:off + k]
        off += k
    T = sum(q_lens)
    q = (torch.randn(T, H, Dq, device=DEV, generator=g) * 0.3).bfloat16()
    qsl = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    sl = torch.tensor(seq, dtype=torch.int32, device=DEV)
    meta = AttentionMetadata(None, None, bt, sl, qsl, n, T, num_decode_reqs=0, max_query_len=max(q_lens),
                             max_seq_len=max(seq), padded_num_reqs=n, padded_num_tokens=T)
    ti = None
    if topk:
        # per token: a random subset of its visible positions, padded with -1, plus out-of-range junk
        ti = torch.full((T, topk), -1, dtype=torch.int32, device=DEV)
        tok = 0
        for r in range(n):
            for j in range(q_lens[r]):
                vis = seq[r] - q_lens[r] + j + 1
                k = min(topk - 2, vis)
                sel = torch.randperm(vis, device=DEV, generator=g)[:k].to(torch.int32)
                ti[tok, :k] = sel
                ti[tok, topk - 1] = seq[r] + 5            # beyond the context: ignored
                tok += 1
    scale = (L + R) ** -0.5
    got, got_lse = cuda.mla_paged_attention(q, cache, meta, scale, L, topk_indices=ti, return_lse=True)
    want, want_lse = ref.mla_paged_attention(q, cache, bt, sl, qsl, scale, L, num_reqs=n, topk_indices=ti,
                                             return_lse=True)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    fin = torch.isfinite(want_lse)
    torch.testing.assert_close(got_lse[fin], want_lse[fin], rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("H,L,R", [(128, 512, 64), (16, 512, 64), (4, 64, 16), (8, 128, 32)])
def test_mla_decode(H, L, R):
    _case([1, 1, 1, 1], [0, 15, 300, 1029], H, L, R)


def test_mla_prefill_and_mixed():
    _case([1, 37, 3, 64], [50, 0, 700, 20], 16, 512, 64)


def test_mla_sparse_topk():
    _case([1, 5, 1], [400, 90, 7], 32, 512, 64, topk=64)


def test_mla_write_cache():
    from vllm_torchtpu_b200.ops import cuda
    T, L, R, nb, bs = 23, 512, 64, 5, 16
    kv = torch.randn(T, L + R + 8, device=DEV).bfloat16()
    kv_c, k_pe = kv[:, :L], kv[:, L:L + R]
    slots = torch.randperm(nb * bs, device=DEV)[:T].to(torch.int32)
    slots[3] = -1
    c1 = torch.zeros(nb, bs, L + R, device=DEV, dtype=torch.bfloat16)
    c2 = c1.clone()
    cuda.mla_write_cache(c1, kv_c, k_pe, slots)
    ref.mla_write_cache(c2, kv_c, k_pe, slots)
    assert torch.equal(c1, c2)


def test_deepseek_style_engine_runs_on_gpu_and_matches_dense_logits():
    """MLA + MoE model through the engine on the GPU: first-token logits against the dense fp32
    forward of the same weights, and graph decode == eager decode."""
    import dataclasses

    import numpy as np

    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.config import model_preset
    from vllm_torchtpu_b200.engine.llm import LLM
    from vllm_torchtpu_b200.models.reference_forward_mla import dense_mla_logits
    from vllm_torchtpu_b200.ops import cuda
    cfg = dataclasses.replace(model_preset("tiny-mla"), dtype=torch.bfloat16)
    rng = np.random.RandomState(0)
    prompts = [rng.randint(0, cfg.vocab_size, size=n).tolist() for n in (5, 17, 40)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)

    def make(**kw):
        return LLM(cfg, device="cuda", max_num_seqs=8, max_num_batched_tokens=128, block_size=16,
                   num_gpu_blocks_override=64, **kw)
    llm = make(enforce_eager=True)
    eng = llm.engine
    eng.add_request(prompts[2], SamplingParams(max_tokens=1))
    out = eng.scheduler.schedule()
    r = eng.runner
    r._update_batch(out)
    prep = r._prepare_inputs(out)
    prep["bufs"].upload(prep["R_pad"])
    _, logits = r._forward_and_sample(prep["bufs"], r._make_meta(prep), prep["T_pad"], prep["R_pad"], True)
    want = dense_mla_logits(r.model, prompts[2])[-1]
    err = (logits[0].float() - want.to(logits.device)).abs().max().item()
    assert err < 0.08 * want.abs().max().item() + 0.05, err
    eager = [o.outputs[0].token_ids for o in make(enforce_eager=True).generate(prompts, sp)]
    graph = [o.outputs[0].token_ids for o in make().generate(prompts, sp)]
    assert eager == graph
    assert cuda.check_status() == 0


@pytest.mark.parametrize("interleaved", [False, True])
def test_mla_absorb_and_unabsorb_match_einsum(interleaved):
    """W_UK / W_UV as grouped GEMMs over the heads, rope of the rope dims, against fp32 einsum + the
    reference rotary embedding."""
    from vllm_torchtpu_b200.ops import cuda
    from vllm_torchtpu_b200.ops import reference as ref
    T, H, nope, rope, L, v = 37, 16, 128, 64, 512, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(T, H, nope + rope, device="cuda", generator=g).bfloat16()
    kv = torch.randn(T, L + rope, device="cuda", generator=g).bfloat16()
    w_uk = (torch.randn(H, nope, L, device="cuda", generator=g) * 0.05).bfloat16()
    w_uv = (torch.randn(H, L, v, device="cuda", generator=g) * 0.05).bfloat16()
    pos = torch.randint(0, 4000, (T,), device="cuda", generator=g, dtype=torch.int32)
    inv_freq = (1.0 / (10000 ** (torch.arange(0, rope, 2, device="cuda").float() / rope))).contiguous()
    q_latent, k_pe = cuda.mla_absorb(q, kv, pos, inv_freq, w_uk.transpose(1, 2).contiguous(), nope, rope, L,
                                     interleaved)
    torch.cuda.synchronize()
    want_ql = torch.einsum("thn,hnl->thl", q[..., :nope].float(), w_uk.float())
    want_qpe = ref.apply_rope(q[..., nope:], pos, inv_freq, interleaved).float()
    want_kpe = ref.apply_rope(kv[:, L:].reshape(T, 1, rope), pos, inv_freq, interleaved).reshape(T, rope).float()
    assert (q_latent[..., :L].float() - want_ql).abs().max() <= 2e-2 * want_ql.abs().max() + 1e-2
    assert (q_latent[..., L:].float() - want_qpe).abs().max() <= 3e-2
    assert (k_pe.float() - want_kpe).abs().max() <= 3e-2
    o_lat = torch.randn(T, H, L, device="cuda", generator=g).bfloat16()
    y = cuda.mla_unabsorb(o_lat, w_uv.transpose(1, 2).contiguous())
    torch.cuda.synchronize()
    want = torch.einsum("thl,hlv->thv", o_lat.float(), w_uv.float()).reshape(T, H * v)
    assert (y.float() - want).abs().max() <= 2e-2 * want.abs().max() + 1e-2
    assert cuda.check_status() == 0
