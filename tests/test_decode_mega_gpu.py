"""Persistent decode kernel (all layers of a decode step in one launch) against the per-layer kernel
chain of the same model on the same inputs, and through the engine."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a GPU", allow_module_level=True)

from vllm_torchtpu_b200.config import ModelConfig  # noqa: E402
from vllm_torchtpu_b200.models.llama import LlamaForCausalLM  # noqa: E402
from vllm_torchtpu_b200.ops import cuda  # noqa: E402
from vllm_torchtpu_b200.runner.attn_metadata import AttentionMetadata  # noqa: E402

DEV = "cuda"
BS = 16


@pytest.fixture(autouse=True)
def _persistent_kernel_on(monkeypatch):
    """The persistent kernel is opt-in (B200_DECODE_MEGAKERNEL); these tests exercise it."""
    from vllm_torchtpu_b200 import envs
    monkeypatch.setenv("B200_DECODE_MEGAKERNEL", "1")
    envs.reset()
    yield
    monkeypatch.delenv("B200_DECODE_MEGAKERNEL", raising=False)
    envs.reset()


def _model(L, H, Hq, Hkv, I, qk_norm=False, bias=False):
    cfg = ModelConfig(name="mega-test", num_layers=L, hidden_size=H, num_q_heads=Hq, num_kv_heads=Hkv, head_dim=128,
                      intermediate_size=I, vocab_size=512, max_model_len=4096, dtype=torch.bfloat16,
                      qk_norm=qk_norm, attention_bias=bias, init_std=0.03)
    m = LlamaForCausalLM(cfg, DEV)
    m.init_dummy()
    g = torch.Generator(device=DEV).manual_seed(5)
    for layer in m.layers:       # non-trivial norm weights / biases so that a swapped pointer shows
        layer.input_ln = (1 + 0.1 * torch.randn(H, device=DEV, generator=g)).bfloat16()
        layer.post_ln = (1 + 0.1 * torch.randn(H, device=DEV, generator=g)).bfloat16()
        a = layer.self_attn
        if qk_norm:
            a.q_norm_w.copy_((1 + 0.1 * torch.randn(128, device=DEV, generator=g)).bfloat16())
            a.k_norm_w.copy_((1 + 0.1 * torch.randn(128, device=DEV, generator=g)).bfloat16())
        if bias:
            a.qkv.bias = (0.1 * torch.randn(a.qkv.out_features, device=DEV, generator=g)).bfloat16()
    return m


def _batch(m, ctx_lens, pad_to=None):
    R = len(ctx_lens)
    Rp = pad_to or R
    Hkv = m.layers[0].self_attn.attn.num_kv_heads
    nblk = [-(-(c + 1) // BS) for c in ctx_lens]
    mb = max(nblk) + 1
    nb = sum(nblk) + 2
    g = torch.Generator(device=DEV).manual_seed(1)
    kvs = [(torch.randn(nb, 2, Hkv, BS, 128, device=DEV, generator=g) * 0.5).bfloat16() for _ in m.layers]
    bt = torch.zeros(Rp, mb, dtype=torch.int32)
    perm = (torch.randperm(nb - 1) + 1).tolist()
    off = 0
    for r in range(R):
        bt[r, :nblk[r]] = torch.tensor(perm[off:off + nblk[r]], dtype=torch.int32)
        off += nblk[r]
    pos = torch.zeros(Rp, dtype=torch.int32)
    pos[:R] = torch.tensor(ctx_lens, dtype=torch.int32)
    slots = torch.full((Rp,), -1, dtype=torch.int32)
    for r, c in enumerate(ctx_lens):
        slots[r] = int(bt[r, c // BS]) * BS + c % BS
    sl = torch.zeros(Rp, dtype=torch.int32)
    sl[:R] = pos[:R] + 1
    qsl = torch.arange(Rp + 1, dtype=torch.int32)
    qsl[R + 1:] = R
    meta = AttentionMetadata(pos.to(DEV), slots.to(DEV), bt.to(DEV).contiguous(), sl.to(DEV), qsl.to(DEV), R, R,
                             num_decode_reqs=R, max_query_len=1, max_seq_len=max(ctx_lens) + 1,
                             padded_num_reqs=Rp, padded_num_tokens=Rp)
    x0 = (torch.randn(Rp, m.cfg.hidden_size, device=DEV, generator=g) * 0.5).bfloat16()
    return kvs, meta, x0


def _run_both(m, ctx_lens, pad_to=None, repeat=1):
    kvs, meta, x0 = _batch(m, ctx_lens, pad_to)
    R = len(ctx_lens)
    kv_a = [k.clone() for k in kvs]
    kv_b = [k.clone() for k in kvs]
    m.decode_mega = None
    ha, ra = m.forward(None, meta, kv_a, hidden=x0.clone())
    want = (ha.float() + ra.float())[:R]
    m.setup_decode_fusion(kv_b)
    assert m.decode_mega is not None, m.decode_mega_reason
    got = None
    for _ in range(repeat):
        for k, k0 in zip(kv_b, kvs):
            k.copy_(k0)
        hb, rb = m.forward(None, meta, kv_b, hidden=x0.clone())
        torch.cuda.synchronize()
        assert cuda.check_status() == 0
        got = (hb.float() + rb.float())[:R]
    return want, got, kv_a, kv_b


def _assert_close(want, got, tol=3e-2):
    assert torch.isfinite(got).all()
    err = (got - want).abs().max() / want.abs().max().clamp_min(1e-6)
    assert err < tol, float(err)


@pytest.mark.parametrize("L,H,Hq,Hkv,I,R", [(2, 1024, 8, 2, 2048, 8), (3, 2048, 16, 4, 1536, 33),
                                            (2, 4096, 32, 8, 14336, 64), (2, 4096, 4, 1, 1792, 64)])
def test_layers_match_per_layer_kernels(L, H, Hq, Hkv, I, R):
    m = _model(L, H, Hq, Hkv, I)
    rng = np.random.RandomState(0)
    ctx = rng.randint(1, 700, size=R).tolist()
    want, got, kv_a, kv_b = _run_both(m, ctx)
    _assert_close(want, got)
    for a, b in zip(kv_a, kv_b):          # the new token's K / V rows landed in the same slots
        assert (a.float() - b.float()).abs().max() <= 0.02 * a.float().abs().max()


def test_qk_norm_bias_padded_rows_and_relaunch():
    m = _model(2, 1024, 8, 4, 1024, qk_norm=True, bias=True)
    want, got, _, _ = _run_both(m, [0, 5, 17, 300, 1023], pad_to=8, repeat=3)
    _assert_close(want, got)


def test_kv_split_merge(monkeypatch):
    from vllm_torchtpu_b200 import envs
    monkeypatch.setenv("B200_ATTN_SPLIT_KV", "4")
    envs.reset()
    try:
        m = _model(2, 1024, 8, 2, 1024)
        want, got, _, _ = _run_both(m, [1500, 3, 64, 900])
        _assert_close(want, got)
    finally:
        monkeypatch.delenv("B200_ATTN_SPLIT_KV")
        envs.reset()


def test_graph_replay_of_persistent_kernel():
    m = _model(2, 1024, 8, 2, 2048)
    kvs, meta, x0 = _batch(m, [10, 200, 33, 64])
    m.setup_decode_fusion(kvs)
    h, r = m.forward(None, meta, kvs, hidden=x0)
    torch.cuda.synchronize()
    eager = (h.float() + r.float()).clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        h2, r2 = m.forward(None, meta, kvs, hidden=x0)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert cuda.check_status() == 0
    _assert_close(eager, h2.float() + r2.float(), tol=1e-3)


def test_engine_decodes_with_and_without_the_persistent_kernel(monkeypatch):
    from vllm_torchtpu_b200 import SamplingParams, envs
    from vllm_torchtpu_b200.engine.llm import LLM
    cfg = ModelConfig(name="mega-engine", num_layers=2, hidden_size=1024, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=2048, vocab_size=4096, max_model_len=512, dtype=torch.bfloat16)
    rng = np.random.RandomState(0)
    prompts = [rng.randint(0, 4096, size=n).tolist() for n in (8, 33, 70, 150)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    toks = {}
    for flag in ("1", "0"):
        monkeypatch.setenv("B200_DECODE_MEGAKERNEL", flag)
        envs.reset()
        llm = LLM(cfg, device="cuda", max_num_seqs=8, max_num_batched_tokens=256, num_gpu_blocks_override=256,
                  init_dist=False)
        assert (llm.engine.runner.model.decode_mega is not None) == (flag == "1")
        toks[flag] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        torch.cuda.synchronize()
        assert cuda.check_status() == 0
    same = sum(a == b for a, b in zip(toks["1"], toks["0"]))
    # random-init logits are nearly flat: a rounding difference may flip an arg-max late in a sequence
    assert same >= 3, toks
    assert all(a[:4] == b[:4] for a, b in zip(toks["1"], toks["0"])), toks
