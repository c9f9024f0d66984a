"""Reference (PyTorch) statements of ops that the kernels are compared against: gated activations."""
import pytest
import torch


def test_gated_activation_family_and_moe_option():
    """silu / gelu / gelu_tanh / swigluoai / clamped silu / situ against their definitions, and the activation
    option of the expert pipeline."""
    import torch.nn.functional as F
    from vllm_torchtpu_b200.ops import reference as ref
    torch.manual_seed(0)
    x = torch.randn(5, 32) * 4
    g, u = x[:, :16], x[:, 16:]
    torch.testing.assert_close(ref.gated_act_and_mul(x, "silu"), F.silu(g) * u)
    torch.testing.assert_close(ref.gated_act_and_mul(x, "gelu_tanh"), F.gelu(g, approximate="tanh") * u)
    gc, uc = g.clamp(max=7.0), u.clamp(-7.0, 7.0)
    torch.testing.assert_close(ref.gated_act_and_mul(x, "swigluoai"), (uc + 1) * gc * torch.sigmoid(1.702 * gc))
    torch.testing.assert_close(ref.gated_act_and_mul(x, "swigluoai:1.5:2"),
                               (u.clamp(-2, 2) + 1) * g.clamp(max=2) * torch.sigmoid(1.5 * g.clamp(max=2)))
    torch.testing.assert_close(ref.gated_act_and_mul(x, "silu_and_mul_with_clamp"),
                               F.silu(g.clamp(max=10.0)) * u.clamp(-10.0, 10.0))
    torch.testing.assert_close(ref.gated_act_and_mul(x, "situ:3:none"), 3 * torch.tanh(g / 3) * torch.sigmoid(g) * u)
    torch.testing.assert_close(ref.gated_act_and_mul(x, "situ:3:2"),
                               3 * torch.tanh(g / 3) * torch.sigmoid(g) * 2 * torch.tanh(u / 2))
    with pytest.raises(ValueError):
        ref.parse_gated_act("relu")
    # experts with another activation
    T, H, I, E, k = 6, 16, 8, 4, 2
    xx = torch.randn(T, H)
    w13, w2 = torch.randn(E, 2 * I, H) * 0.3, torch.randn(E, H, I) * 0.3
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).int()
    wt = torch.rand(T, k)
    got = ref.moe_experts(xx, w13, w2, ids, wt, 0, act="swigluoai")
    want = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(ids[t, j])
            want[t] += wt[t, j] * (ref.gated_act_and_mul((xx[t] @ w13[e].t())[None], "swigluoai")[0] @ w2[e].t())
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)


def test_yarn_rope_frequencies_and_attention_factor():
    """YaRN against the published recipe: fast dimensions keep their frequency, slow ones are divided by the
    factor, a linear ramp in between; cos / sin multiplier 0.1 ln(factor) + 1 unless the config overrides it."""
    import math
    from vllm_torchtpu_b200.ops import reference as ref
    D, theta, factor, old = 64, 150000.0, 32.0, 4096
    sc = {"rope_type": "yarn", "factor": factor, "original_max_position_embeddings": old, "beta_fast": 32.0,
          "beta_slow": 1.0, "truncate": False}
    inv = ref.rope_inv_freq(D, theta, sc).double()
    base = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))

    def corr(rot):
        return D * math.log(old / (rot * 2 * math.pi)) / (2 * math.log(theta))
    lo, hi = corr(32.0), corr(1.0)
    ramp = ((torch.arange(D // 2, dtype=torch.float64) - lo) / (hi - lo)).clamp(0, 1)
    want = base / factor * ramp + base * (1 - ramp)
    torch.testing.assert_close(inv, want, rtol=1e-6, atol=0)
    assert torch.allclose(inv[:3], base[:3], rtol=1e-6) and torch.allclose(inv[-3:], base[-3:] / factor, rtol=1e-6)
    assert abs(ref.rope_attention_factor(sc) - (0.1 * math.log(32.0) + 1)) < 1e-9
    assert ref.rope_attention_factor({**sc, "attention_factor": 1.25}) == 1.25
    assert ref.rope_attention_factor({**sc, "mscale": 1.0, "mscale_all_dim": 1.0}) == 1.0     # DeepSeek-V3
    assert ref.rope_attention_factor({"rope_type": "llama3", "factor": 8.0}) == 1.0
    trunc = ref.rope_inv_freq(D, theta, {**sc, "truncate": True}).double()
    lo_t, hi_t = math.floor(lo), math.ceil(hi)
    ramp_t = ((torch.arange(D // 2, dtype=torch.float64) - lo_t) / (hi_t - lo_t)).clamp(0, 1)
    torch.testing.assert_close(trunc, base / factor * ramp_t + base * (1 - ramp_t), rtol=1e-6, atol=0)


def test_route_padding_mask_and_routing_simulation():
    from vllm_torchtpu_b200.ops import reference as ref
    T, k, E = 10, 4, 16
    ids = torch.randint(0, E, (T, k), dtype=torch.int32)
    w = torch.rand(T, k)
    keep_ids, keep_w = ids.clone(), w.clone()
    ref.moe_route_post(ids, w, E, torch.tensor([7], dtype=torch.int32), "")
    assert torch.equal(ids[:7], keep_ids[:7]) and (ids[7:] == -1).all() and (w[7:] == 0).all()
    torch.testing.assert_close(w[:7], keep_w[:7])
    ref.moe_route_post(ids, w, E, None, "uniform")
    counts = torch.bincount(ids.flatten().long(), minlength=E)
    assert counts.max() - counts.min() <= 1 and torch.allclose(w, torch.full_like(w, 0.25))
    ref.moe_route_post(ids, w, E, None, "hash")
    assert all(len(set(r.tolist())) == k for r in ids) and int(ids.min()) >= 0 and int(ids.max()) < E
    # masked rows contribute nothing to the experts' output
    x = torch.randn(T, 8)
    w13, w2 = torch.randn(E, 12, 8) * 0.3, torch.randn(E, 8, 6) * 0.3
    ref.moe_route_post(ids, w, E, torch.tensor([4], dtype=torch.int32), "")
    y = ref.moe_experts(x, w13, w2, ids, w, 0)
    assert not y[4:].any() and y[:4].abs().sum() > 0
