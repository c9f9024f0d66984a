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
