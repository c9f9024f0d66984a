"""Diffusion runtime on CPU: rotary tables, the fused q/k norm + RoPE statement, attention fallbacks, the
transformer's token layout, the scheduler and the guided sampling loop."""
import math

import pytest
import torch

from vllm_torchtpu_b200.omni import register_omni_b200_platform
from vllm_torchtpu_b200.omni.attention import diffusion_attention, sdpa_bshd
from vllm_torchtpu_b200.omni.backend import B200DiffusionAttentionBackend
from vllm_torchtpu_b200.omni.dit import DiffusionTransformer, DiTConfig
from vllm_torchtpu_b200.omni.ops import qk_norm_rope, qk_norm_rope_reference
from vllm_torchtpu_b200.omni.pipeline import DiffusionPipeline
from vllm_torchtpu_b200.omni.rope import apply_rotary_interleaved, axes_split, rope_table_1d, rope_table_3d
from vllm_torchtpu_b200.omni.scheduler import FlowMatchEulerScheduler


def test_rope_tables_and_interleaved_rotation():
    assert axes_split(128) == (22, 21, 21) and sum(axes_split(64)) == 32
    cos, sin = rope_table_3d((2, 3, 4), 64)
    assert cos.shape == (24, 32)
    nf, nh, nw = axes_split(64)
    # token (f, h, w): the frame band depends on f only, the row band on h only, the column band on w only
    tok = lambda f, h, w: (f * 3 + h) * 4 + w                     # noqa: E731
    assert torch.equal(cos[tok(1, 0, 0), :nf], cos[tok(1, 2, 3), :nf])
    assert torch.equal(cos[tok(0, 2, 0), nf:nf + nh], cos[tok(1, 2, 3), nf:nf + nh])
    assert torch.equal(sin[tok(0, 0, 3), nf + nh:], sin[tok(1, 2, 3), nf + nh:])
    assert torch.all(cos[0] == 1) and torch.all(sin[0] == 0)
    # the rotation as complex multiplication of (even, odd) pairs
    x = torch.randn(24, 2, 64)
    got = apply_rotary_interleaved(x, cos, sin)
    z = torch.view_as_complex(x.view(24, 2, 32, 2).contiguous()) * torch.complex(cos, sin)[:, None]
    torch.testing.assert_close(got, torch.view_as_real(z).flatten(-2), rtol=1e-5, atol=1e-5)
    # relative property along one axis: <R(a) q, R(b) k> depends on a - b
    c1, s1 = rope_table_1d(8, 64)
    q, k = torch.randn(1, 1, 64), torch.randn(1, 1, 64)
    dot = lambda a, b: (apply_rotary_interleaved(q, c1[a:a + 1], s1[a:a + 1])            # noqa: E731
                        * apply_rotary_interleaved(k, c1[b:b + 1], s1[b:b + 1])).sum()
    assert abs(dot(5, 2) - dot(6, 3)) < 1e-3


def test_qk_norm_rope_statement():
    T, H, D = 6, 2, 16
    qkv = torch.randn(T, 3 * H * D)
    wq, wk = torch.rand(H * D) + 0.5, torch.rand(H * D) + 0.5
    cos, sin = rope_table_1d(T, D)
    q, k = qk_norm_rope(qkv, wq, wk, cos, sin, H, H, D, 1e-6)
    # the norm runs over all heads' channels, not per head
    xq = qkv[:, :H * D]
    want = xq / xq.pow(2).mean(-1, keepdim=True).add(1e-6).sqrt() * wq
    torch.testing.assert_close(q, apply_rotary_interleaved(want.view(T, H, D), cos, sin), rtol=1e-5, atol=1e-5)
    q2, k2 = qk_norm_rope_reference(qkv, wq, wk, cos, sin, H, H, D, 1e-6)
    assert torch.equal(q, q2) and torch.equal(k, k2) and k.shape == (T, H, D)
    # rotation keeps the norm of every pair
    torch.testing.assert_close(k.view(T, H, D // 2, 2).norm(dim=-1),
                               apply_rotary_interleaved(k, cos, -sin).view(T, H, D // 2, 2).norm(dim=-1))


def test_attention_fallbacks_and_backend_object():
    q, k, v = torch.randn(2, 7, 4, 16), torch.randn(2, 5, 2, 16), torch.randn(2, 5, 2, 16)
    o = diffusion_attention(q, k, v)                  # cross-attention with grouped heads
    kk, vv = k.repeat_interleave(2, 2), v.repeat_interleave(2, 2)
    p = torch.softmax(torch.einsum("bqhd,bkhd->bhqk", q, kk) / 4.0, -1)
    torch.testing.assert_close(o, torch.einsum("bhqk,bkhd->bqhd", p, vv), rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError):
        diffusion_attention(torch.randn(1, 3, 3, 16), k[:1], v[:1])
    qs = torch.randn(1, 6, 2, 16)
    causal = diffusion_attention(qs, qs, qs, causal=True)
    assert torch.allclose(causal[:, 0], qs[:, 0], atol=1e-5)              # the first token sees itself only
    impl = B200DiffusionAttentionBackend.get_impl_cls()(num_heads=2, head_size=16)
    torch.testing.assert_close(impl.forward(qs, qs, qs), sdpa_bshd(qs, qs, qs))
    assert B200DiffusionAttentionBackend.get_name() == "B200_TCGEN05_ATTN"
    assert register_omni_b200_platform() is None      # no GPU / no omni runtime here


def test_scheduler_integrates_a_known_velocity_field():
    s = FlowMatchEulerScheduler(shift=3.0)
    s.set_timesteps(10)
    assert s.sigmas[0] == 1.0 and s.sigmas[-1] == 0.0 and torch.all(s.sigmas[:-1] > s.sigmas[1:])
    assert s.timesteps.shape == (10,) and s.timesteps[0] == 1000.0
    # straight-line flow: x_t = (1 - sigma) * data + sigma * noise has constant velocity noise - data, so
    # Euler steps recover the data exactly whatever the schedule
    data, noise = torch.randn(4, 8), torch.randn(4, 8)
    x = s.add_noise(data, noise, 1.0)
    for i in range(10):
        x = s.step(noise - data, i, x)
    torch.testing.assert_close(x, data, rtol=1e-4, atol=1e-5)
    with pytest.raises(ValueError):
        s.set_timesteps(0)


def test_dit_token_layout_conditioning_and_checkpoint():
    cfg = DiTConfig(dtype=torch.float32)
    m = DiffusionTransformer(cfg, "cpu")
    lat = torch.randn(2, 16, 2, 4, 6)
    grid = m.grid_of(lat)
    assert grid == (2, 2, 3)
    tok = m.patchify(lat)
    assert tok.shape == (2, 12, 64) and torch.equal(m.unpatchify(tok, grid), lat)
    with pytest.raises(ValueError):
        m.grid_of(torch.randn(1, 16, 1, 3, 4))
    text = torch.randn(2, 5, cfg.text_dim)
    t = torch.tensor([500.0, 500.0])
    v = m.forward(lat, t, text)
    assert v.shape == lat.shape and torch.isfinite(v).all()
    # batch entries are independent; timestep and text both change the output
    v0 = m.forward(lat[:1], t[:1], text[:1])
    torch.testing.assert_close(v0, v[:1], rtol=1e-4, atol=1e-5)
    assert not torch.allclose(m.forward(lat[:1], torch.tensor([100.0]), text[:1]), v0, atol=1e-4)
    assert not torch.allclose(m.forward(lat[:1], t[:1], text[1:]), v0, atol=1e-4)
    # bidirectional attention: a change in the last latent cell moves the prediction of the first token
    lat2 = lat[:1].clone()
    lat2[..., -1, -1, -1] += 5.0
    assert not torch.allclose(m.forward(lat2, t[:1], text[:1])[..., 0, 0, 0], v0[..., 0, 0, 0], atol=1e-6)
    # state dict round trip, and a checkpoint with a wrong shape or a missing tensor is refused
    sd = m.state_dict()
    m2 = DiffusionTransformer(cfg, "cpu", state_dict=sd)
    assert torch.equal(m2.forward(lat, t, text), v)
    bad = dict(sd)
    bad.pop("blocks.1.ffn.2.weight")
    with pytest.raises(ValueError, match="lacks"):
        DiffusionTransformer(cfg, "cpu", state_dict=bad)
    bad = dict(sd, **{"head.weight": torch.zeros(3, 3)})
    with pytest.raises(ValueError, match="shape"):
        DiffusionTransformer(cfg, "cpu", state_dict=bad)


def test_pipeline_guidance_and_determinism():
    cfg = DiTConfig(dtype=torch.float32, num_layers=1)
    p = DiffusionPipeline(cfg, "cpu")
    text = torch.randn(1, 4, cfg.text_dim)
    shape = (16, 1, 4, 4)
    a = p.generate(text, shape, num_steps=3, seed=7)
    assert a.shape == (1, *shape) and torch.equal(a, p.generate(text, shape, num_steps=3, seed=7))
    assert not torch.equal(a, p.generate(text, shape, num_steps=3, seed=8))
    # guidance 1 is the conditional branch alone; guidance g extrapolates from the unconditional one
    g = torch.Generator().manual_seed(0)
    x0 = torch.randn((1, *shape), generator=g)
    neg = torch.zeros_like(text)
    one = p.generate(text, shape, num_steps=1, latents=x0)
    unc = p.generate(neg, shape, num_steps=1, latents=x0)
    two = p.generate(text, shape, num_steps=1, guidance_scale=2.5, negative_text=neg, latents=x0)
    torch.testing.assert_close(two, unc + 2.5 * (one - unc), rtol=1e-4, atol=1e-5)
    assert math.isfinite(float(two.abs().max()))
