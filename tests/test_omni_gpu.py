"""Diffusion runtime on the device: the fused q/k norm + RoPE kernel, dense attention on the tcgen05 kernel,
and the transformer / sampling loop against the fp32 CPU statement of the same weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda")


@pytest.mark.parametrize("T,Hq,Hkv,D,extra", [(300, 12, 12, 128, 12 * 128), (77, 8, 2, 64, 2 * 64 + 8),
                                               (33, 40, 40, 128, 0)])
def test_qk_norm_rope_kernel_matches_the_statement(T, Hq, Hkv, D, extra):
    from vllm_torchtpu_b200.omni.ops import qk_norm_rope, qk_norm_rope_reference
    from vllm_torchtpu_b200.omni.rope import rope_table_1d
    dev = _dev()
    g = torch.Generator().manual_seed(T)
    qkv = (torch.randn(T, (Hq + Hkv) * D + extra, generator=g) * 2).to(dev, torch.bfloat16)
    wq = (torch.rand(Hq * D, generator=g) + 0.5).to(dev, torch.bfloat16)
    wk = (torch.rand(Hkv * D, generator=g) + 0.5).to(dev, torch.bfloat16)
    cos, sin = rope_table_1d(T, D, device=dev)
    q, k = qk_norm_rope(qkv, wq, wk, cos, sin, Hq, Hkv, D, 1e-6)
    rq, rk = qk_norm_rope_reference(qkv.cpu(), wq.cpu(), wk.cpu(), cos.cpu(), sin.cpu(), Hq, Hkv, D, 1e-6)
    assert q.shape == (T, Hq, D) and k.shape == (T, Hkv, D)
    torch.testing.assert_close(q.float().cpu(), rq.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(k.float().cpu(), rk.float(), rtol=2e-2, atol=2e-2)


def test_dense_attention_runs_on_the_tensor_core_kernel():
    from vllm_torchtpu_b200 import ops
    from vllm_torchtpu_b200.omni.attention import diffusion_attention, sdpa_bshd
    dev = _dev()
    g = torch.Generator().manual_seed(1)
    q, k, v = [torch.randn(2, 333, 4, 128, generator=g).to(dev, torch.bfloat16) for _ in range(3)]
    before = ops.launch_count()
    o = diffusion_attention(q, k, v)
    assert ops.launch_count() == before + 1                    # one launch of the package's kernel, not SDPA
    want = sdpa_bshd(q.float().cpu(), k.float().cpu(), v.float().cpu())
    torch.testing.assert_close(o.float().cpu(), want, rtol=3e-2, atol=3e-2)


def test_transformer_and_sampling_loop_match_the_cpu_statement():
    from vllm_torchtpu_b200.omni.dit import DiffusionTransformer, DiTConfig
    from vllm_torchtpu_b200.omni.pipeline import DiffusionPipeline
    dev = _dev()
    cfg = DiTConfig()
    pipe = DiffusionPipeline(cfg, "cuda")
    sd = {n: t.float().cpu() for n, t in pipe.model.state_dict().items()}
    ref = DiffusionTransformer(DiTConfig(dtype=torch.float32), "cpu", state_dict=sd)
    g = torch.Generator().manual_seed(2)
    lat = torch.randn(2, 16, 2, 8, 8, generator=g)
    text = torch.randn(2, 6, cfg.text_dim, generator=g)
    t = torch.tensor([700.0, 300.0])
    v = pipe.model.forward(lat.to(dev), t.to(dev), text.to(dev)).float().cpu()
    want = ref.forward(lat.to(torch.bfloat16).float(), t, text.to(torch.bfloat16).float())
    err = (v - want).norm() / want.norm()
    assert torch.isfinite(v).all() and err < 0.05, float(err)
    out = pipe.generate(text, (16, 2, 8, 8), num_steps=3, guidance_scale=2.0, seed=3)
    assert out.shape == (2, 16, 2, 8, 8) and torch.isfinite(out.float()).all()
    assert len(pipe.step_ms) == 3 and all(ms > 0 for ms in pipe.step_ms)
