"""Quantisation math (CPU): round trips and GEMM oracles against the bf16 result."""
import pytest
import torch

from vllm_torchtpu_b200.quantization import QuantConfig, get_linear_method
from vllm_torchtpu_b200.quantization import fp4, fp8, int4, int8


def test_fp8_block_roundtrip_and_gemm():
    torch.manual_seed(0)
    w = torch.randn(300, 520) * 0.05
    q, s = fp8.quantize_weight_block(w)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (3, 5)
    deq = fp8.dequantize_weight_block(q, s)
    assert (deq - w).abs().max() <= w.abs().max() * 0.07
    x = torch.randn(17, 520)
    got = fp8.fp8_block_gemm_reference(x, q, s, out_dtype=torch.float32)
    want = x @ w.t()
    assert (got - want).abs().max() <= want.abs().max() * 0.08


def test_act_quant_scales_per_group():
    x = torch.zeros(2, 256)
    x[0, :128] = 448.0
    x[0, 128:] = 1.0
    q, s = fp8.quantize_act_1x128(x)
    assert torch.allclose(s[0], torch.tensor([1.0, 1.0 / 448.0]))
    assert torch.allclose(q.float()[0, 128:], torch.full((128,), 448.0))


def test_int8_gemm_close():
    torch.manual_seed(1)
    w, x = torch.randn(64, 256) * 0.1, torch.randn(9, 256)
    q, s = int8.quantize_weight_int8(w)
    got = int8.int8_gemm_reference(x, q, s).float()
    want = x @ w.t()
    assert (got - want).abs().max() <= want.abs().max() * 0.05


def test_mxfp4_and_nvfp4_roundtrip():
    torch.manual_seed(2)
    w = torch.randn(32, 128)
    p, e = fp4.quantize_mxfp4(w)
    assert p.shape == (32, 64) and e.shape == (32, 4)
    d = fp4.dequantize_mxfp4(p, e)
    assert (d - w).abs().max() <= w.abs().max() * 0.3       # 4-bit: coarse but bounded
    exact = torch.tensor([[0.5, -1.5, 6.0, -4.0] * 8])
    p2, e2 = fp4.quantize_mxfp4(exact)
    assert torch.equal(fp4.dequantize_mxfp4(p2, e2), exact)
    pn, bs, gs = fp4.quantize_nvfp4(w)
    dn = fp4.dequantize_nvfp4(pn, bs, gs)
    assert (dn - w).abs().max() <= w.abs().max() * 0.3
    assert torch.equal(fp4.unpack_nibbles(fp4.pack_nibbles(torch.arange(16, dtype=torch.uint8)[None])),
                       torch.arange(16, dtype=torch.uint8)[None])


def test_int4_group_roundtrip():
    torch.manual_seed(3)
    w = torch.randn(16, 256)
    p, s, z = int4.quantize_int4_group(w)
    d = int4.dequantize_int4_group(p, s, z)
    assert (d - w).abs().max() <= (w.max() - w.min()) / 15 * 0.51 + 1e-6


@pytest.mark.parametrize("name", ["fp8_block", "fp8", "online_fp8", "int8", "mxfp4", "nvfp4", "awq"])
def test_linear_methods_apply_on_cpu(name):
    from vllm_torchtpu_b200.layers.linear import ReplicatedLinear
    lin = ReplicatedLinear("model.layers.0.mlp.x", 256, 128, dtype=torch.float32, device="cpu",
                           quant_config=QuantConfig(name))
    lin.init_dummy(0.05, 0)
    x = torch.randn(5, 256)
    y = lin(x)
    from vllm_torchtpu_b200.layers.linear import seeded_normal
    w = seeded_normal("model.layers.0.mlp.x", (128, 256), 0.05, torch.bfloat16, "cpu", 0).float()
    want = x @ w.t()
    tol = 0.35 if name in ("mxfp4", "nvfp4", "awq") else 0.1
    assert (y.float() - want).abs().max() <= want.abs().max() * tol
    assert lin.weight_bytes() < 128 * 256 * 2
    assert get_linear_method(QuantConfig(name, ignored_layers=("lm_head",)), "lm_head").__class__.__name__ == \
        "UnquantizedLinearMethod"


def test_turboquant_4bit_reference_roundtrip():
    from vllm_torchtpu_b200.quantization import turboquant as tq
    g = torch.Generator().manual_seed(0)
    k = torch.randn(64, 128, generator=g)
    v = torch.randn(64, 128, generator=g) * 0.5 + 0.1
    h = tq.hadamard(128)
    torch.testing.assert_close(h @ h.t(), torch.eye(128), atol=1e-5, rtol=0)
    kc, kn, vc, vm = tq.encode(k, v)
    assert kc.shape == (64, 64) and kc.dtype == torch.uint8 and vm.shape == (64, 2)
    kd, vd = tq.decode(kc, kn, vc, vm, dtype=torch.float32)
    cos = torch.nn.functional.cosine_similarity(kd, k, dim=-1)
    assert cos.min() > 0.97                       # 4-bit Lloyd-Max keys: ~1 % relative MSE
    assert (vd - v).abs().max() < (v.amax(-1) - v.amin(-1)).max() / 15 * 0.51 + 0.02
    q8 = tq.quantize_kv_fp8(v.bfloat16(), 0.02)
    assert (tq.dequantize_kv_fp8(q8, 0.02).float() - v).abs().max() < 0.1
