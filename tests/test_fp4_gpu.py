"""W4A16 tcgen05 GEMM (mxfp4 / nvfp4 weights expanded in shared memory) against the dequantised fp32 product."""
import pytest
import torch

from vllm_torchtpu_b200.quantization import fp4 as q

pytestmark = pytest.mark.gpu
DEV = "cuda"


def cu():
    from vllm_torchtpu_b200.ops import cuda
    return cuda


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("T,N,K,bias", [(1, 256, 128, False), (16, 1024, 512, True), (64, 1280, 4096, False),
                                        (100, 200, 192, True), (300, 384, 1024, False), (700, 512, 256, False)])
def test_w4a16_gemm_matches_dequantised_product(fmt, T, N, K, bias):
    g = torch.Generator(device=DEV).manual_seed(T + N)
    x = torch.randn(T, K, device=DEV, generator=g).bfloat16()
    w = torch.randn(N, K, device=DEV, generator=g) * 0.05
    b = torch.randn(N, device=DEV, generator=g).bfloat16() if bias else None
    if fmt == "mxfp4":
        wp, sc = q.quantize_mxfp4(w)
        gs = None
        wd = q.dequantize_mxfp4(wp, sc)
    else:
        wp, sc, gs = q.quantize_nvfp4(w)
        wd = q.dequantize_nvfp4(wp, sc, gs)
    y = cu().w4a16_gemm(x, wp.contiguous(), sc.contiguous(), fmt, gs, b)
    torch.cuda.synchronize()
    assert cu().check_status() == 0
    want = x.float() @ wd.bfloat16().float().t()
    if bias:
        want = want + b.float()
    err = (y.float() - want).abs().max().item()
    assert err <= 1e-2 * want.abs().max().item() + 1e-2, err


def test_w4a16_moe_experts_match_dequantised_experts():
    from vllm_torchtpu_b200.ops import reference as ref
    T, E, k, H, I = 70, 8, 2, 256, 128
    g = torch.Generator(device=DEV).manual_seed(1)
    x = torch.randn(T, H, device=DEV, generator=g).bfloat16()
    w13 = torch.randn(E, 2 * I, H, device=DEV, generator=g) * 0.05
    w2 = torch.randn(E, H, I, device=DEV, generator=g) * 0.05
    q13 = [q.quantize_mxfp4(w13[e]) for e in range(E)]
    q2 = [q.quantize_mxfp4(w2[e]) for e in range(E)]
    w13p, s13 = torch.stack([a for a, _ in q13]), torch.stack([b for _, b in q13])
    w2p, s2 = torch.stack([a for a, _ in q2]), torch.stack([b for _, b in q2])
    ids, w = ref.moe_route(torch.randn(T, E, device=DEV, generator=g), k)
    got = cu().moe_experts_w4a16(x, w13p, s13, w2p, s2, ids, w, 0)
    torch.cuda.synchronize()
    assert cu().check_status() == 0
    d13 = q.dequantize_mxfp4(w13p, s13).bfloat16()
    d2 = q.dequantize_mxfp4(w2p, s2).bfloat16()
    want = ref.moe_experts(x, d13, d2, ids, w, 0)
    err = (got.float() - want.float()).abs().max().item()
    assert err <= 3e-2 * want.float().abs().max().item() + 1e-2, err


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
def test_dequant_kernel_is_bit_exact_and_large_token_counts_use_it(fmt):
    from vllm_torchtpu_b200.ops import cuda_fp4
    g = torch.Generator(device=DEV).manual_seed(2)
    w = torch.randn(384, 512, device=DEV, generator=g) * 0.3
    w[0, :32] *= 200.0                                   # a group with a large scale
    if fmt == "mxfp4":
        wp, sc = q.quantize_mxfp4(w)
        gs, wd = None, q.dequantize_mxfp4(wp, sc)
    else:
        wp, sc, gs = q.quantize_nvfp4(w)
        wd = q.dequantize_nvfp4(wp, sc, gs)
    got = cuda_fp4.dequant_w4(wp.contiguous(), sc.contiguous(), fmt, gs)
    torch.cuda.synchronize()
    assert torch.equal(got, wd.bfloat16())
    x = torch.randn(cuda_fp4.DEQUANT_FROM_TOKENS + 5, 512, device=DEV, generator=g).bfloat16()
    y = cu().w4a16_gemm(x, wp.contiguous(), sc.contiguous(), fmt, gs)
    want = x.float() @ wd.bfloat16().float().t()
    assert (y.float() - want).abs().max() <= 1e-2 * want.abs().max() + 1e-2


@pytest.mark.parametrize("group", [32, 64, 128])
@pytest.mark.parametrize("T,N,K,bias", [(1, 256, 128, False), (16, 1024, 512, True), (64, 1280, 4096, False),
                                        (100, 200, 256, True), (1100, 384, 1024, False)])
def test_int4_group_weights_on_the_w4a16_kernel(group, T, N, K, bias):
    """AWQ / GPTQ style weights (unsigned nibbles, fp16 group scales, zero points) stay packed: the fused kernel
    for decode sizes, the dequant kernel + bf16 GEMM from 1024 tokens; the dequant kernel is bit-exact against
    (nibble - zero) * scale rounded to bf16."""
    from vllm_torchtpu_b200.ops import cuda_fp4
    from vllm_torchtpu_b200.quantization.int4 import dequantize_int4_group, quantize_int4_group
    g = torch.Generator(device=DEV).manual_seed(T + N + group)
    x = torch.randn(T, K, device=DEV, generator=g).bfloat16()
    w = torch.randn(N, K, device=DEV, generator=g) * 0.05 + 0.01
    b = torch.randn(N, device=DEV, generator=g).bfloat16() if bias else None
    wp, sc, zp = quantize_int4_group(w, group)
    wd = dequantize_int4_group(wp, sc, zp, group).bfloat16()
    got_w = cuda_fp4.dequant_int4(wp.contiguous(), sc.half().contiguous(), zp.contiguous(), group)
    assert torch.equal(got_w, wd)
    y = cuda_fp4.w4a16_int4_gemm(x, wp.contiguous(), sc.half().contiguous(), zp.contiguous(), group, b)
    torch.cuda.synchronize()
    assert cu().check_status() == 0
    want = x.float() @ wd.float().t()
    if bias:
        want = want + b.float()
    err = (y.float() - want).abs().max().item()
    assert err <= 1e-2 * want.abs().max().item() + 1e-2, err


def test_int4_linear_method_runs_packed_on_the_device():
    from vllm_torchtpu_b200.layers.linear import ColumnParallelLinear
    from vllm_torchtpu_b200.quantization import QuantConfig
    lin = ColumnParallelLinear("l", 512, [768], dtype=torch.bfloat16, device=DEV, quant_config=QuantConfig("awq"))
    lin.init_dummy(0.05, 0)
    assert lin.weight.dtype == torch.uint8 and lin.weight.shape == (768, 256) and lin.weight_scale_h is not None
    from vllm_torchtpu_b200.quantization.int4 import dequantize_int4_group
    x = torch.randn(20, 512, device=DEV).bfloat16()
    from vllm_torchtpu_b200 import ops
    before = ops.launch_count()
    y = lin(x)
    assert ops.launch_count() - before == 1          # one fused kernel, no dequantised copy of the weight
    want = x.float() @ dequantize_int4_group(lin.weight, lin.weight_scale, lin.weight_zero, lin.group).bfloat16().float().t()
    assert (y.float() - want).abs().max().item() <= 1e-2 * want.abs().max().item() + 1e-2
