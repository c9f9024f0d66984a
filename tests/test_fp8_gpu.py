"""Block-scaled fp8 tcgen05 GEMM vs the fp32 statement of the same quantised computation."""
import pytest
import torch

from vllm_torchtpu_b200.quantization import fp8 as q

pytestmark = pytest.mark.gpu
DEV = "cuda"


def cu():
    from vllm_torchtpu_b200.ops import cuda
    return cuda


def test_quant_act_matches_reference():
    x = (torch.randn(37, 640, device=DEV) * 3).bfloat16()
    xq, xs = cu().quant_act_1x128(x)
    rq, rs = q.quantize_act_1x128(x)
    torch.testing.assert_close(xs, rs, rtol=1e-6, atol=0)
    # e4m3 rounding of x/scale may differ by one ulp between the two conversions
    assert (xq.float() - rq.float()).abs().max() <= 32.0
    assert ((xq.float() * xs.repeat_interleave(128, 1)[:, :640]) - x.float()).abs().max() <= 0.07 * x.float().abs().max()


def test_quant_rows_bounded_by_device_count_and_fused_swiglu():
    """Only the first rows[0] rows are written; with swiglu the quantised values are those of
    quantising SiLU(gate) * up (rounded to bf16) on its own."""
    T, K = 90, 384
    x = (torch.randn(T, 2 * K, device=DEV) * 2).bfloat16()
    rows = torch.tensor([53], dtype=torch.int32, device=DEV)
    xq = torch.zeros(T, K, dtype=torch.float8_e4m3fn, device=DEV)
    xs = torch.full((T, 3), -1.0, device=DEV)
    cu().quant_rows_1x128(x, K, rows=rows, swiglu=True, out=(xq, xs))
    act = (torch.nn.functional.silu(x[:, :K].float()) * x[:, K:].float()).bfloat16()
    rq, rs = cu().quant_act_1x128(act)
    torch.cuda.synchronize()
    assert (xs[53:] == -1.0).all() and (xq[53:].float() == 0).all()
    torch.testing.assert_close(xs[:53], rs[:53], rtol=2e-2, atol=0)
    deq = xq[:53].float() * xs[:53].repeat_interleave(128, 1)
    assert (deq - act[:53].float()).abs().max() <= 0.07 * act.float().abs().max()
    # plain form over all rows equals the per-row kernel
    xq2, xs2 = cu().quant_rows_1x128(x, 2 * K)
    rq2, rs2 = cu().quant_act_1x128(x)
    assert torch.equal(xs2, rs2) and torch.equal(xq2.view(torch.uint8), rq2.view(torch.uint8))


@pytest.mark.parametrize("T,N,K", [(16, 256, 512), (64, 1280, 8192), (100, 384, 1024), (128, 7168, 2048),
                                   (300, 1024, 640), (1, 128, 128),
                                   # more tiles than SMs with a short last wave: main launch + split-K tail launch
                                   (64, 28672, 1024), (16, 20000, 2048)])
def test_fp8_block_gemm(T, N, K):
    g = torch.Generator(device=DEV).manual_seed(T + N)
    x = torch.randn(T, K, device=DEV, generator=g).bfloat16()
    w = torch.randn(N, K, device=DEV, generator=g) * 0.05
    wq, ws = q.quantize_weight_block(w)
    y = cu().fp8_block_gemm(x, wq, ws)
    torch.cuda.synchronize()
    assert cu().check_status() == 0
    want = q.fp8_block_gemm_reference(x, wq, ws, out_dtype=torch.float32)
    err = (y.float() - want).abs().max().item()
    assert err <= 2e-2 * want.abs().max().item() + 1e-2, err


@pytest.mark.parametrize("T,N,K,bias", [(1500, 4096, 1024, False), (4096, 1280, 2048, True), (777, 6152, 640, True),
                                        (129, 28672, 512, False)])
def test_fp8_block_gemm_many_token_kernel(T, N, K, bias):
    """Token-major kernel (tokens on the TMEM lanes): ragged token and weight tiles, bias, N not a multiple
    of the 256-row tile."""
    from vllm_torchtpu_b200.ops import cuda_fp8
    assert cuda_fp8.use_rows_kernel(T, N)
    g = torch.Generator(device=DEV).manual_seed(T + N)
    x = torch.randn(T, K, device=DEV, generator=g).bfloat16()
    w = torch.randn(N, K, device=DEV, generator=g) * 0.05
    b = torch.randn(N, device=DEV, generator=g).bfloat16() if bias else None
    wq, ws = q.quantize_weight_block(w)
    y = cu().fp8_block_gemm(x, wq, ws, b)
    torch.cuda.synchronize()
    assert cu().check_status() == 0
    want = q.fp8_block_gemm_reference(x, wq, ws, out_dtype=torch.float32)
    if bias:
        want = want + b.float()
    err = (y.float() - want).abs().max().item()
    assert err <= 2e-2 * want.abs().max().item() + 1e-2, err


def test_fp8_grouped_gemm_many_token_kernel():
    """Grouped form: uneven groups (one empty, one of a single row) against the per-group reference."""
    from vllm_torchtpu_b200.ops import cuda_fp8
    E, N, K = 6, 1024, 512
    sizes = [700, 0, 1, 1300, 257, 3000]
    R = sum(sizes)
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn(R, K, device=DEV, generator=g).bfloat16()
    w = torch.randn(E, N, K, device=DEV, generator=g) * 0.05
    qs = [q.quantize_weight_block(w[e]) for e in range(E)]
    wq, ws = torch.stack([a for a, _ in qs]), torch.stack([b for _, b in qs])
    off = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device=DEV)
    y = cuda_fp8.grouped_fp8_gemm(x, wq, ws, off, R // E)
    torch.cuda.synchronize()
    assert cu().check_status() == 0
    lo = 0
    for e, n in enumerate(sizes):
        if n:
            want = q.fp8_block_gemm_reference(x[lo:lo + n], wq[e], ws[e], out_dtype=torch.float32)
            err = (y[lo:lo + n].float() - want).abs().max().item()
            assert err <= 2e-2 * want.abs().max().item() + 1e-2, (e, err)
        lo += n


def test_fp8_moe_experts():
    from vllm_torchtpu_b200.ops import reference as ref
    T, E, k, H, I = 50, 8, 2, 512, 256
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(T, H, device=DEV, generator=g).bfloat16()
    w13 = torch.randn(E, 2 * I, H, device=DEV, generator=g) * 0.05
    w2 = torch.randn(E, H, I, device=DEV, generator=g) * 0.05
    q13 = [q.quantize_weight_block(w13[e]) for e in range(E)]
    q2 = [q.quantize_weight_block(w2[e]) for e in range(E)]
    w13q, s13 = torch.stack([a for a, _ in q13]), torch.stack([b for _, b in q13])
    w2q, s2 = torch.stack([a for a, _ in q2]), torch.stack([b for _, b in q2])
    ids, w = ref.moe_route(torch.randn(T, E, device=DEV, generator=g), k)
    got = cu().moe_experts_fp8(x, w13q, s13, w2q, s2, ids, w, 0)
    torch.cuda.synchronize()
    assert cu().check_status() == 0
    d13 = torch.stack([q.dequantize_weight_block(w13q[e], s13[e]) for e in range(E)]).bfloat16()
    d2 = torch.stack([q.dequantize_weight_block(w2q[e], s2[e]) for e in range(E)]).bfloat16()
    want = ref.moe_experts(x, d13, d2, ids, w, 0)
    err = (got.float() - want.float()).abs().max().item()
    assert err <= 6e-2 * want.float().abs().max().item() + 2e-2, err     # activations are fp8 in the kernel path


@pytest.mark.parametrize("T,N,K", [(1, 256, 512), (48, 1024, 4096), (64, 4096, 1024), (200, 640, 2048)])
def test_int8_w8a8_gemm_matches_reference(T, N, K):
    from vllm_torchtpu_b200.ops import cuda
    from vllm_torchtpu_b200.quantization import int8 as q8
    g = torch.Generator(device="cuda").manual_seed(T + N)
    x = torch.randn(T, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    wq, ws = q8.quantize_weight_int8(w)
    xq, xs = cuda.quant_act_int8(x)
    rq, rs = q8.quantize_act_int8(x)
    assert (xq.int() - rq.int()).abs().max() <= 1                    # rounding ties only
    torch.testing.assert_close(xs, rs.squeeze(-1), rtol=1e-5, atol=1e-8)
    got = cuda.int8_gemm(x, wq, ws)
    want = q8.int8_gemm_reference(x, wq, ws)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2 * want.float().abs().max().item())
    assert cuda.check_status() == 0


def test_fp8_per_tensor_linear_quantises_activations_in_one_kernel():
    """Per-tensor weight scale, per-token activation scale: the kernel path against the same arithmetic in fp32."""
    from vllm_torchtpu_b200.ops import launch_count
    T, N, K = 77, 640, 1024
    g = torch.Generator(device=DEV).manual_seed(11)
    x = (torch.randn(T, K, device=DEV, generator=g) * 2).bfloat16()
    w = torch.randn(N, K, device=DEV, generator=g) * 0.05
    s = w.abs().max() / 448.0
    wq = (w / s).clamp(-448, 448).to(torch.float8_e4m3fn)
    before = launch_count()
    y = cu().fp8_per_tensor_gemm(x, wq, s.reshape(1))
    assert launch_count() - before == 2                     # activation quantisation + GEMM
    torch.cuda.synchronize()
    assert cu().check_status() == 0
    xs = x.float().abs().amax(-1, keepdim=True).clamp_min(1e-12) / 448.0
    xq = (x.float() / xs).clamp(-448, 448).to(torch.float8_e4m3fn)
    want = (xq.float() @ wq.float().t()) * xs * s
    err = (y.float() - want).abs().max().item()
    assert err <= 2e-2 * want.abs().max().item() + 1e-2, err
