"""Small CUDA kernels (LoRA bgmv, token bitmask, pool row copies, fp8 KV, TurboQuant) against the
plain-PyTorch statements of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_bgmv_shrink_expand_match_reference():
    from vllm_torchtpu_b200.lora import ops as lops
    g = torch.Generator(device=DEV).manual_seed(0)
    T, K, N, r, S = 37, 512, 768, 16, 4
    x = torch.randn(T, K, device=DEV, generator=g).bfloat16()
    A = (torch.randn(S, r, K, device=DEV, generator=g) * 0.05).bfloat16()
    B = (torch.randn(S, N, r, device=DEV, generator=g) * 0.05).bfloat16()
    idx = torch.randint(-1, S, (T,), device=DEV, generator=g)
    scale = torch.tensor([0.5, 1.0, 2.0, 0.25], device=DEV)
    y0 = torch.randn(T, N + 64, device=DEV, generator=g).bfloat16()
    got = lops.lora_apply(x, y0.clone(), A, B, idx, scale, col_offset=64)
    want = lops.lora_apply(x.cpu(), y0.cpu().clone(), A.cpu(), B.cpu(), idx.cpu(), scale.cpu(), col_offset=64)
    torch.testing.assert_close(got.float().cpu(), want.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_token_bitmask_matches_reference(dtype):
    from vllm_torchtpu_b200.structured import apply_token_bitmask
    g = torch.Generator().manual_seed(1)
    R, V = 6, 1000
    logits = torch.randn(R, V, generator=g).to(dtype)
    bm = torch.randint(-2**31, 2**31 - 1, (3, (V + 31) // 32), generator=g, dtype=torch.int64).to(torch.int32)
    rows = torch.tensor([4, 0, 5])
    want = apply_token_bitmask(logits.clone(), bm, rows)
    got = apply_token_bitmask(logits.clone().to(DEV), bm.to(DEV), rows.to(DEV))
    assert torch.equal(got.cpu(), want)
    assert torch.equal(apply_token_bitmask(logits[:3].clone().to(DEV), bm.to(DEV)).cpu(),
                       apply_token_bitmask(logits[:3].clone(), bm))


def test_copy_rows_between_state_pools():
    from vllm_torchtpu_b200.ops import cuda_misc
    src = torch.randn(9, 4, 32, 24, device=DEV)
    dst = torch.zeros(7, 4, 32, 24, device=DEV)
    di = torch.tensor([3, -1, 0, 6], device=DEV)
    si = torch.tensor([8, 2, 1, -1], device=DEV)
    cuda_misc.copy_rows(dst, src, di, si)
    want = torch.zeros_like(dst)
    want[3], want[0] = src[8], src[1]
    assert torch.equal(dst, want)


def test_fp8_kv_quant_roundtrip():
    from vllm_torchtpu_b200.ops import cuda_misc
    from vllm_torchtpu_b200.quantization import turboquant as tq
    x = (torch.randn(1000, 128, device=DEV) * 3).bfloat16()
    q = cuda_misc.quantize_kv_fp8(x, 0.05)
    assert torch.equal(q.view(torch.uint8).cpu(), tq.quantize_kv_fp8(x.cpu(), 0.05).view(torch.uint8))
    back = cuda_misc.dequantize_kv_fp8(q, 0.05)
    torch.testing.assert_close(back.float().cpu(), tq.dequantize_kv_fp8(q.cpu(), 0.05).float())


def test_turboquant_4bit_matches_reference_and_preserves_dot_products():
    from vllm_torchtpu_b200.ops import cuda_misc
    from vllm_torchtpu_b200.quantization import turboquant as tq
    g = torch.Generator(device=DEV).manual_seed(3)
    k = torch.randn(300, 128, device=DEV, generator=g).bfloat16()
    v = (torch.randn(300, 128, device=DEV, generator=g) * 0.7 + 0.2).bfloat16()
    kc, kn, vc, vm = cuda_misc.tq4_encode(k, v)
    rk, rn, rv, rm = tq.encode(k.cpu(), v.cpu())
    # codes agree except where a coordinate sits on a decision boundary
    assert (kc.cpu() != rk).float().mean() < 0.02
    assert (vc.cpu() != rv).float().mean() < 0.02
    torch.testing.assert_close(kn.float().cpu(), rn.float(), rtol=2e-2, atol=1e-2)
    torch.testing.assert_close(vm.float().cpu(), rm.float(), rtol=1e-2, atol=1e-2)
    kd, vd = cuda_misc.tq4_decode(kc, kn, vc, vm)
    wk, wv = tq.decode(kc.cpu(), kn.cpu(), vc.cpu(), vm.cpu())
    torch.testing.assert_close(kd.float().cpu(), wk.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(vd.float().cpu(), wv.float(), rtol=2e-2, atol=2e-2)
    # quantisation quality: 4-bit keys keep attention scores close
    q = torch.randn(16, 128, device=DEV, generator=g)
    s_ref, s_q = q @ k.float().t(), q @ kd.float().t()
    assert (s_ref - s_q).abs().mean() / s_ref.abs().mean() < 0.15
    assert (vd.float() - v.float()).abs().max() < 0.2
