"""tcgen05 bf16 GEMM vs fp32 matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"

SHAPES = [
    (16, 256, 512), (1, 128, 64), (64, 4096, 4096), (100, 384, 1024), (128, 1024, 2048),
    (300, 1024, 512), (64, 6144, 4096), (64, 4096, 14336), (1024, 2048, 4096), (777, 1000, 520),
    (8192, 1024, 1024),
]


def _run(T, N, K, bias=False, splits=0):
    from vllm_torchtpu_b200.ops import cuda
    g = torch.Generator(device=DEV).manual_seed(T + N + K)
    x = torch.randn(T, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.05).bfloat16()
    b = torch.randn(N, device=DEV, generator=g).bfloat16() if bias else None
    y = cuda.gemm(x, w, b, force_splits=splits)
    torch.cuda.synchronize()
    assert cuda.check_status() == 0
    want = x.float() @ w.float().t()
    if b is not None:
        want = want + b.float()
    err = (y.float() - want).abs().max().item()
    scale = want.abs().max().item()
    assert err <= 2e-2 * scale + 1e-2, f"{(T, N, K)}: max err {err} vs scale {scale}"


@pytest.mark.parametrize("T,N,K", SHAPES)
def test_gemm(T, N, K):
    _run(T, N, K)


@pytest.mark.parametrize("T,N,K,bias", [(64, 28672, 4096, False), (64, 6144, 4096, True), (64, 4096, 4096, False),
                                        (32, 2304, 1024, True), (128, 9600, 2048, False), (300, 4000, 1024, True),
                                        (512, 4096, 4096, False), (17, 19000, 512, False)])
def test_gemm_tile_counts_that_do_not_fill_the_sms(T, N, K, bias):
    """Tile counts that leave SMs idle under whole-tile scheduling (224, 48, 32 ... tiles on 148 SMs), run twice
    (split-K counters and cluster launches are re-armed by the kernel)."""
    _run(T, N, K, bias=bias)
    _run(T, N, K, bias=bias)


def test_gemm_bias():
    _run(64, 512, 1024, bias=True)
    _run(500, 512, 1024, bias=True)


@pytest.mark.parametrize("splits", [2, 3, 7])
def test_gemm_split_k(splits):
    _run(64, 512, 4096, splits=splits)
    _run(64, 512, 4096, bias=True, splits=splits)      # counters were re-armed by the first call


def test_gemm_strided_views():
    from vllm_torchtpu_b200.ops import cuda
    big = torch.randn(64, 4096 + 512, device=DEV).bfloat16()
    x = big[:, :4096]
    w = (torch.randn(256, 4096, device=DEV) * 0.05).bfloat16()
    y = cuda.gemm(x, w)
    want = x.float() @ w.float().t()
    torch.testing.assert_close(y.float(), want, rtol=2e-2, atol=5e-2)


@pytest.mark.parametrize("T,N,K,bias", [(256, 256, 64, False), (1024, 4096, 4096, False), (300, 392, 520, True),
                                        (8192, 1024, 1024, True), (2049, 6144, 4096, False)])
def test_gemm_two_sm(T, N, K, bias, monkeypatch):
    """cta_group::2 kernel (SM pairs, 256 x 256 tiles) against the fp32 product, ragged edges included."""
    from vllm_torchtpu_b200 import envs
    from vllm_torchtpu_b200.ops import cuda
    monkeypatch.setenv("B200_GEMM_2SM_MIN_T", "1")
    envs.reset()
    try:
        g = torch.Generator(device="cuda").manual_seed(T + N)
        x = torch.randn(T, K, device="cuda", generator=g).bfloat16()
        w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
        b = torch.randn(N, device="cuda", generator=g).bfloat16() if bias else None
        y = cuda.gemm(x, w, b)
        want = x.float() @ w.float().t()
        if bias:
            want = want + b.float()
        torch.cuda.synchronize()
        assert cuda.check_status() == 0
        err = (y.float() - want).abs().max().item()
        assert err <= 2e-2 * want.abs().max().item() + 1e-2, err
    finally:
        monkeypatch.delenv("B200_GEMM_2SM_MIN_T")
        envs.reset()


@pytest.mark.parametrize("T,I,K", [(256, 128, 64), (1024, 1024, 512), (300, 200, 520), (4096, 3584, 1024)])
def test_gemm_swiglu_two_sm(T, I, K, monkeypatch):
    """SwiGLU form of the cta_group::2 kernel: gate and up rows share a CTA's accumulator lanes."""
    from vllm_torchtpu_b200 import envs
    from vllm_torchtpu_b200.ops import cuda
    monkeypatch.setenv("B200_GEMM_2SM_MIN_T", "1")
    envs.reset()
    try:
        g = torch.Generator(device="cuda").manual_seed(T + I)
        x = torch.randn(T, K, device="cuda", generator=g).bfloat16()
        w = (torch.randn(2 * I, K, device="cuda", generator=g) * 0.05).bfloat16()
        y = cuda.gemm_swiglu(x, w)
        gu = x.float() @ w.float().t()
        want = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
        torch.cuda.synchronize()
        assert cuda.check_status() == 0
        err = (y.float() - want).abs().max().item()
        assert err <= 2e-2 * want.abs().max().item() + 1e-2, err
    finally:
        monkeypatch.delenv("B200_GEMM_2SM_MIN_T")
        envs.reset()
