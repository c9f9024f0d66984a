"""Gated DeltaNet kernels vs the PyTorch recurrence, including state carried across steps."""
import pytest
import torch

from vllm_torchtpu_b200.ops import gdn_reference as g
from vllm_torchtpu_b200.runner.attn_metadata import AttentionMetadata

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _meta(q_lens, ctx, slots):
    qsl = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    sl = torch.tensor([a + b for a, b in zip(q_lens, ctx)], dtype=torch.int32, device=DEV)
    return AttentionMetadata(None, None, None, sl, qsl, len(q_lens), sum(q_lens),
                             padded_num_reqs=len(q_lens), padded_num_tokens=sum(q_lens),
                             state_slots=torch.tensor(slots, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("Hk,Hv,dk,dv", [(2, 4, 128, 128), (2, 2, 64, 64)])
def test_gdn_forward_two_steps(Hk, Hv, dk, dv):
    from vllm_torchtpu_b200.ops import cuda
    torch.manual_seed(0)
    C = 2 * Hk * dk + Hv * dv
    conv_w = (torch.randn(C, 4, device=DEV) * 0.3).bfloat16()
    A_log = torch.randn(Hv, device=DEV) * 0.3
    dt_bias = torch.randn(Hv, device=DEV) * 0.3
    pools = [(torch.zeros(5, C, 3, device=DEV, dtype=torch.bfloat16), torch.zeros(5, Hv, dk, dv, device=DEV))
             for _ in range(2)]
    for q_lens, ctx in (([17, 1, 40], [0, 0, 0]), ([1, 1, 5], [17, 1, 40])):
        T = sum(q_lens)
        mixed = torch.randn(T, C, device=DEV).bfloat16()
        a, b = torch.randn(T, Hv, device=DEV).bfloat16(), torch.randn(T, Hv, device=DEV).bfloat16()
        meta = _meta(q_lens, ctx, [3, 0, 2])
        got = cuda.gdn_forward(mixed, a, b, meta, pools[0][0], pools[0][1], conv_w, A_log, dt_bias, Hk, Hv, dk, dv)
        want = g.gdn_forward(mixed, a, b, None, meta, pools[1][0], pools[1][1], conv_w, A_log, dt_bias, Hk, Hv, dk, dv)
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 3e-2 * want.float().abs().max().item() + 1e-2, err
    torch.testing.assert_close(pools[0][1], pools[1][1], rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("Hk,Hv,dk,dv,lb", [(2, 2, 128, 128, None), (2, 4, 64, 64, -5.0), (1, 2, 32, 128, None)])
def test_kda_forward_two_steps(Hk, Hv, dk, dv, lb):
    """Per-channel decay (Kimi Delta Attention): both gate forms, state carried across two steps."""
    from vllm_torchtpu_b200.ops import cuda
    torch.manual_seed(1)
    A_log = torch.randn(Hv, device=DEV) * 0.3
    dt_bias = torch.randn(Hv, dk, device=DEV) * 0.3
    pools = [torch.zeros(5, Hv, dk, dv, device=DEV) for _ in range(2)]
    for q_lens, ctx in (([17, 1, 40], [0, 0, 0]), ([1, 1, 5], [17, 1, 40])):
        T = sum(q_lens)
        q = torch.randn(T, Hk, dk, device=DEV).bfloat16()
        k = torch.randn(T, Hk, dk, device=DEV).bfloat16()
        v = torch.randn(T, Hv, dv, device=DEV).bfloat16()
        a = torch.randn(T, Hv, dk, device=DEV).bfloat16()
        b = torch.randn(T, Hv, device=DEV).bfloat16()
        meta = _meta(q_lens, ctx, [3, 0, 2])
        got = cuda.kda_forward(q, k, v, a, b, meta, pools[0], A_log, dt_bias, lb)
        want = g.kda_forward(q, k, v, a, b, meta, pools[1], A_log, dt_bias, lb)
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 3e-2 * want.float().abs().max().item() + 1e-2, err
    torch.testing.assert_close(pools[0], pools[1], rtol=3e-2, atol=3e-2)
