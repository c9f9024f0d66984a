import pytest
import torch

from vllm_torchtpu_b200.lora import LoRAAdapter, LoRAManager, lora_apply


def test_bgmv_matches_per_token_reference():
    torch.manual_seed(0)
    T, K, N, r, S = 9, 32, 24, 4, 3
    x = torch.randn(T, K)
    y = torch.randn(T, N)
    A, B = torch.randn(S, r, K), torch.randn(S, N, r)
    idx = torch.tensor([0, -1, 2, 2, 1, -1, 0, 1, 2])
    scale = torch.tensor([0.5, 2.0, 1.0])
    want = y.clone()
    for t in range(T):
        if idx[t] >= 0:
            s = int(idx[t])
            want[t] += scale[s] * (x[t] @ A[s].t()) @ B[s].t()
    got = lora_apply(x, y.clone(), A, B, idx, scale)
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)


def test_manager_slots_lru_and_pinning():
    m = LoRAManager(max_loras=2, max_rank=8, dtype=torch.float32)
    m.register_layer("l0.q", 16, 16)
    for n in "abc":
        m.add_adapter(LoRAAdapter(n, 4, 8.0, {"l0.q": (torch.ones(4, 16), torch.ones(16, 4))}))
    with pytest.raises(ValueError):
        m.add_adapter(LoRAAdapter("big", 16, 1.0))
    sa, sb = m.activate("a"), m.activate("b")
    assert {sa, sb} == {0, 1}
    m.pin_adapter("a")
    sc = m.activate("c")                      # evicts b (a is pinned)
    assert sc == sb and "b" not in m.slot_of
    assert float(m.scales[sc]) == 2.0 and float(m.layers["l0.q"][0][sc, :4].sum()) == 64.0
    idx = m.token_indices(["a", None, "c"], [2, 1, 3])
    assert idx.tolist() == [sa, sa, -1, sc, sc, sc]
    assert m.remove_adapter("a") and m.list_adapters() == ["b", "c"]
