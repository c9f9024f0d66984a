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


def test_engine_serves_adapter_and_base_requests_in_one_batch():
    """A request with an adapter must generate what a model with merged weights (W + scale * B A)
    generates, while a base request in the same batch is unaffected."""
    import numpy as np

    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.engine.llm import LLM

    def make():
        return LLM("tiny-llama", device="cpu", max_num_seqs=4, max_num_batched_tokens=64, block_size=16,
                   num_gpu_blocks_override=32)
    rng = np.random.RandomState(0)
    llm = make()
    cfg = llm.engine.cfg.model
    prompts = [rng.randint(0, cfg.vocab_size, size=n).tolist() for n in (9, 14)]
    base = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6))]

    g = torch.Generator().manual_seed(1)
    r, alpha = 4, 64.0
    weights, merged = {}, {}
    model = llm.engine.runner.model
    for lin in model.named_linears():
        prefix, leaf = lin.name.rsplit(".", 1)
        if leaf == "qkv_proj":
            size = lin.shard_sizes[0]                          # adapt q_proj only
            A = torch.randn(r, lin.in_features, generator=g) * 0.3
            B = torch.randn(size, r, generator=g) * 0.3
            weights[f"{prefix}.q_proj"] = (A, B)
            merged[lin.name] = (0, size, (alpha / r) * (B @ A))
        elif leaf == "down_proj":
            A = torch.randn(r, lin.in_features, generator=g) * 0.3
            B = torch.randn(lin.out_features, r, generator=g) * 0.3
            weights[lin.name] = (A, B)
            merged[lin.name] = (0, lin.out_features, (alpha / r) * (B @ A))
    assert llm.engine.add_lora("ad1", r, alpha, weights)
    assert llm.engine.list_loras() == ["ad1"]
    sp_l = SamplingParams(temperature=0.0, max_tokens=6, lora_name="ad1")
    sp_b = SamplingParams(temperature=0.0, max_tokens=6)
    outs = llm.generate([prompts[0], prompts[1]], [sp_l, sp_b])
    got_lora, got_base = outs[0].outputs[0].token_ids, outs[1].outputs[0].token_ids
    assert got_base == base[1]

    ref = make()
    for lin in ref.engine.runner.model.named_linears():
        if lin.name in merged:
            lo, size, delta = merged[lin.name]
            lin.weight[lo:lo + size] += delta.to(lin.weight.dtype)
    want = ref.generate([prompts[0]], sp_b)[0].outputs[0].token_ids
    assert got_lora == want
    assert got_lora != base[0]                                # the adapter changes the output
