"""Speculative decoding pieces on CPU: drafter, rejection sampling laws, engine equivalence."""
import numpy as np
import pytest
import torch

from vllm_torchtpu_b200 import SamplingParams
from vllm_torchtpu_b200.engine.llm import LLM
from vllm_torchtpu_b200.sample.rejection_sampler import greedy_accept, rejection_sample
from vllm_torchtpu_b200.spec_decode.ngram import find_ngram_continuation


def test_ngram_lookup():
    t = np.array([1, 2, 3, 4, 5, 9, 9, 2, 3, 4])
    assert find_ngram_continuation(t, 2, 4, 3) == [5, 9, 9]
    assert find_ngram_continuation(np.array([1, 2, 3]), 2, 4, 3) == []


def test_greedy_accept():
    assert greedy_accept([5, 6, 7], [5, 6, 7, 8]) == [5, 6, 7, 8]
    assert greedy_accept([5, 6, 7], [5, 9, 7, 8]) == [5, 9]
    assert greedy_accept([], [3]) == [3]


def test_rejection_sampling_preserves_target_distribution():
    torch.manual_seed(0)
    V = 6
    p = torch.tensor([[0.5, 0.2, 0.1, 0.1, 0.05, 0.05], [0.1, 0.1, 0.6, 0.1, 0.05, 0.05]])
    q = torch.tensor([[0.1, 0.6, 0.1, 0.1, 0.05, 0.05]])
    counts = torch.zeros(V)
    n = 20000
    for _ in range(n):
        d = torch.multinomial(q[0], 1)
        out = rejection_sample(d, p, q, torch.rand(1), torch.rand(2))
        counts[out[0]] += 1
    assert torch.allclose(counts / n, p[0], atol=0.02)


def test_engine_with_ngram_drafts_matches_plain_greedy():
    rng = np.random.RandomState(5)
    base = rng.randint(0, 1024, size=12).tolist()
    prompts = [base * 4, rng.randint(0, 1024, size=30).tolist()]
    sp = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    plain = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    want = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    spec = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False,
               speculative_config={"method": "ngram", "num_speculative_tokens": 3, "prompt_lookup_min": 2})
    got = [o.outputs[0].token_ids for o in spec.generate(prompts, sp)]
    assert got == want
    assert spec.engine.spec.stats["proposed"] > 0
    assert spec.engine.runner.stats.get("spec_accepted", 0) >= 0


def test_adaptive_verification_budget_and_prefixes():
    """The budget maximises expected tokens per millisecond under the cost table; every request keeps a
    prefix of its drafts; cheap rows admit more drafts than expensive rows; padding is refilled."""
    from vllm_torchtpu_b200.spec_decode.adaptive_verification import AdaptiveVerificationManager, StepCostTable
    conf = {"a": [0.9, 0.9, 0.9], "b": [0.5, 0.2, 0.9], "c": [0.05, 0.9, 0.9]}
    flat = AdaptiveVerificationManager(StepCostTable([(1, 1.0), (64, 1.0)]), 3)
    assert flat.select(conf) == {"a": 3, "b": 3, "c": 3}          # rows are free: verify everything
    steep = AdaptiveVerificationManager(StepCostTable([(3, 1.0), (12, 10.0)]), 3)
    keep = steep.select(conf)
    assert keep["a"] >= keep["b"] >= keep["c"] and keep["c"] == 0 and sum(keep.values()) < 9
    # exhaustive check of the optimum over budgets
    surv = sorted((s for c in conf.values() for s in steep.survival(c)), reverse=True)
    rates = [(3 + sum(surv[:b])) / steep.cost_table.cost(3 + b) for b in range(10)]
    assert sum(keep.values()) == max(range(10), key=lambda b: rates[b])
    grown = steep.expand(keep, conf, extra_rows=2)
    assert sum(grown.values()) == sum(keep.values()) + 2 and all(grown[r] >= keep[r] for r in keep)
    expect = steep.select({"a": conf["a"], "b": conf["b"]}, base_rows=3)
    trimmed = steep.trim({"a": [1, 2, 3], "b": [4, 5, 6], "z": [7]}, conf, base_rows=3)
    assert trimmed.get("a", []) == [1, 2, 3][: expect["a"]] and trimmed.get("b", []) == [4, 5, 6][: expect["b"]]
    assert trimmed["z"] == [7] and "c" not in trimmed          # no confidences: drafts kept whole
    # overhead calibration ignores stalls
    steep.observe(3, 1.5)
    assert 0 < steep.overhead_ms < 0.1
    before = steep.overhead_ms
    steep.observe(3, 100.0)
    assert steep.overhead_ms == before
    t = StepCostTable([(8, 1.0), (16, 2.0), (32, 6.0)])
    assert t.cost(12) == 1.5 and t.cost(24) == 4.0 and t.cost(64) == 14.0 and t.cost(1) >= 0.0


def test_engine_with_draft_head_and_adaptive_verification_is_lossless():
    prompts = [np.random.RandomState(7).randint(0, 1024, size=n).tolist() for n in (9, 21)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    plain = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    want = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    spec = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False,
               speculative_config={"method": "mtp", "num_speculative_tokens": 3,
                                   "enable_adaptive_verification": True,
                                   "step_cost_samples": [(1, 1.0), (4, 1.2), (16, 4.0)]})
    got = [o.outputs[0].token_ids for o in spec.generate(prompts, sp)]
    assert got == want
    st = spec.engine.adaptive.stats
    assert st["steps"] > 0 and st["verified"] <= st["proposed"]
    with pytest.raises(ValueError):
        LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False,
            speculative_config={"method": "ngram", "enable_adaptive_verification": True})


def test_medusa_heads_load_from_a_checkpoint_and_reproduce_plain_decoding(tmp_path):
    """Heads written as a Medusa checkpoint (identity-like blocks + the target's own projection) draft the
    token the target would produce next from the same hidden state, so some drafts are accepted, and the
    output equals plain greedy decoding whatever is accepted."""
    import torch
    from safetensors.torch import save_file

    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.engine.llm import LLM
    prompts = [[5, 6, 7, 8, 9, 10, 11], [21, 22, 23, 24], [3, 4, 9, 10, 2, 17]]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    kw = dict(device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    plain_llm = LLM("tiny-llama", **kw)
    plain = [o.outputs[0].token_ids for o in plain_llm.generate(prompts, sp)]
    H = plain_llm.engine.cfg.model.hidden_size
    lm_head = plain_llm.engine.runner.model.lm_head
    tensors = {}
    for i in range(2):
        tensors[f"medusa_heads.{i}.0.linear.weight"] = torch.zeros(H, H)
        tensors[f"medusa_heads.{i}.0.linear.bias"] = torch.zeros(H)
        tensors[f"medusa_heads.{i}.1.weight"] = lm_head.float().clone()
    save_file(tensors, str(tmp_path / "model.safetensors"))
    spec_llm = LLM("tiny-llama", speculative_config={"method": "medusa", "num_speculative_tokens": 2,
                                                      "model": str(tmp_path)}, **kw)
    got = [o.outputs[0].token_ids for o in spec_llm.generate(prompts, sp)]
    assert got == plain
    prop = spec_llm.engine.spec
    assert prop.num_speculative_tokens == 2 and prop.stats["proposed"] > 0
    assert len(prop.blocks) == 2 and prop.heads[0] is not None
    assert spec_llm.engine.runner.stats.get("spec_drafted", 0) > 0
