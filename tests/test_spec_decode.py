"""Speculative decoding pieces on CPU: drafter, rejection sampling laws, engine equivalence."""
import numpy as np
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
