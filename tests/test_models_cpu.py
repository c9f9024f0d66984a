"""Model families on the CPU path vs dense references."""
import numpy as np
import torch

from vllm_torchtpu_b200 import SamplingParams
from vllm_torchtpu_b200.engine.llm import LLM


def _prompts(vocab=1024):
    rng = np.random.RandomState(1)
    return [rng.randint(0, vocab, size=n).tolist() for n in (5, 19, 40)]


def test_mla_moe_engine_matches_non_absorbed_dense_forward():
    from vllm_torchtpu_b200.models.reference_forward_mla import dense_mla_logits
    llm = LLM("tiny-mla", device="cpu", max_num_seqs=4, max_num_batched_tokens=32, block_size=16,
              init_dist=False)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    outs = llm.generate(_prompts(), sp)
    model = llm.engine.runner.model
    for p, o in zip(_prompts(), outs):
        toks = list(p)
        for _ in range(6):
            toks.append(int(dense_mla_logits(model, toks)[-1].argmax()))
        assert o.outputs[0].token_ids == toks[len(p):]
