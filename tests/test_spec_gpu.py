"""Speculative-decoding kernels against the host statement of the same rules, and an engine run whose
verification steps are judged on the device."""
import pytest
import torch

from vllm_torchtpu_b200.sample.rejection_sampler import greedy_accept, rejection_sample

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_spec_accept_kernel_matches_host_rule():
    from vllm_torchtpu_b200.ops import cuda
    g = torch.Generator().manual_seed(0)
    spec_k = [3, 0, 2, 4, 1]
    kmax = max(spec_k)
    R = len(spec_k)
    # each request contributes (some prompt rows +) k + 1 rows whose last k inputs are the drafts
    ids, qsl, target, want = [], [0], [], []
    for r, k in enumerate(spec_k):
        extra = r % 2                                     # rows in front of the verified ones
        drafts = torch.randint(0, 5, (k,), generator=g).tolist()
        tgt = torch.randint(0, 5, (k + 1,), generator=g).tolist()
        if r == 3:
            tgt[:k] = drafts                              # everything accepted: bonus token kept
        ids += [7] * extra + [9] + drafts
        qsl.append(len(ids))
        target += tgt
        want.append(greedy_accept(drafts, tgt))
    out, cnt = cuda.spec_accept(torch.tensor(target, dtype=torch.int32, device=DEV),
                                torch.tensor(ids, dtype=torch.int32, device=DEV),
                                torch.tensor(qsl, dtype=torch.int32, device=DEV),
                                torch.tensor(spec_k, dtype=torch.int32, device=DEV), R, kmax)
    torch.cuda.synchronize()
    for r in range(R):
        n = int(cnt[r])
        assert out[r, :n].tolist() == want[r], (r, out[r].tolist(), want[r])
        assert (out[r, n:] == -1).all()


@pytest.mark.parametrize("with_q", [False, True])
def test_rejection_sample_kernel_matches_host_rule(with_q):
    from vllm_torchtpu_b200.ops import cuda
    g = torch.Generator().manual_seed(1)
    V, spec_k = 503, [3, 2, 0, 3, 1, 3]
    kmax, R = max(spec_k), len(spec_k)
    temps = torch.tensor([1.0, 0.7, 1.0, 0.0, 1.3, 1.0])
    L = sum(k + 1 for k in spec_k)
    logits = torch.randn(L, V, generator=g) * 2
    q = torch.softmax(torch.randn(R, kmax, V, generator=g) * 2, -1) if with_q else None
    drafts = torch.zeros(R, kmax, dtype=torch.int32)
    off = 0
    for r, k in enumerate(spec_k):
        for i in range(k):
            p = torch.softmax(logits[off + i] / max(float(temps[r]), 1e-6), -1)
            # likely tokens so that both acceptance and rejection occur
            drafts[r, i] = int(torch.multinomial(p if not with_q else q[r, i], 1, generator=g))
        if r == 3:
            drafts[r, 0] = int(logits[off].argmax())     # greedy request: first draft accepted
        off += k + 1
    u = torch.rand(R, kmax, generator=g)
    u2 = torch.rand(R, kmax + 1, generator=g)
    out, cnt = cuda.rejection_sample(logits.to(DEV), drafts.to(DEV), q.to(DEV) if with_q else None,
                                     torch.tensor(spec_k, dtype=torch.int32, device=DEV), temps.to(DEV),
                                     u.to(DEV), u2.to(DEV))
    torch.cuda.synchronize()
    off = 0
    accepted_any = rejected_any = False
    for r, k in enumerate(spec_k):
        n = int(cnt[r])
        got = out[r, :n].tolist()
        if float(temps[r]) == 0.0:
            want = greedy_accept(drafts[r, :k].tolist(), logits[off:off + k + 1].argmax(-1).tolist())
        else:
            p = torch.softmax(logits[off:off + k + 1].double() / float(temps[r]), -1).float()
            want = rejection_sample(drafts[r, :k], p, q[r, :k] if with_q else None, u[r, :k], u2[r])
        assert len(got) == len(want), (r, got, want)
        assert got[:-1] == want[:-1], (r, got, want)
        if got[-1] != want[-1]:
            # the inverse CDF may land on a neighbour when the draw sits on a boundary: the two tokens must
            # then both carry mass around the drawn quantile
            assert abs(got[-1] - want[-1]) <= 3, (r, got, want)
        accepted_any |= n > 1
        rejected_any |= n <= k
        off += k + 1
    assert accepted_any and rejected_any


def test_engine_ngram_spec_decode_with_device_acceptance_equals_plain_decode():
    import numpy as np

    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.config import ModelConfig
    from vllm_torchtpu_b200.engine.llm import LLM
    cfg = ModelConfig(name="t", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                      intermediate_size=1024, vocab_size=2048, max_model_len=512, dtype=torch.bfloat16)
    rng = np.random.RandomState(3)
    prompts = [(rng.randint(0, 2048, size=6).tolist() * 4)[:n] for n in (20, 13, 24)]   # repeated n-grams
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    kw = dict(device="cuda", max_num_seqs=8, max_num_batched_tokens=256, num_gpu_blocks_override=512,
              init_dist=False)
    plain = [o.outputs[0].token_ids for o in LLM(cfg, **kw).generate(prompts, sp)]
    spec_llm = LLM(cfg, speculative_config={"method": "ngram", "num_speculative_tokens": 3,
                                            "prompt_lookup_min": 2}, **kw)
    spec = [o.outputs[0].token_ids for o in spec_llm.generate(prompts, sp)]
    assert spec_llm.engine.runner.stats.get("spec_drafted", 0) > 0
    assert spec == plain


def _bf16_cfg():
    from vllm_torchtpu_b200.config import ModelConfig
    return ModelConfig(name="t", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                       intermediate_size=1024, vocab_size=2048, max_model_len=512, dtype=torch.bfloat16)


@pytest.mark.parametrize("method", ["mtp", "eagle", "eagle3"])
def test_draft_layer_engine_run_is_lossless_on_the_device(method):
    """A draft layer with attention (its own KV tensor behind the target's block tables) runs its catch-up
    and look-ahead passes on the package's kernels; the engine's tokens equal plain decoding."""
    import numpy as np
    from vllm_torchtpu_b200 import LLM, SamplingParams
    prompts = [np.random.RandomState(4).randint(0, 2048, size=n).tolist() for n in (9, 40, 23)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    kw = dict(device=DEV, max_num_seqs=4, num_gpu_blocks_override=256, init_dist=False)
    plain = LLM(_bf16_cfg(), max_num_batched_tokens=256, **kw)
    want = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    del plain
    spec = LLM(_bf16_cfg(), max_num_batched_tokens=32,
               speculative_config={"method": method, "num_speculative_tokens": 3}, **kw)
    got = [o.outputs[0].token_ids for o in spec.generate(prompts, sp)]
    assert got == want
    st = spec.engine.spec.stats
    assert st["proposed"] > 0 and st["catch_up_rows"] >= sum(len(p) for p in prompts)


def test_mtp_layer_mirroring_a_bigram_target_is_accepted_on_the_device():
    import numpy as np
    from vllm_torchtpu_b200 import LLM, SamplingParams
    prompts = [np.random.RandomState(5).randint(0, 2048, size=n).tolist() for n in (9, 18)]
    sp = SamplingParams(temperature=0.0, max_tokens=17, ignore_eos=True)
    spec = LLM(_bf16_cfg(), device=DEV, max_num_seqs=4, num_gpu_blocks_override=256, init_dist=False,
               speculative_config={"method": "mtp", "num_speculative_tokens": 3})
    d = spec.engine.spec
    for l in list(spec.engine.runner.model.layers) + [d.layer]:
        l.self_attn.o.weight.zero_()
        l.mlp.down.weight.zero_()
    H = d.fc.shape[0]
    d.fc = torch.cat([torch.eye(H), torch.zeros(H, H)], 1).to(device=d.fc.device, dtype=d.fc.dtype)
    d.out_norm.copy_(spec.engine.runner.model.norm)
    outs = spec.generate(prompts, sp)
    assert all(len(o.outputs[0].token_ids) == 17 for o in outs)
    rs = spec.engine.runner.stats
    assert rs["spec_drafted"] > 0 and rs["spec_accepted"] >= 0.8 * rs["spec_drafted"]


@pytest.mark.parametrize("method,layers", [("dflash", 2), ("dspark", 1)])
def test_block_drafter_engine_run_is_lossless_on_the_device(method, layers):
    """Parallel block drafting on the package's kernels: context K/V written by the RoPE + cache kernel, the block
    rows run as one-row requests over context + block (non-causal inside the block)."""
    import numpy as np
    from vllm_torchtpu_b200 import LLM, SamplingParams
    prompts = [np.random.RandomState(4).randint(0, 2000, size=n).tolist() for n in (9, 40, 23)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    kw = dict(device=DEV, max_num_seqs=4, num_gpu_blocks_override=256, init_dist=False)
    plain = LLM(_bf16_cfg(), max_num_batched_tokens=256, **kw)
    want = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    del plain
    spec = LLM(_bf16_cfg(), max_num_batched_tokens=32,
               speculative_config={"method": method, "num_speculative_tokens": 3, "num_hidden_layers": layers}, **kw)
    got = [o.outputs[0].token_ids for o in spec.generate(prompts, sp)]
    assert got == want
    st = spec.engine.spec.stats
    assert st["proposed"] > 0 and st["context_rows"] >= sum(len(p) for p in prompts)
    from vllm_torchtpu_b200.ops import cuda
    assert cuda.check_status() == 0
