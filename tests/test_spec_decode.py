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


def _spec_llm(method, k=3, **kw):
    sc = {"method": method, "num_speculative_tokens": k}
    sc.update(kw.pop("spec", {}))
    return LLM("tiny-llama", device="cpu", block_size=16, init_dist=False, speculative_config=sc, **kw)


def _logged_drafts(llm, prompts, sp):
    """Generate and return (outputs, {(prompt index, sequence length): drafts})."""
    llm.engine.spec.log = []
    outs = llm.generate(prompts, sp)
    order = {o.request_id: i for i, o in enumerate(outs)}
    return [o.outputs[0].token_ids for o in outs], {(order[r], n): d for r, n, d in llm.engine.spec.log}


@pytest.mark.parametrize("method", ["mtp", "eagle", "eagle3"])
def test_draft_layer_kv_cache_is_consistent_across_batching_and_lossless(method):
    """A draft layer's proposals are a function of the sequence alone: whole-prompt steps and 16-token
    prompt chunks (catch-up passes split differently, other batch composition) give the same drafts at
    the same sequence lengths, and the engine's tokens equal plain decoding."""
    prompts = [np.random.RandomState(11).randint(0, 1024, size=n).tolist() for n in (7, 37, 20)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    plain = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    want = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    a = _spec_llm(method, max_num_seqs=4)
    got_a, drafts_a = _logged_drafts(a, prompts, sp)
    b = _spec_llm(method, max_num_seqs=2, max_num_batched_tokens=16)
    got_b, drafts_b = _logged_drafts(b, prompts, sp)
    assert got_a == want and got_b == want
    common = set(drafts_a) & set(drafts_b)
    assert len(common) >= 6
    for key in common:
        n = min(len(drafts_a[key]), len(drafts_b[key]))
        assert drafts_a[key][:n] == drafts_b[key][:n], key
    st = a.engine.spec.stats
    assert st["proposed"] > 0 and st["catch_up_rows"] >= sum(len(p) for p in prompts)
    assert not a.engine.scheduler.async_mode


def test_mtp_draft_layer_that_mirrors_a_bigram_target_is_accepted_in_full():
    """Target whose layers add nothing (next token = f(last token)) and an MTP module that ignores the
    hidden state and repeats the target's head: every draft is right, so every verification step keeps
    k + 1 tokens; this walks the multi-row acceptance path of the catch-up pass."""
    prompts = [np.random.RandomState(5).randint(0, 1024, size=n).tolist() for n in (9, 18)]
    sp = SamplingParams(temperature=0.0, max_tokens=17, ignore_eos=True)

    def flatten(model_layers):
        for l in model_layers:
            l.self_attn.o.weight.zero_()
            l.mlp.down.weight.zero_()
    plain = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    flatten(plain.engine.runner.model.layers)
    want = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    spec = _spec_llm("mtp", k=3, max_num_seqs=4)
    flatten(spec.engine.runner.model.layers)
    d = spec.engine.spec
    flatten([d.layer])
    H = d.fc.shape[0]
    d.fc = torch.cat([torch.eye(H), torch.zeros(H, H)], 1).to(d.fc.dtype)
    d.out_norm.copy_(spec.engine.runner.model.norm)
    got = [o.outputs[0].token_ids for o in spec.generate(prompts, sp)]
    assert got == want
    rs = spec.engine.runner.stats
    assert rs["spec_drafted"] > 0 and rs["spec_accepted"] == rs["spec_drafted"]


@pytest.mark.parametrize("method", ["mtp", "eagle", "eagle3"])
def test_draft_layer_checkpoints_load(tmp_path, method):
    from safetensors.torch import save_file
    from vllm_torchtpu_b200.config import model_preset
    m = model_preset("tiny-llama")
    H, D, I, V, L = m.hidden_size, m.head_dim, m.intermediate_size, m.vocab_size, m.num_layers
    g = torch.Generator().manual_seed(3)
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.05       # noqa: E731
    attn_in = 2 * H if method == "eagle3" else H
    layer = {"self_attn.q_proj.weight": rnd(m.num_q_heads * D, attn_in),
             "self_attn.k_proj.weight": rnd(m.num_kv_heads * D, attn_in),
             "self_attn.v_proj.weight": rnd(m.num_kv_heads * D, attn_in),
             "self_attn.o_proj.weight": rnd(H, m.num_q_heads * D),
             "mlp.gate_proj.weight": rnd(I, H), "mlp.up_proj.weight": rnd(I, H), "mlp.down_proj.weight": rnd(H, I),
             "post_attention_layernorm.weight": 1 + rnd(H)}
    if method == "mtp":
        pre = f"model.layers.{L}."
        t = {pre + k: v for k, v in layer.items()}
        t.update({pre + "input_layernorm.weight": 1 + rnd(H), pre + "enorm.weight": 1 + rnd(H),
                  pre + "hnorm.weight": 1 + rnd(H), pre + "eh_proj.weight": rnd(H, 2 * H),
                  pre + "shared_head.norm.weight": 1 + rnd(H), pre + "shared_head.head.weight": rnd(V, H),
                  "model.layers.0.input_layernorm.weight": rnd(H)})       # a target tensor: ignored
        fc_name, norm_name = pre + "eh_proj.weight", pre + "shared_head.norm.weight"
    elif method == "eagle":
        t = {"layers.0." + k: v for k, v in layer.items()}
        t.update({"fc.weight": rnd(H, 2 * H), "fc.bias": rnd(H), "embed_tokens.weight": rnd(V, H)})
        fc_name, norm_name = "fc.weight", None
    else:
        t = {"midlayer." + k: v for k, v in layer.items()}
        t.update({"midlayer.input_layernorm.weight": 1 + rnd(H), "midlayer.hidden_norm.weight": 1 + rnd(H),
                  "fc.weight": rnd(H, 3 * H), "norm.weight": 1 + rnd(H), "lm_head.weight": rnd(64, H),
                  "d2t": torch.arange(64) * 3, "t2d": torch.zeros(V, dtype=torch.bool)})
        fc_name, norm_name = "fc.weight", "norm.weight"
    d = tmp_path / method
    d.mkdir()
    save_file({k: v.contiguous() for k, v in t.items()}, str(d / "model.safetensors"))
    llm = _spec_llm(method, max_num_seqs=4, spec={"model": str(d)}, dtype="float32")
    p = llm.engine.spec
    key = next(k for k in t if k.endswith("self_attn.q_proj.weight"))
    stem = key[: -len("self_attn.q_proj.weight")]
    qkv = torch.cat([t[stem + f"self_attn.{x}_proj.weight"] for x in "qkv"], 0)
    torch.testing.assert_close(p.layer.self_attn.qkv.weight, qkv)
    torch.testing.assert_close(p.layer.mlp.down.weight, t[stem + "mlp.down_proj.weight"])
    torch.testing.assert_close(p.layer.post_ln, t[stem + "post_attention_layernorm.weight"])
    torch.testing.assert_close(p.fc, t[fc_name])
    if norm_name:
        torch.testing.assert_close(p.out_norm, t[norm_name])
    if method == "eagle":
        torch.testing.assert_close(p.fc_bias, t["fc.bias"])
        assert p.embed is not None and p.head is None
    if method == "eagle3":
        torch.testing.assert_close(p.hidden_norm, t["midlayer.hidden_norm.weight"])
        assert p.head.shape == (64, H) and p.d2t[5] == 15
    prompts = [np.random.RandomState(2).randint(0, 1024, size=n).tolist() for n in (6, 19)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    plain = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False, dtype="float32")
    assert [o.outputs[0].token_ids for o in llm.generate(prompts, sp)] == \
        [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    if method == "eagle3":          # drafts come from the reduced vocabulary, mapped through d2t
        llm.engine.spec.log = []
        llm.generate(prompts, sp)
        assert all(tok % 4 == 0 and tok < 64 * 4 for _, _, dr in llm.engine.spec.log for tok in dr)


@pytest.mark.parametrize("preset", ["tiny-mla", "tiny-moe"])
def test_mtp_module_takes_the_layer_class_of_its_target(preset):
    """The MTP module of an MLA + MoE target is an MLA + MoE layer with a latent cache of its own."""
    prompts = [np.random.RandomState(4).randint(0, 1024, size=n).tolist() for n in (9, 30)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    plain = LLM(preset, device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    want = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    spec = LLM(preset, device="cpu", max_num_seqs=4, block_size=16, init_dist=False,
               speculative_config={"method": "mtp", "num_speculative_tokens": 2})
    assert [o.outputs[0].token_ids for o in spec.generate(prompts, sp)] == want
    d = spec.engine.spec
    assert type(d.layer) is type(spec.engine.runner.model.layers[-1]) and hasattr(d.layer.mlp, "experts")
    assert d.kv_cache.shape == spec.engine.runner.kv_caches[-1].shape and d.stats["proposed"] > 0


@pytest.mark.parametrize("preset", ["tiny-gdn", "tiny-kda"])
def test_mtp_on_linear_attention_hybrids(preset):
    """The MTP module of a hybrid is a full-attention layer; its drafts are verified in k + 1 rows and the
    recurrent layers' state is rolled back for the rejected ones."""
    prompts = [np.random.RandomState(4).randint(0, 1024, size=n).tolist() for n in (9, 30)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    plain = LLM(preset, device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    want = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    spec = LLM(preset, device="cpu", max_num_seqs=4, block_size=16, init_dist=False,
               speculative_config={"method": "mtp", "num_speculative_tokens": 2})
    assert [o.outputs[0].token_ids for o in spec.generate(prompts, sp)] == want
    d = spec.engine.spec
    assert hasattr(d.layer.self_attn, "qkv") and d.kv_cache.dim() == 5
    assert spec.engine.runner.stats.get("state_rollbacks", 0) > 0 and d.stats["proposed"] > 0


@pytest.mark.parametrize("method,layers", [("dflash", 1), ("dflash", 2), ("dspark", 1)])
def test_block_drafter_is_lossless_and_independent_of_batching(method, layers):
    """Parallel block drafting: context keys / values from the target's hidden states, all k drafts from one
    non-causal block pass.  The engine's tokens equal plain decoding, and the drafts are a function of the
    sequence alone (whole prompts against 16-token chunks with another batch composition)."""
    prompts = [np.random.RandomState(12).randint(0, 1000, size=n).tolist() for n in (7, 37, 20)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    plain = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    want = [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    spec = {"num_hidden_layers": layers}
    a = _spec_llm(method, max_num_seqs=4, spec=spec)
    got_a, drafts_a = _logged_drafts(a, prompts, sp)
    b = _spec_llm(method, max_num_seqs=2, max_num_batched_tokens=16, spec=spec)
    got_b, drafts_b = _logged_drafts(b, prompts, sp)
    assert got_a == want and got_b == want
    common = set(drafts_a) & set(drafts_b)
    assert len(common) >= 6
    for key in common:
        n = min(len(drafts_a[key]), len(drafts_b[key]))
        assert drafts_a[key][:n] == drafts_b[key][:n], key
    d = a.engine.spec
    assert len(d.layers) == layers and len(d.kv_caches) == layers
    assert d.stats["passes"] > 0 and d.stats["context_rows"] >= sum(len(p) for p in prompts)
    assert d.stats["proposed"] <= d.stats["passes"] * 3 * len(prompts)      # one pass drafts all k tokens of a step
    assert a.engine.scheduler.lookahead_extra == 2 and not a.engine.scheduler.async_mode


def test_block_drafter_rows_see_the_whole_block_and_checkpoints_load(tmp_path):
    """A mask row's output depends on LATER block rows too (the block is not causal), and a checkpoint in the
    drafter's naming loads (layers through the package's loader, fc / norm / head / d2t / Markov head)."""
    from safetensors.torch import save_file
    from vllm_torchtpu_b200.config import model_preset
    m = model_preset("tiny-llama")
    H, D, I, V, L = m.hidden_size, m.head_dim, m.intermediate_size, m.vocab_size, m.num_layers
    g = torch.Generator().manual_seed(3)
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.05       # noqa: E731
    t = {"fc.weight": rnd(H, 3 * H), "norm.weight": 1 + rnd(H), "lm_head.weight": rnd(64, H),
         "d2t": torch.arange(64) * 3, "markov_head.embed.weight": rnd(V, 8), "markov_head.proj.weight": rnd(64, 8)}
    for l in range(2):
        pre = f"layers.{l}."
        t.update({pre + "self_attn.q_proj.weight": rnd(m.num_q_heads * D, H),
                  pre + "self_attn.k_proj.weight": rnd(m.num_kv_heads * D, H),
                  pre + "self_attn.v_proj.weight": rnd(m.num_kv_heads * D, H),
                  pre + "self_attn.o_proj.weight": rnd(H, m.num_q_heads * D),
                  pre + "mlp.gate_proj.weight": rnd(I, H), pre + "mlp.up_proj.weight": rnd(I, H),
                  pre + "mlp.down_proj.weight": rnd(H, I), pre + "input_layernorm.weight": 1 + rnd(H),
                  pre + "post_attention_layernorm.weight": 1 + rnd(H)})
    d = tmp_path / "dspark"
    d.mkdir()
    save_file({k: v.contiguous() for k, v in t.items()}, str(d / "model.safetensors"))
    llm = _spec_llm("dspark", max_num_seqs=4, spec={"model": str(d), "num_hidden_layers": 2, "mask_token_id": 5},
                    dtype="float32")
    p = llm.engine.spec
    torch.testing.assert_close(p.fc, t["fc.weight"])
    torch.testing.assert_close(p.layers[1].mlp.down.weight, t["layers.1.mlp.down_proj.weight"])
    torch.testing.assert_close(p.layers[0].input_ln, t["layers.0.input_layernorm.weight"])
    assert p.head.shape == (64, H) and p.markov_embed.shape == (V, 8) and p.mask_token_id == 5
    prompts = [np.random.RandomState(2).randint(0, 1000, size=n).tolist() for n in (6, 19)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    plain = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False, dtype="float32")
    llm.engine.spec.log = []
    assert [o.outputs[0].token_ids for o in llm.generate(prompts, sp)] == \
        [o.outputs[0].token_ids for o in plain.generate(prompts, sp)]
    assert all(tok % 4 == 0 and tok < 64 * 4 for _, _, dr in llm.engine.spec.log for tok in dr)
    # non-causal block: the first mask row changes when a later row's token changes
    q = _spec_llm("dflash", max_num_seqs=4)
    q.generate([prompts[0]], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    dq = q.engine.spec
    bslots, start = np.array([0]), np.array([3])
    meta = dq._block_meta(bslots, start, 3)

    def first_mask_state(last_token):
        ids = torch.tensor([7, dq.mask_token_id, last_token], dtype=torch.int32)
        hidden, residual = ops_embedding(ids, q.engine.runner.model.embed), None
        for lay, cache in zip(dq.layers, dq.kv_caches):
            hidden, residual = lay.forward(hidden, residual, cache, meta)
        return (hidden + residual)[1].clone()
    from vllm_torchtpu_b200.ops import embedding as ops_embedding
    assert not torch.allclose(first_mask_state(11), first_mask_state(12))
