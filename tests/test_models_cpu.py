"""Model families on the CPU path vs dense references."""
import numpy as np
import pytest
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


def _hf_cfg(arch, **kw):
    d = {"architectures": [arch], "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4,
         "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 512, "vocab_size": 1024,
         "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 256, "torch_dtype": "float32"}
    d.update(kw)
    return d


def test_safetensors_roundtrip_dense_and_moe(tmp_path):
    from vllm_torchtpu_b200.models.loader import save_hf_checkpoint
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    for preset, hf in (("tiny-llama", _hf_cfg("LlamaForCausalLM")),
                       ("tiny-moe", _hf_cfg("Qwen3MoeForCausalLM", num_experts=8, num_experts_per_tok=2,
                                            moe_intermediate_size=128, norm_topk_prob=True))):
        src = LLM(preset, device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
        want = [o.outputs[0].token_ids for o in src.generate(_prompts(), sp)]
        d = tmp_path / preset
        save_hf_checkpoint(src.engine.runner.model, str(d), hf)
        dst = LLM(str(d), device="cpu", max_num_seqs=4, block_size=16, init_dist=False, dtype="float32")
        got = [o.outputs[0].token_ids for o in dst.generate(_prompts(), sp)]
        assert got == want, preset
        if preset == "tiny-llama":
            # the same checkpoint named by a URI: configuration pulled to a host-local directory, weights read
            # in place
            import os
            os.environ["HOME"], home = str(tmp_path / "home"), os.environ.get("HOME")
            try:
                uri = LLM(f"file://{d}", device="cpu", max_num_seqs=4, block_size=16, init_dist=False, dtype="float32")
            finally:
                if home is not None:
                    os.environ["HOME"] = home
            assert [o.outputs[0].token_ids for o in uri.generate(_prompts(), sp)] == want
            assert (tmp_path / "home" / ".cache" / "vllm_torchtpu_b200" / "model_source").is_dir()


def _rewrite_checkpoint(d, rename):
    """Rewrite the tensors of a saved checkpoint through ``rename(dict) -> dict``."""
    from safetensors.torch import load_file, save_file
    f = str(d / "model.safetensors")
    save_file({k: v.contiguous() for k, v in rename(load_file(f)).items()}, f)


def test_mixtral_phi3_and_qwen2_moe_checkpoint_layouts(tmp_path):
    """Mixtral (block_sparse_moe / w1 w3 w2 names), Phi-3 (fused qkv_proj and gate_up_proj tensors) and
    Qwen2-MoE (a shared expert behind a sigmoid gate) load into the Llama / Qwen-MoE models and reproduce
    the tokens of the model they were written from."""
    import re
    from vllm_torchtpu_b200.models.loader import save_hf_checkpoint
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)

    def run(path_or_preset, **kw):
        llm = LLM(path_or_preset, device="cpu", max_num_seqs=4, block_size=16, init_dist=False, **kw)
        return llm, [o.outputs[0].token_ids for o in llm.generate(_prompts(), sp)]

    from vllm_torchtpu_b200.config import ModelConfig

    def donor(hf):
        mc = ModelConfig.from_hf_dict(hf)
        mc.dtype, mc.max_model_len = torch.float32, 256
        return run(mc)

    # Mixtral
    hf = _hf_cfg("MixtralForCausalLM", num_local_experts=8, num_experts_per_tok=2, intermediate_size=128)
    src, want = donor(hf)
    assert src.engine.runner.model.layers[0].self_attn.q_norm_w is None
    d = tmp_path / "mixtral"
    save_hf_checkpoint(src.engine.runner.model, str(d), hf)
    back = {"gate_proj": "w1", "up_proj": "w3", "down_proj": "w2"}

    def to_mixtral(t):
        out = {}
        for k, v in t.items():
            k = k.replace(".mlp.", ".block_sparse_moe.")
            k = re.sub(r"(experts\.\d+\.)(gate_proj|up_proj|down_proj)", lambda m: m.group(1) + back[m.group(2)], k)
            out[k] = v
        return out
    _rewrite_checkpoint(d, to_mixtral)
    _, got = run(str(d), dtype="float32")
    assert got == want

    # Phi-3
    src, want = run("tiny-llama")
    d = tmp_path / "phi3"
    save_hf_checkpoint(src.engine.runner.model, str(d), _hf_cfg("Phi3ForCausalLM"))

    def to_phi3(t):
        out = {k: v for k, v in t.items() if not re.search(r"\.(q|k|v|gate|up)_proj\.", k)}
        for i in range(2):
            a, m = f"model.layers.{i}.self_attn.", f"model.layers.{i}.mlp."
            out[a + "qkv_proj.weight"] = torch.cat([t[a + f"{p}_proj.weight"] for p in "qkv"], 0)
            out[m + "gate_up_proj.weight"] = torch.cat([t[m + "gate_proj.weight"], t[m + "up_proj.weight"]], 0)
        return out
    _rewrite_checkpoint(d, to_phi3)
    _, got = run(str(d), dtype="float32")
    assert got == want

    # Qwen2-MoE: the gate is read from the checkpoint and changes the output
    hf = _hf_cfg("Qwen2MoeForCausalLM", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                 shared_expert_intermediate_size=192, norm_topk_prob=False)
    mc = ModelConfig.from_hf_dict(hf)
    assert mc.shared_expert_gate and mc.shared_expert_intermediate_size == 192 and mc.attention_bias
    src, want = donor(hf)
    blk = src.engine.runner.model.layers[0].mlp
    assert blk.shared_gate is not None and blk.shared.down.weight.shape[1] == 192
    x = torch.randn(3, 256)
    full = blk.forward(x)
    gate = torch.sigmoid(x @ blk.shared_gate)[:, None]
    torch.testing.assert_close(full, blk.experts.forward(x) + gate * blk.shared.forward(x), rtol=1e-5, atol=1e-5)
    d = tmp_path / "qwen2moe"
    save_hf_checkpoint(src.engine.runner.model, str(d), hf)
    dst, got = run(str(d), dtype="float32")
    assert got == want
    torch.testing.assert_close(dst.engine.runner.model.layers[1].mlp.shared_gate,
                               src.engine.runner.model.layers[1].mlp.shared_gate)


def test_hf_config_mapping():
    from vllm_torchtpu_b200.config import ModelConfig
    mc = ModelConfig.from_hf_dict({"architectures": ["DeepseekV3ForCausalLM"], "num_hidden_layers": 61,
                                   "hidden_size": 7168, "num_attention_heads": 128, "vocab_size": 129280,
                                   "n_routed_experts": 256, "num_experts_per_tok": 8, "moe_intermediate_size": 2048,
                                   "n_shared_experts": 1, "first_k_dense_replace": 3, "scoring_func": "sigmoid",
                                   "topk_method": "noaux_tc", "n_group": 8, "topk_group": 4, "kv_lora_rank": 512,
                                   "q_lora_rank": 1536, "qk_nope_head_dim": 128, "qk_rope_head_dim": 64,
                                   "v_head_dim": 128, "intermediate_size": 18432, "routed_scaling_factor": 2.5,
                                   "quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128]}})
    assert mc.architecture == "deepseek_v3" and mc.is_mla and mc.moe_score_bias and mc.quantization == "fp8_block"
    assert mc.layer_is_moe(3) and not mc.layer_is_moe(2)


def test_gdn_recurrence_is_chunk_invariant_and_engine_runs_hybrid():
    from vllm_torchtpu_b200.ops import gdn_reference as g
    torch.manual_seed(0)
    T, Hk, Hv, dk, dv = 23, 2, 4, 8, 8
    q, k, v = torch.randn(T, Hk, dk), torch.randn(T, Hk, dk), torch.randn(T, Hv, dv)
    gate, beta = -torch.rand(T, Hv), torch.rand(T, Hv)
    s1 = torch.zeros(Hv, dk, dv)
    full = g.gated_delta_rule(q, k, v, gate, beta, s1)
    s2 = torch.zeros(Hv, dk, dv)
    parts = [g.gated_delta_rule(q[a:b], k[a:b], v[a:b], gate[a:b], beta[a:b], s2) for a, b in ((0, 9), (9, 10), (10, 23))]
    torch.testing.assert_close(torch.cat(parts), full, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(s1, s2, rtol=1e-5, atol=1e-5)
    # conv window carried across chunks
    x, w = torch.randn(T, 6), torch.randn(6, 4)
    c1, c2 = torch.zeros(6, 3), torch.zeros(6, 3)
    a = g.causal_conv1d_update(x, c1, w)
    b = torch.cat([g.causal_conv1d_update(x[:5], c2, w), g.causal_conv1d_update(x[5:], c2, w)])
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-5)
    # hybrid engine: chunked prefill + batching must not change greedy tokens
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    one = LLM("tiny-gdn", device="cpu", max_num_seqs=4, max_num_batched_tokens=256, block_size=16, init_dist=False)
    want = [one.generate([p], sp)[0].outputs[0].token_ids for p in _prompts()]
    many = LLM("tiny-gdn", device="cpu", max_num_seqs=4, max_num_batched_tokens=16, block_size=16, init_dist=False)
    got = [o.outputs[0].token_ids for o in many.generate(_prompts(), sp)]
    assert got == want


def test_kda_recurrence_reduces_to_gdn_and_is_chunk_invariant():
    """Kimi Delta Attention with the same log-decay on every key channel is the gated delta rule, and
    running a sequence in two pieces with the carried state equals running it whole."""
    from vllm_torchtpu_b200.ops import gdn_reference as g
    torch.manual_seed(0)
    T, Hk, Hv, dk, dv = 12, 2, 4, 16, 8
    q, k = torch.randn(T, Hk, dk), torch.randn(T, Hk, dk)
    v = torch.randn(T, Hv, dv)
    gl = -torch.rand(T, Hv)
    beta = torch.rand(T, Hv)
    s1, s2 = torch.zeros(Hv, dk, dv), torch.zeros(Hv, dk, dv)
    o_gdn = g.gated_delta_rule(q, k, v, gl, beta, s1)
    o_kda = g.kda_rule(q, k, v, gl[:, :, None].expand(T, Hv, dk).contiguous(), beta, s2)
    torch.testing.assert_close(o_kda, o_gdn, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(s1, s2, rtol=1e-4, atol=1e-4)
    gk = -torch.rand(T, Hv, dk)
    whole = torch.zeros(Hv, dk, dv)
    o_whole = g.kda_rule(q, k, v, gk, beta, whole)
    part = torch.zeros(Hv, dk, dv)
    o_a = g.kda_rule(q[:5], k[:5], v[:5], gk[:5], beta[:5], part)
    o_b = g.kda_rule(q[5:], k[5:], v[5:], gk[5:], beta[5:], part)
    torch.testing.assert_close(torch.cat([o_a, o_b]), o_whole, rtol=1e-5, atol=1e-5)
    # bounded gate form stays inside [lower_bound, 0]
    gb = g.kda_gate(torch.randn(T, Hv, dk), torch.zeros(Hv), torch.zeros(Hv, dk), lower_bound=-5.0)
    assert float(gb.min()) >= -5.0 and float(gb.max()) <= 0.0


@pytest.mark.parametrize("preset", ["tiny-kda", "tiny-kda-mla"])
def test_kimi_linear_hybrid_engine_is_chunk_and_batch_invariant(preset):
    """KDA layers (conv window + per-channel-decay state in slot pools) next to full attention - grouped-query
    attention, or latent attention without rotary embeddings as in the published layout: chunked prefill and
    batching leave the greedy tokens unchanged."""
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    one = LLM(preset, device="cpu", max_num_seqs=4, max_num_batched_tokens=256, block_size=16, init_dist=False)
    want = [one.generate([p], sp)[0].outputs[0].token_ids for p in _prompts()]
    many = LLM(preset, device="cpu", max_num_seqs=4, max_num_batched_tokens=16, block_size=16, init_dist=False)
    got = [o.outputs[0].token_ids for o in many.generate(_prompts(), sp)]
    assert got == want


def test_kimi_linear_latent_attention_layers_and_config_mapping():
    """The Kimi-Linear configuration with latent attention maps onto the hybrid model: KDA layers keep state pools,
    the full-attention layers get a latent cache, and without rotary embeddings the output does not depend on
    where the rotary base sits."""
    from vllm_torchtpu_b200.config import ModelConfig, model_preset
    hf = {"architectures": ["KimiLinearForCausalLM"], "num_hidden_layers": 4, "hidden_size": 256, "vocab_size": 1024,
          "num_attention_heads": 4, "num_key_value_heads": 4, "head_dim": 72, "intermediate_size": 512,
          "kv_lora_rank": 64, "qk_nope_head_dim": 32, "qk_rope_head_dim": 16, "v_head_dim": 32, "mla_use_nope": True,
          "linear_attn_config": {"full_attn_layers": [4], "kda_layers": [1, 2, 3], "num_heads": 4, "head_dim": 32,
                                 "short_conv_kernel_size": 4}, "torch_dtype": "float32"}
    mc = ModelConfig.from_hf_dict(hf)
    assert mc.architecture == "kimi_linear" and mc.is_mla and mc.mla_use_nope and mc.kv_lora_rank == 64
    llm = LLM("tiny-kda-mla", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    m = llm.engine.runner.model
    kinds = [type(l.self_attn).__name__ for l in m.layers]
    assert kinds == ["KimiDeltaAttention"] * 3 + ["MLAAttention"]
    caches = llm.engine.runner.kv_caches
    assert isinstance(caches[0], tuple) and caches[3].shape[1:] == (16, 64 + 16)
    assert m.kv_bytes_per_block(16, torch.float32) == 16 * 80 * 4
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    base = llm.generate(_prompts(), sp)
    cfg2 = model_preset("tiny-kda-mla")
    cfg2.rope_theta = 123.0                                   # no rotary embeddings: the base must not matter
    other = LLM(cfg2, device="cpu", max_num_seqs=4, block_size=16, init_dist=False).generate(_prompts(), sp)
    assert [o.outputs[0].token_ids for o in other] == [o.outputs[0].token_ids for o in base]
    assert float(m.layers[3].self_attn.inv_freq.abs().max()) == 0.0
    cfg3 = model_preset("tiny-kda-mla")
    cfg3.mla_use_nope = False
    roped = LLM(cfg3, device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    assert float(roped.engine.runner.model.layers[3].self_attn.inv_freq.abs().max()) == 1.0


@pytest.mark.parametrize("preset", ["tiny-gdn", "tiny-kda", "tiny-kda-mla"])
def test_speculative_decoding_on_hybrids_rolls_recurrent_state_back(preset):
    """Verification steps fold k + 1 rows into the recurrent state; rejected drafts are undone from a snapshot
    plus a replay of the accepted rows, so the tokens equal plain decoding.  The drafter of this test knows the
    right continuation and spoils its second draft on every other call: full and partial acceptance both occur."""
    rng = np.random.RandomState(3)
    prompts = [rng.randint(0, 1024, size=n).tolist() for n in (22, 13, 27)]
    sp = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    kw = dict(device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    want = [o.outputs[0].token_ids for o in LLM(preset, **kw).generate(prompts, sp)]
    spec = LLM(preset, speculative_config={"method": "ngram", "num_speculative_tokens": 3}, **kw)

    def propose(out, sampled):
        drafts = {}
        for s in out.scheduled:
            r = s.request
            if not sampled.get(r.request_id) or r.status.finished:
                continue
            i = prompts.index(list(r.prompt_token_ids))
            n = len(r.output_token_ids) + len(sampled[r.request_id])
            d = list(want[i][n:min(n + 3, sp.max_tokens - 1)])
            if n % 2 and len(d) > 1:
                d[1] = (d[1] + 1) % 1024
            if d:
                drafts[r.request_id] = d
        return drafts
    spec.engine.spec.propose = propose
    got = [o.outputs[0].token_ids for o in spec.generate(prompts, sp)]
    st = spec.engine.runner.stats
    assert st.get("spec_drafted", 0) > 0 and 0 < st.get("spec_accepted", 0) < st["spec_drafted"]
    assert st.get("state_rollbacks", 0) > 0
    assert got == want
    assert not spec.engine.scheduler.async_mode


def test_state_rollback_equals_running_only_the_accepted_rows():
    """Layer-level statement: after a step of k + 1 rows per request, rollback(accepted) leaves the pools as
    if only the accepted rows had run."""
    from vllm_torchtpu_b200.config import model_preset
    from vllm_torchtpu_b200.models.qwen3_next import GatedDeltaNet
    from vllm_torchtpu_b200.runner.attn_metadata import AttentionMetadata
    from vllm_torchtpu_b200.runner.spec_boundary_state import StateRollback
    cfg = model_preset("tiny-gdn")
    layer = GatedDeltaNet("l", cfg, "cpu", None)
    layer.init_dummy(0.05, 0)
    torch.manual_seed(0)

    def pools():
        cs, rs = layer.state_shapes(4)
        g = torch.Generator().manual_seed(1)
        return torch.randn(cs, generator=g) * 0.1, torch.randn(rs, generator=g) * 0.1

    def meta(qsl, seq, slots, rb=None):
        t = lambda x: torch.tensor(x, dtype=torch.int32)       # noqa: E731
        return AttentionMetadata(positions=t([0] * qsl[-1]), slot_mapping=t([-1] * qsl[-1]),
                                 block_tables=t([[0]] * len(seq)), seq_lens=t(seq), query_start_loc=t(qsl),
                                 num_reqs=len(seq), num_tokens=qsl[-1], state_slots=t(slots), state_rollback=rb)
    # three requests: a decode row (no drafts), and two verifying requests with k = 3 and k = 2
    x = torch.randn(1 + 4 + 3, cfg.hidden_size) * 0.5
    qsl, pos0, slots = [0, 1, 5, 8], [9, 20, 14], [2, 0, 3]
    seq = [pos0[i] + qsl[i + 1] - qsl[i] for i in range(3)]
    cache = pools()
    rb = StateRollback([1, 2], [0, 3], [1, 5], [4, 3], [20, 14], "cpu")
    layer.forward(x, cache, meta(qsl, seq, slots, rb))
    assert rb.rollback([2, 3]) == 1                   # request 1 keeps 2 of 4 rows, request 2 keeps all 3
    want = pools()
    rows = [0, 1, 2, 5, 6, 7]
    layer.forward(x[rows], want, meta([0, 1, 3, 6], [10, 22, 17], slots))
    for got_pool, want_pool in zip(cache, want):
        torch.testing.assert_close(got_pool, want_pool, rtol=1e-5, atol=1e-6)


def test_checkpoint_features_without_kernels_are_refused():
    from vllm_torchtpu_b200.config import ModelConfig
    base = _hf_cfg("Qwen3NextForCausalLM", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128)
    ModelConfig.from_hf_dict(base)
    for extra, word in (({"partial_rotary_factor": 0.25}, "partial_rotary"), ({"attn_output_gate": True}, "output_gate"),
                        ({"head_dim": 256}, "head_dim")):
        with pytest.raises(ValueError, match=word):
            ModelConfig.from_hf_dict({**base, **extra})


def _gpt_oss_hf_cfg(**kw):
    d = {"architectures": ["GptOssForCausalLM"], "num_hidden_layers": 4, "hidden_size": 192, "num_attention_heads": 4,
         "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 128, "vocab_size": 1024, "rms_norm_eps": 1e-5,
         "rope_theta": 150000.0, "max_position_embeddings": 256, "torch_dtype": "float32", "num_local_experts": 8,
         "num_experts_per_tok": 2, "sliding_window": 8, "swiglu_limit": 7.0, "attention_bias": True,
         "layer_types": ["sliding_attention", "full_attention"] * 2,
         "rope_scaling": {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64,
                          "beta_fast": 32.0, "beta_slow": 1.0, "truncate": False}}
    d.update(kw)
    return d


def _gpt_oss_tensors(model, packed: bool):
    """The model's parameters under the published GPT-OSS names and layouts (expert stacks input-major with gate
    and up interleaved; ``packed``: experts as mxfp4 blocks + scales)."""
    from vllm_torchtpu_b200.quantization.fp4 import quantize_mxfp4
    cfg = model.cfg
    D, H = cfg.head_dim, cfg.hidden_size
    out = {"model.embed_tokens.weight": model.embed, "model.norm.weight": model.norm, "lm_head.weight": model.lm_head}

    def interleave(gate, up):                       # rows: gate_0, up_0, gate_1, up_1, ...
        return torch.stack([gate, up], 1).flatten(0, 1)
    for i, l in enumerate(model.layers):
        pre = f"model.layers.{i}."
        a = l.self_attn
        sizes = [cfg.num_q_heads * D, cfg.num_kv_heads * D, cfg.num_kv_heads * D]
        for nme, w, b in zip("qkv", a.qkv.weight.split(sizes, 0), a.qkv.bias.split(sizes, 0)):
            out[pre + f"self_attn.{nme}_proj.weight"], out[pre + f"self_attn.{nme}_proj.bias"] = w, b
        out[pre + "self_attn.o_proj.weight"], out[pre + "self_attn.o_proj.bias"] = a.o.weight, a.o.bias
        out[pre + "self_attn.sinks"] = l.sinks
        out[pre + "input_layernorm.weight"], out[pre + "post_attention_layernorm.weight"] = l.input_ln, l.post_ln
        moe = l.mlp.experts
        out[pre + "mlp.router.weight"], out[pre + "mlp.router.bias"] = moe.gate.weight, moe.gate.bias
        I = moe.intermediate_size
        w13 = torch.stack([interleave(moe.w13[e, :I], moe.w13[e, I:]) for e in range(moe.num_experts)])   # [E, 2I, H]
        w2 = moe.w2[:, :H]                                                                            # [E, H, I]
        out[pre + "mlp.experts.gate_up_proj_bias"] = torch.stack(
            [interleave(moe.b13[e, :I], moe.b13[e, I:]) for e in range(moe.num_experts)])
        out[pre + "mlp.experts.down_proj_bias"] = moe.b2[:, :H]
        if packed:
            q13 = [quantize_mxfp4(w13[e].float()) for e in range(moe.num_experts)]
            q2 = [quantize_mxfp4(w2[e].float()) for e in range(moe.num_experts)]
            out[pre + "mlp.experts.gate_up_proj_blocks"] = torch.stack([q for q, _ in q13]).unflatten(-1, (-1, 16))
            out[pre + "mlp.experts.gate_up_proj_scales"] = torch.stack([s for _, s in q13])
            out[pre + "mlp.experts.down_proj_blocks"] = torch.stack([q for q, _ in q2]).unflatten(-1, (-1, 16))
            out[pre + "mlp.experts.down_proj_scales"] = torch.stack([s for _, s in q2])
        else:
            out[pre + "mlp.experts.gate_up_proj"] = w13.transpose(1, 2)          # [E, H, 2I]
            out[pre + "mlp.experts.down_proj"] = w2.transpose(1, 2)              # [E, I, H]
    return {k: v.detach().clone().contiguous() for k, v in out.items()}


def test_gpt_oss_engine_and_checkpoint_layouts(tmp_path):
    """GPT-OSS shape: sinks, alternating window / full layers, biased router and experts, OAI SwiGLU, a hidden
    size that is no multiple of the kernels' tile.  Chunked prefill with batching keeps the greedy tokens; the
    published checkpoint layout (bf16 and mxfp4 expert stacks) loads back into the same model."""
    import json
    from safetensors.torch import save_file
    from vllm_torchtpu_b200.config import ModelConfig
    from vllm_torchtpu_b200.quantization.fp4 import dequantize_mxfp4
    prompts = [np.random.RandomState(3).randint(0, 1000, size=n).tolist() for n in (9, 40, 23)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    kw = dict(device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    src = LLM("tiny-gpt-oss", max_num_batched_tokens=256, **kw)
    want = [src.generate([p], sp)[0].outputs[0].token_ids for p in prompts]
    many = LLM("tiny-gpt-oss", max_num_batched_tokens=16, **kw)
    assert [o.outputs[0].token_ids for o in many.generate(prompts, sp)] == want
    model = src.engine.runner.model
    assert [l.self_attn.attn.sliding_window for l in model.layers] == [8, None, 8, None]
    assert model.layers[0].mlp.experts.w2.shape[1] == 256 and model.layers[0].self_attn.attn.sinks is model.layers[0].sinks
    mc = ModelConfig.from_hf_dict(_gpt_oss_hf_cfg())
    assert mc.architecture == "gpt_oss" and mc.moe_bias and mc.hidden_act.startswith("swigluoai") \
        and mc.layer_sliding == (True, False, True, False) and mc.quant_ignored == ("self_attn",)
    # the experts' bias and activation against the definition, one token
    moe = model.layers[1].mlp.experts
    x = torch.randn(1, 192) * 0.5
    ids, w = moe.route(x)
    got = moe.method.apply(moe, x, ids, w)[0]
    ref_out = torch.zeros(192)
    I = moe.intermediate_size
    for j in range(2):
        e = int(ids[0, j])
        h = x[0] @ moe.w13[e].t() + moe.b13[e]
        g, u = h[:I].clamp(max=7.0), h[I:].clamp(-7.0, 7.0)
        act = (u + 1) * g * torch.sigmoid(1.702 * g)
        ref_out += w[0, j] * (act @ moe.w2[e, :192].t() + moe.b2[e, :192])
    torch.testing.assert_close(got, ref_out, rtol=1e-4, atol=1e-4)
    # bf16 checkpoint in the published layout
    d = tmp_path / "bf16"
    d.mkdir()
    save_file(_gpt_oss_tensors(model, packed=False), str(d / "model.safetensors"))
    json.dump(_gpt_oss_hf_cfg(), open(d / "config.json", "w"))
    dst = LLM(str(d), dtype="float32", **kw)
    assert [dst.generate([p], sp)[0].outputs[0].token_ids for p in prompts] == want
    torch.testing.assert_close(dst.engine.runner.model.layers[2].sinks, model.layers[2].sinks)
    # mxfp4 expert stacks stay packed; attention stays unquantised
    d4 = tmp_path / "mxfp4"
    d4.mkdir()
    t4 = _gpt_oss_tensors(model, packed=True)
    save_file(t4, str(d4 / "model.safetensors"))
    json.dump(_gpt_oss_hf_cfg(quantization_config={"quant_method": "mxfp4"}), open(d4 / "config.json", "w"))
    q = LLM(str(d4), dtype="float32", **kw)
    qm = q.engine.runner.model
    e4 = qm.layers[0].mlp.experts
    assert e4.w13.dtype == torch.uint8 and qm.layers[0].self_attn.qkv.weight.dtype == torch.float32
    blocks = t4["model.layers.0.mlp.experts.gate_up_proj_blocks"][3].flatten(-2)
    torch.testing.assert_close(e4.w13[3], torch.cat([blocks[0::2], blocks[1::2]], 0))
    I = e4.intermediate_size
    torch.testing.assert_close(dequantize_mxfp4(e4.w13[3], e4.w13_scale[3])[:I].float(),
                               dequantize_mxfp4(*[t.contiguous() for t in (blocks[0::2], t4["model.layers.0.mlp.experts.gate_up_proj_scales"][3][0::2])]).float())
    outs = q.generate(prompts, sp)
    assert all(len(o.outputs[0].token_ids) == 8 for o in outs)
