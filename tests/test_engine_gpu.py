"""End-to-end engine on the GPU kernels: logits vs a dense fp32 forward, CUDA-graph
decode vs eager decode, async vs sync scheduling."""
import numpy as np
import pytest
import torch

from vllm_torchtpu_b200 import SamplingParams
from vllm_torchtpu_b200.config import ModelConfig
from vllm_torchtpu_b200.engine.llm import LLM

pytestmark = pytest.mark.gpu


def _cfg():
    return ModelConfig(name="t", num_layers=2, hidden_size=512, num_q_heads=8, num_kv_heads=2, head_dim=128,
                       intermediate_size=1024, vocab_size=2048, max_model_len=512, dtype=torch.bfloat16)


def _prompts():
    rng = np.random.RandomState(0)
    return [rng.randint(0, 2048, size=n).tolist() for n in (8, 17, 32, 64, 129)]


def _llm(**kw):
    return LLM(_cfg(), device="cuda", max_num_seqs=8, max_num_batched_tokens=256,
               num_gpu_blocks_override=512, init_dist=False, **kw)


def test_prefill_logits_match_dense():
    from vllm_torchtpu_b200.models.reference_forward import dense_llama_logits
    llm = _llm(enforce_eager=True)
    eng = llm.engine
    p = _prompts()[3]
    eng.add_request(p, SamplingParams(max_tokens=1))
    out = eng.scheduler.schedule()
    r = eng.runner
    r._update_batch(out)
    prep = r._prepare_inputs(out)
    prep["bufs"].upload(prep["R_pad"])
    _, logits = r._forward_and_sample(prep["bufs"], r._make_meta(prep), prep["T_pad"], prep["R_pad"], True)
    want = dense_llama_logits(r.model, p)[-1]
    err = (logits[0].float() - want).abs().max().item()
    assert err < 0.05 * want.abs().max().item() + 0.02, err


def test_graph_decode_equals_eager_and_async():
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    eager = [o.outputs[0].token_ids for o in _llm(enforce_eager=True).generate(_prompts(), sp)]
    graph = [o.outputs[0].token_ids for o in _llm().generate(_prompts(), sp)]
    asyn = [o.outputs[0].token_ids for o in _llm(async_scheduling=True).generate(_prompts(), sp)]
    assert eager == graph
    assert eager == asyn
    from vllm_torchtpu_b200.ops import cuda
    assert cuda.check_status() == 0


def test_random_sampling_runs_and_is_seeded():
    sp = SamplingParams(temperature=0.8, top_k=50, top_p=0.9, max_tokens=8, ignore_eos=True)
    a = [o.outputs[0].token_ids for o in _llm().generate(_prompts()[:2], sp)]
    b = [o.outputs[0].token_ids for o in _llm().generate(_prompts()[:2], sp)]
    assert a == b


def test_lora_request_and_embedding_on_gpu():
    """Adapter requests run through the bgmv kernels next to base requests (which keep their tokens),
    and LLM.embed returns unit vectors."""
    import numpy as np
    llm = _llm(enforce_eager=True)
    prompts = _prompts()[:2]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    base = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    g = torch.Generator().manual_seed(0)
    weights = {}
    for lin in llm.engine.runner.model.named_linears():
        prefix, leaf = lin.name.rsplit(".", 1)
        if leaf == "down_proj":
            weights[lin.name] = (torch.randn(8, lin.in_features, generator=g) * 0.5,
                                 torch.randn(lin.out_features, 8, generator=g) * 0.5)
    assert llm.engine.add_lora("ad", 8, 64.0, weights)
    sp_l = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, lora_name="ad")
    outs = llm.generate(prompts, [sp_l, sp])
    assert outs[1].outputs[0].token_ids == base[1]
    assert outs[0].outputs[0].token_ids != base[0]
    v = llm.embed(prompts[:1])[0]
    assert abs(float(np.square(v).sum()) - 1.0) < 1e-2
    from vllm_torchtpu_b200.ops import cuda
    assert cuda.check_status() == 0


def test_fp8_kv_cache_engine():
    """An e4m3 KV cache (written by the rope kernel, expanded inside the attention kernels) keeps the
    prefill logits close to the dense forward and decodes through CUDA graphs."""
    from vllm_torchtpu_b200.models.reference_forward import dense_llama_logits
    llm = _llm(kv_cache_dtype="fp8")
    eng = llm.engine
    r = eng.runner
    assert r.kv_caches[0].dtype == torch.float8_e4m3fn
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    outs = llm.generate(_prompts(), sp)
    assert all(len(o.outputs[0].token_ids) == 12 for o in outs)
    p = _prompts()[3]
    eng.add_request(p, SamplingParams(max_tokens=1))
    out = eng.scheduler.schedule()
    r._update_batch(out)
    prep = r._prepare_inputs(out)
    prep["bufs"].upload(prep["R_pad"])
    _, logits = r._forward_and_sample(prep["bufs"], r._make_meta(prep), prep["T_pad"], prep["R_pad"], True)
    want = dense_llama_logits(r.model, p)[-1]
    err = (logits[0].float() - want).abs().max().item()
    assert err < 0.12 * want.abs().max().item() + 0.05, err
    from vllm_torchtpu_b200.ops import cuda
    assert cuda.check_status() == 0


@pytest.mark.parametrize("arch,extra", [
    ("qwen3_next", dict(qk_norm=True, full_attention_interval=2, gdn_num_k_heads=2, gdn_num_v_heads=4)),
    ("kimi_linear", dict(full_attention_interval=4, gdn_num_k_heads=4, gdn_num_v_heads=4, kda_gate_rank=32)),
])
def test_hybrid_linear_attention_models_on_gpu(arch, extra):
    """Gated DeltaNet and Kimi Delta Attention hybrids on the CUDA kernels (short conv, recurrence with
    pooled state, paged attention for the full layers): chunked prefill with batching reproduces the
    greedy tokens of one-request-at-a-time serving, and a long decode keeps the state finite."""
    cfg = ModelConfig(name="h", architecture=arch, num_layers=4, hidden_size=512, num_q_heads=8, num_kv_heads=2,
                      head_dim=128, intermediate_size=1024, vocab_size=2048, max_model_len=512,
                      dtype=torch.bfloat16, gdn_head_k_dim=64, gdn_head_v_dim=64, **extra)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    mk = lambda mbt: LLM(cfg, device="cuda", max_num_seqs=8, max_num_batched_tokens=mbt,
                         num_gpu_blocks_override=512, init_dist=False, enforce_eager=True)
    prompts = _prompts()[:4]
    one = mk(256)
    want = [one.generate([p], sp)[0].outputs[0].token_ids for p in prompts]
    got = [o.outputs[0].token_ids for o in mk(64).generate(prompts, sp)]
    same = sum(int(a == b) for a, b in zip(got, want))
    assert same >= len(prompts) - 1, (got, want)      # bf16 ties may flip one continuation
    from vllm_torchtpu_b200.ops import cuda
    assert cuda.check_status() == 0


@pytest.mark.parametrize("arch,extra", [
    ("qwen3_next", dict(qk_norm=True, full_attention_interval=2, gdn_num_k_heads=2, gdn_num_v_heads=4)),
    ("kimi_linear", dict(full_attention_interval=4, gdn_num_k_heads=4, gdn_num_v_heads=4, kda_gate_rank=32)),
])
def test_speculative_decoding_on_hybrids_on_gpu(arch, extra):
    """Verification steps on a hybrid: the recurrent state of requests that rejected drafts is restored from
    the snapshot and the accepted rows are replayed through the recurrence kernels; tokens equal plain
    decoding (a drafter that knows the continuation and spoils every other call's second draft)."""
    cfg = ModelConfig(name="h", architecture=arch, num_layers=4, hidden_size=512, num_q_heads=8, num_kv_heads=2,
                      head_dim=128, intermediate_size=1024, vocab_size=2048, max_model_len=512,
                      dtype=torch.bfloat16, gdn_head_k_dim=64, gdn_head_v_dim=64, **extra)
    sp = SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True)
    kw = dict(device="cuda", max_num_seqs=8, max_num_batched_tokens=256, num_gpu_blocks_override=512,
              init_dist=False, enforce_eager=True)
    prompts = _prompts()[:3]
    want = [o.outputs[0].token_ids for o in LLM(cfg, **kw).generate(prompts, sp)]
    spec = LLM(cfg, speculative_config={"method": "ngram", "num_speculative_tokens": 3}, **kw)

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
                d[1] = (d[1] + 1) % 2048
            if d:
                drafts[r.request_id] = d
        return drafts
    spec.engine.spec.propose = propose
    got = [o.outputs[0].token_ids for o in spec.generate(prompts, sp)]
    st = spec.engine.runner.stats
    assert st.get("spec_drafted", 0) > 0 and st.get("state_rollbacks", 0) > 0
    # a bf16 tie between the 1-row and the (k + 1)-row kernels may flip one continuation
    assert sum(int(a == b) for a, b in zip(got, want)) >= len(prompts) - 1, (got, want)
    from vllm_torchtpu_b200.ops import cuda
    assert cuda.check_status() == 0


def test_moe_engine_with_padded_decode_buckets_on_gpu():
    """Qwen3-MoE shaped model through the engine with captured decode graphs: three requests run in a bucket of
    four rows, the padded row takes no expert (the routing reads the step's real row count from the device),
    and the tokens equal serving the requests one at a time."""
    cfg = ModelConfig(name="m", architecture="qwen3_moe", qk_norm=True, num_layers=2, hidden_size=512, num_q_heads=8,
                      num_kv_heads=2, head_dim=128, intermediate_size=1024, vocab_size=2048, max_model_len=512,
                      dtype=torch.bfloat16, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    kw = dict(device="cuda", max_num_seqs=8, max_num_batched_tokens=256, num_gpu_blocks_override=512, init_dist=False)
    prompts = _prompts()[:3]
    one = LLM(cfg, **kw)
    want = [one.generate([p], sp)[0].outputs[0].token_ids for p in prompts]
    many = LLM(cfg, **kw)
    got = [o.outputs[0].token_ids for o in many.generate(prompts, sp)]
    assert many.engine.runner.stats["graph_steps"] > 0
    assert sum(int(a == b) for a, b in zip(got, want)) >= len(prompts) - 1, (got, want)   # a bf16 tie may flip one
    from vllm_torchtpu_b200.ops import cuda
    assert cuda.check_status() == 0


@pytest.mark.parametrize("quant", [None, "mxfp4"])
def test_gpt_oss_shape_on_gpu(quant):
    """GPT-OSS shape on the device: 64-wide heads with sinks, window and full layers in alternation, YaRN, biased
    router and experts with the OAI SwiGLU, a hidden size below the padded down projection; bf16 experts and mxfp4
    experts on the W4A16 kernel.  Batched chunked prefill repeats one-at-a-time serving."""
    from vllm_torchtpu_b200.config import model_preset
    cfg = model_preset("tiny-gpt-oss")
    cfg.dtype, cfg.quantization = torch.bfloat16, quant
    if quant:
        cfg.quant_ignored = ("self_attn",)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    mk = lambda mbt: LLM(cfg, device="cuda", max_num_seqs=8, max_num_batched_tokens=mbt,
                         num_gpu_blocks_override=256, init_dist=False)
    rng = np.random.RandomState(1)
    prompts = [rng.randint(0, 1000, size=n).tolist() for n in (8, 17, 40, 64)]
    one = mk(256)
    want = [one.generate([p], sp)[0].outputs[0].token_ids for p in prompts]
    if quant:
        assert one.engine.runner.model.layers[0].mlp.experts.w13.dtype == torch.uint8
    got = [o.outputs[0].token_ids for o in mk(32).generate(prompts, sp)]
    assert sum(int(a == b) for a, b in zip(got, want)) >= len(prompts) - 1, (got, want)
    from vllm_torchtpu_b200.ops import cuda
    assert cuda.check_status() == 0


def test_logprobs_min_tokens_prompt_logprobs_on_gpu():
    """The logprob kernel, the min_tokens mask and chunked prompt logprobs on the device path (these
    steps leave the CUDA graphs), against the dense fp32 forward."""
    from vllm_torchtpu_b200.models.reference_forward import dense_llama_logits
    llm = LLM(_cfg(), device="cuda", max_num_seqs=8, max_num_batched_tokens=64, num_gpu_blocks_override=512,
              init_dist=False)
    prompt = _prompts()[4]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    toks = llm.generate([prompt], sp)[0].outputs[0].token_ids
    out = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, logprobs=4,
                                                prompt_logprobs=1))[0]
    assert out.outputs[0].token_ids == toks
    for t, e in zip(toks, out.outputs[0].logprobs):
        assert e["token_id"] == t and e["rank"] == 1 and e["top"][0][0] == t and e["logprob"] <= 0.0
    want = torch.log_softmax(dense_llama_logits(llm.engine.runner.model, prompt).float(), dim=-1)
    plp = out.prompt_logprobs
    assert len(plp) == len(prompt) and plp[0] is None
    err = max(abs(plp[i]["logprob"] - float(want[i - 1, prompt[i]])) for i in range(1, len(prompt)))
    assert err < 0.08, err
    held = SamplingParams(temperature=0.0, max_tokens=8, stop_token_ids=[toks[0]], min_tokens=3)
    got = llm.generate([prompt], held)[0].outputs[0].token_ids
    assert len(got) >= 3 and toks[0] not in got[:3]
    from vllm_torchtpu_b200.ops import cuda
    assert cuda.check_status() == 0


def test_vision_encoder_on_gpu_matches_cpu():
    """ViT blocks on the tcgen05 GEMM and the bidirectional attention kernel against the fp32 CPU stack."""
    from vllm_torchtpu_b200.layers.vision import VisionConfig, VisionEncoder
    kw = dict(patch_dim=96, hidden_size=256, num_heads=4, depth=2, merge=4, out_hidden_size=512)
    cpu = VisionEncoder(VisionConfig(dtype=torch.float32, **kw), "cpu")
    gpu = VisionEncoder(VisionConfig(dtype=torch.bfloat16, **kw), "cuda")
    # random-init draws differ between devices: give the GPU stack the CPU stack's weights
    for name in ("patch_w", "merge_w"):
        setattr(gpu, name, getattr(cpu, name).to("cuda", torch.bfloat16))
    for bc, bg in zip(cpu.blocks, gpu.blocks):
        for name in ("qkv_w", "proj_w", "fc1_w", "fc2_w"):
            setattr(bg, name, getattr(bc, name).to("cuda", torch.bfloat16))
    g = torch.Generator().manual_seed(0)
    counts = [64, 200, 16]
    patches = torch.randn(sum(counts), 96, generator=g)
    want = cpu.forward(patches, counts)
    got = gpu.forward(patches.cuda(), counts)
    for a, b in zip(got, want):
        assert a.shape == b.shape
        err = (a.float().cpu() - b).abs().max().item()
        assert err < 0.05 * b.abs().max().item() + 0.02, err


def test_fp8_block_quantised_engine_matches_its_dequantised_dense_forward():
    """Llama-style model with block-scaled fp8 linears (activation quantisation shared between projections,
    SiLU*mul fused into the down projection's quantisation): prefill logits against the dense fp32 forward
    over the dequantised weights."""
    from vllm_torchtpu_b200.models.reference_forward import dense_llama_logits
    cfg = _cfg()
    cfg.quantization = "fp8_block"
    llm = LLM(cfg, device="cuda", max_num_seqs=8, max_num_batched_tokens=256, num_gpu_blocks_override=512,
              init_dist=False, enforce_eager=True)
    eng = llm.engine
    p = _prompts()[3]
    eng.add_request(p, SamplingParams(max_tokens=1))
    out = eng.scheduler.schedule()
    r = eng.runner
    r._update_batch(out)
    prep = r._prepare_inputs(out)
    prep["bufs"].upload(prep["R_pad"])
    _, logits = r._forward_and_sample(prep["bufs"], r._make_meta(prep), prep["T_pad"], prep["R_pad"], True)
    want = dense_llama_logits(r.model, p)[-1]
    err = (logits[0].float() - want).abs().max().item()
    # activations go through e4m3 in the kernel path and stay bf16 in the dense forward
    assert err < 0.12 * want.abs().max().item() + 0.05, err
    fresh = LLM(cfg, device="cuda", max_num_seqs=8, max_num_batched_tokens=256, num_gpu_blocks_override=512,
                init_dist=False)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    toks = [o.outputs[0].token_ids for o in fresh.generate(_prompts()[:3], sp)]
    assert all(len(t) == 8 for t in toks)
