"""CPU plumbing run: tiny Llama through the paged engine vs a dense PyTorch forward."""
import numpy as np
import pytest
import torch

from vllm_torchtpu_b200 import SamplingParams
from vllm_torchtpu_b200.engine.llm import LLM
from vllm_torchtpu_b200.models.reference_forward import dense_greedy_generate


def _prompts():
    rng = np.random.RandomState(0)
    return [rng.randint(0, 1024, size=n).tolist() for n in (8, 17, 32, 64)]


@pytest.mark.parametrize("async_sched", [False, True])
@pytest.mark.parametrize("max_batched", [8192, 24])
def test_tiny_llama_matches_dense_reference(async_sched, max_batched):
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=8, max_num_batched_tokens=max_batched,
              block_size=16, async_scheduling=async_sched, init_dist=False)
    sp = SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True)
    outs = llm.generate(_prompts(), sp)
    model = llm.engine.runner.model
    for p, o in zip(_prompts(), outs):
        want, _ = dense_greedy_generate(model, p, 16)
        assert o.outputs[0].token_ids == want
        assert o.outputs[0].finish_reason == "length"


def test_logits_match_dense_reference():
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    eng = llm.engine
    p = _prompts()[2]
    eng.add_request(p, SamplingParams(max_tokens=1))
    out = eng.scheduler.schedule()
    r = eng.runner
    r._update_batch(out)
    prep = r._prepare_inputs(out)
    prep["bufs"].upload(prep["R_pad"])
    meta = r._make_meta(prep)
    _, logits = r._forward_and_sample(prep["bufs"], meta, prep["T_pad"], prep["R_pad"], True)
    from vllm_torchtpu_b200.models.reference_forward import dense_llama_logits
    want = dense_llama_logits(r.model, p)[-1]
    torch.testing.assert_close(logits[0].float(), want, rtol=1e-4, atol=1e-4)


def test_prefix_caching_reuses_blocks():
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, enable_prefix_caching=True,
              init_dist=False)
    p = _prompts()[3]
    sp = SamplingParams(max_tokens=4, ignore_eos=True)
    a = llm.generate([p], sp)[0]
    b = llm.generate([p], sp)[0]
    assert a.outputs[0].token_ids == b.outputs[0].token_ids
    assert b.num_cached_tokens == 48      # 3 full blocks of the 64-token prompt (last token recomputed)


def test_tiny_moe_matches_dense_reference():
    llm = LLM("tiny-moe", device="cpu", max_num_seqs=8, max_num_batched_tokens=48, block_size=16,
              init_dist=False)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    outs = llm.generate(_prompts()[:3], sp)
    model = llm.engine.runner.model
    for p, o in zip(_prompts()[:3], outs):
        want, _ = dense_greedy_generate(model, p, 8)
        assert o.outputs[0].token_ids == want


def test_embedding_pooling_matches_dense_hidden_states():
    """LLM.embed: last-token and mean pooling of the final-norm hidden states, also when the prompt is
    prefilled in several chunks."""
    import numpy as np
    import torch

    from vllm_torchtpu_b200.engine.llm import LLM
    from vllm_torchtpu_b200.models.reference_forward import dense_llama_hidden
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, max_num_batched_tokens=32, block_size=16,
              num_gpu_blocks_override=32)
    rng = np.random.RandomState(3)
    vocab = llm.engine.cfg.model.vocab_size
    prompts = [rng.randint(0, vocab, size=n).tolist() for n in (7, 50)]        # 50 > 32: two chunks
    model = llm.engine.runner.model
    for mode in ("last", "mean", "max", "cls", "all"):
        got = llm.embed(prompts, pooling=mode, normalize=False)
        for p, g in zip(prompts, got):
            h = dense_llama_hidden(model, p)                                    # [len, H] after the final norm
            want = {"last": h[-1], "mean": h.mean(0), "max": h.max(0).values, "cls": h[0], "all": h}[mode]
            torch.testing.assert_close(torch.tensor(g), want.float(), rtol=2e-3, atol=2e-3)
    unit = llm.embed(prompts[:1])[0]
    assert abs(sum(a * a for a in unit) - 1.0) < 1e-4


@pytest.mark.parametrize("async_sched", [False, True])
def test_sample_logprobs_min_tokens_and_prompt_logprobs(async_sched):
    """Logprobs of sampled tokens, the on-device min_tokens mask and chunked prompt logprobs, against the
    dense fp32 forward of the same model."""
    from vllm_torchtpu_b200.models.reference_forward import dense_llama_logits
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, max_num_batched_tokens=16, block_size=16,
              init_dist=False, async_scheduling=async_sched)
    prompt = _prompts()[2]
    base = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))[0]
    toks = base.outputs[0].token_ids
    # sampled-token logprobs: greedy tokens are rank 1 and head the top-k list
    out = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True, logprobs=3))[0]
    lps = out.outputs[0].logprobs
    assert out.outputs[0].token_ids == toks and len(lps) == 5
    for t, e in zip(toks, lps):
        assert e["token_id"] == t and e["rank"] == 1 and e["top"][0][0] == t and len(e["top"]) == 3
        assert e["logprob"] <= 0.0 and abs(e["top"][0][1] - e["logprob"]) < 1e-5
    # stop token = the first greedy token: one token without min_tokens, masked until min_tokens with it
    stop = SamplingParams(temperature=0.0, max_tokens=8, stop_token_ids=[toks[0]])
    assert llm.generate([prompt], stop)[0].outputs[0].token_ids == [toks[0]]
    held = SamplingParams(temperature=0.0, max_tokens=8, stop_token_ids=[toks[0]], min_tokens=3)
    got = llm.generate([prompt], held)[0].outputs[0].token_ids
    assert len(got) >= 3 and toks[0] not in got[:3]
    # prompt logprobs over a prefill that takes several chunks (16 tokens per step)
    out = llm.generate([prompt], SamplingParams(temperature=0.0, max_tokens=1, prompt_logprobs=2))[0]
    plp = out.prompt_logprobs
    assert len(plp) == len(prompt) and plp[0] is None
    want = torch.log_softmax(dense_llama_logits(llm.engine.runner.model, prompt).float(), dim=-1)
    for i in range(1, len(prompt)):
        assert plp[i]["token_id"] == prompt[i]
        assert abs(plp[i]["logprob"] - float(want[i - 1, prompt[i]])) < 2e-3, i
        assert len(plp[i]["top"]) == 2


def test_multimodal_embeddings_through_vision_encoder():
    """Image patches -> vision encoder (bidirectional varlen attention, batched under a patch budget,
    padded to a bucket) -> rows that replace the placeholder tokens; chunked prefill across an image
    and batching with a text-only request leave the tokens unchanged."""
    from vllm_torchtpu_b200.layers.vision import VisionConfig, VisionEncoder
    from vllm_torchtpu_b200.runner.mm_encoder import MMEncoderManager, MMItem, chunk_video, patch_buckets
    assert chunk_video(10, 64, 256, temporal_patch=2) == [(0, 8), (8, 2)]
    assert chunk_video(3, 100, 100, temporal_patch=1) == [(0, 1), (1, 1), (2, 1)]
    assert patch_buckets(1000, 256) == [256, 512, 1000]
    with pytest.raises(ValueError):
        chunk_video(4, 300, 256)
    # the encoder treats every item as its own attention segment: batching does not change an item
    vc = VisionConfig(patch_dim=48, hidden_size=64, num_heads=2, depth=2, merge=4, out_hidden_size=256)
    enc = VisionEncoder(vc, "cpu")
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(16, 48, generator=g), torch.randn(40, 48, generator=g)
    alone = enc.forward(a, [16])[0]
    both = enc.forward(torch.cat([a, b]), [16, 40])
    torch.testing.assert_close(both[0], alone, rtol=1e-5, atol=1e-5)
    assert both[1].shape == (10, 256)
    mgr = MMEncoderManager(enc, max_patches_per_batch=48, buckets=[32, 48])
    mgr.add_request("r", [MMItem("r", 0, a, 3), MMItem("r", 1, b, 20)])
    rows = mgr.gather("r", 0, 8)                       # first chunk covers part of item 0 only
    assert len(rows) == 1 and rows[0][0] == 3 and rows[0][1].shape[0] == 4 and mgr.stats["batches"] == 1
    torch.testing.assert_close(rows[0][1], alone, rtol=1e-5, atol=1e-5)
    rows = mgr.gather("r", 22, 40)
    assert rows[0][0] == 0 and rows[0][1].shape[0] == 8 and mgr.stats["batches"] == 2
    assert mgr.stats["padded_patches"] == 32 + 48
    # engine: greedy tokens with image embeddings, whole prompt vs 16-token chunks + a text neighbour
    prompt = _prompts()[3][:48]
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)

    def run(max_batched, extra):
        llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, max_num_batched_tokens=max_batched, block_size=16,
                  init_dist=False)
        llm.engine.enable_vision(vc, max_patches_per_batch=64)
        eng = llm.engine
        rid = eng.add_request(prompt, sp, mm_items=[(a, 5), (b, 30)])
        for p in extra:
            eng.add_request(p, sp)
        done = {r.request_id: r.output_token_ids for r in eng.run_until_done()}
        return done[rid]

    whole = run(256, [])
    chunked = run(16, [_prompts()[1]])
    assert whole == chunked
    plain = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    assert plain.generate([prompt], sp)[0].outputs[0].token_ids != whole      # the image changes the output
    with pytest.raises(ValueError):
        plain.engine.add_request(prompt, sp, mm_items=[(a, 5)])


def test_device_wait_timeout_fails_the_step_not_the_engine():
    """A non-zero device status word (what a bounded wait inside a kernel leaves when it gives up) turns
    into failed requests for that step; the word is cleared and the engine keeps serving."""
    from vllm_torchtpu_b200.runner.model_runner import DeviceWaitTimeout, StepResult
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False, async_scheduling=False)
    eng = llm.engine
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    rid = eng.add_request(_prompts()[0], sp)
    eng.runner.status_dev[0] = 5                       # as if a peer flag never arrived
    done = eng.step()
    assert [r.request_id for r in done] == [rid] and done[0].error.startswith("device_wait_timeout")
    assert done[0].status.value == "error" and int(eng.runner.status_dev[0]) == 0 and eng.device_errors == 1
    out = llm.generate([_prompts()[1]], sp)[0]          # the engine still serves
    assert len(out.outputs[0].token_ids) == 4 and out.error is None
    with pytest.raises(DeviceWaitTimeout) as ei:
        StepResult([], [], None, None, 0, status_host=torch.tensor([3], dtype=torch.int32)).get()
    assert ei.value.code == 3 and "accumulator" in str(ei.value)


def test_scheduler_blocks_split_into_kernel_blocks_generate_the_same_tokens():
    """64-token scheduler blocks over 16-token kernel pages: the block-table rows the kernels read list four
    kernel blocks per scheduler block, and generation (prefix cache on) matches the plain configuration."""
    import numpy as np

    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.engine.llm import LLM
    from vllm_torchtpu_b200.runner.kernel_block_table import KernelBlockTable
    t = KernelBlockTable(2, 16, 4)
    t.set_row(0, [3, 1])
    t.append(0, [7])
    assert t.table[0, :12].tolist() == [12, 13, 14, 15, 4, 5, 6, 7, 28, 29, 30, 31] and t.num_blocks[0] == 12
    rng = np.random.RandomState(1)
    shared = rng.randint(0, 1000, size=70).tolist()
    prompts = [shared + rng.randint(0, 1000, size=n).tolist() for n in (5, 40)] + [rng.randint(0, 1000, size=9).tolist()]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    kw = dict(device="cpu", max_num_seqs=4, max_num_batched_tokens=64, block_size=16, init_dist=False,
              num_gpu_blocks_override=64, enable_prefix_caching=True)
    plain = [o.outputs[0].token_ids for o in LLM("tiny-llama", **kw).generate(prompts, sp)]
    coarse_llm = LLM("tiny-llama", scheduler_block_size=64, **kw)
    coarse = [o.outputs[0].token_ids for o in coarse_llm.generate(prompts, sp)]
    assert coarse == plain
    assert coarse_llm.engine.scheduler.block_size == 64 and coarse_llm.engine.scheduler.kv.pool.num_blocks == 16


def test_kv_block_counts_are_reconciled_per_pipeline_stage():
    import pytest

    from vllm_torchtpu_b200.engine.kv_block_agreement import reconcile, within_tolerance
    assert within_tolerance([1000, 1003, 998]) and not within_tolerance([1000, 990])
    assert within_tolerance([100000, 100400]) and not within_tolerance([100000, 100600])      # 0.5 %
    # two stages of two ranks: each stage settles on its minimum, the engine on the smaller stage
    assert reconcile({0: 1000, 1: 1002, 2: 800, 3: 799}, {0: 0, 1: 0, 2: 1, 3: 1}) == 799
    with pytest.raises(ValueError, match="stage 1"):
        reconcile({0: 1000, 1: 1002, 2: 800, 3: 700}, {0: 0, 1: 0, 2: 1, 3: 1})


def test_update_weights_in_place_changes_the_output_like_a_fresh_engine(tmp_path):
    """Weights handed over in memory (a trainer's step): the engine that took them generates what an engine
    loaded from the same checkpoint generates, and no longer what it generated before."""
    import torch

    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.engine.llm import LLM
    from vllm_torchtpu_b200.models.loader import iter_safetensors, save_hf_checkpoint
    kw = dict(device="cpu", max_num_seqs=4, block_size=16, init_dist=False, enable_prefix_caching=True)
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    prompts = [[5, 6, 7, 8, 9], [100, 101, 102]]
    donor = LLM("tiny-llama", seed=123, **kw)
    save_hf_checkpoint(donor.engine.runner.model, str(tmp_path))
    want = [o.outputs[0].token_ids for o in donor.generate(prompts, sp)]
    llm = LLM("tiny-llama", seed=0, **kw)
    before = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert before != want
    n = llm.engine.update_weights(dict(iter_safetensors(str(tmp_path))))
    assert n > 0
    after = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert after == want
