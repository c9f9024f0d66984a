"""Scheduler policies, block manager and bucket builders (CPU, no device)."""
import pytest

from vllm_torchtpu_b200.config import CacheConfig, SchedulerConfig
from vllm_torchtpu_b200.engine.block_manager import BlockPool, KVCacheManager
from vllm_torchtpu_b200.engine.request import Request, RequestStatus
from vllm_torchtpu_b200.engine.scheduler import Scheduler
from vllm_torchtpu_b200.platform import pad_to_bucket, request_paddings, token_paddings
from vllm_torchtpu_b200.sampling_params import SamplingParams
from vllm_torchtpu_b200.schedulers import get_scheduler_class
from vllm_torchtpu_b200.schedulers.pp_chunk import StepCostModel, chunk_granularity, step_limit


def mk(cls=Scheduler, blocks=64, max_seqs=8, budget=64, caching=False, **kw):
    return cls(SchedulerConfig(max_seqs, budget), CacheConfig(block_size=16, enable_prefix_caching=caching),
               blocks, **kw)


def req(i, n, max_tokens=4, base=0):
    return Request(f"r{i}", [base + j for j in range(n)], SamplingParams(max_tokens=max_tokens, ignore_eos=True))


def run(s, steps=200):
    order = []
    for _ in range(steps):
        if not s.has_unfinished():
            break
        out = s.schedule()
        sampled = {x.request.request_id: [7] for x in out.scheduled if x.samples}
        for r in s.update_from_output(out, sampled):
            order.append(r.request_id)
    return order


def test_token_and_request_buckets():
    assert token_paddings(8192, 16)[:4] == [16, 32, 64, 128] and token_paddings(8192, 16)[-1] == 8192
    assert token_paddings(100, 16) == [16, 32, 64, 100]
    assert 48 in token_paddings(128, 16, extra=[48]) and 96 in token_paddings(128, 16, linear_stride=32)
    assert request_paddings(64, 8) == [8, 16, 32, 64]
    assert request_paddings(4, 8) == [4]
    assert pad_to_bucket(9, [8, 16]) == 16
    with pytest.raises(ValueError):
        pad_to_bucket(17, [8, 16])


def test_block_pool_refcount_and_prefix_cache():
    pool = BlockPool(8, 4, enable_caching=True)
    a = pool.allocate(3)
    assert pool.num_free_blocks == 4 and 0 not in a
    toks = list(range(12))
    pool.cache_full_blocks(toks, a, 12)
    pool.release(a)
    hit = pool.lookup_prefix(toks + [99])
    assert hit == a
    pool.touch(hit)
    assert pool.num_free_blocks == 4
    pool.release(hit)
    # allocating everything evicts cached blocks and drops their hashes
    pool.allocate(7)
    assert pool.lookup_prefix(toks + [99]) == []
    with pytest.raises(RuntimeError):
        pool.allocate(1)


def test_chunked_prefill_and_decode_mix():
    s = mk(budget=32)
    s.add_request(req(0, 50))
    s.add_request(req(1, 10))
    out = s.schedule()
    assert [(x.request.request_id, x.num_new_tokens, x.samples) for x in out.scheduled] == [("r0", 32, False)]
    s.update_from_output(out, {})
    out = s.schedule()
    got = [(x.request.request_id, x.num_new_tokens, x.samples) for x in out.scheduled]
    assert got == [("r0", 18, True), ("r1", 10, True)]
    s.update_from_output(out, {"r0": [5], "r1": [6]})
    out = s.schedule()
    assert out.is_decode_only and out.total_num_tokens == 2


def test_preemption_recomputes_and_abort_policy():
    s = mk(blocks=6, budget=64)          # 5 usable blocks of 16
    s.add_request(req(0, 40, max_tokens=40))
    s.add_request(req(1, 30, max_tokens=40))
    done = run(s, 400)
    assert sorted(done) == ["r0", "r1"] and s.stats["preemptions"] >= 1
    s2 = mk(blocks=6, budget=64, abort_on_preemption=True)
    s2.add_request(req(0, 40, max_tokens=40))
    s2.add_request(req(1, 30, max_tokens=40))
    run(s2, 400)
    statuses = {r.request_id: r.status for r in s2.requests.values()}
    assert RequestStatus.FINISHED_ERROR in statuses.values()
    assert any(r.error == "kv_cache_preempted" for r in s2.requests.values())


def test_async_scheduling_stops_at_max_tokens():
    s = Scheduler(SchedulerConfig(4, 64, async_scheduling=True), CacheConfig(block_size=16), 32)
    s.add_request(req(0, 5, max_tokens=3))
    pending = []
    n_sampling_steps = 0
    for _ in range(20):
        out = s.schedule()
        if out.scheduled:
            n_sampling_steps += sum(1 for x in out.scheduled if x.samples)
            pending.append(out)
        if len(pending) > 1 or (pending and not out.scheduled):
            o = pending.pop(0)
            s.update_from_output(o, {x.request.request_id: [1] for x in o.scheduled if x.samples})
        if not s.has_unfinished() and not pending:
            break
    assert n_sampling_steps == 3
    assert len(s.requests["r0"].output_token_ids) == 3


def test_prefix_aware_prefers_cached_prefix():
    cls = get_scheduler_class("prefix_aware")
    s = mk(cls, caching=True, budget=64, max_seqs=1)
    s.add_request(req(0, 33, base=0))
    run(s)
    s.add_request(req(1, 40, base=1000))
    s.add_request(req(2, 40, base=0))       # shares 32 cached tokens with r0
    out = s.schedule()
    assert out.scheduled[0].request.request_id == "r2"


def test_srpt_orders_by_remaining_prefill_but_does_not_starve():
    cls = get_scheduler_class("srpt")
    s = mk(cls, budget=64, max_seqs=1)
    s.max_skips = 2
    s.add_request(req(0, 60))
    for i in range(1, 6):
        s.add_request(req(i, 5 + i))
    order = run(s, 500)
    assert order[0] == "r1" and order.index("r0") <= 3


def test_dp_scheduler_throttles_prefill():
    cls = get_scheduler_class("dp")
    s = mk(cls, budget=64)
    s.add_request(req(0, 10, max_tokens=50))
    out = s.schedule()
    s.update_from_output(out, {"r0": [1]})
    s.add_request(req(1, 10))
    s.throttle_prefills([10, 0], max_decode_gap=3)
    assert [x.request.request_id for x in s.schedule().scheduled] == ["r0"]


def test_pp_chunk_policies():
    assert chunk_granularity(16, 1024) == 128 and chunk_granularity(48, 1024, True) == 144
    assert step_limit(1000, 4, 128, 1024) == 256 and step_limit(8000, 4, 128, 1024) is None
    samples = [(256, 0, 10.0), (1024, 0, 34.0), (1024, 4096, 74.0)]
    m = StepCostModel.fit(samples, 1024, 0.1)
    assert m.attn_ms_per_pair > 0
    deep = m.max_chunk(16384, [], 128, 1024)
    shallow = m.max_chunk(0, [], 128, 1024)
    assert 0 < deep < shallow == 1024
    cls = get_scheduler_class("pp_chunk")
    s = mk(cls, budget=1024, blocks=512, pp_size=4)
    s.add_request(req(0, 1000))
    out = s.schedule()
    assert out.scheduled[0].num_new_tokens == 256      # lone prompt spread over 4 stages


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("caching,spec", [(False, 0), (True, 0), (True, 3), (False, 2)])
def test_scheduler_randomised_run_keeps_the_block_pool_consistent(seed, caching, spec):
    """Random arrivals (shared prefixes), aborts, speculative tokens with random acceptance and a pool small
    enough to force preemption: after every step the reference counts equal the holders, no free block is
    held by a request, the token budget and the sequence limit are respected, and at the end every block is
    free and every request finished once."""
    import random
    rng = random.Random(1000 * seed + 17 * spec + caching)
    s = mk(blocks=14, max_seqs=5, budget=48, caching=caching, num_spec_tokens=spec)
    pool = s.kv.pool
    finished, submitted, next_id = [], {}, 0
    prefixes = [[rng.randrange(50) for _ in range(32)] for _ in range(3)]
    for step in range(3000):
        if step < 150 and rng.random() < 0.35:
            p = list(rng.choice(prefixes))[:rng.choice([0, 16, 32])] + [rng.randrange(1000) for _ in range(rng.randrange(1, 40))]
            r = Request(f"r{next_id}", p, SamplingParams(max_tokens=rng.randrange(1, 40), ignore_eos=True))
            submitted[r.request_id] = r
            s.add_request(r)
            next_id += 1
        if submitted and rng.random() < 0.03:
            s.abort_request(rng.choice(list(submitted)))
        if not s.has_unfinished():
            if step >= 150:
                break
            continue
        out = s.schedule()
        assert sum(x.num_new_tokens for x in out.scheduled) <= 48 and len(s.running) <= 5
        sampled, spec_next = {}, {}
        for x in out.scheduled:
            if not x.samples:
                continue
            k = len(x.spec_token_ids)
            acc = rng.randrange(0, k + 1)                       # accepted drafts, then the sampled token
            sampled[x.request.request_id] = list(x.spec_token_ids[:acc]) + [rng.randrange(1000)]
            if spec and rng.random() < 0.7:
                spec_next[x.request.request_id] = [rng.randrange(1000) for _ in range(rng.randrange(1, spec + 1))]
        finished += [r.request_id for r in s.update_from_output(out, sampled, spec_next or None)]
        # invariants of the pool
        holders = {}
        for r in list(s.running) + list(s.waiting):
            for b in r.block_ids:
                holders[b] = holders.get(b, 0) + 1
        for blk in pool.blocks[1:]:
            assert blk.ref_cnt == holders.get(blk.block_id, 0), (step, blk.block_id, blk.ref_cnt, holders.get(blk.block_id))
            assert (blk.ref_cnt == 0) == (blk.block_id in pool.free)
        for r in s.running:
            assert len(r.block_ids) * 16 >= r.num_computed_tokens
    assert not s.has_unfinished()
    assert pool.num_free_blocks == pool.num_blocks - 1
    assert len(finished) == len(set(finished))
    assert s.stats["preemptions"] > 0                 # the pool is small enough to force recomputation
    done_or_aborted = {rid for rid, r in submitted.items() if r.status.finished}
    assert done_or_aborted == set(submitted)


def test_priority_scheduler_admits_by_priority_and_preempts_the_least_important():
    """One request fits the batch at a time: the order of completion follows (priority, arrival), whatever the
    order of submission; the default scheduler keeps arrival order."""
    from vllm_torchtpu_b200.engine.llm import LLM
    from vllm_torchtpu_b200.sampling_params import SamplingParams
    sp = SamplingParams(max_tokens=3, ignore_eos=True)
    prompts = [[1, 2, 3], [4, 5, 6], [7, 8, 9], [10, 11, 12]]
    prios = [5, 1, 3, 1]
    order = {}
    for cls in ("priority", "default"):
        llm = LLM("tiny-llama", device="cpu", max_num_seqs=1, block_size=16, init_dist=False, scheduler_cls=cls)
        ids = [llm.engine.add_request(p, sp, priority=pr) for p, pr in zip(prompts, prios)]
        done = []
        while llm.engine.has_unfinished():
            done += [r.request_id for r in llm.engine.step()]
        order[cls] = [ids.index(r) for r in done]
    assert order["priority"] == [1, 3, 2, 0] and order["default"] == [0, 1, 2, 3]
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=1, block_size=16, init_dist=False, scheduler_cls="priority")
    outs = llm.generate(prompts, sp, priority=prios)
    assert [len(o.outputs[0].token_ids) for o in outs] == [3, 3, 3, 3]
