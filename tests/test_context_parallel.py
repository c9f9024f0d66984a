"""Context parallelism on CPU: head-tail plan, ring attention vs full attention, DCP LSE merge."""
import torch

from vllm_torchtpu_b200.ops import reference as ref
from vllm_torchtpu_b200.parallel.dcp import dcp_local_len, dcp_local_positions, dcp_owner
from vllm_torchtpu_b200.parallel.pcp import HeadTailPlan, InProcessRing, interleaved_owner, ring_attention


def test_head_tail_plan_balances_causal_work():
    plan = HeadTailPlan(1024, 4)
    assert plan.ranges(0) == [(0, 128), (896, 1024)] and plan.ranges(3) == [(384, 512), (512, 640)]
    works = [plan.work(r) for r in range(4)]
    assert max(works) / min(works) < 1.01
    cover = torch.cat([plan.positions(r) for r in range(4)]).sort().values
    assert torch.equal(cover, torch.arange(1024))
    assert interleaved_owner(17, 4, 16) == 1 and interleaved_owner(64, 4, 16) == 0


def test_ring_attention_matches_full_causal_attention():
    torch.manual_seed(0)
    P, S, Hq, Hkv, D = 4, 96, 4, 2, 16
    q, k, v = torch.randn(S, Hq, D), torch.randn(S, Hkv, D), torch.randn(S, Hkv, D)
    scale = D ** -0.5
    s = torch.einsum("qhd,khd->hqk", q, k.repeat_interleave(2, 1)) * scale
    s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril()[None], float("-inf"))
    want = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v.repeat_interleave(2, 1))
    plan = HeadTailPlan(S, P)

    def rank_fn(r):
        pos = plan.positions(r)
        return lambda exchange: ring_attention(q[pos], pos, k[pos], v[pos], pos, scale, P, exchange)

    outs = InProcessRing(P).run([rank_fn(r) for r in range(P)])
    got = torch.empty_like(want)
    for r in range(P):
        got[plan.positions(r)] = outs[r]
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)


def test_dcp_sharding_and_merge():
    assert dcp_local_positions(10, 1, 2, 2).tolist() == [2, 3, 6, 7]
    assert [dcp_local_len(10, r, 2, 2) for r in range(2)] == [6, 4]
    assert dcp_owner(5, 4, 1) == 1
    torch.manual_seed(1)
    T, H, D, S = 3, 4, 8, 40
    q, k, v = torch.randn(T, H, D), torch.randn(S, H, D), torch.randn(S, H, D)
    full = torch.einsum("thk,khd->thd", torch.softmax(torch.einsum("thd,khd->thk", q, k), -1), v)
    outs, lses = [], []
    for r in range(4):
        pos = dcp_local_positions(S, r, 4, 2)
        s = torch.einsum("thd,khd->thk", q, k[pos])
        lses.append(torch.logsumexp(s, -1))
        outs.append(torch.einsum("thk,khd->thd", torch.softmax(s, -1), v[pos]))
    # a shard that saw no key contributes nothing
    outs.append(torch.zeros(T, H, D))
    lses.append(torch.full((T, H), float("-inf")))
    got, _ = ref.merge_attn_states(outs, lses)
    torch.testing.assert_close(got, full, rtol=1e-4, atol=1e-4)


def test_pcp_step_split_covers_every_token_once_and_balances_work():
    """The step plan of the engine's prefill context parallelism: pieces are a partition of each chunk, rank 0 owns
    the piece that ends it, causal work is balanced, short chunks and decode tokens stay replicated."""
    from types import SimpleNamespace

    import numpy as np

    from vllm_torchtpu_b200.engine.scheduler import ScheduledRequest
    from vllm_torchtpu_b200.runner.pcp_step import bind_rows, piece_bounds, split_step
    from vllm_torchtpu_b200.sampling_params import SamplingParams
    for lo, n, P in ((0, 64, 2), (37, 101, 4), (5, 16, 2)):
        b = piece_bounds(lo, n, P)
        assert b[0][0] == lo and b[-1][1] == lo + n and all(x[1] == y[0] for x, y in zip(b, b[1:]))
        assert all(hi > lo_ for lo_, hi in b) and max(hi - l for l, hi in b) - min(hi - l for l, hi in b) <= 1
        work = [sum((hi * (hi + 1) - l * (l + 1)) // 2 for l, hi in (b[r], b[2 * P - 1 - r])) for r in range(P)]
        assert max(work) / min(work) < 1.25

    def sched(rid, start, n, **sp):
        req = SimpleNamespace(request_id=rid, sampling_params=SamplingParams(**sp))
        return ScheduledRequest(req, n, start, samples=True)
    scheds = [sched("dec", 40, 1), sched("long", 64, 100), sched("short", 0, 10), sched("plp", 0, 90, prompt_logprobs=1)]
    slot_of = {"dec": 0, "long": 1, "short": 2, "plp": 3}
    bt = np.arange(4 * 32, dtype=np.int32).reshape(4, 32)            # request i owns blocks 32 i .. 32 i + 31
    seen = []
    for rank in range(2):
        local, plan = split_step(scheds, 2, rank, 16, slot_of, bt, 16, "cpu")
        assert [s.request.request_id for s in local] == ["dec", "short", "plp", "long", "long"]
        head, tail = local[3], local[4]
        assert not head.samples and tail.samples and plan.counts == [50, 50] and plan.own == 50
        seen += list(range(head.start, head.start + head.num_new_tokens))
        seen += list(range(tail.start, tail.start + tail.num_new_tokens))
        if rank == 0:
            assert tail.start + tail.num_new_tokens == 164          # the chunk's last token is on rank 0
        # the other rank's rows: positions of its two pieces, slots inside the request's own blocks
        other = split_step(scheds, 2, 1 - rank, 16, slot_of, bt, 16, "cpu")[0]
        want = [p for s in other[3:] for p in range(s.start, s.start + s.num_new_tokens)]
        assert plan.others_pos.tolist() == want
        assert plan.others_slots.tolist() == [(32 + p // 16) * 16 + p % 16 for p in want]
        assert plan.others_idx.tolist() == list(range((1 - rank) * 50, (1 - rank) * 50 + 50))
        bind_rows(plan, [local[0], local[1], local[2], head, tail], "cpu")
        assert plan.mute_rows == [3] and plan.fix_rows.tolist() == [4]
    assert sorted(seen) == list(range(64, 164))
    assert split_step(scheds[:1] + scheds[2:3], 2, 0, 16, slot_of, bt, 16, "cpu")[1] is None
