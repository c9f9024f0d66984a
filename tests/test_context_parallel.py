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
