"""KV connectors on CPU: prefill engine -> decode engine hand-off, failure injection on the control
plane, pull timeout on the producer, offload store hit, signed messages."""
import numpy as np
import pytest
import torch

from vllm_torchtpu_b200 import SamplingParams
from vllm_torchtpu_b200.engine.llm import LLM
from vllm_torchtpu_b200.kv_transfer import base
from vllm_torchtpu_b200.kv_transfer.transport import InProcessChannel, LocalTransport, TcpChannel


def _prompts():
    rng = np.random.RandomState(3)
    return [rng.randint(0, 1024, size=n).tolist() for n in (20, 33, 50)]


def _llm(role, engine_id, **extra):
    cfg = {"kv_connector": "B200P2PConnector", "kv_role": role, "engine_id": engine_id,
           "kv_connector_extra_config": {"transport": "local", "channel": "inproc"}}
    cfg.update(extra)
    return LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, kv_transfer_config=cfg,
               init_dist=False)


def _decode_with_params(dec, prompts, params, n=6):
    sp = SamplingParams(max_tokens=n, ignore_eos=True)
    ids = [dec.engine.add_request(p, sp, kv_transfer_params=kp) for p, kp in zip(prompts, params)]
    dec.engine.run_until_done()
    return [dec.engine.scheduler.requests[i] for i in ids]


def test_prefill_decode_handoff_matches_monolithic():
    mono = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    want = [o.outputs[0].token_ids for o in mono.generate(_prompts(), SamplingParams(max_tokens=6, ignore_eos=True))]
    pre, dec = _llm("kv_producer", "P0"), _llm("kv_consumer", "D0")
    outs = pre.generate(_prompts(), SamplingParams(max_tokens=1, ignore_eos=True))
    params = [o.kv_transfer_params for o in outs]
    assert all(p and p["remote_engine_id"] == "P0" and p["remote_block_ids"] for p in params)
    free_before = pre.engine.scheduler.kv.pool.num_free_blocks
    reqs = _decode_with_params(dec, _prompts(), params)
    assert [r.output_token_ids for r in reqs] == want
    # decode engine computed only the last prompt token itself
    assert all(r.num_cached_tokens == len(p) - 1 for r, p in zip(reqs, _prompts()))
    # producer frees the blocks once the consumer reported the pull
    pre.engine.step()
    for rid in pre.engine.connector.worker.get_finished_sending():
        pre.engine.scheduler.free_delayed(rid)
    assert pre.engine.scheduler.kv.pool.num_free_blocks > free_before
    st = dec.engine.connector.shared.stats.snapshot()
    assert st["loads_ok"] == 3 and st["loads_failed"] == 0


def test_failed_pull_falls_back_to_recompute():
    pre, dec = _llm("kv_producer", "P1"), _llm("kv_consumer", "D1")
    p = _prompts()[:1]
    params = [o.kv_transfer_params for o in pre.generate(p, SamplingParams(max_tokens=1, ignore_eos=True))]
    mono = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    want = mono.generate(p, SamplingParams(max_tokens=6, ignore_eos=True))[0].outputs[0].token_ids
    dec.engine.connector.worker.channel.drop_next = 1          # the handshake message is lost
    reqs = _decode_with_params(dec, p, params)
    assert reqs[0].output_token_ids == want and reqs[0].error is None
    assert dec.engine.connector.shared.stats.snapshot()["loads_failed"] == 1


def test_failed_pull_with_fail_policy_reports_error():
    pre, dec = _llm("kv_producer", "P2"), _llm("kv_consumer", "D2", kv_load_failure_policy="fail")
    p = _prompts()[:1]
    params = [o.kv_transfer_params for o in pre.generate(p, SamplingParams(max_tokens=1, ignore_eos=True))]
    params[0]["remote_engine_id"] = "nobody"
    reqs = _decode_with_params(dec, p, params)
    assert reqs[0].error and "kv_load_failed" in reqs[0].error


def test_unpulled_blocks_expire(monkeypatch):
    monkeypatch.setenv("B200_P2P_WAIT_PULL_TIMEOUT", "0.0")
    from vllm_torchtpu_b200 import envs
    envs.reset()
    pre = _llm("kv_producer", "P3")
    pre.generate(_prompts()[:1], SamplingParams(max_tokens=1, ignore_eos=True))
    free0 = pre.engine.scheduler.kv.pool.num_free_blocks
    pre.engine.step()                                    # the retire path collects expired sends
    for rid in pre.engine.connector.worker.get_finished_sending():
        pre.engine.scheduler.free_delayed(rid)
    assert pre.engine.connector.shared.stats.snapshot()["sends_expired"] == 1
    assert pre.engine.scheduler.kv.pool.num_free_blocks >= free0
    assert not pre.engine.scheduler._delayed_blocks


def test_signed_messages_and_tcp_channel():
    raw = base.sign_message({"op": "PING"}, b"k1")
    assert base.verify_message(raw, b"k1") == {"op": "PING"}
    with pytest.raises(PermissionError):
        base.verify_message(raw, b"other-key")
    with pytest.raises(PermissionError):
        base.verify_message(raw[:-2] + b"x}", b"k1")
    ch = TcpChannel("127.0.0.1", 0, lambda m: {"ok": True, "echo": m["op"]})
    try:
        assert ch.request(ch.address(), {"op": "PING"}, 2.0) == {"ok": True, "echo": "PING"}
        with pytest.raises(OSError):
            ch.request(("127.0.0.1", 1), {"op": "PING"}, 0.5)
    finally:
        ch.close()


def test_offload_store_reuses_prefix():
    cfg = {"kv_connector": "B200OffloadingConnector", "kv_connector_extra_config": {"num_blocks": 32}}
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, kv_transfer_config=cfg, init_dist=False)
    p = _prompts()[2]
    sp = SamplingParams(max_tokens=4, ignore_eos=True)
    a = llm.generate([p], sp)[0]
    st0 = llm.engine.connector.store.stats()
    assert st0["stored"] >= 3
    b = llm.generate([p], sp)[0]
    assert a.outputs[0].token_ids == b.outputs[0].token_ids
    assert b.num_cached_tokens == 48                     # three full blocks came back from the host store
    # eviction keeps working when the slab is full
    for i in range(12):
        llm.generate([[(7 * i + j) % 1000 for j in range(64)]], sp)
    assert llm.engine.connector.store.stats()["evictions"] > 0


def test_offload_store_keeps_lora_and_base_kv_apart_and_releases_pins():
    """KV computed under a LoRA adapter must not be served to a base-model request with the same
    tokens (k_proj / v_proj are adapter targets), and a request whose admission fails after a host
    hit gives its pinned slots back."""
    from types import SimpleNamespace
    from vllm_torchtpu_b200.kv_transfer.offload import HostKVStore, OffloadSchedulerHalf, block_hashes
    store = HostKVStore(1, (2, 1, 16, 8), torch.float32, 16, pin=False)
    half = OffloadSchedulerHalf(store, 16)
    toks = list(range(50))

    def req(rid, lora):
        return SimpleNamespace(request_id=rid, all_token_ids=toks, num_tokens=len(toks), num_computed_tokens=48,
                               error=None, sampling_params=SimpleNamespace(lora_name=lora))
    # a finished adapter request saves three blocks
    delay, _ = half.request_finished(req("a", "adapter-1"), [5, 6, 7])
    assert delay
    for h in half._saves[0][1]:
        store.commit(store.reserve(h), True)
    assert store.stats()["pinned"] == 0
    assert block_hashes(toks, 16, 3, ("adapter-1",)) != block_hashes(toks, 16, 3)
    assert half.get_num_new_matched_tokens(req("base", None), 0) == (0, False)
    assert half.get_num_new_matched_tokens(req("other", "adapter-2"), 0) == (0, False)
    n, _ = half.get_num_new_matched_tokens(req("same", "adapter-1"), 0)
    assert n == 48 and store.stats()["pinned"] == 3
    # the scheduler could not allocate: the pins are returned; a second query does not stack pins
    half.request_not_admitted(req("same", "adapter-1"))
    assert store.stats()["pinned"] == 0
    half.get_num_new_matched_tokens(req("same", "adapter-1"), 0)
    half.get_num_new_matched_tokens(req("same", "adapter-1"), 0)
    assert store.stats()["pinned"] == 3
    half.update_state_after_alloc(req("same", "adapter-1"), [1, 2, 3], 48)
    store.unpin(half._loads[0][1])
    assert store.stats()["pinned"] == 0
    store.close()


# ---- engines of different tensor-parallel degree --------------------------------------------------------
def _rank_pool(full, tp, rank, H):
    """One rank's slice of full caches [N, 2, H, bs, D] (heads replicated when tp > H)."""
    h = max(1, H // tp)
    lo = (rank // max(1, tp // H)) * h
    return [t[:, :, lo:lo + h].contiguous() for t in full]


@pytest.mark.parametrize("H,tp_p,tp_c", [(4, 2, 1), (4, 1, 2), (8, 4, 2), (8, 2, 4), (2, 4, 1), (2, 1, 4), (4, 2, 2)])
def test_reshard_plan_moves_head_ranges_between_tp_degrees(H, tp_p, tp_c):
    from vllm_torchtpu_b200.kv_transfer.reshard import KVGeometry, plan_pull, readers_of
    from vllm_torchtpu_b200.kv_transfer.transport import PoolInfo, copy_block_spans
    torch.manual_seed(0)
    N, bs, D, L = 6, 4, 8, 2
    full = [torch.randn(N, 2, H, bs, D).to(torch.bfloat16) for _ in range(L)]
    prod = [PoolInfo(f"p{r}", _rank_pool(full, tp_p, r, H)) for r in range(tp_p)]
    src_ids, dst_ids = [4, 1, 3], [0, 5, 2]
    reads = {r: set() for r in range(tp_p)}
    for cr in range(tp_c):
        want = _rank_pool(full, tp_c, cr, H)
        dst = PoolInfo("c", [torch.zeros_like(t) for t in want])
        cg = KVGeometry.of_cache(dst.layers[0], tp_c, cr, H)
        pg = KVGeometry.of_cache(prod[0].layers[0], tp_p, 0, H)
        plan = plan_pull(cg, pg)
        for pr, span in plan:
            copy_block_spans(prod[pr], dst, src_ids, dst_ids, span)
            reads[pr].add(cr)
        for got, w in zip(dst.layers, want):
            torch.testing.assert_close(got[dst_ids], w[src_ids])
            untouched = [i for i in range(N) if i not in dst_ids]
            assert not got[untouched].any()
    # the producer's view of who reads from it agrees with what the consumers planned
    for pr in range(tp_p):
        pg = KVGeometry.of_cache(prod[pr].layers[0], tp_p, pr, H)
        proto = KVGeometry.of_cache(_rank_pool(full, tp_c, 0, H)[0], tp_c, 0, H)
        assert set(readers_of(pg, tp_c, proto)) == reads[pr]


def test_reshard_plan_of_latent_caches_and_mismatches():
    from vllm_torchtpu_b200.kv_transfer.reshard import KVGeometry, plan_pull
    lat = torch.zeros(4, 16, 72, dtype=torch.bfloat16)
    c = KVGeometry.of_cache(lat, 4, 3, 1)
    p = KVGeometry.of_cache(lat, 2, 0, 1)
    (pr, span), = plan_pull(c, p)
    assert pr == 1 and span.nbytes == 16 * 72 * 2 and span.chunks == 1
    gqa = KVGeometry.of_cache(torch.zeros(4, 2, 2, 16, 8, dtype=torch.bfloat16), 1, 0, 2)
    with pytest.raises(ValueError):
        plan_pull(gqa, p)
    with pytest.raises(ValueError):
        plan_pull(gqa, KVGeometry(1, 0, 4, gqa.head_bytes, 2 * gqa.block_bytes))


@pytest.mark.parametrize("tp_p,tp_c", [(2, 1), (1, 2)])
def test_worker_halves_pull_across_tp_degrees_and_producers_wait_for_all_readers(tp_p, tp_c):
    """Worker halves of a producer engine and a consumer engine with different degrees, one pair per rank in
    this process: every consumer rank assembles its blocks from the producer ranks that hold its heads, and a
    producer rank releases the transfer only when all its readers have acknowledged."""
    from vllm_torchtpu_b200.kv_transfer.p2p_connector import P2PWorkerHalf, _Shared, rank_engine_id
    from vllm_torchtpu_b200.kv_transfer.reshard import KVGeometry
    torch.manual_seed(1)
    H, N, bs, D, L = 4, 8, 4, 8, 2
    full = [torch.randn(N, 2, H, bs, D).to(torch.bfloat16) for _ in range(L)]
    tag = f"rs{tp_p}{tp_c}"

    def half(base, tp, rank, layers, role):
        eid = rank_engine_id(base, rank, tp)
        tr = LocalTransport(eid)
        tr.register_pool(layers)
        sh = _Shared(eid, role, bs, "recompute", KVGeometry.of_cache(layers[0], tp, rank, H), base)
        return sh, P2PWorkerHalf(sh, tr, lambda h, eid=eid: InProcessChannel(eid, h))
    prods = [half(tag + "P", tp_p, r, _rank_pool(full, tp_p, r, H), base.KVConnectorRole.PRODUCER)
             for r in range(tp_p)]
    cons = [half(tag + "C", tp_c, r, [torch.zeros_like(t) for t in _rank_pool(full, tp_c, r, H)],
                 base.KVConnectorRole.CONSUMER) for r in range(tp_c)]
    remote, local = [5, 2, 7], [1, 3, 0]
    for sh, _ in prods:
        sh.pending_sends["u1"] = base.SendMeta("req", "u1", remote, 12, base.now() + 60)
    geom = prods[0][0].geometry.to_dict()
    for cr, (sh, w) in enumerate(cons):
        lm = base.LoadMeta("req", "u1", tag + "P", remote, local, 12, remote_geometry=geom)
        w.start_load_kv(base.ConnectorMetadata([], [lm], []))
        assert w.get_finished_recving() == ["req"] and not sh.load_failed
        for got, want in zip(LocalTransport._pools[sh.engine_id].layers, _rank_pool(full, tp_c, cr, H)):
            torch.testing.assert_close(got[local], want[remote])
        done = [bool(pw.get_finished_sending()) for _, pw in prods]
        if cr < tp_c - 1 and tp_p == 1:
            assert done == [False]              # the second reader has not reported yet
    assert all(not sh.pending_sends for sh, _ in prods)
    for _, w in prods + cons:
        w.close()


# ---- controller -------------------------------------------------------------------------------------------
def test_controller_registry_heartbeats_picks_and_unreachable_marking():
    from vllm_torchtpu_b200.kv_transfer.controller import ControllerClient, KVController
    now = [100.0]
    ctl = KVController("127.0.0.1", 0, ttl_s=5.0, clock=lambda: now[0])
    try:
        cl = ControllerClient(ctl.address())
        assert cl.pick("prefill") is None
        assert not cl.register(engine_id="", role="prefill")["ok"]
        for eid, role, url in (("p0", "prefill", "http://p0"), ("p1", "prefill", "http://p1"),
                               ("d0", "decode", "http://d0"), ("b0", "both", "http://b0")):
            assert cl.register(engine_id=eid, role=role, http_url=url, tp=2, model="m")["ok"]
        cl.heartbeat("p0", {"running": 4, "waiting": 3, "free_blocks": 10})
        cl.heartbeat("p1", {"running": 1, "waiting": 0, "free_blocks": 900})
        cl.heartbeat("b0", {"running": 9, "waiting": 9})
        assert cl.pick("prefill")["engine_id"] == "p1"              # least loaded
        assert cl.pick("prefill", exclude=["p1"])["engine_id"] == "p0"
        assert cl.pick("decode")["engine_id"] == "d0"
        assert cl.pick("decode", model="other") is None
        # a reported engine is skipped until it answers again
        cl.report_unreachable("p1", reporter="d0")
        assert cl.pick("prefill")["engine_id"] == "p0"
        cl.heartbeat("p1", {"running": 0, "waiting": 0})
        assert cl.pick("prefill")["engine_id"] == "p1"
        # no heartbeat within the time-to-live: not alive, not picked
        now[0] += 6.0
        cl.heartbeat("p0", {"running": 0, "waiting": 0})
        assert cl.pick("prefill")["engine_id"] == "p0"
        alive = {e["engine_id"]: e["alive"] for e in cl.list("prefill")}
        assert alive == {"p0": True, "p1": False, "b0": False}
        # a restarted controller forgets the engines; the next heartbeat registers again
        ctl.engines.clear()
        cl._engine = {"engine_id": "p0", "role": "prefill", "http_url": "http://p0"}
        assert cl.heartbeat("p0", {"running": 0})["ok"] and cl.pick("prefill")["engine_id"] == "p0"
        cl.deregister("p0")
        assert cl.pick("prefill") is None
    finally:
        ctl.close()


def test_proxy_picks_from_the_controller_and_reports_dead_instances():
    """The proxy asks the controller for instances; a prefill instance that cannot be connected to is reported
    and the retry goes to the other one."""
    import asyncio
    from vllm_torchtpu_b200.kv_transfer.controller import ControllerClient, KVController
    from vllm_torchtpu_b200.kv_transfer.proxy import build_proxy_app
    ctl = KVController("127.0.0.1", 0, ttl_s=60.0)
    try:
        cl = ControllerClient(ctl.address())
        cl.register(engine_id="dead", role="prefill", http_url="http://dead")
        cl.register(engine_id="live", role="prefill", http_url="http://live")
        cl.register(engine_id="dec", role="decode", http_url="http://dec")
        cl.heartbeat("live", {"running": 5})           # the dead one looks idle, so it is picked first
        posts = []

        class Resp:
            def __init__(self, data): self.status, self._d = 200, data
            async def json(self): return self._d
            async def text(self): return ""
            async def __aenter__(self): return self
            async def __aexit__(self, *a): return False

        class Client:
            async def __aenter__(self): return self
            async def __aexit__(self, *a): return False

            def post(self, url, json=None):
                posts.append(url)
                if url.startswith("http://dead"):
                    raise ConnectionError("Cannot connect to host dead")
                if url.startswith("http://live"):
                    return Resp({"kv_transfer_params": {"uuid": "u", "remote_block_ids": [1]}})
                return Resp({"choices": [{"text": "ok"}], "seen": json.get("kv_transfer_params")})
        app = build_proxy_app([], [], retries=2, client_factory=Client, controller=cl)
        from starlette.testclient import TestClient
        r = TestClient(app).post("/v1/completions", json={"prompt": "x", "max_tokens": 4})
        assert r.status_code == 200 and r.json()["seen"]["uuid"] == "u"
        assert posts[0].startswith("http://dead") and posts[1].startswith("http://live") and posts[2].startswith("http://dec")
        assert app.state.counts["reported_unreachable"] == 1
        assert {e["engine_id"]: e["alive"] for e in cl.list("prefill")}["dead"] is False
    finally:
        ctl.close()


def test_engines_register_with_the_controller_and_report_load():
    from vllm_torchtpu_b200.kv_transfer.controller import ControllerClient, KVController
    ctl = KVController("127.0.0.1", 0, ttl_s=60.0)
    try:
        addr = "%s:%d" % ctl.address()
        extra = {"transport": "local", "channel": "inproc", "controller": addr, "heartbeat_s": 0.05}
        pre = _llm("kv_producer", "PC", kv_connector_extra_config={**extra, "http_url": "http://pre:8100"})
        dec = _llm("kv_consumer", "DC", kv_connector_extra_config={**extra, "http_url": "http://dec:8200"})
        cl = ControllerClient(ctl.address())
        got = {e["engine_id"]: e for e in cl.list()}
        assert got["PC"]["role"] == "prefill" and got["DC"]["role"] == "decode"
        assert got["PC"]["http_url"] == "http://pre:8100" and got["PC"]["geometry"]["num_kv_heads"] > 0
        assert cl.pick("prefill")["engine_id"] == "PC" and cl.pick("decode")["engine_id"] == "DC"
        import time
        deadline = time.time() + 5
        while time.time() < deadline and "free_blocks" not in {e["engine_id"]: e for e in cl.list()}["PC"]["load"]:
            time.sleep(0.05)
        assert {e["engine_id"]: e for e in cl.list()}["PC"]["load"]["free_blocks"] > 0     # the scheduler's counts
        pre.engine.connector.controller.stop()
        dec.engine.connector.controller.stop()
    finally:
        ctl.close()
