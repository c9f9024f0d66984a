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
