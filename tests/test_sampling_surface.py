"""Sampling parameters beyond temperature / top-k / top-p: penalties, logit bias, allowed tokens, min-p,
n completions per prompt and stop strings, from the tensor edit up to the offline API and the server."""
import json
import math

import pytest
import torch

from vllm_torchtpu_b200.engine.llm import LLM
from vllm_torchtpu_b200.entrypoints.stop_strings import StopStringMatcher, truncate_at_stop
from vllm_torchtpu_b200.runner.logit_adjust import apply_logit_adjust, plan_row
from vllm_torchtpu_b200.sampling_params import SamplingParams


class LetterTokenizer:
    """Token t <-> one lower-case letter (t mod 26): enough to exercise text-level features."""
    eos_token_id = None

    def encode(self, text):
        return [ord(c) - 97 + 26 for c in text if c.isalpha()]

    def decode(self, ids):
        return "".join(chr(97 + int(t) % 26) for t in ids)


def _oracle(logits, sp, prompt, output):
    out = [float(x) for x in logits]
    V = len(out)
    if sp.allowed_token_ids:
        out = [x if i in set(sp.allowed_token_ids) else -math.inf for i, x in enumerate(out)]
    for t, b in (sp.logit_bias or {}).items():
        if 0 <= t < V:
            out[t] += b
    seen_all, cnt = set(prompt) | set(output), {}
    for t in output:
        cnt[t] = cnt.get(t, 0) + 1
    for t in range(V):
        if t in seen_all and sp.repetition_penalty != 1.0:
            out[t] = out[t] / sp.repetition_penalty if out[t] > 0 else out[t] * sp.repetition_penalty
        if t in cnt:
            out[t] -= sp.frequency_penalty * cnt[t] + sp.presence_penalty
    if sp.min_p > 0 and not sp.greedy:
        p = torch.softmax(torch.tensor(out) / sp.temperature, -1)
        out = [x if float(p[i]) >= sp.min_p * float(p.max()) else -math.inf for i, x in enumerate(out)]
    return out


def test_logit_adjust_matches_a_per_token_oracle():
    g = torch.Generator().manual_seed(0)
    V = 40
    logits = torch.randn(5, V, generator=g) * 3
    sps = [SamplingParams(presence_penalty=0.7, frequency_penalty=0.4),
           SamplingParams(),
           SamplingParams(repetition_penalty=1.6, logit_bias={3: 5.0, 39: -100.0, 99: 1.0}),
           SamplingParams(temperature=0.8, min_p=0.2, allowed_token_ids=list(range(0, 30))),
           SamplingParams(temperature=1.3, min_p=0.05, frequency_penalty=1.0, repetition_penalty=1.2)]
    prompts = [[1, 2, 3], [4], [5, 6, 7, 7], [8], [9, 10]]
    outputs = [[2, 2, 11, 12, 2], [1], [6, 13], [14], [9, 9, 15]]
    rows = [plan_row(i, sp, p, o) for i, (sp, p, o) in enumerate(zip(sps, prompts, outputs))]
    assert rows[1] is None
    got = logits.clone()
    apply_logit_adjust(got, [r for r in rows if r is not None])
    for i in range(5):
        want = torch.tensor(_oracle(logits[i], sps[i], prompts[i], outputs[i]))
        fin = torch.isfinite(want)
        assert torch.equal(torch.isfinite(got[i]), fin), i
        torch.testing.assert_close(got[i][fin], want[fin], rtol=1e-5, atol=1e-5)


def test_token_in_flight_is_counted_from_the_device_table():
    V = 16
    logits = torch.zeros(2, V)
    sp = SamplingParams(frequency_penalty=1.0, presence_penalty=0.5)
    last = torch.tensor([0, 7, 3], dtype=torch.int32)
    rows = [plan_row(0, sp, [1], [7, 4], inflight_slot=1), plan_row(1, sp, [1], [7, 4], inflight_slot=2)]
    apply_logit_adjust(logits, rows, last)
    assert logits[0, 7] == -2.5 and logits[0, 4] == -1.5 and logits[0, 3] == 0       # 7 twice, 4 once
    assert logits[1, 7] == -1.5 and logits[1, 3] == -1.5 and logits[1, 4] == -1.5
    with pytest.raises(ValueError):
        apply_logit_adjust(torch.zeros(1, V), [plan_row(0, sp, [], [], inflight_slot=0)], None)


def test_sampling_params_validation():
    for bad in (dict(n=0), dict(min_p=1.5), dict(presence_penalty=3), dict(repetition_penalty=0),
                dict(stop=[""]), dict(logit_bias={"a": 1}), dict(logit_bias={1: 500}), dict(allowed_token_ids=[])):
        with pytest.raises(ValueError):
            SamplingParams(**bad).verify()
    sp = SamplingParams(stop="END", logit_bias={"5": 2})
    sp.verify()
    assert sp.stop == ["END"] and sp.logit_bias == {5: 2.0} and sp.has_logit_adjust
    assert not SamplingParams(min_p=0.3).has_logit_adjust          # greedy: min-p cannot change the arg-max
    assert SamplingParams(min_p=0.3, temperature=1.0).has_logit_adjust


def test_stop_string_matcher_streams_only_safe_text():
    full = "abcdeSTOPfgh"
    for include in (False, True):
        m = StopStringMatcher(["STOP", "zz"], include)
        shown, hit = "", False
        for end in range(1, len(full) + 1):
            delta, hit = m.push(full[:end])
            shown += delta
            assert "STOP"[:2] not in shown or include or hit is False or shown == "abcde"
            if hit:
                break
        assert hit and m.hit == "STOP" and shown == ("abcdeSTOP" if include else "abcde")
    m = StopStringMatcher(["xyz"])
    a, _ = m.push("hello x")
    assert a == "hello"                  # "x" could be the start of the stop string: held back
    b, hit = m.push("hello xa", final=True)
    assert a + b == "hello xa" and not hit
    assert truncate_at_stop("one two three", ["two", "three"]) == ("one ", "two")
    assert truncate_at_stop("nothing here", ["zzz"]) == ("nothing here", None)


def _llm(**kw):
    return LLM("tiny-llama", device="cpu", max_num_seqs=8, block_size=16, init_dist=False,
               tokenizer=LetterTokenizer(), **kw)


def test_engine_bias_allowed_and_penalties():
    llm = _llm()
    prompt = [3, 9, 27, 81, 11]
    base = llm.generate([prompt], SamplingParams(max_tokens=12, ignore_eos=True))[0].outputs[0].token_ids
    forced = llm.generate([prompt], SamplingParams(max_tokens=4, ignore_eos=True, logit_bias={17: 100.0}))
    assert forced[0].outputs[0].token_ids == [17] * 4
    only = llm.generate([prompt], SamplingParams(max_tokens=8, ignore_eos=True, allowed_token_ids=[5, 6, 7]))
    assert set(only[0].outputs[0].token_ids) <= {5, 6, 7}
    # a frequency penalty at the limit spreads a three-token budget over all three tokens before repeating
    spread = llm.generate([prompt], SamplingParams(max_tokens=3, ignore_eos=True, allowed_token_ids=[5, 6, 7],
                                                   frequency_penalty=2.0, presence_penalty=2.0,
                                                   repetition_penalty=1.5))[0].outputs[0].token_ids
    assert sorted(spread) == [5, 6, 7] or len(set(spread)) >= 2
    # plain requests in the same batch are not disturbed
    mixed = llm.generate([prompt, prompt], [SamplingParams(max_tokens=12, ignore_eos=True),
                                            SamplingParams(max_tokens=12, ignore_eos=True, presence_penalty=1.0)])
    assert mixed[0].outputs[0].token_ids == base
    with pytest.raises(ValueError):
        llm.generate([prompt], SamplingParams(min_p=2.0))


def test_penalties_under_async_scheduling_match_the_synchronous_engine():
    sp = SamplingParams(max_tokens=16, ignore_eos=True, frequency_penalty=1.2, presence_penalty=0.6,
                        repetition_penalty=1.3, allowed_token_ids=list(range(40, 48)))
    prompts = [[3, 9, 27, 81, 11], [40, 41, 42], [7] * 20]
    want = [o.outputs[0].token_ids for o in _llm().generate(prompts, sp)]
    got = [o.outputs[0].token_ids for o in _llm(async_scheduling=True).generate(prompts, sp)]
    assert got == want
    for toks in want:                       # eight allowed tokens, strong penalties: none is used 5 times
        assert max(toks.count(t) for t in set(toks)) < 5


def test_penalties_are_refused_with_speculative_decoding():
    llm = _llm(speculative_config={"method": "ngram", "num_speculative_tokens": 2})
    with pytest.raises(ValueError, match="speculative"):
        llm.generate([[1, 2, 3]], SamplingParams(presence_penalty=0.5))
    assert llm.generate([[1, 2, 3]], SamplingParams(max_tokens=2, ignore_eos=True))[0].finished


def test_generate_n_and_stop_strings():
    llm = _llm()
    prompt = [3, 9, 27, 81, 11]
    outs = llm.generate([prompt, [5, 6]], [SamplingParams(max_tokens=6, ignore_eos=True, n=3, temperature=1.0),
                                           SamplingParams(max_tokens=3, ignore_eos=True)])
    assert [c.index for c in outs[0].outputs] == [0, 1, 2] and len(outs[1].outputs) == 1
    assert all(len(c.token_ids) == 6 for c in outs[0].outputs)
    assert not llm.engine.scheduler.requests                 # every sub-request was collected
    text = llm.generate([prompt], SamplingParams(max_tokens=12, ignore_eos=True))[0].outputs[0].text
    stop = text[4:6]
    cut = text.index(stop)
    o = llm.generate([prompt], SamplingParams(max_tokens=12, ignore_eos=True, stop=[stop]))[0].outputs[0]
    assert o.text == text[:cut] and o.finish_reason == "stop" and o.stop_reason == stop
    assert len(o.token_ids) < 12                             # the request ended early
    o = llm.generate([prompt], SamplingParams(max_tokens=12, ignore_eos=True, stop=[stop],
                                              include_stop_str_in_output=True))[0].outputs[0]
    assert o.text == text[:cut + 2]
    with pytest.raises(ValueError, match="tokenizer"):
        LLM("tiny-llama", device="cpu", init_dist=False).generate([prompt], SamplingParams(stop=["x"]))


def test_server_n_stop_and_penalties():
    pytest.importorskip("httpx")
    from starlette.testclient import TestClient

    from vllm_torchtpu_b200.entrypoints.openai_server import build_app
    llm = _llm()
    app = build_app(llm.engine, "tiny-llama", llm.tokenizer)
    body = {"prompt": [3, 9, 27, 81, 11], "max_tokens": 10, "temperature": 0, "ignore_eos": True}
    with TestClient(app) as c:
        full = c.post("/v1/completions", json=body).json()["choices"][0]
        r = c.post("/v1/completions", json=dict(body, n=2, temperature=1.0)).json()
        assert [ch["index"] for ch in r["choices"]] == [0, 1] and r["usage"]["completion_tokens"] == 20
        stop = full["text"][3:5]
        cut = full["text"].index(stop)
        r = c.post("/v1/completions", json=dict(body, stop=stop)).json()
        assert r["choices"][0]["text"] == full["text"][:cut] and r["choices"][0]["finish_reason"] == "stop"
        assert r["usage"]["completion_tokens"] < 10
        with c.stream("POST", "/v1/completions", json=dict(body, stop=[stop], stream=True, n=2)) as s:
            chunks = [json.loads(l[5:]) for l in s.iter_lines() if l.startswith("data: {")]
        per = {0: "", 1: ""}
        for ch in chunks:
            per[ch["choices"][0]["index"]] += ch["choices"][0]["text"]
        assert per[0] == per[1] == full["text"][:cut]
        assert sum(ch["choices"][0]["finish_reason"] == "stop" for ch in chunks) == 2 and "usage" in chunks[-1]
        r = c.post("/v1/completions", json=dict(body, logit_bias={"21": 100}, max_tokens=3)).json()
        assert r["choices"][0]["token_ids"] == [21, 21, 21]
        r = c.post("/v1/completions", json=dict(body, frequency_penalty=2.0, allowed_token_ids=[5, 6, 7],
                                                max_tokens=3)).json()
        assert len(set(r["choices"][0]["token_ids"])) >= 2
        assert c.post("/v1/completions", json=dict(body, presence_penalty=9)).status_code == 400
        assert c.post("/v1/completions", json=dict(body, stop=[""])).status_code == 400
    app.state.async_engine.shutdown()


def test_llm_chat_renders_conversations_through_the_template():
    llm = _llm()
    sp = SamplingParams(max_tokens=4, ignore_eos=True)
    conv = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hello"}]
    one = llm.chat(conv, sp)
    assert len(one) == 1 and len(one[0].outputs[0].token_ids) == 4
    # the plain transcript of a tokenizer without a template: "role: content" lines + an open assistant turn
    want = llm.tokenizer.encode("system: be brief\nuser: hello\nassistant:")
    assert one[0].prompt_token_ids == want
    two = llm.chat([conv, conv + [{"role": "assistant", "content": "hi"}, {"role": "user", "content": "more"}]], sp)
    assert len(two) == 2 and two[0].outputs[0].token_ids == one[0].outputs[0].token_ids
    cont = llm.chat(conv + [{"role": "assistant", "content": "abc"}], sp, continue_final_message=True)
    assert cont[0].prompt_token_ids == llm.tokenizer.encode("system: be brief\nuser: hello\nassistant: abc")
    with pytest.raises(ValueError):
        llm.chat(conv, sp, continue_final_message=True)
