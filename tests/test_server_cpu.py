"""OpenAI server routes on a CPU engine (in-process ASGI client), and the P/D flow through two servers' apps."""
import numpy as np
import pytest

httpx = pytest.importorskip("httpx")
from starlette.testclient import TestClient

from vllm_torchtpu_b200.engine.llm import LLM
from vllm_torchtpu_b200.entrypoints.openai_server import build_app


@pytest.fixture(scope="module")
def client():
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    app = build_app(llm.engine, "tiny-llama", None)
    with TestClient(app) as c:
        yield c
    app.state.async_engine.shutdown()


def test_completions_models_metrics(client):
    r = client.post("/v1/completions", json={"prompt": [1, 2, 3, 4, 5], "max_tokens": 4, "temperature": 0,
                                             "ignore_eos": True})
    assert r.status_code == 200
    body = r.json()
    assert len(body["choices"][0]["token_ids"]) == 4 and body["usage"]["completion_tokens"] == 4
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny-llama"
    assert "b200_generation_tokens_total" in client.get("/metrics").text
    assert client.get("/health").json()["status"] == "ok"


def test_streaming_and_chat(client):
    with client.stream("POST", "/v1/completions", json={"prompt": [7, 8, 9], "max_tokens": 3, "temperature": 0,
                                                       "ignore_eos": True, "stream": True}) as r:
        lines = [l for l in r.iter_lines() if l.startswith("data:")]
    assert lines[-1] == "data: [DONE]" and len(lines) >= 2
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}]})
    assert r.status_code == 400          # no tokenizer: text prompts are rejected with a clear error


def test_bad_requests(client):
    assert client.post("/v1/completions", json={"prompt": [1, 2], "seed": 3}).status_code == 400
    assert client.post("/v1/completions", json={"prompt": [1] * 5000, "max_tokens": 4}).status_code == 500


def test_completion_logprobs_and_prompt_logprobs(client):
    r = client.post("/v1/completions", json={"prompt": [1, 2, 3, 4, 5, 6], "max_tokens": 3, "temperature": 0,
                                             "ignore_eos": True, "logprobs": 2, "prompt_logprobs": 1})
    assert r.status_code == 200
    ch = r.json()["choices"][0]
    lp = ch["logprobs"]
    assert lp["token_ids"] == ch["token_ids"] and len(lp["token_logprobs"]) == 3
    assert all(len(t) == 2 for t in lp["top_logprobs"]) and all(v <= 0 for v in lp["token_logprobs"])
    plp = ch["prompt_logprobs"]
    assert len(plp) == 6 and plp[0] is None and [e["token_id"] for e in plp[1:]] == [2, 3, 4, 5, 6]


def test_multimodal_items_over_http():
    """Image patches in the request body reach the vision encoder; without one the request fails cleanly."""
    from vllm_torchtpu_b200.layers.vision import VisionConfig
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    hidden = llm.engine.cfg.model.hidden_size
    llm.engine.enable_vision(VisionConfig(patch_dim=12, hidden_size=32, num_heads=2, depth=1, merge=4,
                                          out_hidden_size=hidden))
    app = build_app(llm.engine, "tiny-llama", None)
    rng = np.random.RandomState(0)
    prompt = list(range(1, 25))
    body = {"prompt": prompt, "max_tokens": 3, "temperature": 0, "ignore_eos": True}
    with TestClient(app) as c:
        plain = c.post("/v1/completions", json=body).json()["choices"][0]["token_ids"]
        item = {"patches": rng.randn(16, 12).tolist(), "offset": 4}
        r = c.post("/v1/completions", json=dict(body, mm_items=[item]))
        assert r.status_code == 200 and len(r.json()["choices"][0]["token_ids"]) == 3
        assert r.json()["choices"][0]["token_ids"] != plain
        assert c.post("/v1/completions", json=dict(body, mm_items=[{"offset": 1}])).status_code == 400
        bad = dict(body, mm_items=[dict(item, offset=23)])          # runs past the prompt
        assert c.post("/v1/completions", json=bad).status_code == 500
    app.state.async_engine.shutdown()


def test_embeddings_and_lora_adapter_routes(client, tmp_path):
    import torch
    from safetensors.torch import save_file
    r = client.post("/v1/embeddings", json={"input": [[1, 2, 3, 4], [9, 8, 7]], "pooling": "mean"})
    assert r.status_code == 200
    data = r.json()["data"]
    assert len(data) == 2 and abs(sum(a * a for a in data[0]["embedding"]) - 1.0) < 1e-3
    assert r.json()["usage"]["prompt_tokens"] == 7
    assert client.post("/v1/embeddings", json={"input": [1, 2], "pooling": "median"}).status_code == 400
    body = {"prompt": [3, 1, 4, 1, 5, 9, 2, 6], "max_tokens": 4, "temperature": 0, "ignore_eos": True}
    base = client.post("/v1/completions", json=body).json()["choices"][0]["token_ids"]
    g = torch.Generator().manual_seed(0)
    tensors = {}
    for li in range(2):
        k = f"model.layers.{li}.mlp.down_proj"
        tensors[k + ".lora_A.weight"] = torch.randn(4, 512, generator=g) * 0.5
        tensors[k + ".lora_B.weight"] = torch.randn(256, 4, generator=g) * 0.5
    path = str(tmp_path / "ad.safetensors")
    save_file(tensors, path)
    r = client.post("/v1/load_lora_adapter", json={"lora_name": "ad", "lora_path": path, "alpha": 32})
    assert r.status_code == 200 and r.json()["loaded"]
    with_ad = client.post("/v1/completions", json=dict(body, lora_name="ad")).json()["choices"][0]["token_ids"]
    assert with_ad != base
    assert client.post("/v1/completions", json=body).json()["choices"][0]["token_ids"] == base
    assert client.post("/v1/unload_lora_adapter", json={"lora_name": "ad"}).json()["unloaded"]
    assert client.post("/v1/load_lora_adapter", json={"lora_name": "x", "lora_path": "/nonexistent"}).status_code == 400


def test_chat_prompt_continue_final_message_with_and_without_template_support():
    import pytest

    from vllm_torchtpu_b200.entrypoints.chat_template import build_chat_prompt

    class Tok:
        """Template: <role>content</s> per message, generation prompt '<assistant>'."""
        supports_continue = True

        def apply_chat_template(self, messages, add_generation_prompt=False, tokenize=True,
                                continue_final_message=None, **kw):
            if continue_final_message is not None and not self.supports_continue:
                raise TypeError("unexpected keyword continue_final_message")
            text = ""
            for i, m in enumerate(messages):
                last = i == len(messages) - 1
                text += f"<{m['role']}>{m['content']}" + ("" if last and continue_final_message else "</s>")
            if add_generation_prompt:
                text += "<assistant>"
            return [ord(c) for c in text] if tokenize else text

    enc = lambda s: [ord(c) for c in s]
    dec = lambda ids: "".join(chr(i) for i in ids)
    msgs = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "The answer is"}]
    tok = Tok()
    assert dec(build_chat_prompt(tok, enc, msgs[:1])) == "<user>hi</s><assistant>"
    want = "<user>hi</s><assistant>The answer is"
    assert dec(build_chat_prompt(tok, enc, msgs, continue_final_message=True)) == want
    tok.supports_continue = False                      # a template that always closes the last message
    assert dec(build_chat_prompt(tok, enc, msgs, continue_final_message=True)) == want
    assert dec(build_chat_prompt(None, enc, msgs, continue_final_message=True)) == "user: hi\nassistant: The answer is"
    with pytest.raises(ValueError):
        build_chat_prompt(tok, enc, msgs[:1], continue_final_message=True)


def test_update_weights_and_reload_kernel_routes(tmp_path):
    """/update_weights loads checkpoint-named tensors from disk into the running model (the outputs change, the
    prefix cache is dropped); /reload_kernel calls the engine's kernel reload and reports a busy engine as 409."""
    import torch
    from safetensors.torch import save_file
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    app = build_app(llm.engine, "tiny-llama", None)
    with TestClient(app) as c:
        body = {"prompt": list(range(3, 20)), "max_tokens": 6, "temperature": 0.0, "ignore_eos": True}
        before = c.post("/v1/completions", json=body).json()["choices"][0]
        g = torch.Generator().manual_seed(5)
        mc = llm.engine.cfg.model
        new = {"lm_head.weight": torch.randn(mc.vocab_size, mc.hidden_size, generator=g) * 0.05}
        f = tmp_path / "delta.safetensors"
        save_file(new, str(f))
        r = c.post("/update_weights", json={"path": str(f)})
        assert r.status_code == 200 and r.json()["tensors"] == 1
        torch.testing.assert_close(llm.engine.runner.model.lm_head, new["lm_head.weight"])
        after = c.post("/v1/completions", json=body).json()["choices"][0]
        assert after != before
        assert c.post("/update_weights", json={"path": str(tmp_path / "missing")}).status_code == 400
        calls = []
        llm.engine.reload_kernels = lambda path=None: calls.append(path) or "lib.so"
        r = c.post("/reload_kernel", json={"path": "/x/lib.so"})
        assert r.status_code == 200 and r.json()["library"] == "lib.so" and calls == ["/x/lib.so"]

        def busy(path=None):
            raise RuntimeError("reload_kernels needs an idle engine")
        llm.engine.reload_kernels = busy
        assert c.post("/reload_kernel").status_code == 409
    app.state.async_engine.shutdown()


def test_launch_exports_once_then_serves_the_artifact(tmp_path):
    """``launch`` splits the serve command line, exports into a cache keyed by model + export flags, and
    replaces itself with the server over the artifact; a second launch reuses the artifact."""
    import json
    import os
    import socket
    import subprocess
    import sys
    import time
    import urllib.request

    from vllm_torchtpu_b200.entrypoints.cli import main
    cache = str(tmp_path / "exports")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    argv = ["launch", "tiny-llama", "--device", "cpu", "--host", "127.0.0.1", "--port", str(port), "--max-num-seqs", "4",
            "--max-model-len", "128", "--scheduler-cls", "default", "--export-cache", cache]
    env = dict(os.environ, B200_LOG_LEVEL="WARNING")
    out = subprocess.run([sys.executable, "-m", "vllm_torchtpu_b200"] + argv + ["--dry-run"], capture_output=True,
                         text=True, env=env, timeout=120)
    plan = json.loads(out.stdout.strip().splitlines()[-1])
    assert plan["cached"] is False and plan["world_size"] == 1
    assert "--max-num-seqs" in plan["export"] and "--port" not in plan["export"]
    assert "--port" in plan["serve"] and "--max-num-seqs" not in plan["serve"] and plan["serve"][4] == plan["artifact"]
    # other export flags -> another artifact; other front-end flags -> the same one
    alt = subprocess.run([sys.executable, "-m", "vllm_torchtpu_b200"] + argv + ["--dry-run", "--block-size", "32"],
                         capture_output=True, text=True, env=env, timeout=120)
    assert json.loads(alt.stdout.strip().splitlines()[-1])["artifact"] != plan["artifact"]
    proc = subprocess.Popen([sys.executable, "-m", "vllm_torchtpu_b200"] + argv, env=env, stdout=subprocess.PIPE,
                            stderr=subprocess.STDOUT, text=True)
    try:
        deadline, up = time.time() + 180, False
        while time.time() < deadline and proc.poll() is None:
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                    up = r.status == 200
                    break
            except OSError:
                time.sleep(0.5)
        assert up, "the server did not come up"
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions", method="POST",
                                     headers={"Content-Type": "application/json"},
                                     data=json.dumps({"prompt": [1, 2, 3, 4], "max_tokens": 3, "temperature": 0,
                                                      "ignore_eos": True}).encode())
        with urllib.request.urlopen(req, timeout=60) as r:
            body = json.loads(r.read())
        assert len(body["choices"][0]["token_ids"]) == 3
    finally:
        proc.terminate()
        try:
            proc.wait(30)
        except subprocess.TimeoutExpired:
            proc.kill()
    assert os.path.isfile(os.path.join(plan["artifact"], "metadata.json"))
    with open(os.path.join(plan["artifact"], "metadata.json")) as f:
        meta = json.load(f)
    assert meta["engine"]["max_num_seqs"] == 4 and meta["engine"]["max_model_len"] == 128
    assert main(argv + ["--dry-run"]) == 0          # the artifact is found again (printed as cached)
    again = subprocess.run([sys.executable, "-m", "vllm_torchtpu_b200"] + argv + ["--dry-run"], capture_output=True,
                           text=True, env=env, timeout=120)
    assert json.loads(again.stdout.strip().splitlines()[-1])["cached"] is True


class _PieceTokenizer:
    """Token id -> a fixed piece of text; enough for structured decoding and function calling over HTTP."""

    def __init__(self, vocab):
        self.vocab = vocab

    def __len__(self):
        return len(self.vocab)

    def encode(self, text):
        return [3 + (ord(c) % 50) for c in text][:64] or [3]

    def decode(self, ids):
        return "".join(self.vocab[t] for t in ids)


def test_function_calling_batched_prompts_and_utility_routes():
    import json

    from vllm_torchtpu_b200.entrypoints.tool_calls import extract_tool_calls, structured_spec_for, validate_tools
    tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {
        "type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"enum": [0, 7]}}, "required": ["ok", "n"]}}},
        {"type": "function", "function": {"name": "noop"}}]
    # the parser and the request checks on their own
    assert validate_tools({}) == ([], None) and validate_tools({"tools": tools})[1] == "auto"
    assert validate_tools({"tools": tools, "tool_choice": {"type": "function", "function": {"name": "noop"}}})[1] == "noop"
    for bad in ({"tool_choice": "required"}, {"tools": [{"type": "function"}]},
                {"tools": tools, "tool_choice": {"function": {"name": "missing"}}}, {"tools": tools, "tool_choice": "x"}):
        with pytest.raises(ValueError):
            validate_tools(bad)
    assert structured_spec_for(tools, "auto") is None and "json" in structured_spec_for(tools, "required")
    text = 'Let me look.\n<tool_call>\n{"name": "get_weather", "arguments": {"ok": true, "n": 3}}\n</tool_call>' \
           '<tool_call>{"name": "unknown", "arguments": {}}</tool_call>'
    content, calls = extract_tool_calls(text, tools, "auto")
    assert content == "Let me look." and len(calls) == 1 and calls[0]["function"]["name"] == "get_weather"
    assert json.loads(calls[0]["function"]["arguments"]) == {"ok": True, "n": 3}
    assert extract_tool_calls("plain answer", tools, "auto") == ("plain answer", [])
    assert extract_tool_calls(text, tools, "none") == (text, [])
    _, calls = extract_tool_calls('[{"name": "noop", "parameters": {}}]', tools, "required")
    assert calls[0]["function"] == {"name": "noop", "arguments": "{}"}

    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    V = llm.engine.cfg.model.vocab_size
    pieces = ['{', '}', '"', ':', ',', ' ', 'ok', 'n', 'true', 'false', '0', '1', '7', '42', 'x', 'y']
    tok = _PieceTokenizer(pieces + [f"<{i}>" for i in range(V - len(pieces))])
    llm.engine.eos_token_id = V - 1
    app = build_app(llm.engine, "tiny-llama", tok)
    msgs = [{"role": "user", "content": "weather?"}]
    with TestClient(app) as c:
        # a named function: the arguments are constrained to its parameter schema
        r = c.post("/v1/chat/completions", json={
            "messages": msgs, "tools": tools, "max_tokens": 40, "temperature": 0,
            "tool_choice": {"type": "function", "function": {"name": "get_weather"}}})
        assert r.status_code == 200, r.text
        ch = r.json()["choices"][0]
        assert ch["finish_reason"] == "tool_calls" and ch["message"]["content"] is None
        call = ch["message"]["tool_calls"][0]
        args = json.loads(call["function"]["arguments"])
        assert call["function"]["name"] == "get_weather" and isinstance(args["ok"], bool) and args["n"] in (0, 7)
        # the same as a stream: the calls come as one delta of the last chunk
        with c.stream("POST", "/v1/chat/completions", json={
                "messages": msgs, "tools": tools, "max_tokens": 40, "temperature": 0, "stream": True,
                "tool_choice": {"type": "function", "function": {"name": "get_weather"}}}) as s:
            chunks = [json.loads(l[5:]) for l in s.iter_lines() if l.startswith("data: {")]
        last = chunks[-1]["choices"][0]
        assert last["finish_reason"] == "tool_calls" and last["delta"]["tool_calls"][0]["index"] == 0
        assert c.post("/v1/chat/completions", json={"messages": msgs, "tool_choice": "required"}).status_code == 400
        # several prompts in one completion request
        r = c.post("/v1/completions", json={"prompt": [[1, 2, 3], [4, 5, 6, 7]], "max_tokens": 2, "temperature": 0,
                                            "ignore_eos": True, "n": 2}).json()
        assert [ch["index"] for ch in r["choices"]] == [0, 1, 2, 3]
        assert r["usage"] == dict(r["usage"], prompt_tokens=7, completion_tokens=8, total_tokens=15)
        assert c.post("/v1/completions", json={"prompt": [[1], [2]], "stream": True}).status_code == 400
        # utility routes
        t = c.post("/tokenize", json={"prompt": "abc"}).json()
        assert t["count"] == 3 and t["tokens"] == tok.encode("abc")
        assert c.post("/tokenize", json={"messages": msgs}).json()["count"] > 0
        assert c.post("/detokenize", json={"tokens": [0, 6, 1]}).json() == {"prompt": "{ok}"}
        assert c.post("/detokenize", json={"tokens": "x"}).status_code == 400
        assert c.get("/version").json()["version"] and c.get("/ping").json() == {"status": "ok"}
    app.state.async_engine.shutdown()


def test_metrics_histograms_and_vllm_compatible_names(client):
    for n in (2, 5):
        r = client.post("/v1/completions", json={"prompt": [9, 8, 7, 6], "max_tokens": n, "temperature": 0,
                                                 "ignore_eos": True})
        assert r.status_code == 200
    text = client.get("/metrics").text
    series = {}
    for line in text.splitlines():
        if line and not line.startswith("#"):
            name, val = line.rsplit(" ", 1)
            series[name] = float(val)
    lab = 'model_name="tiny-llama"'
    assert series["b200_generation_tokens_total"] == series[f"vllm:generation_tokens_total{{{lab}}}"] >= 7
    assert series["vllm:request_success_total{" + lab + ',finished_reason="length"}'] >= 2
    cnt = series[f"vllm:time_to_first_token_seconds_count{{{lab}}}"]
    assert cnt >= 2 and series[f'vllm:time_to_first_token_seconds_bucket{{{lab},le="+Inf"}}'] == cnt
    assert series[f"vllm:e2e_request_latency_seconds_sum{{{lab}}}"] >= series[f"vllm:time_to_first_token_seconds_sum{{{lab}}}"]
    assert series[f"vllm:time_per_output_token_seconds_count{{{lab}}}"] >= 2
    assert series[f"vllm:request_queue_time_seconds_count{{{lab}}}"] == cnt
    assert series["b200_request_generation_tokens_sum"] >= 7 and series["b200_prefix_cache_queries_total"] >= 8
    # cumulative buckets never decrease
    buckets = [v for k, v in series.items() if k.startswith("b200_e2e_request_latency_seconds_bucket")]
    assert buckets == sorted(buckets)
    assert "# TYPE vllm:num_requests_running gauge" in text and "# TYPE b200_kv_cache_usage gauge" in text


def test_metrics_carry_offload_and_transfer_statistics():
    """A second request with the same prompt is served from the host store: the external prefix-cache counters and
    the renderer's view of a P2P connector's statistics."""
    from vllm_torchtpu_b200.entrypoints.metrics import ServingMetrics
    from vllm_torchtpu_b200.kv_transfer.stats import KVConnectorStats
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False,
              kv_transfer_config={"kv_connector": "B200OffloadingConnector", "kv_role": "kv_both",
                                  "kv_connector_extra_config": {"num_blocks": 32}})
    app = build_app(llm.engine, "tiny-llama", None)
    body = {"prompt": list(range(1, 50)), "max_tokens": 2, "temperature": 0, "ignore_eos": True}
    with TestClient(app) as c:
        assert c.post("/v1/completions", json=body).status_code == 200
        assert c.post("/v1/completions", json=body).status_code == 200
        text = c.get("/metrics").text
    app.state.async_engine.shutdown()
    vals = {l.rsplit(" ", 1)[0]: float(l.rsplit(" ", 1)[1]) for l in text.splitlines() if l and l[0] != "#"}
    assert vals["b200_external_prefix_cache_hits_total"] >= 32          # two full blocks of the repeated prompt
    assert vals["b200_external_prefix_cache_queries_total"] >= 49
    compat = vals['vllm:external_prefix_cache_hits_total{model_name="tiny-llama"}']
    assert compat == vals["b200_external_prefix_cache_hits_total"]
    # P2P statistics through the same renderer
    from types import SimpleNamespace
    st = KVConnectorStats()
    st.record_load(4, 0.01, ok=True)
    st.record_send(3, expired=False)
    st.record_send(2, expired=True)
    conn = SimpleNamespace(scheduler=SimpleNamespace(s=SimpleNamespace(stats=st)), worker=SimpleNamespace(s=SimpleNamespace(stats=st)))
    lines = ServingMetrics._connector_lines(conn, 'model_name="m"')
    assert 'b200_kv_loads_total{result="ok"} 1' in lines and 'b200_kv_blocks_total{direction="out"} 3' in lines
    assert 'b200_kv_sends_total{result="expired"} 1' in lines and sum(l.startswith("b200_kv_loads_total") for l in lines) == 2
