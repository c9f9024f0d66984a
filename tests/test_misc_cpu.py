"""Envs registry, env validation, profile options, phase classification, parallel layouts, CLI parsing."""
import os
import pytest

from vllm_torchtpu_b200 import env_validation, envs
from vllm_torchtpu_b200.parallel.state import dcp_groups, layout_ranks
from vllm_torchtpu_b200.tracing.profiler import classify_phase, parse_profile_options


def test_envs_typed_lazy_and_validated(monkeypatch):
    assert envs.B200_FUSED_TP is True
    monkeypatch.setenv("B200_FUSED_TP", "0")
    assert envs.B200_FUSED_TP is True            # cached
    envs.reset()
    assert envs.B200_FUSED_TP is False
    monkeypatch.setenv("B200_TP_COMM", "carrier-pigeon")
    envs.reset()
    with pytest.raises(ValueError):
        envs.B200_TP_COMM
    with pytest.raises(AttributeError):
        envs.B200_DOES_NOT_EXIST
    monkeypatch.setenv("B200_TOKEN_BUCKET_EXTRA", "48, 96")
    envs.reset()
    assert envs.B200_TOKEN_BUCKET_EXTRA == [48, 96]


def test_env_validation_flags_typos():
    unknown = env_validation.find_unknown({"B200_FUSED_TPP": "1", "B200_FUSED_TP": "1", "HOME": "/x"})
    assert [u.name for u in unknown] == ["B200_FUSED_TPP"] and unknown[0].suggestion == "B200_FUSED_TP"
    assert env_validation.validate_values({"B200_SYMM_HEAP_MB": "abc"})


def test_profile_options_and_phases():
    o = parse_profile_options("dir:/tmp/x;python:1;shapes:0")
    assert o["dir"] == "/tmp/x" and o["python"] and not o["shapes"]
    with pytest.raises(ValueError):
        parse_profile_options("bogus:1")
    assert classify_phase(900, 10) == "prefill_heavy" and classify_phase(0, 64) == "decode_heavy"
    assert classify_phase(100, 100) == "balanced" and classify_phase(0, 0) == "idle"


def test_rank_layouts():
    lay = layout_ranks(16, tp=4, pp=2, dp=2)
    assert lay["tp"][0] == [0, 1, 2, 3] and lay["pp"][0] == [0, 4] and lay["dp"][0] == [0, 8]
    assert lay["ep"][0] == [0, 1, 2, 3, 8, 9, 10, 11]
    assert dcp_groups([0, 1, 2, 3], 2) == [[0, 1], [2, 3]]
    lay = layout_ranks(8, tp=2, pp=1, dp=2, pcp=2)
    assert lay["pcp"][0] == [0, 2] and lay["tp"][1] == [2, 3]


def test_cli_parses_vllm_style_flags():
    import argparse
    from vllm_torchtpu_b200.entrypoints.cli import add_engine_args
    ap = argparse.ArgumentParser()
    add_engine_args(ap)
    a = ap.parse_args(["llama-3.1-8b", "-tp", "8", "--enable-expert-parallel", "--kv-cache-dtype", "fp8",
                       "--kv-transfer-config", '{"kv_connector": "B200P2PConnector", "kv_role": "kv_producer"}',
                       "--speculative-config", '{"method": "ngram", "num_speculative_tokens": 3}'])
    assert a.tensor_parallel_size == 8 and a.kv_transfer_config["kv_role"] == "kv_producer"
    assert a.speculative_config["method"] == "ngram"


def test_platform_rejects_bad_configs():
    from vllm_torchtpu_b200.config import EngineConfig, model_preset
    from vllm_torchtpu_b200.platform import B200Platform
    from vllm_torchtpu_b200.sampling_params import SamplingParams
    cfg = EngineConfig(model=model_preset("tiny-llama"))
    cfg.model.quantization = "int3"
    with pytest.raises(ValueError):
        cfg.finalize()
    cfg = EngineConfig(model=model_preset("tiny-llama"))
    cfg.parallel.tensor_parallel_size = 3
    cfg.parallel.world_size = 3
    with pytest.raises(ValueError):
        cfg.finalize()
    with pytest.raises(ValueError):
        B200Platform.validate_request(SamplingParams(seed=1))
    with pytest.raises(ValueError):
        B200Platform.validate_request(SamplingParams(logprobs=-1))
    cfg = EngineConfig(model=model_preset("tiny-llama"), kv_transfer={"kv_connector": "Nope"})
    with pytest.raises(ValueError):
        cfg.finalize()


def test_export_serving_dir_roundtrip_and_validation(tmp_path):
    """Export -> validate -> load gives the same greedy tokens; a corrupted file and a wrong format
    version are reported."""
    import json
    import os
    import numpy as np
    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.engine.llm import LLM
    from vllm_torchtpu_b200.entrypoints.cli import main
    from vllm_torchtpu_b200.export import export_serving_dir, load_serving_dir, validate_serving_dir
    src = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    prompts = [np.random.RandomState(3).randint(0, 1024, size=n).tolist() for n in (5, 19)]
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in src.generate(prompts, sp)]
    d = str(tmp_path / "serving")
    meta = export_serving_dir(src, d)
    assert meta["plan"]["request_buckets"] and "serving_checkpoint/model.safetensors" in meta["manifest"]
    assert validate_serving_dir(d) == [] and main(["validate-export", d]) == 0
    dst = load_serving_dir(d, device="cpu", init_dist=False)
    assert [o.outputs[0].token_ids for o in dst.generate(prompts, sp)] == want
    with open(os.path.join(d, "serving_checkpoint", "config.json"), "a") as f:
        f.write(" ")
    assert any("config.json" in p for p in validate_serving_dir(d))
    m = json.load(open(os.path.join(d, "metadata.json")))
    m["format_version"] = 99
    json.dump(m, open(os.path.join(d, "metadata.json"), "w"))
    assert any("format_version" in p for p in validate_serving_dir(d))
    assert main(["validate-export", d]) == 1


def test_merge_rank_traces(tmp_path):
    import json
    import os
    from vllm_torchtpu_b200.tracing.merge_traces import main, merge_dir
    for rank, skew in ((0, 0), (1, 500)):
        d = tmp_path / f"rank_{rank}"
        d.mkdir()
        ev = [{"ph": "M", "name": "process_name", "pid": 7, "tid": 0, "args": {"name": "python"}},
              {"ph": "X", "name": "barrier", "pid": 7, "tid": 1, "ts": 1000 + skew, "dur": 5},
              {"ph": "X", "name": "step", "pid": 7, "tid": 1, "ts": 1100 + skew, "dur": 50}]
        (d / "trace_1.json").write_text(json.dumps({"traceEvents": ev}))
    out = str(tmp_path / "m.json")
    info = merge_dir(str(tmp_path), out, "barrier")
    assert info["ranks"] == [0, 1]
    ev = json.load(open(out))["traceEvents"]
    steps = sorted((e["pid"], e["ts"]) for e in ev if e.get("name") == "step")
    assert steps[0][0] != steps[1][0] and steps[0][1] == steps[1][1] == 1100      # skew removed
    names = [e["args"]["name"] for e in ev if e.get("name") == "process_name"]
    assert names == ["rank 0: python", "rank 1: python"]
    assert main([str(tmp_path), "-o", out]) == 0 and os.path.getsize(out) > 0


def test_pad_q_heads_keeps_the_kv_group_mapping():
    import torch
    from vllm_torchtpu_b200.models.llama import pad_q_heads
    Hkv, G, Gp, D, H = 2, 3, 4, 8, 5
    w = torch.arange(Hkv * G * D * H, dtype=torch.float32).reshape(Hkv * G * D, H)
    p = pad_q_heads(w, 0, Hkv, G, Gp, D)
    assert p.shape == (Hkv * Gp * D, H)
    p4 = p.reshape(Hkv, Gp, D, H)
    torch.testing.assert_close(p4[:, :G].reshape(-1, H), w)          # real heads keep their group and order
    assert float(p4[:, G:].abs().sum()) == 0.0                       # padded heads are zero
    o = torch.arange(H * Hkv * G * D, dtype=torch.float32).reshape(H, Hkv * G * D)
    po = pad_q_heads(o, 1, Hkv, G, Gp, D)
    assert po.shape == (H, Hkv * Gp * D)
    torch.testing.assert_close(po.reshape(H, Hkv, Gp, D)[:, :, :G].reshape(H, -1), o)


def test_fused_ep_plane_is_called_once_per_call_tokens_rows():
    """A step longer than the plane's call size goes through it in several calls, the same number on
    every rank (the agreed row count decides, not this rank's own)."""
    import types

    import torch

    from vllm_torchtpu_b200.layers.moe import FusedMoE

    calls = []

    class Method:
        def apply_fused_ep(self, moe, x, ids, w, comm):
            calls.append(x.shape[0])
            return x * 2

    moe = FusedMoE.__new__(FusedMoE)
    moe.method = Method()
    comm = types.SimpleNamespace(heap=types.SimpleNamespace(ep_state=types.SimpleNamespace(max_tokens=4)))
    x = torch.arange(22, dtype=torch.float32).reshape(11, 2)
    ids = torch.zeros(11, 2, dtype=torch.int32)
    w = torch.ones(11, 2)
    y = moe._fused_ep_calls(x, ids, w, comm)
    assert calls == [4, 4, 3] and torch.equal(y, x * 2)
    calls.clear()
    y = moe._fused_ep_calls(x[:3], ids[:3], w[:3], comm, rows=9)      # peers hold 9 rows: three calls here too
    assert calls == [3, 0, 0] and torch.equal(y, x[:3] * 2)
    calls.clear()
    moe._fused_ep_calls(x[:4], ids[:4], w[:4], comm)
    assert calls == [4]


def test_docs_list_every_environment_variable_and_guided_choice_maps_to_a_regex():
    import os
    import re
    from vllm_torchtpu_b200 import envs
    from vllm_torchtpu_b200.entrypoints.openai_server import _structured_spec
    doc = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "docs", "reference",
                            "env_vars.md")).read()
    missing = [n for n in envs.declared() if f"`{n}`" not in doc]
    assert not missing, f"docs/reference/env_vars.md lacks {missing}"
    spec = _structured_spec({"guided_choice": ["yes", "no way", "a.b"]})
    rx = re.compile(spec["regex"])
    assert all(rx.fullmatch(s) for s in ("yes", "no way", "a.b")) and not rx.fullmatch("axb")
    assert _structured_spec({"response_format": {"type": "json_object"}}) == {"json_object": True}


def test_example_scripts_run_on_cpu():
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for name in ("offline_inference", "offline_lora_inference", "multi_modal_inference"):
        spec = importlib.util.spec_from_file_location(name, os.path.join(root, "examples", name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        out = mod.main(["--device", "cpu", "--model", "tiny-llama"])
        assert out
    spec = importlib.util.spec_from_file_location("oi", os.path.join(root, "examples", "offline_inference.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    outs = mod.main(["--device", "cpu", "--speculative-config", '{"method": "ngram", "num_speculative_tokens": 2}'])
    assert len(outs) == 2


def _pull_worker(uri, cache, q):
    from vllm_torchtpu_b200.models import model_source as ms
    q.put(ms.ensure_local_aux_files(uri, cache))


def test_aux_files_of_a_uri_model_are_pulled_once_per_host(tmp_path):
    """Ranks that share a host serialise on a lock: one pulls the non-weight files, the others find them; a
    pull that died half-way is started over; weights are never copied."""
    import multiprocessing as mp
    import shutil

    from vllm_torchtpu_b200.models import model_source as ms
    src = tmp_path / "bucket" / "model"
    src.mkdir(parents=True)
    for name, body in (("config.json", "{}"), ("tokenizer.json", "{}"), ("merges.txt", "a b"),
                       ("modeling_custom.py", "x = 1"), ("model-00001.safetensors", "W" * 64), ("notes.bin", "b")):
        (src / name).write_text(body)
    log = tmp_path / "fetch.log"

    def counting_fetch(uri, name, dst):
        with open(log, "a") as f:
            f.write(name + "\n")
        shutil.copyfile(os.path.join(uri[len("count://"):], name), dst)
    ms.register_fetcher("count", lambda uri: sorted(os.listdir(uri[len("count://"):])), counting_fetch)
    uri, cache = f"count://{src}", str(tmp_path / "cache")
    ctx = mp.get_context("fork")
    q = ctx.Queue()
    procs = [ctx.Process(target=_pull_worker, args=(uri, cache, q)) for _ in range(4)]
    [p.start() for p in procs]
    dirs = {q.get(timeout=60) for _ in procs}
    [p.join(60) for p in procs]
    assert len(dirs) == 1 and all(p.exitcode == 0 for p in procs)
    local = dirs.pop()
    assert local == ms.local_dir_for(uri, cache) and ms.is_complete(local)
    assert sorted(log.read_text().split()) == ["config.json", "merges.txt", "modeling_custom.py", "tokenizer.json"]
    assert not os.path.exists(os.path.join(local, "model-00001.safetensors"))
    # a crashed pull: the mark of a pull in progress without the completion mark
    os.remove(os.path.join(local, ".b200_aux_complete"))
    open(os.path.join(local, ".b200_pulling"), "w").close()
    os.remove(os.path.join(local, "tokenizer.json"))
    assert ms.ensure_local_aux_files(uri, cache) == local and os.path.exists(os.path.join(local, "tokenizer.json"))
    assert len(log.read_text().split()) == 8
    # file:// models: aux files local, weights read in place; plain paths pass through; unknown schemes refuse
    aux, weights = ms.resolve_model(f"file://{src}", cache)
    assert weights == str(src) and os.path.exists(os.path.join(aux, "config.json")) and aux != str(src)
    assert ms.resolve_model(str(src)) == (str(src), str(src))
    with pytest.raises(ValueError, match="fetcher"):
        ms.ensure_local_aux_files("s3://bucket/model", cache)
    (src / "config.json").unlink()
    with pytest.raises(FileNotFoundError):
        ms.ensure_local_aux_files(f"file://{src}", str(tmp_path / "cache2"))
