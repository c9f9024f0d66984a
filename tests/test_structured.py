import torch

from vllm_torchtpu_b200.structured import (ChoiceGrammar, RegexGrammar, StructuredDecodingManager,
                                           apply_token_bitmask, pack_bitmask)


def test_bitmask_roundtrip_and_apply():
    V = 70
    m = torch.from_numpy(pack_bitmask([0, 31, 32, 69], V))[None]
    logits = torch.zeros(2, V)
    apply_token_bitmask(logits, m, torch.tensor([1]))
    assert torch.isfinite(logits[0]).all()
    assert torch.isfinite(logits[1]).nonzero().flatten().tolist() == [0, 31, 32, 69]


def test_choice_grammar_walks_trie():
    g = ChoiceGrammar([[5, 6, 7], [5, 9]], eos_token_id=2)
    assert sorted(g.allowed_token_ids()) == [5]
    assert g.accept(5) and sorted(g.allowed_token_ids()) == [6, 9]
    assert not g.accept(4)
    assert g.accept(9) and g.finished and g.allowed_token_ids() == [2]


def test_regex_grammar_masks_vocab():
    vocab = ["a", "b", "1", "2", "ab", "-"]
    g = RegexGrammar(r"[a-b]+-\d\d", vocab, eos_token_id=99)
    assert sorted(g.allowed_token_ids()) == [0, 1, 4]
    for t in (4, 5, 2):
        assert g.accept(t)
    assert sorted(g.allowed_token_ids()) == [2, 3]
    assert g.accept(3) and 99 in g.allowed_token_ids()


def test_manager_drives_constrained_sampling():
    mgr = StructuredDecodingManager(vocab_size=16, eos_token_id=0)
    mgr.add_request("r1", {"choice": [[3, 4], [7]]})
    out = []
    for _ in range(3):
        bm, rows = mgr.build_bitmask(["r0", "r1"])
        logits = torch.randn(2, 16)
        apply_token_bitmask(logits, bm, rows)
        tok = int(logits[1].argmax())
        mgr.accept_tokens({"r1": [tok]})
        out.append(tok)
        if tok == 0:
            break
    assert out in ([3, 4, 0], [7, 0])


def test_engine_respects_choice_constraint():
    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.engine.llm import LLM
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=4, block_size=16, init_dist=False)
    llm.engine.eos_token_id = 0
    sp = SamplingParams(temperature=0.0, max_tokens=8, structured={"choice": [[11, 12, 13], [500]]})
    free = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    outs = llm.generate([[1, 2, 3, 4], [5, 6, 7]], [sp, free])
    assert outs[0].outputs[0].token_ids in ([11, 12, 13, 0], [500, 0])
    assert len(outs[1].outputs[0].token_ids) == 4


def test_json_schema_regex_accepts_exactly_the_schema():
    import json

    import regex

    from vllm_torchtpu_b200.structured.json_schema import any_json_object_regex, schema_to_regex
    schema = {
        "type": "object",
        "properties": {
            "name": {"type": "string", "maxLength": 8},
            "age": {"type": "integer"},
            "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "minItems": 1, "maxItems": 3},
            "score": {"type": ["number", "null"]},
            "address": {"$ref": "#/$defs/addr"},
        },
        "required": ["name", "age"],
        "$defs": {"addr": {"type": "object", "properties": {"zip": {"type": "string", "pattern": "^[0-9]{5}$"}},
                           "required": ["zip"]}},
    }
    rx = regex.compile(schema_to_regex(schema))
    good = [
        {"name": "ann", "age": 3},
        {"name": "", "age": -12, "tags": ["a", "b"], "score": 1.5e3},
        {"name": "x", "age": 0, "score": None, "address": {"zip": "12345"}},
    ]
    for g in good:
        assert rx.fullmatch(json.dumps(g)) is not None, g
        assert rx.fullmatch(json.dumps(g, separators=(",", ":"))) is not None, g
    bad = [
        '{"age": 3}',                                      # required property missing
        '{"name": "toolongname", "age": 3}',               # maxLength
        '{"name": "a", "age": 3.5}',                       # integer
        '{"name": "a", "age": 3, "tags": []}',             # minItems
        '{"name": "a", "age": 3, "tags": ["c"]}',          # enum
        '{"name": "a", "age": 3, "extra": 1}',             # undeclared property
        '{"age": 3, "name": "a"}',                         # declaration order
        '{"name": "a", "age": 3, "address": {"zip": "1234"}}',
    ]
    for b in bad:
        assert rx.fullmatch(b) is None, b
    # a prefix of a valid text is a partial match (what the token mask is built from)
    assert rx.fullmatch('{"name": "an', partial=True) is not None
    anyobj = regex.compile(any_json_object_regex())
    assert anyobj.fullmatch('{"a": [1, {"b": null}], "c": "d"}') is not None
    assert anyobj.fullmatch('[1, 2]') is None


def test_engine_generates_json_that_satisfies_a_schema():
    import json

    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.engine.llm import LLM
    llm = LLM("tiny-llama", device="cpu", max_num_seqs=2, init_dist=False)
    V = llm.engine.cfg.model.vocab_size
    # a toy vocabulary: JSON punctuation, digits, letters, and filler tokens that never fit
    pieces = ['{', '}', '"', ':', ',', ' ', 'ok', 'n', 'true', 'false', '0', '1', '7', '42', 'x', 'y']
    vocab = pieces + [f"<{i}>" for i in range(V - len(pieces))]
    eos = V - 1
    llm.engine.vocab_strings, llm.engine.eos_token_id = vocab, eos
    schema = {"type": "object", "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer"}},
              "required": ["ok", "n"]}
    sp = SamplingParams(temperature=0.0, max_tokens=40, structured={"json": schema}, stop_token_ids=[eos])
    out = llm.generate([[1, 2, 3]], sp)[0].outputs[0].token_ids
    text = "".join(vocab[t] for t in out if t != eos)
    obj = json.loads(text)
    assert set(obj) == {"ok", "n"} and isinstance(obj["ok"], bool) and isinstance(obj["n"], int)
