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
