"""Speculative decoding: drafters propose k tokens, the target model verifies them in one step
and a rejection sampler decides how many are kept.

Drafters: ``ngram`` (prompt lookup), ``suffix`` (longest-suffix match over prompt + output), ``medusa``
(K residual-block heads on the target's hidden state, loaded from a checkpoint and run batched on the
device), ``mtp`` / ``eagle`` / ``eagle3`` (one transformer layer with attention and its own KV cache behind
the target's block tables, ``draft_layer.py``), ``dflash`` / ``dspark`` (parallel block drafting: context keys and
values from the target's hidden states, all k drafts from one non-causal block pass, ``dflash.py``).
(reference: src/vllm_torchtpu/spec_decode/, docs/user_guide/speculative_decoding.md:5-16)"""
from __future__ import annotations


DRAFT_LAYER_METHODS = ("mtp", "eagle", "eagle3", "dflash", "dspark")      # drafters that keep KV caches of their own


def create_proposer(cfg, runner):
    sc = cfg.speculative or {}
    method = sc.get("method", "ngram")
    k = int(sc.get("num_speculative_tokens", 3))
    if method in ("ngram", "suffix"):
        from .ngram import NgramProposer
        return NgramProposer(k, int(sc.get("prompt_lookup_min", 2)), int(sc.get("prompt_lookup_max", 4)),
                             suffix=(method == "suffix"))
    if method == "medusa":
        from .medusa import MedusaProposer
        return MedusaProposer(cfg, runner, k, sc.get("model"), int(sc.get("num_hidden_layers", 1)))
    if method in ("dflash", "dspark"):
        from .dflash import DFlashProposer
        return DFlashProposer(cfg, runner, k, method, sc.get("model"), int(sc.get("num_hidden_layers", 1)),
                              sc.get("mask_token_id"))
    if method in DRAFT_LAYER_METHODS:
        from .draft_layer import DraftLayerProposer
        return DraftLayerProposer(cfg, runner, k, method, sc.get("model"))
    raise ValueError(f"unknown speculative method {method!r}")
