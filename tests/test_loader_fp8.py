"""Block-scaled fp8 Hugging Face checkpoints: every ``weight`` comes with a ``weight_scale_inv`` grid,
in whatever order the file lists them; the loader shards both for the rank and the dequantised result
equals the dequantised checkpoint's shard (bit-exact when the shard lies on block boundaries)."""
import json
import os

import pytest
import torch

from vllm_torchtpu_b200.config import ModelConfig
from vllm_torchtpu_b200.models.loader import load_safetensors
from vllm_torchtpu_b200.models.registry import get_model_class
from vllm_torchtpu_b200.parallel import state as pstate
from vllm_torchtpu_b200.quantization.fp8 import dequantize_weight_block, quantize_weight_block

HF = {"architectures": ["Qwen3MoeForCausalLM"], "num_hidden_layers": 2, "hidden_size": 256,
      "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 512,
      "vocab_size": 512, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 256,
      "torch_dtype": "bfloat16", "num_experts": 4, "num_experts_per_tok": 2, "moe_intermediate_size": 256,
      "norm_topk_prob": True, "mlp_only_layers": [0],
      "quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128]}}


def _write_checkpoint(path, scales_last: bool):
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(0)
    H, D, I, E, Im = 256, 64, 512, 4, 256
    dense, tensors = {}, {}

    def lin(name, n, k):
        w = torch.randn(n, k, generator=g) * 0.05
        q, s = quantize_weight_block(w)
        dense[name] = dequantize_weight_block(q, s)
        tensors[name + ".weight"], tensors[name + ".weight_scale_inv"] = q, s

    tensors["model.embed_tokens.weight"] = (torch.randn(512, H, generator=g) * 0.05).bfloat16()
    tensors["lm_head.weight"] = (torch.randn(512, H, generator=g) * 0.05).bfloat16()
    tensors["model.norm.weight"] = torch.ones(H).bfloat16()
    for li in range(2):
        p = f"model.layers.{li}."
        tensors[p + "input_layernorm.weight"] = torch.ones(H).bfloat16()
        tensors[p + "post_attention_layernorm.weight"] = torch.ones(H).bfloat16()
        tensors[p + "self_attn.q_norm.weight"] = torch.ones(D).bfloat16()
        tensors[p + "self_attn.k_norm.weight"] = torch.ones(D).bfloat16()
        lin(p + "self_attn.q_proj", 4 * D, H)
        lin(p + "self_attn.k_proj", 2 * D, H)
        lin(p + "self_attn.v_proj", 2 * D, H)
        lin(p + "self_attn.o_proj", H, 4 * D)
        if li == 0:
            lin(p + "mlp.gate_proj", I, H); lin(p + "mlp.up_proj", I, H); lin(p + "mlp.down_proj", H, I)
        else:
            tensors[p + "mlp.gate.weight"] = torch.randn(E, H, generator=g).bfloat16()
            for e in range(E):
                lin(p + f"mlp.experts.{e}.gate_proj", Im, H)
                lin(p + f"mlp.experts.{e}.up_proj", Im, H)
                lin(p + f"mlp.experts.{e}.down_proj", H, Im)
    os.makedirs(path, exist_ok=True)
    names = sorted(tensors, key=lambda n: (n.endswith("weight_scale_inv") == scales_last, n))
    half = len(names) // 2
    # two files, the second holding what sorts last: scales arrive in another file than their weights
    save_file({n: tensors[n].contiguous() for n in names[:half]}, os.path.join(path, "model-00001-of-00002.safetensors"))
    save_file({n: tensors[n].contiguous() for n in names[half:]}, os.path.join(path, "model-00002-of-00002.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(HF, f)
    return dense


def _close(got, want, exact):
    if exact:
        assert torch.equal(got, want)
    else:
        assert (got - want).abs().max() <= want.abs().max() * 0.07


@pytest.mark.parametrize("tp,rank", [(1, 0), (2, 1)])
@pytest.mark.parametrize("scales_last", [True, False])
def test_block_fp8_checkpoint_loads_with_scales(tmp_path, tp, rank, scales_last):
    dense = _write_checkpoint(str(tmp_path), scales_last)
    cfg = ModelConfig.from_hf_dict(HF)
    assert cfg.quantization == "fp8_block"
    cfg.dtype = torch.bfloat16
    try:
        if tp > 1:
            pstate.set_state_for_test(rank=rank, world_size=tp, tp=pstate.Group("tp", list(range(tp)), rank))
        model = get_model_class(cfg)(cfg, "cpu")
        load_safetensors(model, str(tmp_path))
        D = 64
        for li, layer in enumerate(model.layers):
            p = f"model.layers.{li}."
            a = layer.self_attn
            full = torch.cat([dense[p + f"self_attn.{x}_proj"] for x in "qkv"], 0)
            _close(dequantize_weight_block(a.qkv.weight, a.qkv.weight_scale_inv), a.qkv.shard_of(full), exact=tp == 1)
            _close(dequantize_weight_block(a.o.weight, a.o.weight_scale_inv), a.o.shard_of(dense[p + "self_attn.o_proj"]),
                   exact=True)
            if li == 0:
                gu = torch.cat([dense[p + "mlp.gate_proj"], dense[p + "mlp.up_proj"]], 0)
                _close(dequantize_weight_block(layer.mlp.gate_up.weight, layer.mlp.gate_up.weight_scale_inv),
                       layer.mlp.gate_up.shard_of(gu), exact=True)
                _close(dequantize_weight_block(layer.mlp.down.weight, layer.mlp.down.weight_scale_inv),
                       layer.mlp.down.shard_of(dense[p + "mlp.down_proj"]), exact=True)
            else:
                moe = layer.mlp.experts
                I = moe.intermediate_size
                for e in range(4):
                    g, u, d = (dense[p + f"mlp.experts.{e}.{x}_proj"] for x in ("gate", "up", "down"))
                    if tp > 1:
                        g, u, d = g[rank * I:(rank + 1) * I], u[rank * I:(rank + 1) * I], d[:, rank * I:(rank + 1) * I]
                    _close(dequantize_weight_block(moe.w13[e], moe.w13_scale[e]), torch.cat([g, u], 0), exact=True)
                    _close(dequantize_weight_block(moe.w2[e], moe.w2_scale[e]), d, exact=True)
    finally:
        pstate.set_state_for_test()


def test_fp8_weight_without_scale_is_refused(tmp_path):
    from safetensors.torch import save_file
    _write_checkpoint(str(tmp_path), True)
    # drop one scale tensor from the second file
    from safetensors import safe_open
    f2 = os.path.join(str(tmp_path), "model-00002-of-00002.safetensors")
    with safe_open(f2, framework="pt") as sf:
        kept = {k: sf.get_tensor(k) for k in sf.keys() if k != "model.layers.0.self_attn.o_proj.weight_scale_inv"}
    save_file(kept, f2)
    cfg = ModelConfig.from_hf_dict(HF)
    model = get_model_class(cfg)(cfg, "cpu")
    with pytest.raises(ValueError, match="weight_scale_inv"):
        load_safetensors(model, str(tmp_path))
