"""Two requests in one batch, one through a LoRA adapter and one through the base model.
The adapter here is random (rank 4 on q_proj and down_proj of every layer); a real one is passed as
{"model.layers.N.self_attn.q_proj": (A [r, in], B [out, r]), ...}."""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_torchtpu_b200 import LLM, SamplingParams  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-llama")
    ap.add_argument("--device", default="cuda")
    a = ap.parse_args(argv)
    llm = LLM(a.model, device=a.device, init_dist=False, max_num_seqs=8, block_size=16)
    mc = llm.engine.cfg.model
    g = torch.Generator().manual_seed(0)
    weights = {}
    for i in range(mc.num_layers):
        pre = f"model.layers.{i}."
        weights[pre + "self_attn.q_proj"] = (torch.randn(4, mc.hidden_size, generator=g) * 0.2,
                                             torch.randn(mc.num_q_heads * mc.head_dim, 4, generator=g) * 0.2)
        weights[pre + "mlp.down_proj"] = (torch.randn(4, mc.intermediate_size, generator=g) * 0.2,
                                          torch.randn(mc.hidden_size, 4, generator=g) * 0.2)
    assert llm.engine.add_lora("demo", 4, 8.0, weights)
    prompt = list(range(10, 30))
    sps = [SamplingParams(temperature=0.0, max_tokens=8, lora_name="demo"),
           SamplingParams(temperature=0.0, max_tokens=8)]
    outs = llm.generate([prompt, prompt], sps)
    print("with adapter:", outs[0].outputs[0].token_ids)
    print("base model  :", outs[1].outputs[0].token_ids)
    print("adapters    :", llm.engine.list_loras())
    return outs


if __name__ == "__main__":
    main()
