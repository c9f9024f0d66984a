"""Image patches through the vision encoder into placeholder rows of the prompt.  An item is
(patches [num_patches, patch_dim], offset of its first placeholder token in the prompt); the encoder merges
`merge` patches into one embedding row, so an item of 16 patches with merge 4 fills 4 placeholder positions."""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_torchtpu_b200 import LLM, SamplingParams  # noqa: E402
from vllm_torchtpu_b200.layers.vision import VisionConfig  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-llama")
    ap.add_argument("--device", default="cuda")
    a = ap.parse_args(argv)
    llm = LLM(a.model, device=a.device, init_dist=False, max_num_seqs=8, block_size=16)
    mc = llm.engine.cfg.model
    vc = VisionConfig(patch_dim=48, hidden_size=64, num_heads=2, depth=2, merge=4, out_hidden_size=mc.hidden_size)
    llm.engine.enable_vision(vc, max_patches_per_batch=256)
    g = torch.Generator().manual_seed(0)
    image = torch.randn(16, 48, generator=g).to(mc.dtype)            # 16 patches -> 4 rows
    video = torch.randn(40, 48, generator=g).to(mc.dtype)            # 40 patches -> 10 rows
    prompt = list(range(100, 148))
    sp = SamplingParams(temperature=0.0, max_tokens=8)
    rid = llm.engine.add_request(prompt, sp, mm_items=[(image, 5), (video, 30)])
    done = {r.request_id: r for r in llm.engine.run_until_done()}
    print("with image + video:", done[rid].output_token_ids)
    print("text only         :", llm.generate([prompt], sp)[0].outputs[0].token_ids)
    return done[rid].output_token_ids


if __name__ == "__main__":
    main()
