"""Offline generation.  `python examples/offline_inference.py --model /path/to/checkpoint --tensor-parallel-size 1`
(with several GPUs: `python -m torch.distributed.run --nproc-per-node N examples/offline_inference.py ...`).
Without a checkpoint a preset with random weights (`tiny-llama`, `llama-3.1-8b`, ...) runs on token ids."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from vllm_torchtpu_b200 import LLM, SamplingParams  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-llama")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--enable-prefix-caching", action="store_true")
    ap.add_argument("--speculative-config", default=None, help='JSON, e.g. {"method": "ngram", "num_speculative_tokens": 3}')
    a = ap.parse_args(argv)
    import json
    llm = LLM(a.model, device=a.device, tensor_parallel_size=a.tensor_parallel_size,
              enable_prefix_caching=a.enable_prefix_caching, init_dist=a.tensor_parallel_size > 1,
              speculative_config=json.loads(a.speculative_config) if a.speculative_config else None,
              max_num_seqs=8, block_size=16)
    sp = SamplingParams(temperature=a.temperature, top_p=a.top_p, max_tokens=a.max_tokens)
    if llm.tokenizer is not None:
        prompts = ["The capital of France is", "Blackwell tensor cores keep their accumulators in"]
    else:
        prompts = [[11, 12, 13, 14, 15, 16], [21, 22, 23, 24, 25, 26, 27, 28, 29]]
    outs = llm.generate(prompts, sp)
    for p, o in zip(prompts, outs):
        print("prompt:", p, "->", o.outputs[0].text if llm.tokenizer is not None else o.outputs[0].token_ids)
    return outs


if __name__ == "__main__":
    main()
