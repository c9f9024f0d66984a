"""Child process: the same prompts through a TP engine (fused NVLink plane or NCCL plane);
rank 0 prints the generated tokens as JSON."""
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    import faulthandler
    faulthandler.dump_traceback_later(90, exit=True)      # a stuck rank prints where it is and exits
    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.config import ModelConfig
    from vllm_torchtpu_b200.engine.llm import LLM
    from vllm_torchtpu_b200.ops import cuda
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cfg = ModelConfig(name="tp-test", num_layers=2, hidden_size=1024, num_q_heads=8, num_kv_heads=8, head_dim=128,
                      intermediate_size=2048, vocab_size=4096, max_model_len=512, dtype=torch.bfloat16)
    ep = "--moe" in sys.argv
    if ep:
        cfg = ModelConfig(name="ep-test", architecture="qwen3_moe", num_layers=2, hidden_size=1024, num_q_heads=8,
                          num_kv_heads=8, head_dim=128, intermediate_size=2048, vocab_size=4096,
                          max_model_len=512, dtype=torch.bfloat16, qk_norm=True, num_experts=8,
                          num_experts_per_tok=2, moe_intermediate_size=256)
    par = dict(tensor_parallel_size=world)
    if "--mqa" in sys.argv or "--dcp" in sys.argv:
        cfg.num_kv_heads = 1
    if "--dcp" in sys.argv and world > 1:           # the cache of the one KV head dealt over the ranks by position
        par.update(decode_context_parallel_size=world, cp_kv_cache_interleave_size=1)
    if "--pp" in sys.argv:
        par = dict(pipeline_parallel_size=world)
    if "--dpep" in sys.argv:                       # data-parallel attention, experts sharded over the replicas
        par = dict(data_parallel_size=world)
        ep = True
    llm = LLM(cfg, device="cuda", max_num_seqs=8, max_num_batched_tokens=256,
              num_gpu_blocks_override=256, enforce_eager="--eager" in sys.argv, enable_expert_parallel=ep, **par)
    rng = np.random.RandomState(0)
    prompts = [rng.randint(0, 4096, size=n).tolist() for n in (8, 33, 70, 150)]
    rank = int(os.environ.get("RANK", "0"))
    mine = prompts
    if "--dpep" in sys.argv:
        mine = [p for i, p in enumerate(prompts) if i % world == rank]
    lp = "--lp" in sys.argv
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True, logprobs=1 if lp else None,
                        prompt_logprobs=0 if lp else None)
    outs = llm.generate(mine, sp)
    torch.cuda.synchronize()
    status = cuda.check_status()
    toks = [o.outputs[0].token_ids for o in outs]
    if "--dpep" in sys.argv and world > 1:
        import torch.distributed as dist
        every = [None] * world
        dist.all_gather_object(every, toks)
        merged = [None] * len(prompts)
        for r, part in enumerate(every):
            for j, t in enumerate(part):
                merged[r + j * world] = t
        toks = merged
    res = {"tokens": toks, "status": status,
           "persistent_decode": getattr(llm.engine.runner.model, "decode_mega", None) is not None}
    if lp:
        # log-probabilities of the sampled tokens (decode steps) and of every prompt token (prefill)
        res["sample_lp"] = [[e["logprob"] for e in o.outputs[0].logprobs] for o in outs]
        res["prompt_lp"] = [[e["logprob"] for e in o.prompt_logprobs[1:]] for o in outs]
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    if world > 1:
        import torch.distributed as dist
        from vllm_torchtpu_b200.parallel.state import leave_process
        dist.barrier()
        leave_process(0)


if __name__ == "__main__":
    main()
