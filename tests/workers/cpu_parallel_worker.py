"""Child process of the CPU multi-rank tests (gloo, launched by torch.distributed.run): the same
prompts through an engine with tensor or pipeline parallelism; rank 0 prints the tokens as JSON."""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    import faulthandler
    faulthandler.dump_traceback_later(150, exit=True)
    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.engine.llm import LLM
    world = int(os.environ.get("WORLD_SIZE", "1"))
    mode = sys.argv[1] if len(sys.argv) > 1 else "tp"
    model = sys.argv[2] if len(sys.argv) > 2 else "tiny-llama"
    kw = {}
    if mode in ("tp", "tplora"):
        kw["tensor_parallel_size"] = world
    elif mode == "dcp":
        # KV cache dealt over the ranks by position (runs of 2 tokens), attention merged by log-sum-exp
        kw["tensor_parallel_size"] = world
        kw["decode_context_parallel_size"] = world
        kw["cp_kv_cache_interleave_size"] = 2 if "--il2" in sys.argv else 1
    elif mode == "pcp":
        # prefill chunks of 16 tokens and more are cut into pieces over the ranks
        os.environ["B200_PCP_MIN_TOKENS"] = "16"
        kw["prefill_context_parallel_size"] = world if "--tp2" not in sys.argv else world // 2
        kw["tensor_parallel_size"] = 1 if "--tp2" not in sys.argv else 2
    elif mode == "pp":
        kw["pipeline_parallel_size"] = world
    elif mode == "ep":
        kw["tensor_parallel_size"] = world
        kw["enable_expert_parallel"] = True
    elif mode == "dpep":
        kw["data_parallel_size"] = world
        kw["enable_expert_parallel"] = True
    if "--moe-pipeline" in sys.argv:
        # the all-gather plane in three chunks per step, chunks of at least two tokens
        os.environ["B200_MOE_PIPELINE_CHUNKS"], os.environ["B200_MOE_PIPELINE_MIN_CHUNK_TOKENS"] = "3", "2"
    if "--dp-vocab" in sys.argv:
        kw["additional_config"] = {"dp_vocab_parallel": True}
    llm = LLM(model, device="cpu", max_num_seqs=8, max_num_batched_tokens=64, block_size=16,
              num_gpu_blocks_override=64, async_scheduling="--async" in sys.argv, **kw)
    rng = np.random.RandomState(0)
    vocab = llm.engine.cfg.model.vocab_size
    prompts = [rng.randint(0, vocab, size=n).tolist() for n in (5, 23, 70)]
    rank = int(os.environ.get("RANK", "0"))
    mine = prompts
    if mode == "dpep":
        # every replica serves its own requests: rank 0 gets two prompts, rank 1 one (uneven on purpose)
        mine = [p for i, p in enumerate(prompts) if i % world == rank]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    if mode == "tplora":
        # one adapter on a fused column-parallel target, a plain column-parallel sub-projection and a
        # row-parallel target; full-size matrices, identical on every rank, sharded by the wiring
        import torch
        mc = llm.engine.cfg.model
        g = torch.Generator().manual_seed(11)
        weights = {}
        for li in range(mc.num_layers):
            pre = f"model.layers.{li}."
            weights[pre + "self_attn.q_proj"] = (torch.randn(4, mc.hidden_size, generator=g) * 0.3,
                                                 torch.randn(mc.num_q_heads * mc.head_dim, 4, generator=g) * 0.3)
            weights[pre + "mlp.up_proj"] = (torch.randn(4, mc.hidden_size, generator=g) * 0.3,
                                            torch.randn(mc.intermediate_size, 4, generator=g) * 0.3)
            weights[pre + "mlp.down_proj"] = (torch.randn(4, mc.intermediate_size, generator=g) * 0.3,
                                              torch.randn(mc.hidden_size, 4, generator=g) * 0.3)
        assert llm.engine.add_lora("ad", 4, 16.0, weights)
        sp = [SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True, lora_name="ad" if i != 1 else None)
              for i in range(len(mine))]
    if "--closed-loop" in sys.argv:
        # the benchmark's client: at most one request in flight per replica, new ones added as others finish,
        # two serves back to back (the replicas must leave each serve in the same step)
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
        import bench
        toks = None
        for _ in range(2):
            done = bench.serve(llm.engine, mine, sp, 1)
            by_prompt = {tuple(r.prompt_token_ids): r.output_token_ids for r in done}
            toks = [list(by_prompt[tuple(p)]) for p in mine]
    else:
        outs = llm.generate(mine, sp)
        toks = [o.outputs[0].token_ids for o in outs]
    if mode == "dpep":
        import torch.distributed as dist
        every = [None] * world
        dist.all_gather_object(every, toks)
        merged = [None] * len(prompts)
        for r, part in enumerate(every):
            for j, t in enumerate(part):
                merged[r + j * world] = t
        toks = merged
    if "--export" in sys.argv:
        # every rank calls the exporter; rank 0 writes the directory
        from vllm_torchtpu_b200.export import export_serving_dir
        export_serving_dir(llm, sys.argv[sys.argv.index("--export") + 1])
    if "--dp-vocab" in sys.argv:
        # each replica keeps half of the embedding table and of the lm_head
        m = llm.engine.runner.model
        assert m.embed.shape[0] == -(-vocab // world) and m.lm_head.shape[0] == -(-vocab // world), m.embed.shape
    if mode == "pcp":
        assert llm.engine.runner.stats.get("pcp_split_steps", 0) >= 2, llm.engine.runner.stats
    if "--moe-pipeline" in sys.argv:
        from vllm_torchtpu_b200.layers import moe as moe_layer
        assert moe_layer.PIPELINED_CALLS > 0
    if rank == 0:
        print("RESULT " + json.dumps({"tokens": toks}), flush=True)
    if world > 1:
        import torch.distributed as dist
        from vllm_torchtpu_b200.parallel.state import leave_process
        dist.barrier()
        leave_process(0)


if __name__ == "__main__":
    main()
