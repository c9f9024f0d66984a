"""Child process of the multi-rank serving tests (launched by torch.distributed.run): a tensor-parallel
engine behind the OpenAI app.  Only rank 0 receives the HTTP requests (in-process ASGI client); the
other ranks follow the broadcast request stream.  Rank 0 prints the generated tokens as JSON."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    import faulthandler
    faulthandler.dump_traceback_later(150, exit=True)
    import numpy as np
    from vllm_torchtpu_b200.engine.llm import LLM
    from vllm_torchtpu_b200.parallel.state import leave_process
    device = sys.argv[1] if len(sys.argv) > 1 else "cpu"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    # the CUDA kernels take bf16; the preset's fp32 is the CPU oracle's dtype
    kw = dict(num_gpu_blocks_override=64) if device == "cpu" else dict(num_gpu_blocks_override=256, dtype="bfloat16")
    llm = LLM("tiny-llama", device=device, tensor_parallel_size=world, max_num_seqs=8, max_num_batched_tokens=64,
              block_size=16, async_scheduling="--async" in sys.argv, **kw)
    eng = llm.engine
    assert eng.enable_request_sync()
    if rank != 0:
        eng.follow()
        leave_process(0)
    from starlette.testclient import TestClient
    from vllm_torchtpu_b200.entrypoints.openai_server import build_app
    rng = np.random.RandomState(0)
    prompts = [rng.randint(0, eng.cfg.model.vocab_size, size=n).tolist() for n in (5, 23, 70)]
    app = build_app(eng, "tiny-llama", None)
    toks = []
    with TestClient(app) as c:
        for p in prompts:
            r = c.post("/v1/completions", json={"prompt": p, "max_tokens": 8, "temperature": 0, "ignore_eos": True})
            assert r.status_code == 200, r.text
            toks.append(r.json()["choices"][0]["token_ids"])
        # a request the leader refuses never reaches the followers
        assert c.post("/v1/completions", json={"prompt": [1] * 5000, "max_tokens": 4}).status_code == 500
    app.state.async_engine.shutdown()          # tells the followers to leave
    print("RESULT " + json.dumps({"tokens": toks}), flush=True)
    leave_process(0)


if __name__ == "__main__":
    main()
