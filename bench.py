"""Serving throughput benchmark: output tok/s for a fixed request set.

One "step" of this benchmark is one complete serve of the workload named by
BASELINE.json: 512 requests of uniform-random token ids, 1024 input / 128 output
tokens (EOS ignored), at most 64 requests in flight, block size 16, on a
random-init Llama-3.1-8B-shaped bf16 model with TP = number of GPUs.  W warm-up
serves are followed by exactly K timed serves between barrier + synchronize.

``--model`` selects the other target configurations (their request shapes become
the defaults): ``llama-3.1-70b-fp8`` (TP, block-scaled fp8 weights, 2048 / 256,
c128), ``qwen3-30b-a3b`` and ``deepseek-v3`` (``--parallelism ep-dp``: experts
sharded over all GPUs, attention data parallel, every rank serves its share of
the requests in lockstep).  ``--num-layers`` runs a shallower copy of a preset
(recorded in ``config``; such a line is kernel evidence, not a headline).

Two numbers come out of the same timed serves:
  * ``value``   - output tokens / device time, where device time is the sum of the
    CUDA-event durations of every engine step (forward + sampling kernels), max
    over ranks;
  * ``e2e``     - output tokens / wall time through the public ``LLM`` engine API,
    which every step copies that step's inputs from pinned host memory to the
    device and reads the sampled tokens back to the host.

Launch:  python bench.py --gpus 1            (single process)
         python -m torch.distributed.run --nnodes=1 --nproc-per-node N \
             --master-addr 127.0.0.1 --master-port P bench.py --gpus N
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

REFERENCE_UNAVAILABLE = (
    "the reference is a TPU-only vLLM plugin: it installs with --no-deps into baseline/_ref but "
    "`import vllm_torchtpu.platforms.tpu_platform` fails (portpicker / torch_tpu / jax / libtpu are "
    "not installable offline) and it contains no CUDA or NCCL code path")


# no number is published for these configurations; the closest published ones (TPU v7x-8, other shapes)
PROXIES = {
    "llama-3.1-8b": {"note": "closest published proxy: Fin-R1-7B TP8 1024/1024 c64 on TPU v7x-8", "tok_s": 9654},
    "qwen3-30b-a3b": {"note": "closest published proxy: Qwen3-Coder-30B-A3B TP8+EP 1024/1024 c64 on TPU v7x-8",
                      "tok_s": 5589},
    "deepseek-v3": {"note": "closest published proxy: DeepSeek-V2 TP8+EP 1024/1024 c64 on TPU v7x-8", "tok_s": 1619},
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--parallelism", default=None, choices=["tp", "ep-dp"],
                    help="tp: tensor parallel over all GPUs; ep-dp: expert parallel + data-parallel attention")
    ap.add_argument("--num-layers", type=int, default=0, help="run the first N layers of the preset (0 = all)")
    ap.add_argument("--num-requests", type=int, default=None)
    ap.add_argument("--input-len", type=int, default=None)
    ap.add_argument("--output-len", type=int, default=None)
    ap.add_argument("--concurrency", type=int, default=None)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--kv-cache-dtype", default="auto", help="auto (= model dtype) or fp8 (e4m3 cache; not the headline config)")
    ap.add_argument("--sync-scheduling", action="store_true")
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--warmup-requests", type=int, default=0,
                    help="requests per warm-up serve (0 = the full workload)")
    a = ap.parse_args()
    # request shapes of the target configurations (BASELINE.json configs 2-5)
    shapes = {"llama-3.1-8b": (512, 1024, 128, 64, "tp"), "llama-3.1-70b-fp8": (512, 2048, 256, 128, "tp"),
              "llama-3.1-70b": (512, 2048, 256, 128, "tp"), "qwen3-30b-a3b": (1024, 1024, 256, 256, "ep-dp"),
              "deepseek-v3": (512, 2048, 512, 256, "ep-dp")}
    n, i, o, c, par = shapes.get(a.model, shapes["llama-3.1-8b"])
    a.num_requests = a.num_requests or n
    a.input_len = a.input_len or i
    a.output_len = a.output_len or o
    a.concurrency = a.concurrency or c
    a.parallelism = a.parallelism or par
    return a


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, path: str):
        self.path, self.proc, self.gpu = path, None, gpu_index

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1])); mx.append(float(parts[2])); power.append(float(parts[3]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        if sm:
            # samples taken while idle between serves would pull the median down: keep the samples
            # drawn under load (power well above idle), or all of them when none qualifies
            busy = [c for c, w in zip(sm, power) if w >= 0.5 * max(power)]
            loaded = busy or sm
            out.update(sm_mhz=statistics.median(loaded), sm_max_mhz=max(mx), reasons=sorted(reasons),
                       samples=len(sm), power_w_max=max(power))
        return out


def make_prompts(n, input_len, vocab, seed):
    import numpy as np
    rng = np.random.RandomState(seed)
    return [rng.randint(0, vocab, size=input_len).tolist() for _ in range(n)]


def serve(engine, prompts, sp, concurrency):
    """Closed-loop client: keeps at most `concurrency` requests in flight."""
    nxt, inflight, done = 0, 0, []
    n = len(prompts)
    while nxt < n or inflight > 0 or engine.has_unfinished():
        while nxt < n and inflight < concurrency:
            engine.add_request(prompts[nxt], sp, request_id=f"r{engine.step_count}-{nxt}-{time.monotonic_ns()}")
            nxt += 1
            inflight += 1
        finished = engine.step()
        inflight -= len(finished)
        done += finished
    done += engine.drain()
    for r in done:
        engine.scheduler.requests.pop(r.request_id, None)
    return done


def main():
    args = parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    import torch
    import torch.distributed as dist
    from vllm_torchtpu_b200 import SamplingParams
    from vllm_torchtpu_b200.engine.llm import LLM
    from vllm_torchtpu_b200.ops import cuda as cuda_ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # re-exec under torchrun so that `python bench.py --gpus N` also works
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                   f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port", "29541",
                   os.path.abspath(__file__)] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"WORLD_SIZE={world} does not match --gpus {args.gpus}")

    ep_dp = args.parallelism == "ep-dp" and args.gpus > 1
    model = args.model
    if args.num_layers:
        from vllm_torchtpu_b200.config import model_preset
        model = model_preset(args.model)
        if args.num_layers < model.num_layers:
            model.num_layers = args.num_layers
            model.name = f"{model.name}[first {args.num_layers} layers]"
    # data-parallel attention: every replica keeps its share of the requests in flight
    per_rank_conc = -(-args.concurrency // world) if ep_dp else args.concurrency
    par = (dict(data_parallel_size=args.gpus, enable_expert_parallel=True) if ep_dp
           else dict(tensor_parallel_size=args.gpus, enable_expert_parallel=args.parallelism == "ep-dp"))
    llm = LLM(model, device="cuda", max_num_seqs=per_rank_conc,
              max_num_batched_tokens=args.max_num_batched_tokens, block_size=16,
              kv_cache_dtype=args.kv_cache_dtype,
              max_model_len=args.input_len + args.output_len + 16,
              async_scheduling=not args.sync_scheduling, enforce_eager=args.enforce_eager, **par)
    eng = llm.engine
    runner = eng.runner
    mcfg = eng.cfg.model
    sp = SamplingParams(temperature=0.0, max_tokens=args.output_len, ignore_eos=True)
    prompts = make_prompts(args.num_requests, args.input_len, mcfg.vocab_size, seed=0)
    if ep_dp:
        prompts = prompts[rank::world]
    args.concurrency_total, args.concurrency = args.concurrency, per_rank_conc

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        wp = prompts if not args.warmup_requests else prompts[: args.warmup_requests]
        serve(eng, wp, sp, args.concurrency)
    barrier()
    sampler = ClockSampler(local_rank, f"/tmp/bench_clocks_{rank}.csv")
    if rank == 0:
        sampler.start()
    runner.timing_events = []
    launches0 = runner.launch_counter
    h2d0, d2h0, steps0 = runner.stats["h2d_bytes"], runner.stats["d2h_bytes"], runner.stats["steps"]
    out_tokens, ttfts, tpots = 0, [], []
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        done = serve(eng, prompts, sp, args.concurrency)
        for r in done:
            n_out = len(r.output_token_ids)
            out_tokens += n_out
            if r.first_token_time is not None:
                ttfts.append(r.first_token_time - r.arrival_time)
                if n_out > 1 and r.finish_time is not None:
                    tpots.append((r.finish_time - r.first_token_time) / (n_out - 1))
    barrier()
    wall_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else {}
    durs = [(a.elapsed_time(b), dec, ntok) for a, b, dec, ntok in runner.timing_events]
    device_ms = sum(d for d, _, _ in durs)
    dec_ms = sorted(d for d, dec, _ in durs if dec)
    pre_ms = sorted(d for d, dec, ntok in durs if not dec and ntok >= args.max_num_batched_tokens // 2)
    engine_steps = runner.stats["steps"] - steps0
    status = cuda_ops.check_status()
    t = torch.tensor([wall_s, device_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    wall_s, device_ms = float(t[0]), float(t[1])
    if ep_dp:
        # every replica served its own requests: the job's output is the sum
        tok = torch.tensor([out_tokens], dtype=torch.int64, device="cuda")
        dist.all_reduce(tok)
        out_tokens = int(tok[0])
        st_t = torch.tensor([status], dtype=torch.int32, device="cuda")
        dist.all_reduce(st_t, op=dist.ReduceOp.MAX)
        status = int(st_t[0])
    proxy = None if args.num_layers else PROXIES.get(mcfg.name)
    if rank == 0:
        value = out_tokens / (device_ms / 1e3)
        e2e = out_tokens / wall_s
        line = {
            "metric": f"output tok/s (serving, {args.input_len} in / {args.output_len} out, "
                      f"c{args.concurrency_total})", "value": round(value, 1),
            "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(device_ms / args.steps, 2), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: uniform-random token ids, random-init N(0,0.02) weights",
            "config": {"model": mcfg.name, "global_batch": args.concurrency_total, "seq_len": args.input_len,
                       "parallelism": (f"ep{args.gpus}+dp{args.gpus}-attention" if ep_dp else f"tp{args.gpus}"),
                       "num_layers": mcfg.num_layers, "quantization": mcfg.quantization,
                       "num_requests": args.num_requests,
                       "input_len": args.input_len, "output_len": args.output_len,
                       "max_concurrency": args.concurrency_total, "block_size": 16,
                       "kv_cache_dtype": args.kv_cache_dtype,
                       "step_definition": "one full serve of the request set",
                       "l2": "inputs larger than L2: every engine step streams the weights "
                             "(>= 2 GB per rank) and the KV cache through the 126 MB L2",
                       "timing": "value: sum of per-engine-step CUDA event durations; e2e: wall clock",
                       "async_scheduling": not args.sync_scheduling},
            "e2e": {"value": round(e2e, 1), "unit": "tok/s",
                    "h2d_bytes_per_step": (runner.stats["h2d_bytes"] - h2d0) // args.steps,
                    "d2h_bytes_per_step": (runner.stats["d2h_bytes"] - d2h0) // args.steps,
                    "wall_s_per_step": round(wall_s / args.steps, 3)},
            "gpu_launches": runner.launch_counter - launches0,
            "engine_steps": engine_steps,
            "decode_step_ms_p50": round(dec_ms[len(dec_ms) // 2], 3) if dec_ms else None,
            "decode_steps": len(dec_ms),
            "prefill_step_ms_p50": round(pre_ms[len(pre_ms) // 2], 3) if pre_ms else None,
            "prefill_steps": len(pre_ms),
            "p50_ttft_ms": round(statistics.median(ttfts) * 1e3, 2) if ttfts else None,
            "p50_tpot_ms": round(statistics.median(tpots) * 1e3, 3) if tpots else None,
            "clocks": clocks, "device_status": status,
            "proxy_baseline": proxy and dict(proxy, ratio=round(e2e / proxy["tok_s"], 3)),
        }
        print(json.dumps(line))
    sys.stdout.flush()
    if world == 1:
        return 0
    dist.barrier()
    # Captured CUDA graphs hold NCCL kernels and destroying the communicator under them can block, so
    # multi-rank processes skip interpreter teardown; the registered at-exit handlers still run first.
    from vllm_torchtpu_b200.parallel.state import leave_process
    leave_process(0)


if __name__ == "__main__":
    sys.exit(main())
