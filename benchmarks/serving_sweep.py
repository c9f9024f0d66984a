#!/usr/bin/env python3
"""Closed-loop serving sweep over (input length, output length, concurrency) cells.

Every cell serves ``--num-prompts`` synthetic requests through the engine's public API at a fixed number
of requests in flight and writes ``isl<I>_osl<O>_c<C>.json`` (output / total tokens per second, median TTFT
and TPOT, completed requests) into ``--results-dir`` — the files ``benchmarks/check_regression.py`` gates.
Cells come from ``--cells I:O:C[,I:O:C...]`` or from a JSON config ``{"model": ..., "engine": {...},
"cells": [[I, O, C], ...]}`` (the reference keeps one such config per model,
reference: scripts/vllm/benchmarking/configs/, scripts/vllm/benchmarking/run_benchmarks.sh).

Under tensor parallelism launch with ``python -m torch.distributed.run``; rank 0 writes the files."""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def run_cell(llm, isl: int, osl: int, conc: int, num_prompts: int, seed: int) -> dict:
    import numpy as np

    from vllm_torchtpu_b200.sampling_params import SamplingParams
    eng = llm.engine
    rng = np.random.default_rng(seed)
    vocab = eng.cfg.model.vocab_size
    prompts = [rng.integers(10, vocab - 10, size=isl).tolist() for _ in range(num_prompts)]
    sp = SamplingParams(temperature=0.0, max_tokens=osl, ignore_eos=True)
    pending, live, done = list(range(num_prompts)), {}, []
    t0 = time.perf_counter()
    while pending or live:
        while pending and len(live) < conc:
            i = pending.pop(0)
            rid = eng.add_request(prompts[i], sp)
            live[rid] = time.perf_counter()
        for req in eng.step():
            start = live.pop(req.request_id, None)
            if start is None:
                continue
            end = time.perf_counter()
            first = req.first_token_time or end
            n_out = len(req.output_token_ids)
            ttft = max(0.0, first - req.arrival_time)
            tpot = (end - first) / max(1, n_out - 1)
            done.append((ttft, tpot, n_out))
    wall = time.perf_counter() - t0
    out_tokens = sum(n for _, _, n in done)
    return {"isl": isl, "osl": osl, "concurrency": conc, "num_prompts": num_prompts, "completed": len(done),
            "output_tok_s": out_tokens / wall, "total_tok_s": (out_tokens + isl * len(done)) / wall,
            "p50_ttft_ms": statistics.median(t for t, _, _ in done) * 1e3 if done else None,
            "p50_tpot_ms": statistics.median(t for _, t, _ in done) * 1e3 if done else None,
            "wall_s": wall}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", help="JSON file with model, engine arguments and cells")
    ap.add_argument("--model", default="tiny-llama")
    ap.add_argument("--cells", default="128:16:4", help="I:O:C[,I:O:C...]")
    ap.add_argument("--num-prompts", type=int, default=0, help="per cell (default 4 x concurrency)")
    ap.add_argument("--results-dir", default="benchmark_results")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--tensor-parallel-size", type=int, default=int(os.environ.get("WORLD_SIZE", "1")))
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    engine_args, model = {}, a.model
    cells = [tuple(int(v) for v in c.split(":")) for c in a.cells.split(",")]
    if a.config:
        cfg = json.loads(Path(a.config).read_text())
        model = cfg.get("model", model)
        engine_args = dict(cfg.get("engine", {}))
        cells = [tuple(c) for c in cfg.get("cells", cells)]
    from vllm_torchtpu_b200.engine.llm import LLM
    need = max(i + o for i, o, _ in cells) + 16
    engine_args.setdefault("max_model_len", need)
    engine_args.setdefault("max_num_seqs", max(c for _, _, c in cells))
    llm = LLM(model, device=a.device, tensor_parallel_size=a.tensor_parallel_size, seed=a.seed, **engine_args)
    rank = int(os.environ.get("RANK", "0"))
    out = Path(a.results_dir)
    if rank == 0:
        out.mkdir(parents=True, exist_ok=True)
    for isl, osl, conc in cells:
        n = a.num_prompts or 4 * conc
        run_cell(llm, isl, osl, conc, min(n, conc), a.seed)            # warm-up: shapes, graphs
        r = run_cell(llm, isl, osl, conc, n, a.seed + 1)
        if rank == 0:
            (out / f"isl{isl}_osl{osl}_c{conc}.json").write_text(json.dumps(r, indent=2) + "\n")
            print(json.dumps(r))
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        from vllm_torchtpu_b200.parallel.state import leave_process
        leave_process(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
