#!/usr/bin/env python3
"""Gate a benchmark run against stored baselines.

Two kinds of result are understood:

* perf cells written by ``benchmarks/serving_sweep.py``: one JSON per (input length, output length,
  concurrency) cell, named ``isl<I>_osl<O>_c<C>.json``.  Latencies may grow and throughputs may shrink by
  at most ``--tolerance`` (5 % unless told otherwise); a cell that completed fewer than 95 % of the
  baseline's requests fails whatever its speed.
* accuracy numbers (``--mode eval``): ``{"task": {"metric": x, "metric_stderr": s}}``.  The gate is on the
  difference of two independent runs, so its noise is hypot(stderr_baseline, stderr_run); the run fails when
  it is below the baseline by more than ``max(tolerance, 1.645 * that)`` (one-sided 95 %).

``--calibrate DIR [DIR ...]`` writes a baseline from the medians of several runs of the same code.
Behaviour of the reference's gate (reference: scripts/vllm/benchmarking/check_regression.py:121-230).
"""
from __future__ import annotations

import argparse
import json
import math
import re
import statistics
import sys
from pathlib import Path

CELL = re.compile(r"^isl(\d+)_osl(\d+)_c(\d+)$")
# (field, +1 if larger is better / -1 if smaller is better)
PERF_FIELDS = (("output_tok_s", +1), ("total_tok_s", +1), ("p50_ttft_ms", -1), ("p50_tpot_ms", -1))
COMPLETED_FLOOR = 0.95
Z95 = 1.645
EPS = 1e-9


def load_cells(directory: Path) -> dict:
    cells = {}
    for f in sorted(directory.glob("isl*_osl*_c*.json")):
        if CELL.match(f.stem):
            cells[f.stem] = json.loads(f.read_text())
    return cells


def gate_perf(results: dict, baseline: dict, tolerance: float) -> tuple[list, int]:
    """Rows (cell, field, actual, baseline, ratio, verdict) and the number of failures."""
    rows, failed = [], 0
    for cell in sorted(set(results) | set(baseline)):
        if cell not in baseline:
            rows.append((cell, "-", None, None, None, "no baseline"))
            continue
        if cell not in results:
            rows.append((cell, "-", None, None, None, "FAIL (no result)"))
            failed += 1
            continue
        got, base = results[cell], baseline[cell]
        if base.get("completed") and got.get("completed") is not None:
            ratio = got["completed"] / base["completed"]
            if ratio < COMPLETED_FLOOR:
                rows.append((cell, "completed", got["completed"], base["completed"], ratio, "FAIL"))
                failed += 1
        for field, sign in PERF_FIELDS:
            a, b = got.get(field), base.get(field)
            if a is None or not b:
                continue                      # a field the baseline does not carry is not gated
            ratio = float(a) / float(b)
            ok = ratio >= 1.0 - tolerance - EPS if sign > 0 else ratio <= 1.0 + tolerance + EPS
            rows.append((cell, field, float(a), float(b), ratio, "pass" if ok else "FAIL"))
            failed += 0 if ok else 1
    return rows, failed


def calibrate_perf(directories: list, ttft_max_concurrency=None) -> dict:
    """Median of every gated field over the given runs.  Under closed-loop load beyond what one prefill step
    admits, median TTFT is queue position rather than latency: cells above ``ttft_max_concurrency`` leave
    it out so that the gate ignores it."""
    per_cell: dict = {}
    for d in directories:
        for cell, r in load_cells(Path(d)).items():
            slot = per_cell.setdefault(cell, {"completed": []})
            slot["completed"].append(r.get("completed", 0))
            for field, _ in PERF_FIELDS:
                if r.get(field) is not None:
                    slot.setdefault(field, []).append(float(r[field]))
    out = {}
    for cell, slot in per_cell.items():
        conc = int(CELL.match(cell).group(3))
        entry = {"completed": int(statistics.median(slot["completed"])), "runs": len(slot["completed"])}
        for field, _ in PERF_FIELDS:
            if field == "p50_ttft_ms" and ttft_max_concurrency is not None and conc > ttft_max_concurrency:
                continue
            if slot.get(field):
                entry[field] = statistics.median(slot[field])
        out[cell] = entry
    return out


def gate_eval(results: dict, baseline: dict, tolerance: float) -> tuple[list, int]:
    rows, failed = [], 0
    for task in sorted(baseline):
        if task not in results:
            rows.append((task, "-", None, None, None, "FAIL (no result)"))
            failed += 1
            continue
        for metric, b in baseline[task].items():
            if metric.endswith("_stderr") or metric not in results[task]:
                continue
            a = float(results[task][metric])
            se = math.hypot(float(baseline[task].get(metric + "_stderr", 0.0)),
                            float(results[task].get(metric + "_stderr", 0.0)))
            allowed = max(tolerance, Z95 * se)
            ok = a - float(b) >= -allowed - EPS
            rows.append((task, metric, a, float(b), a - float(b), "pass" if ok else "FAIL"))
            failed += 0 if ok else 1
    return rows, failed


def print_rows(rows, title):
    print(f"\n## {title}\n")
    print("| key | metric | actual | baseline | ratio / delta | verdict |")
    print("|---|---|---:|---:|---:|---|")
    for key, metric, a, b, r, verdict in rows:
        fmt = lambda v: "-" if v is None else f"{v:.4g}"
        print(f"| `{key}` | {metric} | {fmt(a)} | {fmt(b)} | {fmt(r)} | {verdict} |")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--mode", choices=["perf", "eval"], default="perf")
    ap.add_argument("--results-dir", nargs="+", required=True)
    ap.add_argument("--baseline")
    ap.add_argument("--tolerance", type=float, default=0.05)
    ap.add_argument("--calibrate", action="store_true", help="write a baseline from the runs in --results-dir")
    ap.add_argument("--gate-ttft-max-concurrency", type=int, default=None)
    ap.add_argument("--output", help="where --calibrate writes (default: stdout)")
    a = ap.parse_args(argv)
    if a.calibrate:
        if a.mode != "perf":
            ap.error("--calibrate is for perf results")
        text = json.dumps(calibrate_perf(a.results_dir, a.gate_ttft_max_concurrency), indent=2, sort_keys=True)
        if a.output:
            Path(a.output).write_text(text + "\n")
        else:
            print(text)
        return 0
    if not a.baseline:
        ap.error("--baseline is required unless --calibrate is given")
    baseline = json.loads(Path(a.baseline).read_text())
    if a.mode == "perf":
        rows, failed = gate_perf(load_cells(Path(a.results_dir[0])), baseline, a.tolerance)
        print_rows(rows, f"perf gate, tolerance {a.tolerance * 100:.1f} %")
    else:
        results = json.loads((Path(a.results_dir[0]) / "eval.json").read_text())
        rows, failed = gate_eval(results, baseline, a.tolerance)
        print_rows(rows, f"accuracy gate, floor {a.tolerance:.3f} or 1.645 x stderr of the difference")
    print(f"\n{failed} failure(s)")
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
