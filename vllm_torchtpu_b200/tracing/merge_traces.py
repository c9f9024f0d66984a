"""Merge the per-rank Chrome traces of a profiling session into one timeline.

Every rank writes ``<dir>/rank_<N>/trace_*.json`` (see profiler.py).  The merged file keeps all
events, gives each rank its own process-id range (so the ranks appear as separate process groups in
Perfetto / chrome://tracing) and labels the groups ``rank N``.  Clock skew between ranks can be
removed by aligning a named event that every rank records at the same moment (a barrier annotation).

    python -m vllm_torchtpu_b200.tracing.merge_traces /tmp/b200_profile -o merged.json [--align barrier]

(reference: src/vllm_torchtpu/tools/merge_xplane.py — merges the per-host profiler planes of a
multi-host run into one file.)
"""
from __future__ import annotations

import argparse
import glob
import gzip
import json
import os
import re
from typing import Optional

PID_STRIDE = 1_000_000


def _load(path: str) -> dict:
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rt") as f:
        data = json.load(f)
    return {"traceEvents": data} if isinstance(data, list) else data


def find_rank_traces(root: str) -> dict:
    """rank -> newest trace file under ``root/rank_<N>/``."""
    out = {}
    for d in sorted(glob.glob(os.path.join(root, "rank_*"))):
        m = re.search(r"rank_(\d+)$", d)
        files = sorted(glob.glob(os.path.join(d, "trace*.json")) + glob.glob(os.path.join(d, "trace*.json.gz")),
                       key=os.path.getmtime)
        if m and files:
            out[int(m.group(1))] = files[-1]
    return out


def merge(traces: dict, align_event: Optional[str] = None) -> dict:
    """``traces``: rank -> loaded trace dict.  Returns one trace dict."""
    events, offsets = [], {}
    if align_event:
        firsts = {}
        for rank, tr in traces.items():
            ts = [e["ts"] for e in tr.get("traceEvents", []) if e.get("name") == align_event and "ts" in e]
            if ts:
                firsts[rank] = min(ts)
        if firsts:
            base = min(firsts.values())
            offsets = {r: base - t for r, t in firsts.items()}
    for rank in sorted(traces):
        shift = offsets.get(rank, 0)
        seen_pids = set()
        for e in traces[rank].get("traceEvents", []):
            e = dict(e)
            pid = e.get("pid", 0)
            pid = pid if isinstance(pid, int) else (hash(str(pid)) % (PID_STRIDE - 1))
            e["pid"] = rank * PID_STRIDE + (pid % PID_STRIDE)
            seen_pids.add(e["pid"])
            if shift and "ts" in e:
                e["ts"] = e["ts"] + shift
            if e.get("ph") == "M" and e.get("name") == "process_name":
                args = dict(e.get("args") or {})
                args["name"] = f"rank {rank}: {args.get('name', '')}".rstrip(": ")
                e["args"] = args
            events.append(e)
        for pid in sorted(seen_pids):
            events.append({"ph": "M", "name": "process_sort_index", "pid": pid, "tid": 0,
                           "args": {"sort_index": pid}})
    return {"traceEvents": events, "displayTimeUnit": "ms",
            "otherData": {"ranks": sorted(traces), "aligned_on": align_event if offsets else None}}


def merge_dir(root: str, out_path: str, align_event: Optional[str] = None) -> dict:
    files = find_rank_traces(root)
    if not files:
        raise FileNotFoundError(f"no rank_*/trace*.json under {root}")
    merged = merge({r: _load(p) for r, p in files.items()}, align_event)
    opener = gzip.open if out_path.endswith(".gz") else open
    with opener(out_path, "wt") as f:
        json.dump(merged, f)
    return {"ranks": sorted(files), "events": len(merged["traceEvents"]), "output": out_path}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("root")
    ap.add_argument("-o", "--output", default="merged_trace.json")
    ap.add_argument("--align", default=None, help="name of an event all ranks record at the same moment")
    a = ap.parse_args(argv)
    print(json.dumps(merge_dir(a.root, a.output, a.align)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
