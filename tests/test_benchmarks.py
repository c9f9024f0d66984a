"""The serving sweep and the regression gate that reads its files."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "benchmarks"))

import check_regression as cr  # noqa: E402


def _cell(out=1000.0, total=9000.0, ttft=50.0, tpot=10.0, completed=64):
    return {"output_tok_s": out, "total_tok_s": total, "p50_ttft_ms": ttft, "p50_tpot_ms": tpot,
            "completed": completed}


def test_perf_gate_directions_tolerance_and_completion_floor():
    base = {"isl1024_osl128_c64": _cell()}
    ok = {"isl1024_osl128_c64": _cell(out=960.0, ttft=52.0)}          # -4 % throughput, +4 % latency
    assert cr.gate_perf(ok, base, 0.05)[1] == 0
    slow = {"isl1024_osl128_c64": _cell(out=940.0)}                    # -6 %
    rows, failed = cr.gate_perf(slow, base, 0.05)
    assert failed == 1 and any(r[1] == "output_tok_s" and r[5] == "FAIL" for r in rows)
    late = {"isl1024_osl128_c64": _cell(tpot=10.6)}
    assert cr.gate_perf(late, base, 0.05)[1] == 1
    dropped = {"isl1024_osl128_c64": _cell(completed=60)}              # 93.75 % of the requests
    assert cr.gate_perf(dropped, base, 0.05)[1] == 1
    assert cr.gate_perf({}, base, 0.05)[1] == 1                        # a missing cell fails
    assert cr.gate_perf({"isl8_osl8_c1": _cell()}, {}, 0.05)[1] == 0   # a cell without baseline is reported only


def test_calibrate_takes_medians_and_can_leave_ttft_ungated(tmp_path):
    for i, v in enumerate((900.0, 1000.0, 1100.0)):
        d = tmp_path / f"run{i}"
        d.mkdir()
        (d / "isl128_osl16_c256.json").write_text(json.dumps(_cell(out=v, ttft=100.0 * (i + 1))))
    runs = [tmp_path / f"run{i}" for i in range(3)]
    b = cr.calibrate_perf(runs)
    assert b["isl128_osl16_c256"]["output_tok_s"] == 1000.0 and b["isl128_osl16_c256"]["p50_ttft_ms"] == 200.0
    b = cr.calibrate_perf(runs, ttft_max_concurrency=64)
    assert "p50_ttft_ms" not in b["isl128_osl16_c256"]
    # a result 3x later in TTFT passes against that baseline
    assert cr.gate_perf({"isl128_osl16_c256": _cell(ttft=600.0)}, b, 0.05)[1] == 0


def test_accuracy_gate_scales_with_the_stderr_of_the_difference():
    base = {"gsm8k": {"exact_match": 0.90, "exact_match_stderr": 0.01}}
    near = {"gsm8k": {"exact_match": 0.88, "exact_match_stderr": 0.01}}   # -0.02 < 1.645 * 0.0141
    assert cr.gate_eval(near, base, 0.0)[1] == 0
    far = {"gsm8k": {"exact_match": 0.86, "exact_match_stderr": 0.01}}
    assert cr.gate_eval(far, base, 0.0)[1] == 1
    assert cr.gate_eval(far, base, 0.05)[1] == 0                          # the absolute floor is wider
    assert cr.gate_eval({}, base, 0.05)[1] == 1


def test_sweep_writes_cells_the_gate_accepts(tmp_path):
    out = tmp_path / "res"
    r = subprocess.run([sys.executable, str(ROOT / "benchmarks" / "serving_sweep.py"), "--device", "cpu",
                        "--cells", "16:4:2", "--num-prompts", "4", "--results-dir", str(out)],
                       capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    cell = json.loads((out / "isl16_osl4_c2.json").read_text())
    assert cell["completed"] == 4 and cell["output_tok_s"] > 0 and cell["p50_tpot_ms"] is not None
    base = out.parent / "baseline.json"
    assert cr.main(["--calibrate", "--results-dir", str(out), "--output", str(base)]) == 0
    assert cr.main(["--results-dir", str(out), "--baseline", str(base)]) == 0
