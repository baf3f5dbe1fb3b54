"""bench.py on a machine without a GPU: the arm that times the CPU restatement prints ONE JSON line with the contract's keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_port_arm_prints_one_json_line(oracle_lib):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "port", "--workload", "C1", "--cpu-sample", "0.1"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "steps", "warmup", "ms_per_step", "higher_is_better", "dtype", "data", "config", "cpu_baseline"):
        assert key in d, key
    assert d["impl"] == "port" and d["unit"] == "frames/s" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert "workload" in d["config"] and "model" not in d["config"]
