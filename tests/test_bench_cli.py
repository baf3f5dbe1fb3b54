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


def test_reference_arm_imports_leave_this_library_unloaded():
    """bench.py --impl reference drives the reference's operators through this repository's frame loop; nothing it
    imports for that may load (or even map) libflashgs_b200.so, or the comparison of the two arms would be tainted."""
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "from flashgs_b200.rasterizer import DeviceScene, Rasterizer, TorchCamera\n"
        "from flashgs_b200 import parallel, scenes, _lib\n"
        "assert _lib._lib is None\n"
        "assert 'flashgs_b200.ops' not in sys.modules\n"
        "assert 'libflashgs_b200' not in open('/proc/self/maps').read()\n" % ROOT)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    # and the script itself imports the operator module only inside the branch of its own arm
    src = open(os.path.join(ROOT, "bench.py")).read()
    head = src[: src.index("ours = args.impl ==")]
    assert "from flashgs_b200 import ops" not in head and "_lib" not in head
