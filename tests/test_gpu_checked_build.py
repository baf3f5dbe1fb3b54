"""The small GPU cases once more under the checked flavour of the library.

libflashgs_b200_checked.so is the same source built with -DFGS_DEBUG_BOUNDS: every kernel compares each global
store, each index it derived from data and each computed shared-memory index with its extent before the access,
skips an access that falls outside and counts it (include/flashgs_b200_test.h). It stands in for a memory checker,
which cannot be run on the machines these tests run on. The cases run in a child pytest process whose
FLASHGS_B200_LIB points at the checked flavour; a fixture in conftest.py then asserts after every test that no
violation was counted. Nothing here faults or traps a GPU: the one test that makes the check fire does so on a pair
of plain integers inside a one-thread kernel.
"""
import ctypes
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKED = os.path.join(ROOT, "flashgs_b200", "libflashgs_b200_checked.so")
IN_CHILD = os.environ.get("FLASHGS_B200_LIB", "") == CHECKED


@pytest.mark.skipif(IN_CHILD, reason="this is the child run")
def test_small_cases_under_the_checked_flavour():
    if not os.path.exists(CHECKED):
        pytest.skip("checked flavour not built (python -m flashgs_b200.build --checked)")
    env = dict(os.environ, FLASHGS_B200_LIB=CHECKED)
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider",
                        os.path.join(ROOT, "tests", "test_gpu_parity.py"), os.path.join(ROOT, "tests", "test_gpu_checked_build.py"),
                        "-k", "not full_size and not example_script"],
                       capture_output=True, text=True, timeout=1500, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
    assert "passed" in r.stdout and "test_the_check_counts_and_skips" not in r.stdout.split("short test summary")[-1]


@pytest.mark.skipif(not IN_CHILD, reason="runs in the child process, under the checked flavour")
@pytest.mark.allow_bounds_violations
def test_the_check_counts_and_skips():
    from flashgs_b200 import _lib
    L = _lib.load()
    assert hasattr(L, "fgs_debug_bounds_selftest"), "the child must have loaded the checked flavour"
    out = (ctypes.c_ulonglong * 12)()
    assert L.fgs_debug_bounds_report(out, 1) == 0
    touched = torch.zeros(1, device="cuda:0", dtype=torch.int32)
    assert L.fgs_debug_bounds_selftest(3, 4, touched.data_ptr(), None) == 0       # inside: the access happens
    torch.cuda.synchronize()
    assert int(touched[0]) == 1 and L.fgs_debug_bounds_report(out, 0) == 0
    touched.zero_()
    assert L.fgs_debug_bounds_selftest(7, 4, touched.data_ptr(), None) == 0       # outside: counted, recorded, skipped
    assert L.fgs_debug_bounds_selftest(-1, 4, touched.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert int(touched[0]) == 0
    assert L.fgs_device_status(0, None) & _lib.ERR_BOUNDS
    assert L.fgs_debug_bounds_report(out, 1) == 2
    assert list(out[:8]) == [0] * 8 and out[8] == 2 and out[10] == 7 and out[11] == 4 and out[9] > 0
    assert L.fgs_device_status(1, None) == 0                                        # cleared by the report above
