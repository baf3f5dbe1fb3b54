import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    config.addinivalue_line("markers", "allow_bounds_violations: the test provokes the checked build's index check itself")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle_lib():
    from oracle import build, oracle
    build.build_oracle()
    return oracle


@pytest.fixture(autouse=True)
def _no_index_violations(request):
    """Under the checked flavour of the library (FLASHGS_B200_LIB pointing at libflashgs_b200_checked.so) every GPU
    test also asserts that no kernel met an index outside its extent."""
    yield
    if "gpu" not in request.keywords or "allow_bounds_violations" in request.keywords:
        return
    from flashgs_b200 import _lib
    lib = _lib._lib
    if lib is not None and hasattr(lib, "fgs_debug_bounds_report"):
        import ctypes
        out = (ctypes.c_ulonglong * 12)()
        total = lib.fgs_debug_bounds_report(out, 1)
        assert total == 0, "index violations (count, line, index, extent) x (preprocess, sort, render): %s" % list(out)
