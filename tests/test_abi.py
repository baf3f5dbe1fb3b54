"""CPU-side checks of the C ABI: the library loads, exports what the header declares, and its host-only logic."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from flashgs_b200 import _lib, scenes
from helpers import identity_camera

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols(header="flashgs_b200.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fgs_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), "missing export " + n
        assert n in _lib.SIGNATURES, "no ctypes prototype for " + n
    hooks = _declared_symbols("flashgs_b200_test.h")      # the test-only switches have a header of their own
    assert sorted(hooks) == sorted(_lib.TEST_HOOKS + _lib.CHECKED_HOOKS)
    for n in _lib.TEST_HOOKS:
        assert hasattr(lib, n), "missing export " + n
    for n in _lib.CHECKED_HOOKS:       # the checked flavour's own exports are not in the product library
        assert not hasattr(lib, n), n
    if os.path.exists(_lib.LIB_CHECKED_PATH):
        checked = C.CDLL(_lib.LIB_CHECKED_PATH)
        for n in names + list(_lib.TEST_HOOKS + _lib.CHECKED_HOOKS):
            assert hasattr(checked, n), "checked flavour: missing export " + n
    assert lib.fgs_abi_version() == 3
    assert _lib.status_string(0) == "ok"
    assert "overflow" in _lib.status_string(_lib.ERR_PAIR_OVERFLOW)


def test_view_proj_matches_oracle(oracle_lib):
    lib = _lib.load()
    for name in ("C1", "C2", "C5"):
        w = scenes.WORKLOADS[name]
        for cam in scenes.make_cameras(w)[:3] + [identity_camera()]:
            v = np.zeros(16, np.float32)
            p = np.zeros(16, np.float32)
            pos = np.ascontiguousarray(cam.position, np.float32)
            rot = np.ascontiguousarray(cam.rotation, np.float32)
            st = lib.fgs_view_proj_matrices(cam.width, cam.height, pos.ctypes.data, rot.ctypes.data,
                                            cam.focal_x, cam.focal_y, cam.zFar, cam.zNear, v.ctypes.data, p.ctypes.data)
            assert st == 0
            ov, op = oracle_lib.view_proj(cam)
            assert (v.view(np.uint32) == ov.view(np.uint32)).all()
            assert (p.view(np.uint32) == op.view(np.uint32)).all()
            # p_view = R^T (p - pos): the camera position maps to the origin, +z is forward
            M = v.reshape(4, 4).T
            np.testing.assert_allclose(M @ np.append(pos, 1.0), [0, 0, 0, 1], atol=2e-5)
            fwd = rot[:, 2]
            np.testing.assert_allclose((M @ np.append(pos + fwd, 1.0))[:3], [0, 0, 1], atol=2e-5)


def test_argument_checks_need_no_gpu():
    lib = _lib.load()
    assert lib.fgs_view_proj_matrices(0, 10, None, None, 1.0, 1.0, 100.0, 0.01, None, None) == _lib.ERR_BAD_ARG
    assert lib.fgs_sort_pairs(-1, 64, 64, 16, 16, None, 0, None, None, None, None, None) == _lib.ERR_BAD_ARG
    assert lib.fgs_sort_pairs(0, 64, 64, 16, 16, None, 0, None, None, None, None, None) == _lib.OK
    assert lib.fgs_sort_pairs(5, 64, 64, 16, 16, None, 0, None, None, None, None, None) == _lib.ERR_BAD_ARG
    assert lib.fgs_render_ex(8, 8, 0, 64, 64, None, None, None, None, None, None, None, 0, -1,
                             None, None, None, None, None, None, None) == _lib.ERR_BAD_ARG
    assert lib.fgs_preprocess(-1, *([None] * 4), 64, 64, 16, 16, None, None, 1.0, 1.0, 100.0, 0.01,
                              *([None] * 5), 0, None, None) == _lib.ERR_BAD_ARG
    assert lib.fgs_tile_ranges(0, 0, None, None, None) == _lib.ERR_BAD_ARG
    # scratch for the index list of the Gaussians that reach a strip must hold P + 1 ints (checked before anything runs)
    assert lib.fgs_preprocess_strip_culled(-1, *([None] * 4), 64, 64, 16, 16, None, None, 1.0, 1.0, 100.0, 0.01, 0, 2,
                                           *([None] * 5), 0, None, None, 0, None) == _lib.ERR_BAD_ARG   # a negative count first
    assert lib.fgs_sort_pairs_static(-1, 64, 64, 16, 16, None, None, None, None, None) == _lib.ERR_BAD_ARG
    assert lib.fgs_sort_pairs_stable(-1, 64, 64, 16, 16, None, 0, None, None, None, None, None) == _lib.ERR_BAD_ARG
    dummy = (C.c_int * 4)()
    assert lib.fgs_preprocess_strip_culled(10, *([None] * 4), 64, 64, 16, 16, None, None, 1.0, 1.0, 100.0, 0.01, 0, 2,
                                           *([None] * 5), 0, None, C.addressof(dummy), 4, None) == _lib.ERR_TEMP_TOO_SMALL


def test_sort_temp_bytes_is_monotone_and_covers_alternate_buffers():
    lib = _lib.load()
    prev = 0
    for n in (0, 1, 4095, 4096, 4097, 1 << 20, 1 << 27):
        b = lib.fgs_sort_temp_bytes(n)
        assert b >= 12 * n and b >= prev and b % 256 == 0
        prev = b
    assert lib.fgs_sort_temp_bytes(1 << 27) < 2.2 * (1 << 30)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU fallback"):
        _lib.load()


def test_integration_shim_compiles_against_the_reference_header(tmp_path):
    """The C++ binding shown in INTEGRATION.md (the reference's operators implemented on top of this library's C ABI)
    is real code: it compiles against the reference's csrc/ops.h where a checkout of the reference is present."""
    import shutil
    import subprocess
    from oracle import build as oracle_build
    ops_h = os.path.join(oracle_build.REFERENCE_ROOT, "csrc", "ops.h")
    cuda_inc = os.path.join(oracle_build.CUDA_HOME, "include")
    if not (os.path.exists(ops_h) and os.path.exists(os.path.join(cuda_inc, "cuda_runtime.h")) and shutil.which(oracle_build.CXX)):
        pytest.skip("needs the reference checkout, the CUDA headers and a C++ compiler")
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    code = re.search(r"```cpp\n(.*?)```", text, flags=re.S).group(1)
    assert "namespace flashgs" in code and "fgs_preprocess(" in code and "fgs_sort_pairs(" in code and "fgs_render_16x16(" in code
    src = tmp_path / "ops_b200.cpp"
    src.write_text(code)
    r = subprocess.run([oracle_build.CXX, "-std=c++17", "-fsyntax-only", "-Wall", "-I", os.path.dirname(ops_h),
                        "-I", os.path.join(ROOT, "include"), "-I", cuda_inc, str(src)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
