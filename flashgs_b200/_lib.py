"""ctypes loader for ``libflashgs_b200.so`` (the C ABI declared in ``include/flashgs_b200.h``).

There is no CPU fallback: if the library is missing the import of the operator
module fails with instructions to build it.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FLASHGS_B200_LIB") or os.path.join(HERE, "libflashgs_b200.so")

TILE_COUNT_WORDS = 65536   # FGS_TILE_COUNT_WORDS
OK, ERR_BAD_ARG, ERR_CUDA, ERR_PAIR_OVERFLOW, ERR_LOOKBACK_TIMEOUT, ERR_TEMP_TOO_SMALL = 0, 1, 2, 4, 8, 16

_p = C.c_void_p
_i = C.c_int
_f = C.c_float
_i64 = C.c_int64

# name -> (restype, argtypes); mirrors include/flashgs_b200.h one to one
SIGNATURES = {
    "fgs_abi_version": (_i, []),
    "fgs_status_string": (C.c_char_p, [_i]),
    "fgs_device_status": (_i, [_i, _p]),
    "fgs_view_proj_matrices": (_i, [_i, _i, _p, _p, _f, _f, _f, _f, _p, _p]),
    "fgs_preprocess": (_i, [_i, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _f, _f, _f, _f,
                            _p, _p, _p, _p, _p, _i64, _p, _p]),
    "fgs_preprocess_strip": (_i, [_i, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _f, _f, _f, _f, _i, _i,
                                  _p, _p, _p, _p, _p, _i64, _p, _p]),
    "fgs_preprocess_strip_culled": (_i, [_i, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _f, _f, _f, _f, _i, _i,
                                         _p, _p, _p, _p, _p, _i64, _p, _p, _i64, _p]),
    "fgs_scene_bounds": (_i, [_i, _p, _p, _p, _p, _p]),
    "fgs_preprocess_prepared": (_i, [_i, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _f, _f, _f, _f, _i, _i,
                                     _p, _p, _p, _p, _p, _i64, _p, _p, _i64, _p, _p, _p]),
    "fgs_preprocess_profile": (_i, [_i, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _f, _f, _f, _f, _i, _i,
                                    _p, _p, _p, _p, _p, _i64, _p, _p, _i64, _p, _p, _p, _p]),
    "fgs_sort_temp_bytes": (C.c_size_t, [_i64]),
    "fgs_sort_pairs": (_i, [_i, _i, _i, _i, _i, _p, C.c_size_t, _p, _p, _p, _p, _p]),
    "fgs_sort_pairs_stable": (_i, [_i, _i, _i, _i, _i, _p, C.c_size_t, _p, _p, _p, _p, _p]),
    "fgs_sort_pairs_counted": (_i, [_i, _i, _i, _i, _i, _p, C.c_size_t, _p, _p, _p, _p, _p, _p]),
    "fgs_sort_static_max_pairs": (_i, []),
    "fgs_sort_pairs_static": (_i, [_i, _i, _i, _i, _i, _p, _p, _p, _p, _p]),
    "fgs_sort_pairs_profile": (_i, [_i, _i, _i, _i, _i, _p, C.c_size_t, _p, _p, _p, _p, _p, _p, _p, _p, _i, _p]),
    "fgs_render_16x16": (_i, [_i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p]),
    "fgs_render_32x16": (_i, [_i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p]),
    "fgs_render_32x32": (_i, [_i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p]),
    "fgs_render_ex": (_i, [_i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _i, _i, _p, _p, _p, _p, _p, _p, _p]),
    "fgs_render_frame": (_i, [_i, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _f, _f, _f, _f, _p, _p, _p, _p, _p, _p, _p, _p, _i64,
                              _p, C.c_size_t, _p, _p, _i, _i, _p, _p, _p, _p, _p]),
    "fgs_tile_ranges": (_i, [_i, _i, _p, _p, _p]),
    "fgs_ply_vertex_count": (C.c_longlong, [C.c_char_p]),
    "fgs_ply_load": (_i, [C.c_char_p, C.c_longlong, _p, _p, _p, _p]),
}

TEST_HOOKS = ("fgs_debug_preprocess_no_column_cull", "fgs_debug_sort_plain", "fgs_debug_sort_skip_publish",
              "fgs_debug_chained_launches")
CHECKED_HOOKS = ("fgs_debug_bounds_report", "fgs_debug_bounds_selftest")   # exported by the checked flavour only
LIB_CHECKED_PATH = os.path.join(HERE, "libflashgs_b200_checked.so")
ERR_BOUNDS = 32

_lib = None


class FlashGSError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, func: str, status: int):
        self.status = status
        super().__init__("%s failed: %s (status %d)" % (func, status_string(status), status))


def load():
    """Load the shared library (once) and attach the prototypes."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "flashgs_b200: %s is missing. Build it with `python -m flashgs_b200.build` "
                "(needs nvcc; there is no CPU fallback)." % LIB_PATH)
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        for name in TEST_HOOKS:   # include/flashgs_b200_test.h: switches for the test-suite, not part of the operator ABI
            fn = getattr(lib, name)
            fn.restype = None
            fn.argtypes = [_i]
        if hasattr(lib, "fgs_debug_bounds_report"):   # the checked flavour (FLASHGS_B200_LIB points at it)
            lib.fgs_debug_bounds_report.restype = C.c_longlong
            lib.fgs_debug_bounds_report.argtypes = [_p, _i]
            lib.fgs_debug_bounds_selftest.restype = _i
            lib.fgs_debug_bounds_selftest.argtypes = [_i, _i, _p, _p]
        _lib = lib
    return _lib


def status_string(status: int) -> str:
    return load().fgs_status_string(int(status)).decode()


def check(func: str, status: int) -> None:
    if status != OK:
        raise FlashGSError(func, status)
