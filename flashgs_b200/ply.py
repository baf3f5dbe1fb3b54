"""Scene loading: the reference's ``ops.loadPly`` (csrc/pybind.cpp:58-120) on top of the C ABI.

``load_ply(path)`` returns ``(num_vertex, position[N,3], shs[N,48], opacity[N], cov3d[N,6])`` as fp32
CPU tensors, like the reference. ``save_ply`` writes the same 62-float record layout from raw model
parameters; tests and tools use it to make PLY files.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib

HEADER_PROPS = (["x", "y", "z", "nx", "ny", "nz"] + ["f_dc_%d" % i for i in range(3)] +
                ["f_rest_%d" % i for i in range(45)] + ["opacity"] + ["scale_%d" % i for i in range(3)] +
                ["rot_%d" % i for i in range(4)])


def load_ply(path: str):
    lib = _lib.load()
    lib.fgs_ply_vertex_count.restype = C.c_longlong
    lib.fgs_ply_vertex_count.argtypes = [C.c_char_p]
    lib.fgs_ply_load.restype = C.c_int
    lib.fgs_ply_load.argtypes = [C.c_char_p, C.c_longlong] + [C.c_void_p] * 4
    n = int(lib.fgs_ply_vertex_count(str(path).encode()))
    if n <= 0:
        raise RuntimeError("loadPly: cannot read a positive vertex count from %s" % path)
    pos = torch.empty((n, 3), dtype=torch.float32)
    shs = torch.empty((n, 48), dtype=torch.float32)
    opa = torch.empty((n,), dtype=torch.float32)
    cov = torch.empty((n, 6), dtype=torch.float32)
    st = lib.fgs_ply_load(str(path).encode(), n, pos.data_ptr(), shs.data_ptr(), opa.data_ptr(), cov.data_ptr())
    _lib.check("loadPly", st)
    return n, pos, shs, opa, cov


def save_ply(path: str, position, f_dc, f_rest, opacity_logit, log_scale, rotation) -> None:
    """Write a 3DGS model: f_dc [N,3], f_rest [N,45] channel-major (15 coefficients of R, then G, then B)."""
    position = np.asarray(position, np.float32)
    n = position.shape[0]
    rec = np.zeros((n, 62), np.float32)
    rec[:, 0:3] = position
    rec[:, 6:9] = np.asarray(f_dc, np.float32)
    rec[:, 9:54] = np.asarray(f_rest, np.float32).reshape(n, 45)
    rec[:, 54] = np.asarray(opacity_logit, np.float32).reshape(n)
    rec[:, 55:58] = np.asarray(log_scale, np.float32)
    rec[:, 58:62] = np.asarray(rotation, np.float32)
    header = "ply\nformat binary_little_endian 1.0\nelement vertex %d\n" % n
    header += "".join("property float %s\n" % p for p in HEADER_PROPS) + "end_header\n"
    with open(path, "wb") as f:
        f.write(header.encode())
        f.write(rec.tobytes())
