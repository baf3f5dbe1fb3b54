"""numpy front end of the CPU oracle (``fgs_oracle.cpp``). Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.ORACLE_SO
        if not os.path.exists(path):
            path = _build.build_oracle()
        L = C.CDLL(path)
        p, i, f, i64 = C.c_void_p, C.c_int, C.c_float, C.c_int64
        L.fgso_set_contract.restype = i
        L.fgso_set_contract.argtypes = [i]
        L.fgso_max_threads.restype = i
        L.fgso_view_proj.restype = None
        L.fgso_view_proj.argtypes = [i, i, p, p, f, f, f, f, p, p]
        L.fgso_preprocess.restype = i64
        L.fgso_preprocess.argtypes = [i, p, p, p, p, i, i, i, i, p, p, f, f, f, f, i, i, p, p, p, p, p, i64, p]
        L.fgso_higher_msb.restype = C.c_uint32
        L.fgso_higher_msb.argtypes = [C.c_uint32]
        L.fgso_sort.restype = None
        L.fgso_sort.argtypes = [i64, i, i, i, i, p, p, p, p]
        L.fgso_ranges.restype = None
        L.fgso_ranges.argtypes = [i64, p, i, p]
        L.fgso_render.restype = None
        L.fgso_render.argtypes = [i, i, i, i, p, p, p, p, p, p, i, i, p, p, p, p, p]
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def max_threads() -> int:
    return int(lib().fgso_max_threads())


def view_proj(cam):
    v = np.zeros(16, np.float32)
    pr = np.zeros(16, np.float32)
    pos, rot = _f32(cam.position), _f32(cam.rotation)
    lib().fgso_view_proj(cam.width, cam.height, _ptr(pos), _ptr(rot), cam.focal_x, cam.focal_y, cam.zFar, cam.zNear,
                         _ptr(v), _ptr(pr))
    return v, pr


def preprocess(scene, cam, block=(16, 16), rows=(0, -1), capacity=None, feats=None):
    """Returns dict(xy, rgb_depth, conic_opacity, keys, values, counters[P1,P2,V,R])."""
    P = scene.num_vertex
    if feats is None:
        xy = np.zeros((P, 2), np.float32)
        rd = np.zeros((P, 4), np.float32)
        co = np.zeros((P, 4), np.float32)
    else:
        xy, rd, co = feats
    pos, sh, op, cov = _f32(scene.position), _f32(scene.shs), _f32(scene.opacity), _f32(scene.cov3d)
    cpos, crot = _f32(cam.position), _f32(cam.rotation)
    cap = int(capacity) if capacity is not None else max(1 << 20, 16 * P)
    while True:
        keys = np.zeros(cap, np.uint64)
        vals = np.zeros(cap, np.uint32)
        cnt = np.zeros(4, np.int64)
        R = lib().fgso_preprocess(P, _ptr(pos), _ptr(sh), _ptr(op), _ptr(cov), cam.width, cam.height, block[0], block[1],
                                  _ptr(cpos), _ptr(crot), cam.focal_x, cam.focal_y, cam.zFar, cam.zNear,
                                  rows[0], rows[1], _ptr(xy), _ptr(rd), _ptr(co), _ptr(keys), _ptr(vals), cap, _ptr(cnt))
        if R >= 0 or capacity is not None:
            break
        cap = int(cnt[3])
    n = max(int(R), 0)
    return dict(xy=xy, rgb_depth=rd, conic_opacity=co, keys=keys[:n], values=vals[:n], counters=cnt, overflow=R < 0)


def sort_pairs(keys, values, width, height, block=(16, 16)):
    keys = np.ascontiguousarray(keys, np.uint64)
    values = np.ascontiguousarray(values, np.uint32)
    ko, vo = np.empty_like(keys), np.empty_like(values)
    lib().fgso_sort(keys.size, width, height, block[0], block[1], _ptr(keys), _ptr(values), _ptr(ko), _ptr(vo))
    return ko, vo


def tile_ranges(keys_sorted, num_tiles):
    keys_sorted = np.ascontiguousarray(keys_sorted, np.uint64)
    r = np.zeros((num_tiles, 2), np.int32)
    lib().fgso_ranges(keys_sorted.size, _ptr(keys_sorted), num_tiles, _ptr(r))
    return r


def render(width, height, xy, rgb_depth, conic_opacity, values_sorted, ranges, bg=(0, 0, 0), block=(16, 16),
           rows=(0, -1), floats=True):
    gx, gy = (width + block[0] - 1) // block[0], (height + block[1] - 1) // block[1]
    u8 = np.zeros((height, width, 3), np.uint8)
    rgb = np.zeros((height, width, 3), np.float32) if floats else None
    alpha = np.zeros((height, width), np.float32) if floats else None
    depth = np.zeros((height, width), np.float32) if floats else None
    consumed = np.zeros(gx * gy, np.int32)
    bgv = _f32(np.asarray(bg))
    vs = np.ascontiguousarray(values_sorted, np.uint32)
    rg = np.ascontiguousarray(ranges, np.int32)
    lib().fgso_render(width, height, block[0], block[1], _ptr(_f32(xy)), _ptr(_f32(rgb_depth)), _ptr(_f32(conic_opacity)),
                      _ptr(vs), _ptr(rg), _ptr(bgv), rows[0], rows[1], _ptr(u8), _ptr(rgb), _ptr(alpha), _ptr(depth),
                      _ptr(consumed))
    return dict(u8=u8, rgb=rgb, alpha=alpha, depth=depth, consumed=consumed)


def render_frame(scene, cam, bg=(0, 0, 0), block=(16, 16), rows=(0, -1), floats=True):
    """Whole pipeline on the CPU; returns every intermediate."""
    gx, gy = (cam.width + block[0] - 1) // block[0], (cam.height + block[1] - 1) // block[1]
    pre = preprocess(scene, cam, block, rows)
    ks, vs = sort_pairs(pre["keys"], pre["values"], cam.width, cam.height, block)
    rg = tile_ranges(ks, gx * gy)
    out = render(cam.width, cam.height, pre["xy"], pre["rgb_depth"], pre["conic_opacity"], vs, rg, bg, block, rows, floats)
    out.update(pre)
    out.update(keys_sorted=ks, values_sorted=vs, ranges=rg)
    return out
