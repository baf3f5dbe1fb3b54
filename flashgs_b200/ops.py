"""Operator API of the reference, backed by the sm_100a library.

Same function names, positional arguments and argument meaning as the module the
reference binds with pybind11 (``flash_gaussian_splatting.ops``,
csrc/pybind.cpp:122-271): PyTorch tensors in, results written into caller-owned
tensors. Each function is a thin shim that hands raw pointers to the C ABI of
``libflashgs_b200.so``; camera position/rotation and the background colour are
read on the host and therefore must be CPU tensors (csrc/pybind.cpp:131-143,177),
everything else must live on the current CUDA device.

Differences from the reference, all on the strict side:
  * a non-zero status of the C ABI raises ``RuntimeError`` (the reference checks
    no launch at all);
  * output tensors must be contiguous (the reference would silently write into a
    temporary, csrc/pybind.cpp:145-148);
  * the render ops never write outside the image (the reference does for empty
    tiles on a partial last tile row, csrc/cuda_rasterizer/render.cu:530-546).
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import FlashGSError  # noqa: F401  (re-exported)

_L = _lib.load()


def _stream() -> int:
    # The reference always launches on the legacy default stream (its bindings pass no
    # stream); torch's current stream is that stream unless the caller changed it.
    return torch.cuda.current_stream().cuda_stream


def _dev(t: torch.Tensor, name: str, dtype=None) -> int:
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor" % name)
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError("%s must have dtype %s, got %s" % (name, dtype, t.dtype))
    return t.data_ptr()


def _in(t: torch.Tensor, name: str, dtype) -> torch.Tensor:
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor" % name)
    if t.dtype != dtype:
        raise RuntimeError("%s must have dtype %s, got %s" % (name, dtype, t.dtype))
    return t if t.is_contiguous() else t.contiguous()


def _out(t: torch.Tensor, name: str, dtype) -> torch.Tensor:
    if not t.is_contiguous():
        raise RuntimeError("%s is written in place and must be contiguous" % name)
    return _in(t, name, dtype)


def _host(t: torch.Tensor, name: str, n: int) -> torch.Tensor:
    if t.is_cuda:
        raise RuntimeError("%s is read on the host and must be a CPU tensor" % name)
    t = t.to(torch.float32).contiguous()
    if t.numel() < n:
        raise RuntimeError("%s needs %d elements" % (name, n))
    return t


def loadPly(path: str):
    """Scene loading is not part of the per-frame path; see ``flashgs_b200.ply.load_ply``."""
    from .ply import load_ply
    return load_ply(path)


def preprocess(orig_points, shs, opacities, cov3Ds, width, height, block_x, block_y,
               position, rotation, focal_x, focal_y, zFar, zNear,
               points_xy, rgb_depth, conic_opacity,
               gaussian_keys_unsorted, gaussian_values_unsorted, curr_offset,
               tile_row_begin: int = 0, tile_row_end: int = -1, cull_scratch=None, scene_bounds=None,
               tile_counts=None) -> None:
    """csrc/pybind.cpp:122-150. The trailing keyword arguments restrict the pairs to a strip of tile rows;
    ``cull_scratch`` (int32 CUDA tensor, at least P + 1 elements) lets a strip list the Gaussians that can reach it
    first and run the expensive kernel on those only; ``scene_bounds`` (what ``prepare_scene`` returned for these
    arrays) makes that first kernel read 16 bytes per Gaussian instead of 40; ``tile_counts`` (int32 CUDA tensor of
    65536 elements) receives the pairs per tile, which ``sort_gaussian(..., tile_counts=)`` then need not count again."""
    f32 = torch.float32
    pts = _in(orig_points, "orig_points", f32)
    sh = _in(shs, "shs", f32)
    op = _in(opacities, "opacities", f32)
    cov = _in(cov3Ds, "cov3Ds", f32)
    pos = _host(position, "position", 3)
    rot = _host(rotation, "rotation", 9)
    xy = _out(points_xy, "points_xy", f32)
    rd = _out(rgb_depth, "rgb_depth", f32)
    co = _out(conic_opacity, "conic_opacity", f32)
    keys = _out(gaussian_keys_unsorted, "gaussian_keys_unsorted", torch.int64)
    vals = _out(gaussian_values_unsorted, "gaussian_values_unsorted", torch.int32)
    off = _out(curr_offset, "curr_offset", torch.int32)
    P = int(op.size(0))
    cap = min(int(keys.numel()), int(vals.numel()))
    scratch = None if cull_scratch is None else _out(cull_scratch, "cull_scratch", torch.int32)
    bounds = None
    if scene_bounds is not None:
        bounds = _in(scene_bounds, "scene_bounds", f32)
        if scratch is None or bounds.numel() != 4 * P or not scene_bounds.is_contiguous():
            raise RuntimeError("scene_bounds needs cull_scratch and one contiguous [4] record per Gaussian")
    counts = None
    if tile_counts is not None:
        counts = _out(tile_counts, "tile_counts", torch.int32)
        if counts.numel() < _lib.TILE_COUNT_WORDS:
            raise RuntimeError("tile_counts needs %d elements" % _lib.TILE_COUNT_WORDS)
    st = _L.fgs_preprocess_prepared(P, pts.data_ptr(), sh.data_ptr(), op.data_ptr(), cov.data_ptr(),
                                    int(width), int(height), int(block_x), int(block_y),
                                    pos.data_ptr(), rot.data_ptr(),
                                    float(focal_x), float(focal_y), float(zFar), float(zNear),
                                    int(tile_row_begin), int(tile_row_end),
                                    xy.data_ptr(), rd.data_ptr(), co.data_ptr(),
                                    keys.data_ptr(), vals.data_ptr(), cap, off.data_ptr(),
                                    None if scratch is None else scratch.data_ptr(),
                                    0 if scratch is None else int(scratch.numel()),
                                    None if bounds is None else bounds.data_ptr(),
                                    None if counts is None else counts.data_ptr(), _stream())
    _lib.check("preprocess", st)


def prepare_scene(orig_points, opacities, cov3Ds, out=None):
    """Once per scene (no reference counterpart): the ``[P, 4]`` float32 records -- position and
    trace(covariance) * ln(256 * opacity) -- that ``preprocess(..., cull_scratch=, scene_bounds=)`` streams to list the
    Gaussians that can reach a strip. They depend on the scene only, not on the camera."""
    f32 = torch.float32
    pts, op, cov = _in(orig_points, "orig_points", f32), _in(opacities, "opacities", f32), _in(cov3Ds, "cov3Ds", f32)
    P = int(op.size(0))
    if out is None:
        out = torch.empty((P, 4), device=op.device, dtype=f32)
    out = _out(out, "out", f32)
    if out.numel() < 4 * P:
        raise RuntimeError("out needs 4 floats per Gaussian")
    _lib.check("prepare_scene", _L.fgs_scene_bounds(P, pts.data_ptr(), op.data_ptr(), cov.data_ptr(), out.data_ptr(), _stream()))
    return out


def get_sort_buffer_size(num_rendered: int) -> int:
    """csrc/pybind.cpp:165-168."""
    return int(_L.fgs_sort_temp_bytes(int(num_rendered)))


def sort_gaussian(num_rendered, width, height, block_x, block_y, list_sorting_space,
                  gaussian_keys_unsorted, gaussian_values_unsorted,
                  gaussian_keys_sorted, gaussian_values_sorted, stable: bool = False, tile_counts=None) -> None:
    """csrc/pybind.cpp:152-163. Pairs with identical sorted key bits come out in ascending order of their values
    (the frame is then the same bytes every run); ``stable=True`` keeps them in input order, which is the reference's
    library-sort contract, through the slower look-back passes (see ``fgs_sort_pairs`` in include/flashgs_b200.h).
    ``tile_counts``: the table ``preprocess(..., tile_counts=)`` filled for this pair list; the sort starts from it."""
    n = int(num_rendered)
    ki = _in(gaussian_keys_unsorted, "gaussian_keys_unsorted", torch.int64)
    vi = _in(gaussian_values_unsorted, "gaussian_values_unsorted", torch.int32)
    ko = _out(gaussian_keys_sorted, "gaussian_keys_sorted", torch.int64)
    vo = _out(gaussian_values_sorted, "gaussian_values_sorted", torch.int32)
    if n > min(ki.numel(), vi.numel(), ko.numel(), vo.numel()):
        raise RuntimeError("sort_gaussian: num_rendered (%d) exceeds the pair buffers" % n)
    tmp = list_sorting_space
    if not tmp.is_cuda or not tmp.is_contiguous():
        raise RuntimeError("list_sorting_space must be a contiguous CUDA tensor")
    args = (n, int(width), int(height), int(block_x), int(block_y), tmp.data_ptr(), tmp.numel() * tmp.element_size(),
            ki.data_ptr(), vi.data_ptr(), ko.data_ptr(), vo.data_ptr())
    if stable:
        st = _L.fgs_sort_pairs_stable(*args, _stream())
    elif tile_counts is not None:
        counts = _in(tile_counts, "tile_counts", torch.int32)
        if counts.numel() < _lib.TILE_COUNT_WORDS or not tile_counts.is_contiguous():
            raise RuntimeError("tile_counts needs %d contiguous elements" % _lib.TILE_COUNT_WORDS)
        st = _L.fgs_sort_pairs_counted(*args, counts.data_ptr(), _stream())
    else:
        st = _L.fgs_sort_pairs(*args, _stream())
    _lib.check("sort_gaussian", st)


def _check_frame_buffers(block_x, block_y, width, height, ranges, out_color, num_rendered=None, records=(), lists=()):
    """Size checks shared by the render entry points: a short caller buffer must raise here, not become an
    out-of-bounds store on the device."""
    tiles = ((int(width) + block_x - 1) // block_x) * ((int(height) + block_y - 1) // block_y)
    if ranges.numel() < 2 * tiles:
        raise RuntimeError("ranges holds %d tiles, the image has %d" % (ranges.numel() // 2, tiles))
    if out_color is not None:
        if not out_color.is_cuda or not out_color.is_contiguous() or out_color.element_size() != 1:
            raise RuntimeError("out_color must be a contiguous CUDA int8/uint8 tensor")
        if out_color.numel() < int(width) * int(height) * 3:
            raise RuntimeError("out_color is smaller than height*width*3")
    if num_rendered is not None:
        for t, nm in lists:
            if t.numel() < int(num_rendered):
                raise RuntimeError("%s holds %d pairs, num_rendered is %d" % (nm, t.numel(), int(num_rendered)))
    rows = None
    for t, nm, per in records:
        if t.numel() % per:
            raise RuntimeError("%s must have %d floats per Gaussian" % (nm, per))
        rows = t.numel() // per if rows is None else rows
        if t.numel() // per != rows:
            raise RuntimeError("points_xy, rgb_depth and conic_opacity must describe the same number of Gaussians")
    return tiles


def _render(fn_name, block_x, block_y, num_rendered, width, height, points_xy, rgb_depth, conic_opacity,
            gaussian_keys_sorted, gaussian_values_sorted, ranges, bg_color, out_color, tile_order=None, consumed=None):
    if tile_order is not None or consumed is not None:   # the keyword extensions live in the general entry point
        return render_ex(block_x, block_y, num_rendered, width, height, points_xy, rgb_depth, conic_opacity,
                         gaussian_keys_sorted, gaussian_values_sorted, ranges, bg_color, out_color=out_color,
                         consumed=consumed, tile_order=tile_order)
    f32 = torch.float32
    xy = _in(points_xy, "points_xy", f32)
    rd = _in(rgb_depth, "rgb_depth", f32)
    co = _in(conic_opacity, "conic_opacity", f32)
    ks = _in(gaussian_keys_sorted, "gaussian_keys_sorted", torch.int64)
    vs = _in(gaussian_values_sorted, "gaussian_values_sorted", torch.int32)
    rg = _out(ranges, "ranges", torch.int32)
    bg = _host(bg_color, "bg_color", 3)
    if out_color is None:
        raise RuntimeError("out_color is required")
    _check_frame_buffers(block_x, block_y, width, height, rg, out_color, num_rendered,
                         records=((xy, "points_xy", 2), (rd, "rgb_depth", 4), (co, "conic_opacity", 4)),
                         lists=((ks, "gaussian_keys_sorted"), (vs, "gaussian_values_sorted")))
    st = getattr(_L, fn_name)(int(num_rendered), int(width), int(height),
                              xy.data_ptr(), rd.data_ptr(), co.data_ptr(), ks.data_ptr(), vs.data_ptr(),
                              rg.data_ptr(), bg.data_ptr(), out_color.data_ptr(), _stream())
    _lib.check(fn_name, st)


def render_16x16(num_rendered, width, height, points_xy, rgb_depth, conic_opacity,
                 gaussian_keys_sorted, gaussian_values_sorted, ranges, bg_color, out_color,
                 tile_order=None, consumed=None) -> None:
    """csrc/pybind.cpp:170-188. Keyword extensions: see ``render_ex``."""
    _render("fgs_render_16x16", 16, 16, num_rendered, width, height, points_xy, rgb_depth, conic_opacity,
            gaussian_keys_sorted, gaussian_values_sorted, ranges, bg_color, out_color, tile_order, consumed)


def render_32x16(num_rendered, width, height, points_xy, rgb_depth, conic_opacity,
                 gaussian_keys_sorted, gaussian_values_sorted, ranges, bg_color, out_color,
                 tile_order=None, consumed=None) -> None:
    """csrc/pybind.cpp:190-208. Keyword extensions: see ``render_ex``."""
    _render("fgs_render_32x16", 32, 16, num_rendered, width, height, points_xy, rgb_depth, conic_opacity,
            gaussian_keys_sorted, gaussian_values_sorted, ranges, bg_color, out_color, tile_order, consumed)


def render_32x32(num_rendered, width, height, points_xy, rgb_depth, conic_opacity,
                 gaussian_keys_sorted, gaussian_values_sorted, ranges, bg_color, out_color,
                 tile_order=None, consumed=None) -> None:
    """csrc/pybind.cpp:210-228. Keyword extensions: see ``render_ex``."""
    _render("fgs_render_32x32", 32, 32, num_rendered, width, height, points_xy, rgb_depth, conic_opacity,
            gaussian_keys_sorted, gaussian_values_sorted, ranges, bg_color, out_color, tile_order, consumed)


def render_ex(block_x, block_y, num_rendered, width, height, points_xy, rgb_depth, conic_opacity,
              gaussian_keys_sorted, gaussian_values_sorted, ranges, bg_color,
              out_color=None, out_rgb=None, out_alpha=None, out_depth=None, consumed=None,
              tile_row_begin: int = 0, tile_row_end: int = -1, tile_order=None) -> None:
    """General render call (no reference counterpart): strips of tile rows, optional float outputs, the number of
    splats blended per tile (``consumed``, int32 per tile of the frame) and the order in which the tiles are taken up
    (``tile_order``, int32 whole-frame tile ids, every tile of the rendered rows once). The image does not depend on
    the order, the time does: a launch ends with its slowest tiles, so ``tile_order_from(consumed, ...)`` of the
    previous frame of the same view -- heaviest tiles first -- shortens its tail."""
    f32 = torch.float32
    bg = _host(bg_color, "bg_color", 3)
    ptr = lambda t: 0 if t is None else t.data_ptr()  # noqa: E731
    xy, rd, co = _in(points_xy, "points_xy", f32), _in(rgb_depth, "rgb_depth", f32), _in(conic_opacity, "conic_opacity", f32)
    ks = _in(gaussian_keys_sorted, "gaussian_keys_sorted", torch.int64)
    vs = _in(gaussian_values_sorted, "gaussian_values_sorted", torch.int32)
    rg = _out(ranges, "ranges", torch.int32)
    tiles = _check_frame_buffers(int(block_x), int(block_y), width, height, rg, out_color, num_rendered,
                                 records=((xy, "points_xy", 2), (rd, "rgb_depth", 4), (co, "conic_opacity", 4)),
                                 lists=((ks, "gaussian_keys_sorted"), (vs, "gaussian_values_sorted")))
    pixels = int(width) * int(height)
    for t, nm, dt, need in ((out_rgb, "out_rgb", f32, 3 * pixels), (out_alpha, "out_alpha", f32, pixels),
                            (out_depth, "out_depth", f32, pixels), (consumed, "consumed", torch.int32, tiles)):
        if t is not None:
            _out(t, nm, dt)
            if t.numel() < need:
                raise RuntimeError("%s needs %d elements, has %d" % (nm, need, t.numel()))
    order = None
    if tile_order is not None:
        order = _in(tile_order, "tile_order", torch.int32)
        gx = (int(width) + int(block_x) - 1) // int(block_x)
        gy = (int(height) + int(block_y) - 1) // int(block_y)
        r0 = max(0, int(tile_row_begin))
        r1 = gy if int(tile_row_end) < 0 or int(tile_row_end) > gy else int(tile_row_end)
        if not tile_order.is_contiguous() or order.numel() < max(0, r1 - r0) * gx:
            raise RuntimeError("tile_order needs one contiguous entry per tile of the rendered rows (%d)" % (max(0, r1 - r0) * gx))
    st = _L.fgs_render_ex(int(block_x), int(block_y), int(num_rendered), int(width), int(height),
                          xy.data_ptr(), rd.data_ptr(), co.data_ptr(), ks.data_ptr(), vs.data_ptr(),
                          rg.data_ptr(), bg.data_ptr(),
                          int(tile_row_begin), int(tile_row_end),
                          ptr(out_color), ptr(out_rgb), ptr(out_alpha), ptr(out_depth), ptr(consumed),
                          None if order is None else order.data_ptr(), _stream())
    _lib.check("render_ex", st)


def tile_order_from(consumed, width, height, block_x: int = 16, block_y: int = 16, tile_row_begin: int = 0, tile_row_end: int = -1):
    """The tiles of the rendered rows in descending order of ``consumed`` (what ``render_ex(..., consumed=)`` wrote for
    an earlier frame of the same view), as the int32 tensor ``render_ex(..., tile_order=)`` takes."""
    gx = (int(width) + block_x - 1) // block_x
    gy = (int(height) + block_y - 1) // block_y
    r0 = max(0, int(tile_row_begin))
    r1 = gy if int(tile_row_end) < 0 or int(tile_row_end) > gy else int(tile_row_end)
    part = consumed[r0 * gx: r1 * gx]
    return (torch.argsort(part, descending=True, stable=True) + r0 * gx).to(torch.int32)


def render_frame(orig_points, shs, opacities, cov3Ds, width, height, block_x, block_y,
                 position, rotation, focal_x, focal_y, zFar, zNear, bg_color,
                 points_xy, rgb_depth, conic_opacity,
                 gaussian_keys_unsorted, gaussian_values_unsorted, gaussian_keys_sorted, gaussian_values_sorted,
                 list_sorting_space, ranges, curr_offset, out_color,
                 tile_row_begin: int = 0, tile_row_end: int = -1, consumed=None, tile_order=None, scene_bounds=None) -> None:
    """One frame in one call with no host round trip (no reference counterpart): what ``preprocess``,
    ``sort_gaussian`` and ``render_*`` do in sequence, the pair count staying in ``curr_offset`` on the device.
    Read ``curr_offset`` afterwards if the count is wanted; an overflow of the pair buffers shows in ``device_status``."""
    f32 = torch.float32
    pos = _host(position, "position", 3)
    rot = _host(rotation, "rotation", 9)
    bg = _host(bg_color, "bg_color", 3)
    ku = _out(gaussian_keys_unsorted, "gaussian_keys_unsorted", torch.int64)
    vu = _out(gaussian_values_unsorted, "gaussian_values_unsorted", torch.int32)
    ks = _out(gaussian_keys_sorted, "gaussian_keys_sorted", torch.int64)
    vs = _out(gaussian_values_sorted, "gaussian_values_sorted", torch.int32)
    cap = min(int(ku.numel()), int(vu.numel()), int(ks.numel()), int(vs.numel()))
    tmp = list_sorting_space
    if not tmp.is_cuda or not tmp.is_contiguous():
        raise RuntimeError("list_sorting_space must be a contiguous CUDA tensor")
    if out_color is None:
        raise RuntimeError("out_color is required")
    op = _in(opacities, "opacities", f32)
    P = int(op.size(0))
    xy, rd, co = _out(points_xy, "points_xy", f32), _out(rgb_depth, "rgb_depth", f32), _out(conic_opacity, "conic_opacity", f32)
    rg = _out(ranges, "ranges", torch.int32)
    tiles = _check_frame_buffers(int(block_x), int(block_y), width, height, rg, out_color)
    if (consumed is not None and consumed.numel() < tiles) or (tile_order is not None and not tile_order.is_contiguous()):
        raise RuntimeError("consumed needs one element per tile (%d); tile_order must be contiguous" % tiles)
    if tile_order is not None:
        gx = (int(width) + int(block_x) - 1) // int(block_x)
        gy = (int(height) + int(block_y) - 1) // int(block_y)
        r1 = gy if int(tile_row_end) < 0 or int(tile_row_end) > gy else int(tile_row_end)
        if tile_order.numel() < max(0, r1 - max(0, int(tile_row_begin))) * gx:
            raise RuntimeError("tile_order needs one entry per tile of the rendered rows")
    if xy.numel() < 2 * P or rd.numel() < 4 * P or co.numel() < 4 * P:
        raise RuntimeError("points_xy, rgb_depth and conic_opacity need one record per Gaussian (%d)" % P)
    bounds = None
    if scene_bounds is not None:
        bounds = _in(scene_bounds, "scene_bounds", f32)
        if bounds.numel() != 4 * P or not scene_bounds.is_contiguous():
            raise RuntimeError("scene_bounds needs one contiguous [4] record per Gaussian")
    st = _L.fgs_render_frame(P, _in(orig_points, "orig_points", f32).data_ptr(), _in(shs, "shs", f32).data_ptr(),
                             op.data_ptr(), _in(cov3Ds, "cov3Ds", f32).data_ptr(),
                             int(width), int(height), int(block_x), int(block_y), pos.data_ptr(), rot.data_ptr(),
                             float(focal_x), float(focal_y), float(zFar), float(zNear), bg.data_ptr(),
                             xy.data_ptr(), rd.data_ptr(), co.data_ptr(),
                             ku.data_ptr(), vu.data_ptr(), ks.data_ptr(), vs.data_ptr(), cap,
                             tmp.data_ptr(), tmp.numel() * tmp.element_size(),
                             rg.data_ptr(), _out(curr_offset, "curr_offset", torch.int32).data_ptr(),
                             int(tile_row_begin), int(tile_row_end), out_color.data_ptr(),
                             None if consumed is None else _out(consumed, "consumed", torch.int32).data_ptr(),
                             None if tile_order is None else _in(tile_order, "tile_order", torch.int32).data_ptr(),
                             None if bounds is None else bounds.data_ptr(), _stream())
    _lib.check("render_frame", st)


def device_status(reset: bool = True) -> int:
    """OR of the error bits raised by kernels on the current device since the last reset (synchronises)."""
    return int(_L.fgs_device_status(1 if reset else 0, _stream()))
