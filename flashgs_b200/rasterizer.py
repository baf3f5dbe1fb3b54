"""Statically allocated rasterizer: the host-side frame loop of the reference's example.

Mirrors ``Scene`` / ``Rasterizer.forward`` of the reference (example.py:10-27, 45-94):
all scratch (pair buffers, sort space, tile ranges, feature records) is allocated once,
and a frame is ``preprocess -> read the pair count -> sort_gaussian -> render_16x16``
through the operator API. The operator module is a parameter so that the same loop can
drive any implementation of that API.

Additions that the reference does not have:
  * ``rows=(begin, end)`` renders only a strip of tile rows (one frame split across GPUs);
  * the output image can be a caller-owned, reused buffer instead of a fresh
    ``torch.zeros`` per frame (example.py:89).
"""
from __future__ import annotations

import torch

from .scenes import Camera, Scene


def _default_ops():
    """This repository's operator module. Imported on first use only, so that driving ANOTHER implementation of the
    operator API through the classes below (``ops=`` given) never loads this repository's shared library."""
    from . import ops
    return ops


class DeviceScene:
    """Gaussian buffers on the device (example.py:10-27)."""

    def __init__(self, scene: Scene, device):
        self.device = torch.device(device)
        self.num_vertex = scene.num_vertex
        self.position = torch.from_numpy(scene.position).to(self.device)
        self.shs = torch.from_numpy(scene.shs).to(self.device)
        self.opacity = torch.from_numpy(scene.opacity).to(self.device)
        self.cov3d = torch.from_numpy(scene.cov3d).to(self.device)


class TorchCamera:
    """Camera with CPU tensors for position / rotation, as example.py:30-41 builds it."""

    def __init__(self, cam: Camera):
        self.id, self.img_name = cam.id, cam.img_name
        self.width, self.height = cam.width, cam.height
        self.position = torch.from_numpy(cam.position.copy())
        self.rotation = torch.from_numpy(cam.rotation.copy())
        self.focal_x, self.focal_y = cam.focal_x, cam.focal_y
        self.zFar, self.zNear = cam.zFar, cam.zNear


class Rasterizer:
    def __init__(self, scene: DeviceScene, MAX_NUM_RENDERED: int, MAX_NUM_TILES: int, ops=None, block=(16, 16)):
        dev = scene.device
        ops = ops if ops is not None else _default_ops()
        self.ops = ops
        self.block = block
        z = lambda n, dt: torch.zeros(n, device=dev, dtype=dt)  # noqa: E731
        self.gaussian_keys_unsorted = z(MAX_NUM_RENDERED, torch.int64)
        self.gaussian_values_unsorted = z(MAX_NUM_RENDERED, torch.int32)
        self.gaussian_keys_sorted = z(MAX_NUM_RENDERED, torch.int64)
        self.gaussian_values_sorted = z(MAX_NUM_RENDERED, torch.int32)
        self.MAX_NUM_RENDERED = MAX_NUM_RENDERED
        self.MAX_NUM_TILES = MAX_NUM_TILES
        self.SORT_BUFFER_SIZE = ops.get_sort_buffer_size(MAX_NUM_RENDERED)
        self.list_sorting_space = z(self.SORT_BUFFER_SIZE, torch.int8)
        self.ranges = z((MAX_NUM_TILES, 2), torch.int32)
        self.curr_offset = z(1, torch.int32)
        self.points_xy = z((scene.num_vertex, 2), torch.float32)
        self.rgb_depth = z((scene.num_vertex, 4), torch.float32)
        self.conic_opacity = z((scene.num_vertex, 4), torch.float32)
        self.num_rendered = 0
        # The sort's scratch is idle while preprocess runs: its head holds preprocess's list of the Gaussians that can
        # reach the image (P + 1 ints), so that the expensive kernel only runs on those.
        need = 4 * (scene.num_vertex + 1)
        ours = hasattr(ops, "render_frame")   # another operator module (the reference's) has no such argument
        self.cull_scratch = (self.list_sorting_space[:need].view(torch.int32) if ours and self.SORT_BUFFER_SIZE >= need else None)
        # ... and that list is found from 16-byte records prepared once per scene (position and a bound on the reach)
        self.scene_bounds = (ops.prepare_scene(scene.position, scene.opacity, scene.cov3d)
                             if self.cull_scratch is not None and hasattr(ops, "prepare_scene") else None)
        # preprocess knows every pair's tile when it emits it: it counts the pairs per tile for the sort that follows
        self.tile_counts = z(65536, torch.int32) if ours else None
        # Tiles are taken up heaviest first (by what the blend consumed per tile a few frames ago): a launch ends with its
        # slowest tiles. The order is refreshed every `order_refresh` frames; 0 turns it off.
        self.order_refresh = 16 if ours and hasattr(ops, "tile_order_from") else 0
        self.tile_consumed = z(MAX_NUM_TILES, torch.int32) if self.order_refresh else None
        self._order, self._order_key, self._frames = None, None, 0
        self._count_host, self._count_ready = None, None
        self._render = {(16, 16): "render_16x16", (32, 16): "render_32x16", (32, 32): "render_32x32"}[tuple(block)]

    def forward(self, scene: DeviceScene, camera, bg_color, out_color=None, rows=None):
        """One frame (example.py:67-94). Returns the int8 [H,W,3] image tensor."""
        self.begin(scene, camera, rows=rows)
        return self.finish(scene, camera, bg_color, out_color=out_color, rows=rows)

    def begin(self, scene: DeviceScene, camera, rows=None):
        """First half of a frame, nothing waited for: preprocess on the current stream (example.py:67-78). A caller
        that keeps two rasterizers on two streams calls ``begin`` of the next frame before ``finish`` of this one, so
        that the GPU has work while the host waits for this frame's pair count."""
        ops, (bx, by) = self.ops, self.block
        self.curr_offset.fill_(0)
        extra = {} if rows is None else dict(tile_row_begin=rows[0], tile_row_end=rows[1])
        if self.cull_scratch is not None:
            extra["cull_scratch"] = self.cull_scratch
            if self.scene_bounds is not None:
                extra["scene_bounds"] = self.scene_bounds
        if self.tile_counts is not None:
            extra["tile_counts"] = self.tile_counts
        ops.preprocess(scene.position, scene.shs, scene.opacity, scene.cov3d,
                       camera.width, camera.height, bx, by,
                       camera.position, camera.rotation,
                       camera.focal_x, camera.focal_y, camera.zFar, camera.zNear,
                       self.points_xy, self.rgb_depth, self.conic_opacity,
                       self.gaussian_keys_unsorted, self.gaussian_values_unsorted,
                       self.curr_offset, **extra)
        if self._count_host is None:
            self._count_host = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._count_ready = torch.cuda.Event()
        self._count_host.copy_(self.curr_offset, non_blocking=True)   # example.py:79, through pinned memory
        self._count_ready.record()

    def finish(self, scene: DeviceScene, camera, bg_color, out_color=None, rows=None):
        """Second half: wait for the pair count (the one host synchronisation the operator signatures impose), sort,
        render (example.py:79-94). Runs on the current stream, which must be the one ``begin`` ran on."""
        ops, (bx, by) = self.ops, self.block
        self._count_ready.synchronize()
        num_rendered = int(self._count_host[0])
        if num_rendered >= self.MAX_NUM_RENDERED:
            raise RuntimeError("Too many k-v pairs! (%d >= %d)" % (num_rendered, self.MAX_NUM_RENDERED))
        self.num_rendered = num_rendered
        sort_extra = {"tile_counts": self.tile_counts} if self.tile_counts is not None else {}
        ops.sort_gaussian(num_rendered, camera.width, camera.height, bx, by,
                          self.list_sorting_space,
                          self.gaussian_keys_unsorted, self.gaussian_values_unsorted,
                          self.gaussian_keys_sorted, self.gaussian_values_sorted, **sort_extra)
        if out_color is None:
            out_color = torch.zeros((camera.height, camera.width, 3), device=scene.device, dtype=torch.int8)
        order_extra = self._tile_order_arguments(camera, rows)
        if rows is None:
            getattr(ops, self._render)(num_rendered, camera.width, camera.height,
                                       self.points_xy, self.rgb_depth, self.conic_opacity,
                                       self.gaussian_keys_sorted, self.gaussian_values_sorted,
                                       self.ranges, bg_color, out_color, **order_extra)
        else:
            ops.render_ex(bx, by, num_rendered, camera.width, camera.height,
                          self.points_xy, self.rgb_depth, self.conic_opacity,
                          self.gaussian_keys_sorted, self.gaussian_values_sorted,
                          self.ranges, bg_color, out_color=out_color,
                          tile_row_begin=rows[0], tile_row_end=rows[1], **order_extra)
        return out_color

    def _tile_order_arguments(self, camera, rows):
        """Keyword arguments of the render call that concern the order of the tiles: every frame the blend records what
        it consumed per tile; every ``order_refresh`` frames of one (image size, strip) that record becomes the order."""
        if not self.order_refresh:
            return {}
        bx, by = self.block
        tiles = ((camera.width + bx - 1) // bx) * ((camera.height + by - 1) // by)
        if tiles > self.tile_consumed.numel():
            return {}
        key = (camera.width, camera.height, rows)
        if key != self._order_key:
            self._order, self._order_key, self._frames = None, key, 0
        elif self._frames % self.order_refresh == 1:      # the previous frame of this view has left its counts
            r = rows or (0, -1)
            self._order = self.ops.tile_order_from(self.tile_consumed[:tiles], camera.width, camera.height, bx, by, r[0], r[1])
        self._frames += 1
        extra = {"consumed": self.tile_consumed[:tiles]}
        if self._order is not None:
            extra["tile_order"] = self._order
        return extra


    def forward_fused(self, scene: DeviceScene, camera, bg_color, out_color=None, rows=None):
        """One frame through the single-call entry point: nothing waits for the GPU, the pair count stays in
        ``self.curr_offset`` (read it later if needed). Same image as ``forward``."""
        if out_color is None:
            out_color = torch.zeros((camera.height, camera.width, 3), device=scene.device, dtype=torch.int8)
        r = rows or (0, -1)
        self.ops.render_frame(scene.position, scene.shs, scene.opacity, scene.cov3d,
                              camera.width, camera.height, self.block[0], self.block[1],
                              camera.position, camera.rotation, camera.focal_x, camera.focal_y, camera.zFar, camera.zNear,
                              bg_color, self.points_xy, self.rgb_depth, self.conic_opacity,
                              self.gaussian_keys_unsorted, self.gaussian_values_unsorted,
                              self.gaussian_keys_sorted, self.gaussian_values_sorted,
                              self.list_sorting_space, self.ranges, self.curr_offset, out_color,
                              tile_row_begin=r[0], tile_row_end=r[1], scene_bounds=self.scene_bounds,
                              **self._tile_order_arguments(camera, rows))
        return out_color


def strip_rows(grid_y: int, world_size: int, rank: int):
    """Tile rows [begin, end) of ``rank`` when ``grid_y`` rows are dealt out as evenly as possible."""
    base, rem = divmod(grid_y, world_size)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def save_ppm(image: torch.Tensor, path: str) -> None:
    """Binary PPM writer (example.py:97-102)."""
    image = image.cpu()
    assert image.dim() >= 3 and image.size(2) == 3
    with open(path, "wb") as f:
        f.write(b"P6\n" + f"{image.size(1)} {image.size(0)}\n255\n".encode() + image.numpy().tobytes())
