"""One frame on several GPUs: horizontal strips of tile rows, one gather at the end.

The reference is single-GPU; this is the multi-GPU form of the same path. Every rank
holds the whole scene, runs the pipeline restricted to its strip of tile rows
(``preprocess`` drops every Gaussian whose tile rectangle misses the strip, keys keep
their whole-frame tile ids) and ends up with the pixel rows of its strip. There is no
collective inside the frame. When a single image is wanted on one DEVICE, the strips are
gathered on one rank (``gather_strips``: one ``gather`` of equally padded strips, over NVLink
when the backend is NCCL); when it is wanted on the HOST, every rank copies its own strip into
one host image that all ranks of the node share (``HostFrames``), so that the frame leaves
through all PCIe links at once and nothing crosses between GPUs.

The helpers here are backend-agnostic (they work on CPU tensors over gloo as well), so the
partition and gather logic is testable without a GPU.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def strip_rows(grid_y: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Tile rows [begin, end) owned by ``rank``: rows dealt out as evenly as possible, low ranks first."""
    base, rem = divmod(grid_y, world_size)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def views_of_rank(num_views: int, world_size: int, rank: int) -> List[int]:
    """Independent views of one scene dealt out round-robin (view batches: every rank holds the scene and renders its
    views alone; nothing crosses between ranks)."""
    return list(range(rank, num_views, world_size))


def balanced_strip_rows(row_cost: List[float], world_size: int) -> List[Tuple[int, int]]:
    """Contiguous strips whose summed cost (e.g. pairs per tile row of the previous frame) is about equal.

    Greedy prefix split: strip r ends at the first row where the running cost reaches
    (r+1)/world_size of the total; every strip keeps at least one row while rows remain.
    """
    n = len(row_cost)
    total = float(sum(row_cost))
    bounds = [0]
    acc = 0.0
    row = 0
    for r in range(world_size - 1):
        target = total * (r + 1) / world_size
        # leave at least one row for each of the remaining strips
        limit = n - (world_size - 1 - r)
        while row < limit and (acc + row_cost[row] <= target or row == bounds[-1]):
            acc += row_cost[row]
            row += 1
            if acc >= target:
                break
        bounds.append(min(max(row, bounds[-1]), n))
    bounds.append(n)
    return [(bounds[i], bounds[i + 1]) for i in range(world_size)]


def strip_pixel_rows(rows: Tuple[int, int], block_y: int, height: int) -> Tuple[int, int]:
    """Pixel rows [y0, y1) covered by tile rows ``rows``."""
    return min(height, rows[0] * block_y), min(height, rows[1] * block_y)


def gather_strips(local_image: torch.Tensor, all_rows: List[Tuple[int, int]], block_y: int, height: int,
                  dst: int = 0, group=None) -> Optional[torch.Tensor]:
    """Gather the strips of a frame on rank ``dst``.

    ``local_image`` is this rank's full-size ``[H, W, 3]`` image of which only its own strip
    rows are valid. Strips are padded to the tallest strip so that one fixed-size gather
    moves them; ``dst`` returns the assembled ``[H, W, 3]`` image, the other ranks ``None``.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    spans = [strip_pixel_rows(r, block_y, height) for r in all_rows]
    tallest = max(1, max(y1 - y0 for y0, y1 in spans))
    y0, y1 = spans[rank]
    W, C = local_image.shape[1], local_image.shape[2]
    send = torch.zeros((tallest, W, C), dtype=local_image.dtype, device=local_image.device)
    if y1 > y0:
        send[: y1 - y0] = local_image[y0:y1]
    recv = None
    if rank == dst:
        recv = [torch.empty_like(send) for _ in range(world)]
    dist.gather(send, recv, dst=dst, group=group)
    if rank != dst:
        return None
    out = torch.empty_like(local_image)
    for r, (a, b) in enumerate(spans):
        if b > a:
            out[a:b] = recv[r][: b - a]
    return out


class HostFrames:
    """A ring of ``count`` host images ``[H, W, 3]`` in POSIX shared memory, mapped -- and, with ``register=True``,
    page-locked for CUDA -- in every rank of the group on one node. Each rank copies the pixel rows of its own strip
    into the current image with one asynchronous copy over its own PCIe link, so a whole frame reaches the host
    through N links at once instead of being funnelled through the link of the rank that gathered it. There is no
    collective and no peer traffic at all; the ranks meet in a few counters kept in the same shared memory:
    ``publish(k)`` says that this rank's strip of frame ``k`` has landed, ``wait_produced(k)`` (the consumer, rank
    ``dst``) waits for every rank's, ``consume(k)`` releases the image for reuse and ``wait_consumed(k)`` (every
    rank, before it overwrites an image of the ring) waits for that release. Every wait is bounded: it raises
    ``TimeoutError`` after ``timeout_s`` seconds, so a rank that died or never joined ends the others with an error
    instead of leaving them spinning.

    The reference renders on one GPU and copies the image with ``image.cpu()`` (example.py:98); this is the form that
    copy takes when one frame is rendered as strips on several GPUs.
    """

    def __init__(self, count: int, height: int, width: int, group=None, dst: int = 0, register: bool = True,
                 timeout_s: float = 20.0):
        import time
        from multiprocessing import shared_memory

        import numpy as np
        self._time = time
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.dst, self.count, self.timeout_s = dst, count, timeout_s
        image_bytes = height * width * 3
        flag_bytes = 8 * (self.world + 1)
        total = count * image_bytes + 4096 + flag_bytes
        names = [None]
        if self.rank == dst:
            self.shm = shared_memory.SharedMemory(create=True, size=total)
            names[0] = self.shm.name
        if self.world > 1:
            dist.broadcast_object_list(names, src=dst, group=group)
        if self.rank != dst:
            self.shm = shared_memory.SharedMemory(name=names[0])
            try:   # the creating rank removes the segment; attaching ranks must not try to at exit
                from multiprocessing import resource_tracker
                resource_tracker.unregister(self.shm._name, "shared_memory")
            except Exception:
                pass
        buf = np.ndarray((total,), dtype=np.uint8, buffer=self.shm.buf)
        self._np = buf
        self.images = [torch.from_numpy(buf[i * image_bytes:(i + 1) * image_bytes].reshape(height, width, 3)).view(torch.int8)
                       for i in range(count)]
        off = (count * image_bytes + 4095) // 4096 * 4096
        self.flags = np.ndarray((self.world + 1,), dtype=np.int64, buffer=self.shm.buf, offset=off)
        if self.rank == dst:
            self.flags[:] = -1
        self.registered = False
        if register and torch.cuda.is_available():
            rc = torch.cuda.cudart().cudaHostRegister(buf.ctypes.data, count * image_bytes, 0)
            self.registered = int(rc) == 0
        if self.world > 1:
            dist.barrier(group=group)   # the flags are initialised before anybody polls them

    def _spin(self, ready, what: str) -> None:
        t0 = self._time.perf_counter()
        while not ready():
            if self._time.perf_counter() - t0 > self.timeout_s:
                raise TimeoutError("HostFrames: %s not reached within %.1f s (flags %s)" % (what, self.timeout_s, self.flags.tolist()))

    def publish(self, frame: int) -> None:
        """This rank's strip of ``frame`` is complete in host memory (call it after the copy's event has completed)."""
        self.flags[self.rank] = frame

    def wait_produced(self, frame: int) -> None:
        self._spin(lambda: bool((self.flags[: self.world] >= frame).all()), "frame %d from every rank" % frame)

    def consume(self, frame: int) -> None:
        self.flags[self.world] = frame

    def wait_consumed(self, frame: int) -> None:
        if frame >= 0:
            self._spin(lambda: int(self.flags[self.world]) >= frame, "release of frame %d" % frame)

    def close(self) -> None:
        if self.registered:
            torch.cuda.cudart().cudaHostUnregister(self._np.ctypes.data)
            self.registered = False
        self.images, self.flags, self._np = [], None, None
        if self.world > 1:
            dist.barrier(group=self.group)
        try:
            self.shm.close()
            if self.rank == self.dst:
                self.shm.unlink()
        except Exception:
            pass
