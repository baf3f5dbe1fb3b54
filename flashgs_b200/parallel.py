"""One frame on several GPUs: horizontal strips of tile rows, one gather at the end.

The reference is single-GPU; this is the multi-GPU form of the same path. Every rank
holds the whole scene, runs the pipeline restricted to its strip of tile rows
(``preprocess`` drops every Gaussian whose tile rectangle misses the strip, keys keep
their whole-frame tile ids) and ends up with the pixel rows of its strip. There is no
collective inside the frame. Only when a single image is wanted are the strips gathered
on one rank (one ``gather`` of equally padded strips, over NVLink when the backend is NCCL).

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


class PeerFrames:
    """``count`` frame buffers that live on rank ``dst`` and are mapped into every rank of the group (torch symmetric
    memory: peer mappings over NVLink). A rank passes ``frames[i]`` as the output image of its strip, so its blend
    kernel stores the strip's pixels straight into the destination's buffer with ordinary stores; ``barrier()``
    (device side, on the current stream) then tells the destination that every strip has landed. No gather follows.
    Raises whatever the symmetric-memory set-up raises when peer mappings are not available; callers fall back to
    ``gather_strips``."""

    def __init__(self, count: int, height: int, width: int, device, dst: int = 0, group=None):
        import os
        # only plain peer stores are used: ask the allocator not to bind the buffers to an NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        shape = (count, height, width, 3)
        self.local = symm_mem.empty(shape, dtype=torch.int8, device=device)
        self.handle = symm_mem.rendezvous(self.local, group)
        target = self.handle.get_buffer(dst, shape, torch.int8)
        self.frames = [target[i] for i in range(count)]
        self.dst = dst

    def barrier(self) -> None:
        self.handle.barrier(channel=0)
