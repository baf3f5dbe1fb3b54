"""Host-side logic of the multi-GPU strip split, exercised with two CPU ranks over gloo.

Each rank "renders" its strip with the CPU oracle (the renderer is injected; the product
code under test is the partition and gather logic of flashgs_b200.parallel).
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashgs_b200 import parallel, scenes


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle
        w, sc, cams = scenes.make_workload("C1", 6000)
        cam = cams[0]
        gy = scenes.tile_grid(cam.width, cam.height)[1]
        rows = [parallel.strip_rows(gy, world, r) for r in range(world)]
        mine = oracle.render_frame(sc, cam, rows=rows[rank], floats=False)
        local = torch.from_numpy(mine["u8"])
        # rows outside the strip must not matter: poison them
        y0, y1 = parallel.strip_pixel_rows(rows[rank], 16, cam.height)
        local[:y0] = 77
        local[y1:] = 77
        full = parallel.gather_strips(local, rows, 16, cam.height, dst=0)
        counts = torch.tensor([mine["keys"].size], dtype=torch.int64)
        dist.all_reduce(counts)
        # view batches: the ranks' views together are every view exactly once
        seen = torch.zeros(7, dtype=torch.int64)
        seen[parallel.views_of_rank(7, world, rank)] += 1
        dist.all_reduce(seen)
        assert (seen == 1).all()
        if rank == 0:
            ref = oracle.render_frame(sc, cam, floats=False)
            ok = bool((full.numpy() == ref["u8"]).all()) and int(counts[0]) == ref["keys"].size
            with open(out_path, "w") as f:
                f.write("ok" if ok else "mismatch")
        else:
            assert full is None
    finally:
        dist.destroy_process_group()


def test_two_rank_strip_gather(tmp_path, oracle_lib):
    out = tmp_path / "result.txt"
    mp.spawn(_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    assert out.read_text() == "ok"


def test_strip_rows_cover_grid_exactly():
    for gy in (1, 7, 50, 68, 135):
        for world in (1, 2, 3, 4, 8):
            rows = [parallel.strip_rows(gy, world, r) for r in range(world)]
            assert rows[0][0] == 0 and rows[-1][1] == gy
            assert all(rows[i][1] == rows[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in rows]
            assert max(sizes) - min(sizes) <= 1


def test_balanced_strips_follow_cost():
    cost = [1.0] * 10 + [9.0] * 10
    rows = parallel.balanced_strip_rows(cost, 4)
    assert rows[0][0] == 0 and rows[-1][1] == 20
    assert all(rows[i][1] == rows[i + 1][0] for i in range(3))
    sums = [sum(cost[a:b]) for a, b in rows]
    assert max(sums) <= 1.5 * (sum(cost) / 4)
    assert all(b > a for a, b in parallel.balanced_strip_rows([0.0] * 8, 8))
    assert parallel.strip_pixel_rows((60, 68), 16, 1080) == (960, 1080)


def _host_frames_worker(rank, world, port, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        H, W = 96, 40
        rows = [parallel.strip_rows(H // 16, world, r) for r in range(world)]
        y0, y1 = parallel.strip_pixel_rows(rows[rank], 16, H)
        ring = parallel.HostFrames(2, H, W, register=False, timeout_s=20.0)
        ok = True
        for k in range(6):
            ring.wait_consumed(k - 2)                       # image k % 2 is free again
            ring.images[k % 2][y0:y1] = (10 * k + rank) % 100   # this rank's strip of frame k
            ring.publish(k)
            if rank == 0:
                ring.wait_produced(k)
                img = ring.images[k % 2].numpy()
                for r, rr in enumerate(rows):
                    a, b = parallel.strip_pixel_rows(rr, 16, H)
                    ok = ok and bool((img[a:b] == (10 * k + r) % 100).all())
                ring.consume(k)
        # a frame that one rank never delivers: the consumer's wait runs out instead of spinning for ever
        timed_out = False
        if rank == 0:
            ring.timeout_s = 0.3
            try:
                ring.wait_produced(99)
            except TimeoutError:
                timed_out = True
        ring.close()
        if rank == 0:
            with open(out_path, "w") as f:
                f.write("ok" if ok and timed_out else "bad ok=%s timeout=%s" % (ok, timed_out))
    finally:
        dist.destroy_process_group()


def test_host_frame_ring_two_ranks(tmp_path):
    """Every rank writes the rows of its own strip into a host image shared by all ranks; the consumer sees whole
    frames, the ring's images are reused only after their release, and a missing strip ends the wait with an error."""
    out = tmp_path / "ring.txt"
    mp.spawn(_host_frames_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    assert out.read_text() == "ok"
