"""One frame on two GPUs: each rank renders its strip of tile rows and copies it into the host image both ranks share.

Needs two CUDA devices (skipped otherwise). Two child processes, one per GPU, NCCL for the rendezvous and for the
gathered strips the host image is compared with. Nothing here waits on another GPU from device code; the ranks meet
in the host-side counters of ``parallel.HostFrames`` (bounded waits) and in NCCL's own collectives, with NVLS off.
"""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist
    from flashgs_b200 import ops, parallel, scenes
    from flashgs_b200.rasterizer import DeviceScene, Rasterizer, TorchCamera
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        w, sc, cams = scenes.make_workload("C1", 60000)
        cam = cams[0]
        H, W = cam.height, cam.width
        gy = scenes.tile_grid(W, H)[1]
        all_rows = [parallel.strip_rows(gy, world, r) for r in range(world)]
        rows = all_rows[rank]
        y0, y1 = parallel.strip_pixel_rows(rows, 16, H)
        ds = DeviceScene(sc, dev)
        ras = Rasterizer(ds, 1 << 21, 1 << 12)
        tc, bg = TorchCamera(cam), torch.tensor([0.1, 0.2, 0.3])
        ring = parallel.HostFrames(2, H, W, dst=0, timeout_s=30.0)
        assert ring.registered and ring.images[0].is_pinned()
        img = torch.full((H, W, 3), 0x55, device=dev, dtype=torch.int8)
        ok = True
        for k in range(3):   # three frames through the two-image ring
            ring.wait_consumed(k - 2)
            ras.forward(ds, tc, bg, out_color=img, rows=rows)
            ring.images[k % 2][y0:y1].copy_(img[y0:y1], non_blocking=True)
            torch.cuda.current_stream().synchronize()
            ring.publish(k)
            full = parallel.gather_strips(img, all_rows, 16, H, dst=0)      # the same strips over NCCL
            if rank == 0:
                ring.wait_produced(k)
                ok = ok and bool((ring.images[k % 2] == full.cpu()).all())
                ring.consume(k)
        if rank == 0:
            whole = ras.forward(ds, tc, bg).cpu().numpy().view(np.uint8)    # the frame on one GPU
            got = ring.images[0].numpy().view(np.uint8)
            d = np.abs(whole.astype(int) - got.astype(int))
            ok = ok and d.max() <= 1 and (d > 0).mean() <= 1e-5
        status = ops.device_status()
        ring.close()
        if rank == 0:
            with open(out_path, "w") as f:
                f.write("ok" if ok and status == 0 else "bad ok=%s status=%d" % (ok, status))
    finally:
        dist.destroy_process_group()


def test_strips_on_two_gpus_meet_in_one_host_image(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    import torch.multiprocessing as mp
    out = tmp_path / "two.txt"
    mp.spawn(_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    assert out.read_text() == "ok"
