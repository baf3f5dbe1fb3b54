"""Records golden vectors from the REFERENCE's own CUDA build (needs a GPU and oracle/_ref).

Run on a GPU box:  python tests/golden/make_golden.py [out_dir]
For each spec below the seeded scene is rendered with the unmodified reference operators
(preprocess -> sort_gaussian -> render_16x16) and the outputs that define parity are stored in
a compressed .npz: pair count, canonical sorted value list, tile ranges, the 8-bit image,
order-independent checksums of the pair set and of the feature records, and every 8th visible
Gaussian's feature records in full. The inputs are not stored: the tests regenerate them from
the spec with flashgs_b200.scenes.

The reference's blend kernel reads an uninitialised register for tiles that hold exactly one
or two splats (csrc/cuda_rasterizer/render.cu:268-306) and writes out of bounds for empty tiles
of a ragged image (render.cu:530-546), so a spec is only recorded if no tile of its frame has
fewer than three splats; the script checks this on the reference's own sorted keys before it
calls the reference's render.
"""
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from flashgs_b200 import scenes  # noqa: E402
from oracle import ref  # noqa: E402

SPECS = {
    "ref_c1like_256x192": dict(n=30000, clusters=64, workload="C1", seed=7, width=256, height=192,
                               radius=15.0, hfov=60.0, az=34.0, el=17.0),
    "ref_c1like_250x180_ragged": dict(n=30000, clusters=64, workload="C1", seed=8, width=250, height=180,
                                      radius=15.0, hfov=60.0, az=120.0, el=-10.0),
    "ref_needles_320x176": dict(n=40000, clusters=64, workload="C4", seed=9, width=320, height=176,
                                radius=12.0, hfov=50.0, az=34.0, el=17.0),
}


def build_inputs(spec):
    sc = scenes.make_scene(spec["n"], spec["clusters"], scenes.WORKLOADS[spec["workload"]].log_scale, seed=spec["seed"])
    cam = scenes.look_at_camera(spec["width"], spec["height"], spec["radius"], spec["hfov"], spec["az"], spec["el"])
    return sc, cam


def bits_checksum(a):
    """Order-independent checksum of an array's 32-bit patterns (sum modulo 2^64)."""
    return int(np.ascontiguousarray(a).view(np.uint32).astype(np.uint64).sum(dtype=np.uint64))


def pair_checksum(keys, values):
    k = np.asarray(keys, np.uint64)
    v = np.asarray(values, np.uint64)
    return int((k * np.uint64(0x9E3779B97F4A7C15) + v * np.uint64(0xC2B2AE3D27D4EB4F) + (k ^ (v << np.uint64(17)))).sum(dtype=np.uint64))


def record(name, spec, ops, out_dir):
    dev = torch.device("cuda:0")
    sc, cam = build_inputs(spec)
    P, W, H = sc.num_vertex, cam.width, cam.height
    gx, gy = scenes.tile_grid(W, H)
    cap = 1 << 20
    t = lambda a: torch.from_numpy(a).to(dev)  # noqa: E731
    z = lambda shape, dt: torch.zeros(shape, device=dev, dtype=dt)  # noqa: E731
    xy, rd, co = z((P, 2), torch.float32), z((P, 4), torch.float32), z((P, 4), torch.float32)
    ku, vu, ks, vs = z(cap, torch.int64), z(cap, torch.int32), z(cap, torch.int64), z(cap, torch.int32)
    off = z(1, torch.int32)
    ops.preprocess(t(sc.position), t(sc.shs), t(sc.opacity), t(sc.cov3d), W, H, 16, 16,
                   torch.from_numpy(cam.position.copy()), torch.from_numpy(cam.rotation.copy()),
                   cam.focal_x, cam.focal_y, cam.zFar, cam.zNear, xy, rd, co, ku, vu, off)
    R = int(off.cpu()[0])
    tmp = z(ops.get_sort_buffer_size(cap), torch.int8)
    ops.sort_gaussian(R, W, H, 16, 16, tmp, ku, vu, ks, vs)
    torch.cuda.synchronize()
    cnt = torch.bincount(ks[:R] >> 32, minlength=gx * gy)
    if int((cnt < 3).sum()) != 0:
        print(name, "SKIPPED: %d tiles hold fewer than three splats" % int((cnt < 3).sum()))
        return False
    ranges = z((gx * gy, 2), torch.int32)
    img = torch.full((H + 32, W, 3), 0, device=dev, dtype=torch.int8)
    ops.render_16x16(R, W, H, xy, rd, co, ks, vs, ranges, torch.zeros(3), img)
    torch.cuda.synchronize()
    ksn = ks[:R].cpu().numpy().view(np.uint64)
    vsn = vs[:R].cpu().numpy().view(np.uint32)
    order = np.lexsort((vsn, ksn))          # canonical order inside runs of identical keys
    assert (ksn[order] == ksn).all()
    vis = np.unique(vsn)
    xyn, rdn, con = xy.cpu().numpy(), rd.cpu().numpy(), co.cpu().numpy()
    sample = vis[::8]
    np.savez_compressed(
        os.path.join(out_dir, name + ".npz"),
        spec=json.dumps(spec), num_rendered=R,
        values_sorted=vsn[order], ranges=ranges.cpu().numpy(),
        depth_bits_sorted_crc=bits_checksum((ksn & np.uint64(0xFFFFFFFF)).astype(np.uint32)),
        pair_checksum=pair_checksum(ku[:R].cpu().numpy().view(np.uint64), vu[:R].cpu().numpy().view(np.uint32)),
        visible=vis.astype(np.uint32),
        xy_crc=bits_checksum(xyn[vis]), rd_crc=bits_checksum(rdn[vis]), co_crc=bits_checksum(con[vis]),
        sample=sample.astype(np.uint32), xy=xyn[sample], rgb_depth=rdn[sample], conic_opacity=con[sample],
        image=img[:H].cpu().numpy().view(np.uint8))
    print(name, "recorded: R=%d visible=%d" % (R, vis.size))
    return True


if __name__ == "__main__":
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__))
    os.makedirs(out_dir, exist_ok=True)
    m = ref.load()
    if m is None:
        sys.exit("the reference build (oracle/_ref) is not available")
    for name, spec in SPECS.items():
        record(name, spec, m.ops, out_dir)
