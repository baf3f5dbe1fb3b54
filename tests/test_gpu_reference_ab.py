"""A/B of the sm_100a kernels against the reference's own CUDA build on the same device and inputs.

Runs only where oracle/_ref (the unmodified reference compiled from its sources) is present.
Expected: pair sets, sorted lists (runs of identical keys ordered by value), tile ranges and the
three feature arrays bit-exact; 8-bit images within one level on a small fraction of pixels.
The reference's render is invoked only on frames where no tile holds one or two splats, because
for those it reads an uninitialised register (csrc/cuda_rasterizer/render.cu:268-306).
"""
import numpy as np
import pytest
import torch

from flashgs_b200 import scenes
from helpers import canonical_pairs, canonical_sorted_values, psnr_u8

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(ops, sc, cam, pad_rows=32, render_guard=True):
    P, W, H = sc.num_vertex, cam.width, cam.height
    gx, gy = scenes.tile_grid(W, H)
    cap = max(1 << 20, 24 * P)
    t = lambda a: torch.from_numpy(a).to(DEV)  # noqa: E731
    z = lambda shape, dt: torch.zeros(shape, device=DEV, dtype=dt)  # noqa: E731
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
    out = dict(R=R, ku=ku[:R].cpu().numpy().view(np.uint64), vu=vu[:R].cpu().numpy().view(np.uint32),
               ks=ks[:R].cpu().numpy().view(np.uint64), vs=vs[:R].cpu().numpy().view(np.uint32),
               xy=xy.cpu().numpy(), rd=rd.cpu().numpy(), co=co.cpu().numpy())
    cnt = torch.bincount(ks[:R] >> 32, minlength=gx * gy)
    out["sparse_tiles"] = int((cnt < 3).sum())
    if not render_guard or out["sparse_tiles"] == 0:
        ranges = z((gx * gy, 2), torch.int32)
        img = z((H + pad_rows, W, 3), torch.int8)
        ops.render_16x16(R, W, H, xy, rd, co, ks, vs, ranges, torch.zeros(3), img)
        torch.cuda.synchronize()
        out["ranges"] = ranges.cpu().numpy()
        out["img"] = img[:H].cpu().numpy().view(np.uint8)
    return out


@pytest.fixture(scope="module")
def ref_ops():
    from oracle import ref
    m = ref.load() if ref.available() else None
    if m is None:
        pytest.skip("reference build not present")
    return m.ops


@pytest.mark.parametrize("name,n,size", [("C1", 100000, None), ("C1", 400000, None), ("C2", 300000, (960, 540)), ("C4", 200000, (1280, 720))])
def test_against_reference_build(ref_ops, name, n, size):
    from flashgs_b200 import ops as my_ops
    w = scenes.WORKLOADS[name]
    sc = scenes.make_scene(n, w.clusters, w.log_scale, seed=w.seed)
    W, H = size or (w.width, w.height)
    cam = scenes.look_at_camera(W, H, w.radius, w.hfov_deg, w.azimuth_deg, w.elevation_deg)
    a = _run(my_ops, sc, cam, render_guard=False)
    b = _run(ref_ops, sc, cam)
    assert a["R"] == b["R"]
    ka, va = canonical_pairs(a["ku"], a["vu"])
    kb, vb = canonical_pairs(b["ku"], b["vu"])
    assert (ka == kb).all() and (va == vb).all()
    assert (a["ks"] == b["ks"]).all()
    assert (canonical_sorted_values(a["ks"], a["vs"]) == canonical_sorted_values(b["ks"], b["vs"])).all()
    vis = np.unique(b["vu"])
    for f in ("xy", "rd", "co"):
        assert (a[f][vis].view(np.uint32) == b[f][vis].view(np.uint32)).all(), f
    if "img" in b:
        assert (a["ranges"] == b["ranges"]).all()
        d = np.abs(a["img"].astype(int) - b["img"].astype(int))
        assert d.max() <= 1 and (d > 0).mean() <= 1e-4
        assert psnr_u8(a["img"], b["img"]) > 60.0
    assert my_ops.device_status() == 0


@pytest.mark.parametrize("name", ["C3", "C4"])
def test_full_size_pair_sets_against_reference_build(ref_ops, name):
    """The whole workload (C4: 6 M Gaussians, 29.4 M pairs): every (tile, Gaussian) pair the reference's build emits and
    no other. Splats tangent to a tile edge make this sensitive to which multiply-add pairs of the exact tile test are
    fused; the forms pinned in the kernel were found with this comparison."""
    from flashgs_b200 import ops
    w, sc, cams = scenes.make_workload(name)
    cam = cams[0]
    P, W, H = sc.num_vertex, cam.width, cam.height
    t = lambda a: torch.from_numpy(a).to(DEV)  # noqa: E731
    z = lambda shape, dt: torch.zeros(shape, device=DEV, dtype=dt)  # noqa: E731
    pos, shs, opa, cov = t(sc.position), t(sc.shs), t(sc.opacity), t(sc.cov3d)
    cap = 1 << 26

    def pairs(o):
        xy, rd, co = z((P, 2), torch.float32), z((P, 4), torch.float32), z((P, 4), torch.float32)
        ku, vu, off = z(cap, torch.int64), z(cap, torch.int32), z(1, torch.int32)
        o.preprocess(pos, shs, opa, cov, W, H, 16, 16, torch.from_numpy(cam.position.copy()),
                     torch.from_numpy(cam.rotation.copy()), cam.focal_x, cam.focal_y, cam.zFar, cam.zNear,
                     xy, rd, co, ku, vu, off)
        R = int(off.cpu()[0])
        assert R < cap
        return torch.sort((ku[:R] >> 32) * (1 << 23) + vu[:R].long())[0]   # (tile, Gaussian), P < 2^23

    theirs = pairs(ref_ops)
    ours = pairs(ops)
    assert ours.numel() == theirs.numel()
    assert bool((ours == theirs).all())
