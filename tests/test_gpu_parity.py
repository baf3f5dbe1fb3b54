"""Parity of the sm_100a kernels with the CPU oracle (and with the reference's CUDA build when present).

Everything here goes through the C ABI of libflashgs_b200.so via the ctypes shims in
flashgs_b200.ops. Tolerances (stated where used):
  * integer / index results (pair sets, sorted lists, tile ranges): exact, after ordering runs
    of identical 64-bit keys by value (the reference's order inside such a run is the arrival
    order of its atomics and is not defined);
  * float images: max-abs 2e-3 on RGB, 1e-4 on alpha and depth-per-unit-depth, PSNR > 60 dB;
  * 8-bit images: at most 1 level on a small fraction of pixels (truncating quantisation).
"""
import numpy as np
import pytest
import torch

from flashgs_b200 import scenes
from helpers import canonical_pairs, canonical_sorted_values, identity_camera, make_scene, psnr_u8

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from flashgs_b200 import ops as o
    return o


def _t(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.view(dtype) if t.element_size() == torch.empty((), dtype=dtype).element_size() else t.to(dtype)
    return t.to(DEV)


class Frame:
    """Runs the three ops stage by stage and keeps every intermediate on the host."""

    def __init__(self, ops, scene, cam, block=(16, 16), capacity=None, rows=None, bg=(0.0, 0.0, 0.0), floats=True, cull=False):
        P = scene.num_vertex
        bx, by = block
        gx, gy = scenes.tile_grid(cam.width, cam.height, bx, by)
        cap = capacity if capacity is not None else max(1 << 16, 24 * P)
        z = lambda shape, dt: torch.zeros(shape, device=DEV, dtype=dt)  # noqa: E731
        self.pos, self.shs = _t(scene.position), _t(scene.shs)
        self.opa, self.cov = _t(scene.opacity), _t(scene.cov3d)
        self.xy, self.rd, self.co = z((P, 2), torch.float32), z((P, 4), torch.float32), z((P, 4), torch.float32)
        self.ku, self.vu = z(cap, torch.int64), z(cap, torch.int32)
        self.ks, self.vs = z(cap, torch.int64), z(cap, torch.int32)
        self.off = z(1, torch.int32)
        self.cpos, self.crot = torch.from_numpy(cam.position.copy()), torch.from_numpy(cam.rotation.copy())
        extra = {} if rows is None else dict(tile_row_begin=rows[0], tile_row_end=rows[1])
        if cull:   # scratch for the index list of the Gaussians that reach the strip; its contents do not matter
            extra["cull_scratch"] = torch.full((P + 1,), 0x7F7F7F7F, device=DEV, dtype=torch.int32)
            if cull == "bounds":   # ... found from the 16-byte records prepared once per scene
                extra["scene_bounds"] = ops.prepare_scene(self.pos, self.opa, self.cov)
        sort_extra = {}
        if cull == "bounds":       # the whole set of extensions: preprocess also counts the pairs per tile for the sort
            self.counts = torch.full((65536,), 0x7F7F7F7F, device=DEV, dtype=torch.int32)
            extra["tile_counts"] = sort_extra["tile_counts"] = self.counts
        ops.preprocess(self.pos, self.shs, self.opa, self.cov, cam.width, cam.height, bx, by, self.cpos, self.crot,
                       cam.focal_x, cam.focal_y, cam.zFar, cam.zNear, self.xy, self.rd, self.co,
                       self.ku, self.vu, self.off, **extra)
        self.R = int(self.off.cpu()[0])
        self.capacity = cap
        if self.R > cap:
            return
        R = self.R
        self.temp = z(ops.get_sort_buffer_size(max(R, 1)), torch.int8)
        ops.sort_gaussian(R, cam.width, cam.height, bx, by, self.temp, self.ku, self.vu, self.ks, self.vs, **sort_extra)
        self.ranges = z((gx * gy, 2), torch.int32)
        self.img = z((cam.height, cam.width, 3), torch.uint8)
        bgt = torch.tensor(bg, dtype=torch.float32)
        if floats or rows is not None:
            self.rgb, self.alpha = z((cam.height, cam.width, 3), torch.float32), z((cam.height, cam.width), torch.float32)
            self.depth, self.consumed = z((cam.height, cam.width), torch.float32), z(gx * gy, torch.int32)
            r = rows or (0, -1)
            ops.render_ex(bx, by, R, cam.width, cam.height, self.xy, self.rd, self.co, self.ks, self.vs, self.ranges, bgt,
                          out_color=self.img, out_rgb=self.rgb, out_alpha=self.alpha, out_depth=self.depth,
                          consumed=self.consumed, tile_row_begin=r[0], tile_row_end=r[1])
        else:
            fn = {(16, 16): ops.render_16x16, (32, 16): ops.render_32x16, (32, 32): ops.render_32x32}[block]
            fn(R, cam.width, cam.height, self.xy, self.rd, self.co, self.ks, self.vs, self.ranges, bgt, self.img)
        torch.cuda.synchronize()

    def np(self, name, n=None):
        t = getattr(self, name)
        a = (t if n is None else t[:n]).cpu().numpy()
        if a.dtype == np.int64:
            a = a.view(np.uint64)
        if a.dtype == np.int32 and name in ("vu", "vs"):
            a = a.view(np.uint32)
        return a


def _check_against_oracle(f, o, cam, block, max_pair_mismatch=0):
    R = f.R
    ka, va = canonical_pairs(f.np("ku", R), f.np("vu", R))
    kb, vb = canonical_pairs(o["keys"], o["values"])
    if max_pair_mismatch == 0:
        assert R == o["keys"].size
        assert (ka == kb).all() and (va == vb).all()
    else:
        sa = set(zip(ka.tolist(), va.tolist()))
        sb = set(zip(kb.tolist(), vb.tolist()))
        assert len(sa ^ sb) <= max_pair_mismatch
        return
    # sorted list: exact up to the order inside runs of identical keys
    assert (f.np("ks", R) == o["keys_sorted"]).all()
    assert (canonical_sorted_values(f.np("ks", R), f.np("vs", R)) ==
            canonical_sorted_values(o["keys_sorted"], o["values_sorted"])).all()
    assert (f.np("ranges") == o["ranges"]).all()
    vis = np.unique(o["values"])
    assert (f.np("xy")[vis].view(np.uint32) == o["xy"][vis].view(np.uint32)).all()
    # conic terms are IEEE arithmetic on both sides; log2(opacity) and the colour use approximate instructions
    assert (f.np("co")[vis, :3].view(np.uint32) == o["conic_opacity"][vis, :3].view(np.uint32)).all()
    np.testing.assert_allclose(f.np("co")[vis, 3], o["conic_opacity"][vis, 3], rtol=0, atol=2e-6)
    np.testing.assert_allclose(f.np("rd")[vis, :3], o["rgb_depth"][vis, :3], rtol=0, atol=2e-6)
    assert (f.np("rd")[vis, 3].view(np.uint32) == o["rgb_depth"][vis, 3].view(np.uint32)).all()
    # images
    if hasattr(f, "rgb"):
        assert np.abs(f.np("rgb") - o["rgb"]).max() <= 2e-3
        assert np.abs(f.np("alpha") - o["alpha"]).max() <= 1e-4
        zmax = max(1.0, float(o["rgb_depth"][vis, 3].max()))
        assert np.abs(f.np("depth") - o["depth"]).max() <= 1e-4 * zmax
        same = (f.np("consumed") == o["consumed"]).mean()
        assert same >= 0.999, same
    d = np.abs(f.np("img").astype(int) - o["u8"].astype(int))
    assert d.max() <= 1
    assert (d > 0).mean() <= 1e-3
    assert psnr_u8(f.np("img"), o["u8"]) > 60.0


@pytest.mark.parametrize("n", [3000, 20000, 100000])
def test_frame_matches_oracle_c1(ops, oracle_lib, n):
    w, sc, cams = scenes.make_workload("C1", n)
    cam = cams[0]
    f = Frame(ops, sc, cam)
    o = oracle_lib.render_frame(sc, cam)
    _check_against_oracle(f, o, cam, (16, 16))
    assert ops.device_status() == 0


@pytest.mark.parametrize("block", [(32, 16), (32, 32)])
def test_other_tile_shapes_match_oracle(ops, oracle_lib, block):
    w, sc, cams = scenes.make_workload("C1", 30000)
    cam = cams[0]
    f = Frame(ops, sc, cam, block=block)
    o = oracle_lib.render_frame(sc, cam, block=block)
    _check_against_oracle(f, o, cam, block)
    # the plain entry points (no float outputs) give the same bytes as the general one
    g = Frame(ops, sc, cam, block=block, floats=False)
    d = np.abs(g.np("img").astype(int) - f.np("img").astype(int))
    assert d.max() <= 1 and (d > 0).mean() <= 1e-4


def test_needle_splats_match_oracle(ops, oracle_lib):
    # anisotropic splats stress the exact ellipse-vs-tile test (the headline workload's distribution)
    w = scenes.WORKLOADS["C4"]
    sc = scenes.make_scene(60000, 64, w.log_scale, seed=3)
    cam = scenes.look_at_camera(640, 360, 12.0, 50.0, 34.0, 17.0)
    f = Frame(ops, sc, cam)
    o = oracle_lib.render_frame(sc, cam)
    _check_against_oracle(f, o, cam, (16, 16))


def test_crowded_tiles_match_oracle(ops, oracle_lib):
    # a small image of a whole dense scene: a third of the tiles hold far more splats than the in-block sort takes (4096), so the
    # frame goes through the long-list sort, and the blend's early stop decides almost every tile
    w = scenes.WORKLOADS["C3"]
    sc = scenes.make_scene(300000, 16, w.log_scale, seed=5)
    cam = scenes.look_at_camera(160, 112, 25.0, 50.0, 20.0, 10.0)   # the whole scene in 70 tiles
    f = Frame(ops, sc, cam)
    o = oracle_lib.render_frame(sc, cam)
    lengths = o["ranges"][:, 1] - o["ranges"][:, 0]
    assert (lengths > 4096).sum() >= 10, lengths.max()
    _check_against_oracle(f, o, cam, (16, 16))
    assert ops.device_status() == 0


@pytest.mark.parametrize("name,n,size", [("C1", 100000, (800, 800)), ("C4", 300000, (1920, 1080)), ("C3", 200000, (1280, 720))])
def test_column_culling_changes_nothing(ops, name, n, size):
    """Narrowing each row's column range before the exact tile test must not change the pair set."""
    from flashgs_b200 import _lib
    L = _lib.load()
    w = scenes.WORKLOADS[name]
    sc = scenes.make_scene(n, w.clusters, w.log_scale, seed=11)
    cam = scenes.look_at_camera(size[0], size[1], w.radius, w.hfov_deg, w.azimuth_deg, w.elevation_deg)
    a = Frame(ops, sc, cam, floats=False)
    L.fgs_debug_preprocess_no_column_cull(1)
    try:
        b = Frame(ops, sc, cam, floats=False)
    finally:
        L.fgs_debug_preprocess_no_column_cull(0)
    assert a.R == b.R
    ka, va = canonical_pairs(a.np("ku", a.R), a.np("vu", a.R))
    kb, vb = canonical_pairs(b.np("ku", b.R), b.np("vu", b.R))
    assert (ka == kb).all() and (va == vb).all()
    # extreme needles and huge splats: axis ratios up to e^8, some covering the whole image
    sc2 = scenes.make_scene(4000, 8, ((-0.5, 1.5), (-6.0, 1.0), (-6.0, 1.0)), seed=12)
    a = Frame(ops, sc2, cam, floats=False, capacity=1 << 24)
    L.fgs_debug_preprocess_no_column_cull(1)
    try:
        b = Frame(ops, sc2, cam, floats=False, capacity=1 << 24)
    finally:
        L.fgs_debug_preprocess_no_column_cull(0)
    assert a.R == b.R and a.R > 20000
    ka, va = canonical_pairs(a.np("ku", a.R), a.np("vu", a.R))
    kb, vb = canonical_pairs(b.np("ku", b.R), b.np("vu", b.R))
    assert (ka == kb).all() and (va == vb).all()


def test_partial_tiles_and_no_write_outside_image(ops, oracle_lib):
    # 203 x 117: ragged in both directions, byte-store path; the bytes after the image must stay untouched
    cam = scenes.look_at_camera(203, 117, 15.0, 60.0, 34.0, 17.0)
    sc = scenes.make_scene(20000, 64, scenes.WORKLOADS["C1"].log_scale, seed=5)
    o = oracle_lib.render_frame(sc, cam, bg=(0.2, 0.4, 0.6))
    f = Frame(ops, sc, cam, bg=(0.2, 0.4, 0.6))
    _check_against_oracle(f, o, cam, (16, 16))
    guard = torch.full((cam.height + 16, cam.width, 3), 0x5A, device=DEV, dtype=torch.uint8)
    ops.render_16x16(f.R, cam.width, cam.height, f.xy, f.rd, f.co, f.ks, f.vs, f.ranges,
                     torch.tensor([0.2, 0.4, 0.6]), guard)
    torch.cuda.synchronize()
    assert (guard[cam.height:] == 0x5A).all()
    assert (guard[:cam.height].cpu().numpy() == f.np("img")).all()
    # 1920-wide, 1080-high geometry (last tile row partial, vector-store path) at reduced size: 320 x 184
    cam2 = scenes.look_at_camera(320, 184, 15.0, 60.0, 34.0, 17.0)
    o2 = oracle_lib.render_frame(sc, cam2)
    f2 = Frame(ops, sc, cam2)
    _check_against_oracle(f2, o2, cam2, (16, 16))
    guard = torch.full((cam2.height + 16, cam2.width, 3), 0x5A, device=DEV, dtype=torch.uint8)
    ops.render_16x16(f2.R, cam2.width, cam2.height, f2.xy, f2.rd, f2.co, f2.ks, f2.vs, f2.ranges, torch.zeros(3), guard)
    torch.cuda.synchronize()
    assert (guard[cam2.height:] == 0x5A).all()


def test_empty_inputs(ops):
    cam = identity_camera(64, 48, 30.0)
    # no Gaussians at all
    e = lambda *s: torch.zeros(s, device=DEV)  # noqa: E731
    off = torch.zeros(1, device=DEV, dtype=torch.int32)
    ku, vu = torch.zeros(16, device=DEV, dtype=torch.int64), torch.zeros(16, device=DEV, dtype=torch.int32)
    ops.preprocess(e(0, 3), e(0, 48), e(0), e(0, 6), 64, 48, 16, 16, torch.zeros(3), torch.eye(3), 30.0, 30.0, 100.0, 0.01,
                   e(0, 2), e(0, 4), e(0, 4), ku, vu, off)
    assert int(off.cpu()[0]) == 0
    # nothing to sort, nothing to blend: background everywhere, ranges all (0,0)
    tmp = torch.zeros(ops.get_sort_buffer_size(0), device=DEV, dtype=torch.int8)
    ops.sort_gaussian(0, 64, 48, 16, 16, tmp, ku, vu, ku.clone(), vu.clone())
    ranges = torch.full((12, 2), 7, device=DEV, dtype=torch.int32)
    img = torch.zeros((48, 64, 3), device=DEV, dtype=torch.int8)
    ops.render_16x16(0, 64, 48, e(1, 2), e(1, 4), e(1, 4), ku, vu, ranges, torch.tensor([1.0, 0.5, 0.0]), img)
    torch.cuda.synchronize()
    assert (ranges == 0).all()
    assert (img.view(torch.uint8).cpu().numpy() == np.array([255, 127, 0], np.uint8)).all()
    # all Gaussians culled (behind the camera)
    sc = make_scene([[0, 0, -1.0], [0, 0, 0.1]], 0.1, [0.9, 0.9])
    f = Frame(ops, sc, cam)
    assert f.R == 0 and (f.np("img") == 0).all()


def test_pair_overflow_is_reported_not_written(ops, oracle_lib):
    w, sc, cams = scenes.make_workload("C1", 20000)
    cam = cams[0]
    R = int(oracle_lib.preprocess(sc, cam)["counters"][3])
    cap = 1000
    f = Frame.__new__(Frame)
    P = sc.num_vertex
    z = lambda shape, dt: torch.zeros(shape, device=DEV, dtype=dt)  # noqa: E731
    ku = torch.full((cap + 64,), -1, device=DEV, dtype=torch.int64)
    vu = torch.full((cap + 64,), -1, device=DEV, dtype=torch.int32)
    off = z(1, torch.int32)
    assert ops.device_status() == 0
    ops.preprocess(_t(sc.position), _t(sc.shs), _t(sc.opacity), _t(sc.cov3d), cam.width, cam.height, 16, 16,
                   torch.from_numpy(cam.position.copy()), torch.from_numpy(cam.rotation.copy()),
                   cam.focal_x, cam.focal_y, cam.zFar, cam.zNear, z((P, 2), torch.float32), z((P, 4), torch.float32),
                   z((P, 4), torch.float32), ku[:cap], vu[:cap], off)
    assert int(off.cpu()[0]) == R                      # the counter keeps counting (example.py:81 compares it)
    assert (ku[cap:] == -1).all() and (vu[cap:] == -1).all()
    from flashgs_b200 import _lib
    assert ops.device_status() & _lib.ERR_PAIR_OVERFLOW
    assert ops.device_status() == 0                    # reading with reset clears it
    with pytest.raises(RuntimeError):
        ops.sort_gaussian(R, cam.width, cam.height, 16, 16, z(1 << 20, torch.int8), ku[:cap], vu[:cap], ku[:cap].clone(), vu[:cap].clone())


def _sort_case(ops, oracle_lib, keys, vals, width, height, junk=False):
    """Both sort entry points against the oracle's stable sort. ``stable=True``: the same bytes. Default: the same
    keys and the same multiset of pairs, and every run of identical keys in ascending order of its values (with
    ``junk`` -- bits above the sorted width in the keys -- only the order on the sorted bits is defined)."""
    n = keys.size
    ki, vi = _t(keys.view(np.int64)), _t(vals.view(np.int32))
    tmp = torch.zeros(ops.get_sort_buffer_size(n), device=DEV, dtype=torch.int8)
    ek, ev = oracle_lib.sort_pairs(keys, vals, width, height)
    mask = np.uint64((1 << scenes.sort_end_bit(width, height)) - 1)
    for stable in (True, False):
        ko, vo = torch.zeros_like(ki), torch.zeros_like(vi)
        ops.sort_gaussian(n, width, height, 16, 16, tmp, ki, vi, ko, vo, stable=stable)
        torch.cuda.synchronize()
        k, v = ko.cpu().numpy().view(np.uint64), vo.cpu().numpy().view(np.uint32)
        if stable:
            assert (k == ek).all()
            assert (v == ev).all()      # stable: values follow exactly
            continue
        assert ((k & mask) == (ek & mask)).all()
        o1, o2 = np.lexsort((v, k)), np.lexsort((ev, ek))
        assert (k[o1] == ek[o2]).all() and (v[o1] == ev[o2]).all()      # the same pairs
        if not junk:
            assert (k == ek).all()
            same = k[1:] == k[:-1]
            assert (v[1:][same] >= v[:-1][same]).all()                  # ties in ascending order of value
    assert (ki.cpu().numpy().view(np.uint64) == keys).all()    # inputs preserved
    assert (vi.cpu().numpy().view(np.uint32) == vals).all()


@pytest.mark.parametrize("n", [1, 2, 31, 4095, 4096, 4097, 100003, 1 << 20])
def test_sort_random_sizes(ops, oracle_lib, n):
    rng = np.random.default_rng(n)
    W, H = 3840, 2160    # 47 live bits
    tiles = 240 * 135
    keys = (rng.integers(0, tiles, n, dtype=np.uint64) << np.uint64(32)) | rng.integers(0, 1 << 32, n, dtype=np.uint64)
    vals = rng.integers(0, 1 << 32, n, dtype=np.uint64).astype(np.uint32)
    _sort_case(ops, oracle_lib, keys, vals, W, H)


def test_sort_images_with_more_tiles_than_the_bucketed_path_takes(ops, oracle_lib):
    # 8192 x 8192: 262 144 tiles = 18 tile bits, 51 sorted bits -> seven plain digit passes, no in-block tile sorts
    rng = np.random.default_rng(5)
    n = 300000
    W = H = 8192
    tiles = 512 * 512
    keys = (rng.integers(0, tiles, n, dtype=np.uint64) << np.uint64(32)) | rng.integers(0, 1 << 32, n, dtype=np.uint64)
    keys[::7] = keys[3]   # runs of equal keys: stability
    vals = np.arange(n, dtype=np.uint32)
    _sort_case(ops, oracle_lib, keys, vals, W, H)
    assert ops.device_status() == 0


def test_sort_adversarial(ops, oracle_lib):
    rng = np.random.default_rng(1)
    n = 50000
    vals = np.arange(n, dtype=np.uint32)
    W, H = 800, 800      # 44 live bits
    base = (rng.integers(0, 2500, n, dtype=np.uint64) << np.uint64(32)) | rng.integers(0, 1 << 32, n, dtype=np.uint64)
    _sort_case(ops, oracle_lib, np.full(n, base[0], np.uint64), vals, W, H)                  # all equal: stability
    _sort_case(ops, oracle_lib, np.sort(base), vals, W, H)                                    # already sorted
    _sort_case(ops, oracle_lib, np.sort(base)[::-1].copy(), vals, W, H)                       # reversed
    _sort_case(ops, oracle_lib, base & np.uint64(0xFFFFFFFF0000FF00), vals, W, H)             # many duplicates
    # bits at and above the sorted width are carried along but never compared (sort.cu:39)
    junk = base | (rng.integers(0, 1 << 19, n, dtype=np.uint64) << np.uint64(44))
    _sort_case(ops, oracle_lib, junk, vals, W, H, junk=True)
    # values in no particular order: ties of the default sort still come out by value
    _sort_case(ops, oracle_lib, base & np.uint64(0xFFFFFFFF0000FF00), rng.permutation(n).astype(np.uint32), W, H)
    # the same pair twice
    _sort_case(ops, oracle_lib, np.repeat(base[: n // 2], 2), np.repeat(vals[: n // 2], 2), W, H)
    # tiny image: 1 tile -> 33 live bits, the last digit is a single bit
    _sort_case(ops, oracle_lib, (rng.integers(0, 2, n, dtype=np.uint64) << np.uint64(32)) | (base & np.uint64(0xFFFFFFFF)), vals, 16, 16)


def test_bucketed_and_plain_sort_agree(ops):
    """The tile-bucketed path (tile digit passes + in-block depth sort) and the plain six-pass sort give the same bytes."""
    from flashgs_b200 import _lib
    L = _lib.load()
    rng = np.random.default_rng(7)
    for n, W, H in ((300000, 800, 800), (2000000, 3840, 2160), (5000, 64, 64)):
        tiles = ((W + 15) // 16) * ((H + 15) // 16)
        keys = (rng.integers(0, tiles, n, dtype=np.uint64) << np.uint64(32)) | (rng.integers(0, 1 << 20, n, dtype=np.uint64) << np.uint64(8))
        ki, vi = _t(keys.view(np.int64)), _t(np.arange(n, dtype=np.int32))
        tmp = torch.zeros(ops.get_sort_buffer_size(n), device=DEV, dtype=torch.int8)
        outs = []
        for plain in (0, 1):
            ko, vo = torch.zeros_like(ki), torch.zeros_like(vi)
            L.fgs_debug_sort_plain(plain)
            try:
                ops.sort_gaussian(n, W, H, 16, 16, tmp, ki, vi, ko, vo)
                torch.cuda.synchronize()
            finally:
                L.fgs_debug_sort_plain(0)
            outs.append((ko, vo))
        assert (outs[0][0] == outs[1][0]).all() and (outs[0][1] == outs[1][1]).all()
        tk, ti = torch.sort(ki, stable=True)
        assert (tk == outs[0][0]).all() and (vi[ti] == outs[0][1]).all()
    # one tile whose depths pile up at two values (the bucket sort hands over to the bitonic network), one tile
    # with all depths equal, and lists too long for the in-block sort (sorted by the block's radix passes in
    # global memory): two depth values, all depths equal, every depth byte in use, a ragged last chunk
    for n, depths in ((3000, [1, 1 << 30]), (3000, [12345]), (6000, [1, 1 << 30]), (4096, list(range(1, 4097))),
                      (4097, [7]), (50000, [12345]), (100003, None), (8192, None), (12289, [3, 1 << 8, 1 << 16, 1 << 24])):
        keys = rng.integers(0, 1 << 32, n, dtype=np.uint64) if depths is None else rng.choice(np.array(depths, dtype=np.uint64), n)
        ki, vi = _t(keys.view(np.int64)), _t(np.arange(n, dtype=np.int32))
        ko, vo = torch.zeros_like(ki), torch.zeros_like(vi)
        tmp = torch.zeros(ops.get_sort_buffer_size(n), device=DEV, dtype=torch.int8)
        ops.sort_gaussian(n, 16, 16, 16, 16, tmp, ki, vi, ko, vo)
        torch.cuda.synchronize()
        tk, ti = torch.sort(ki, stable=True)
        assert (tk == ko).all() and (vi[ti] == vo).all()
    assert ops.device_status() == 0


def test_long_tile_lists_among_short_ones(ops, oracle_lib):
    """Close-up views pile tens of thousands of splats on some tiles: those lists take the long-list path of the tile
    sort while their neighbours take the in-block sorts; the result is the stable sort of the whole list, and bits
    above the sorted width travel with their keys."""
    rng = np.random.default_rng(11)
    W, H = 800, 800
    tiles = 50 * 50
    n = 600000
    t = rng.integers(0, tiles, n, dtype=np.uint64)
    t[:150000] = rng.choice(np.array([3, 4, 1200, 2499], dtype=np.uint64), 150000)   # four lists of about 37500
    t[150000:160000] = 77                                                             # and one of about 10000
    depth = rng.integers(0, 1 << 32, n, dtype=np.uint64)
    depth[rng.random(n) < 0.3] &= np.uint64(0xFFFF0000)                               # many equal depths
    keys = (t << np.uint64(32)) | depth
    vals = np.arange(n, dtype=np.uint32)
    _sort_case(ops, oracle_lib, keys, vals, W, H)
    junk = keys | (rng.integers(0, 1 << 19, n, dtype=np.uint64) << np.uint64(44))
    _sort_case(ops, oracle_lib, junk, vals, W, H, junk=True)
    _sort_case(ops, oracle_lib, keys, rng.permutation(n).astype(np.uint32), W, H)
    assert ops.device_status() == 0


def test_tile_ranges_match_oracle(ops, oracle_lib):
    from flashgs_b200 import _lib
    L = _lib.load()
    rng = np.random.default_rng(2)
    for ntiles, n in ((1, 10), (50, 0), (2500, 1), (2500, 30000), (32400, 200000)):
        t = np.sort(rng.integers(0, ntiles, n, dtype=np.uint64)) if n else np.zeros(0, np.uint64)
        if n > 10:
            t[t == 3] = 4        # make sure some tiles are empty
        keys = (t << np.uint64(32)) | rng.integers(0, 1 << 32, n, dtype=np.uint64)
        kd = _t(keys.view(np.int64)) if n else torch.zeros(1, device=DEV, dtype=torch.int64)
        r = torch.full((ntiles, 2), -5, device=DEV, dtype=torch.int32)
        assert L.fgs_tile_ranges(n, ntiles, kd.data_ptr(), r.data_ptr(), None) == 0
        torch.cuda.synchronize()
        assert (r.cpu().numpy() == oracle_lib.tile_ranges(keys, ntiles)).all()


def test_bounded_lookback_wait_reports_timeout(ops):
    """A partition that never publishes makes its successors' bounded wait run out: the sort
    returns, the device status carries the timeout bit, and the context stays usable."""
    from flashgs_b200 import _lib
    L = _lib.load()
    rng = np.random.default_rng(3)
    n = 40 * 4096
    keys = (rng.integers(0, 2500, n, dtype=np.uint64) << np.uint64(32)) | rng.integers(0, 1 << 32, n, dtype=np.uint64)
    ki, vi = _t(keys.view(np.int64)), _t(np.arange(n, dtype=np.int32))
    ko, vo = torch.zeros_like(ki), torch.zeros_like(vi)
    tmp = torch.zeros(ops.get_sort_buffer_size(n), device=DEV, dtype=torch.int8)
    assert ops.device_status() == 0
    L.fgs_debug_sort_skip_publish(3)
    try:
        ops.sort_gaussian(n, 800, 800, 16, 16, tmp, ki, vi, ko, vo, stable=True)   # the look-back lives in the stable path
        torch.cuda.synchronize()
    finally:
        L.fgs_debug_sort_skip_publish(-1)
    assert ops.device_status() & _lib.ERR_LOOKBACK_TIMEOUT
    ops.sort_gaussian(n, 800, 800, 16, 16, tmp, ki, vi, ko, vo, stable=True)          # works again
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert (torch.sort(ki, stable=True)[0] == ko).all()


@pytest.mark.parametrize("name,n,strips,cull", [("C1", 60000, 3, False), ("C1", 60000, 3, True), ("C4", 200000, 8, True),
                                                ("C1", 60000, 3, "bounds"), ("C4", 200000, 8, "bounds"), ("C3", 150000, 5, "bounds")])
def test_strips_union_equals_frame(ops, name, n, strips, cull):
    """One frame split into strips of tile rows: the strips' pairs together are the frame's pairs, and the strips'
    pixels are the frame's pixels -- with and without the index list of the Gaussians that reach a strip."""
    w, sc, cams = scenes.make_workload(name, n)
    cam = cams[0] if name == "C1" else scenes.look_at_camera(1280, 720, 12.0, 50.0, 34.0, 17.0)
    full = Frame(ops, sc, cam)
    gy = scenes.tile_grid(cam.width, cam.height)[1]
    from flashgs_b200.parallel import strip_rows
    keys, vals = [], []
    img = np.zeros_like(full.np("img"))
    for r in range(strips):
        rows = strip_rows(gy, strips, r)
        part = Frame(ops, sc, cam, rows=rows, cull=cull)
        keys.append(part.np("ku", part.R)); vals.append(part.np("vu", part.R))
        img[rows[0] * 16: rows[1] * 16] = part.np("img")[rows[0] * 16: rows[1] * 16]
        vis = np.unique(part.np("vu", part.R))   # feature records of the strip's visible Gaussians are the frame's
        assert (part.np("xy")[vis].view(np.uint32) == full.np("xy")[vis].view(np.uint32)).all()
        assert (part.np("rd")[vis].view(np.uint32) == full.np("rd")[vis].view(np.uint32)).all()
        assert (part.np("co")[vis].view(np.uint32) == full.np("co")[vis].view(np.uint32)).all()
    ka, va = canonical_pairs(np.concatenate(keys), np.concatenate(vals))
    kb, vb = canonical_pairs(full.np("ku", full.R), full.np("vu", full.R))
    assert (ka == kb).all() and (va == vb).all()
    # same per-tile lists -> same pixels (splats of identical depth may swap: allow a few 1-level differences)
    d = np.abs(img.astype(int) - full.np("img").astype(int))
    assert d.max() <= 1 and (d > 0).mean() <= 1e-5
    assert ops.device_status() == 0


def test_rasterizer_loop_matches_stage_calls(ops):
    from flashgs_b200.rasterizer import DeviceScene, Rasterizer, TorchCamera
    w, sc, cams = scenes.make_workload("C1", 20000)
    cam = cams[0]
    ds = DeviceScene(sc, DEV)
    r = Rasterizer(ds, 1 << 20, 1 << 12)
    img = r.forward(ds, TorchCamera(cam), torch.zeros(3))
    f = Frame(ops, sc, cam, floats=False)
    assert img.dtype == torch.int8 and tuple(img.shape) == (cam.height, cam.width, 3)
    d = np.abs(img.cpu().numpy().view(np.uint8).astype(int) - f.np("img").astype(int))
    assert d.max() <= 1 and (d > 0).mean() <= 1e-5
    # drop-in module name of the reference extension
    import flash_gaussian_splatting
    assert flash_gaussian_splatting.ops.render_16x16 is ops.render_16x16


def test_example_flow_from_ply(ops, oracle_lib, tmp_path):
    """The call sequence of the reference's example.py (loadPly -> Scene on device -> Rasterizer.forward -> PPM),
    through the drop-in module name, on a PLY written from raw model parameters."""
    import flash_gaussian_splatting
    from flashgs_b200 import ply
    from flashgs_b200.rasterizer import Rasterizer, TorchCamera, save_ppm
    rng = np.random.default_rng(21)
    n = 20000
    path = str(tmp_path / "point_cloud.ply")
    ply.save_ply(path, rng.normal(size=(n, 3)) * 2.0, rng.normal(size=(n, 3)) * 0.5, rng.normal(size=(n, 45)) * 0.05,
                 rng.normal(size=n) * 2.0, rng.normal(size=(n, 3)) * 0.8 - 4.0, rng.normal(size=(n, 4)))
    num_vertex, pos, shs, opa, cov = flash_gaussian_splatting.ops.loadPly(path)
    assert num_vertex == n

    class DevScene:   # example.py:10-27
        device = torch.device(DEV)
    sc = DevScene()
    sc.num_vertex, sc.position, sc.shs, sc.opacity, sc.cov3d = n, pos.to(DEV), shs.to(DEV), opa.to(DEV), cov.to(DEV)
    cam = scenes.look_at_camera(640, 480, 9.0, 60.0, 20.0, 10.0)
    ras = Rasterizer(sc, 1 << 21, 1 << 12, ops=flash_gaussian_splatting.ops)
    img = ras.forward(sc, TorchCamera(cam), torch.zeros(3))
    out = tmp_path / "view.ppm"
    save_ppm(img, str(out))
    assert out.read_bytes().startswith(b"P6\n640 480\n255\n") and out.stat().st_size == 15 + 640 * 480 * 3
    host = scenes.Scene(position=pos.numpy(), shs=shs.numpy(), opacity=opa.numpy(), cov3d=cov.numpy())
    want = oracle_lib.render_frame(host, cam, floats=False)
    assert ras.num_rendered == int(want["counters"][3])
    d = np.abs(img.cpu().numpy().view(np.uint8).astype(int) - want["u8"].astype(int))
    assert d.max() <= 1 and (d > 0).mean() <= 1e-3


def test_full_size_properties(ops):
    """Headline workload at full size (6 M Gaussians, 3840x2160): properties that need no oracle run.
    Sortedness and permutation of the pair list, tile ranges consistent with the keys, stand-alone stages equal to
    the frame loop, every pixel written."""
    from flashgs_b200.rasterizer import DeviceScene, Rasterizer, TorchCamera
    w, sc, cams = scenes.make_workload("C4")
    cam = cams[0]
    ds = DeviceScene(sc, DEV)
    ras = Rasterizer(ds, 1 << 25, 1 << 16)
    img = torch.full((cam.height, cam.width, 3), 0x5A, device=DEV, dtype=torch.int8)
    ras.forward(ds, TorchCamera(cam), torch.tensor([1.0, 0.0, 1.0]), out_color=img)
    torch.cuda.synchronize()
    R = ras.num_rendered
    assert 25_000_000 < R < (1 << 25)
    ku, vu = ras.gaussian_keys_unsorted[:R], ras.gaussian_values_unsorted[:R]
    ks, vs = ras.gaussian_keys_sorted[:R], ras.gaussian_values_sorted[:R]
    assert (ks[1:] >= ks[:-1]).all()                                     # sorted
    assert int(ku.sum()) == int(ks.sum()) and int(vu.sum(dtype=torch.int64)) == int(vs.sum(dtype=torch.int64))
    assert int((ku ^ (vu.long() << 20)).sum()) == int((ks ^ (vs.long() << 20)).sum())   # pairs stay together
    gx, gy = scenes.tile_grid(cam.width, cam.height)
    tiles = ks >> 32
    assert int(tiles.max()) < gx * gy
    counts = torch.bincount(tiles, minlength=gx * gy)
    rg = ras.ranges[: gx * gy].long()
    assert ((rg[:, 1] - rg[:, 0]) == counts).all()
    nonempty = counts > 0
    assert (rg[nonempty, 0] == (torch.cumsum(counts, 0) - counts)[nonempty]).all()
    # depth bits of a key are the depth stored for its Gaussian
    sample = torch.randint(0, R, (200000,), device=DEV)
    assert ((ks[sample] & 0xFFFFFFFF) == ras.rgb_depth[vs[sample].long(), 3].view(torch.int32).long()).all()
    # magenta background, dense scene: no untouched byte pattern left, image not constant
    u8 = img.view(torch.uint8)
    assert not bool((u8 == 0x5A).all(dim=2).any()) or int((u8 == 0x5A).all(dim=2).sum()) < 100
    assert u8.float().std() > 5
    assert ops.device_status() == 0


def test_render_scene_driver(tmp_path, oracle_lib):
    """Model directory in, PPM files out: the driver that mirrors the reference's example script."""
    from flashgs_b200 import ply, render_scene
    rng = np.random.default_rng(33)
    n = 8000
    d = tmp_path / "model"
    (d / "point_cloud" / "iteration_30000").mkdir(parents=True)
    ply.save_ply(str(d / "point_cloud" / "iteration_30000" / "point_cloud.ply"), rng.normal(size=(n, 3)) * 2.0,
                 rng.normal(size=(n, 3)) * 0.5, rng.normal(size=(n, 45)) * 0.05, rng.normal(size=n) * 2.0,
                 rng.normal(size=(n, 3)) * 0.8 - 4.0, rng.normal(size=(n, 4)))
    cams = [scenes.look_at_camera(320, 240, 9.0, 60.0, az, 10.0, cam_id=i) for i, az in enumerate((0.0, 120.0))]
    import json
    (d / "cameras.json").write_text(json.dumps([render_scene.camera_to_json(c) for c in cams]))
    times = render_scene.render_scene(str(d), test_performance=True, max_num_rendered=1 << 21, max_num_tiles=1 << 12)
    assert set(times) == {"view000", "view001"}
    _, pos, shs, opa, cov = ply.load_ply(str(d / "point_cloud" / "iteration_30000" / "point_cloud.ply"))
    host = scenes.Scene(position=pos.numpy(), shs=shs.numpy(), opacity=opa.numpy(), cov3d=cov.numpy())
    for c in cams:
        raw = (d / "test_out" / (c.img_name + ".ppm")).read_bytes()
        head = b"P6\n320 240\n255\n"
        assert raw.startswith(head)
        img = np.frombuffer(raw[len(head):], np.uint8).reshape(240, 320, 3)
        want = oracle_lib.render_frame(host, c, floats=False)["u8"]
        diff = np.abs(img.astype(int) - want.astype(int))
        assert diff.max() <= 1 and (diff > 0).mean() <= 1e-3


def test_fused_frame_equals_stage_calls(ops, oracle_lib):
    """fgs_render_frame (no host read-back, device-side pair count) against the three stage calls."""
    from flashgs_b200 import _lib
    from flashgs_b200.rasterizer import DeviceScene, Rasterizer, TorchCamera
    for name, n, block in (("C1", 60000, (16, 16)), ("C4", 150000, (16, 16)), ("C1", 30000, (32, 32))):
        w = scenes.WORKLOADS[name]
        sc = scenes.make_scene(n, w.clusters, w.log_scale, seed=4)
        cam = scenes.look_at_camera(960, 544, w.radius, w.hfov_deg, w.azimuth_deg, w.elevation_deg)
        ds = DeviceScene(sc, DEV)
        tc = TorchCamera(cam)
        bg = torch.tensor([0.1, 0.2, 0.3])
        ras = Rasterizer(ds, 1 << 22, 1 << 14, block=block)
        a = ras.forward(ds, tc, bg).cpu().numpy().view(np.uint8)
        R = ras.num_rendered
        ks_a = ras.gaussian_keys_sorted[:R].clone()
        vs_a = ras.gaussian_values_sorted[:R].clone()
        ras.gaussian_keys_sorted.zero_(); ras.gaussian_values_sorted.zero_()
        b = ras.forward_fused(ds, tc, bg).cpu().numpy().view(np.uint8)
        assert int(ras.curr_offset.cpu()[0]) == R
        assert (ras.gaussian_keys_sorted[:R] == ks_a).all()
        assert (canonical_sorted_values(ks_a.cpu().numpy().view(np.uint64), vs_a.cpu().numpy().view(np.uint32)) ==
                canonical_sorted_values(ras.gaussian_keys_sorted[:R].cpu().numpy().view(np.uint64),
                                        ras.gaussian_values_sorted[:R].cpu().numpy().view(np.uint32))).all()
        d = np.abs(a.astype(int) - b.astype(int))
        assert d.max() <= 1 and (d > 0).mean() <= 1e-5
        # that call took the tiles up heaviest first (the order comes from the first frame's consumed counts) and left
        # its own counts; further frames, whatever order they use, are the same bytes
        gxy = scenes.tile_grid(cam.width, cam.height, *block)
        T = gxy[0] * gxy[1]
        assert ras._order is not None and ras._order.numel() == T
        consumed = ras.tile_consumed[:T].clone()
        for _ in range(2):
            assert (ras.forward_fused(ds, tc, bg).cpu().numpy().view(np.uint8) == b).all()
            assert (ras.tile_consumed[:T] == consumed).all()
        # a strip through the fused call
        gy = scenes.tile_grid(cam.width, cam.height, *block)[1]
        rows = (gy // 3, 2 * gy // 3)
        c = ras.forward_fused(ds, tc, bg, rows=rows).cpu().numpy().view(np.uint8)
        y0, y1 = rows[0] * block[1], min(cam.height, rows[1] * block[1])
        d = np.abs(a[y0:y1].astype(int) - c[y0:y1].astype(int))
        assert d.max() <= 1 and (d > 0).mean() <= 1e-5
        assert ops.device_status() == 0
    # pair buffers too small: the call still completes, the overflow is reported, the context stays usable
    small = Rasterizer(ds, 4096, 1 << 14, block=(32, 32))
    small.list_sorting_space = torch.zeros(ops.get_sort_buffer_size(4096), device=DEV, dtype=torch.int8)
    small.forward_fused(ds, tc, bg)
    torch.cuda.synchronize()
    assert int(small.curr_offset.cpu()[0]) > 4096
    assert ops.device_status() & _lib.ERR_PAIR_OVERFLOW
    assert ops.device_status() == 0


def test_reference_example_script_runs_unchanged(tmp_path):
    """The reference's own example.py (placed beside the reference build by oracle/build.py, byte for byte the
    reference's file), run as a script in a fresh interpreter with this repository first on the module path: its
    ``import flash_gaussian_splatting`` resolves to the drop-in package, and the PPM files it writes are the ones this
    repository's own driver writes."""
    import hashlib
    import json
    import os
    import subprocess
    import sys
    from flashgs_b200 import ply, render_scene
    from oracle import build as oracle_build
    script = oracle_build.REF_EXAMPLE
    if not os.path.exists(script):
        pytest.skip("the reference's example.py is not present beside the reference build")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    rng = np.random.default_rng(34)
    n = 30000
    d = tmp_path / "model"
    (d / "point_cloud" / "iteration_30000").mkdir(parents=True)
    ply.save_ply(str(d / "point_cloud" / "iteration_30000" / "point_cloud.ply"), rng.normal(size=(n, 3)) * 2.0,
                 rng.normal(size=(n, 3)) * 0.5, rng.normal(size=(n, 45)) * 0.05, rng.normal(size=n) * 2.0,
                 rng.normal(size=(n, 3)) * 0.8 - 4.0, rng.normal(size=(n, 4)))
    cams = [scenes.look_at_camera(400, 304, 9.0, 60.0, az, 10.0, cam_id=i) for i, az in enumerate((0.0, 120.0, 240.0))]
    (d / "cameras.json").write_text(json.dumps([render_scene.camera_to_json(c) for c in cams]))
    code = ("import sys, runpy\n"
            "sys.path.insert(0, %r)\n"
            "sys.argv = [%r, %r]\n"
            "runpy.run_path(%r, run_name='__main__')\n"
            "import flash_gaussian_splatting, flashgs_b200.ops\n"
            "assert flash_gaussian_splatting.ops is flashgs_b200.ops\n" % (root, script, str(d), script))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    assert "num_vertex = %d" % n in r.stdout and "fps = " in r.stdout
    theirs = {c.img_name: (d / "test_out" / (c.img_name + ".ppm")).read_bytes() for c in cams}
    for c in cams:
        os.remove(str(d / "test_out" / (c.img_name + ".ppm")))
    render_scene.render_scene(str(d), max_num_rendered=1 << 22, max_num_tiles=1 << 12)
    for c in cams:
        mine = (d / "test_out" / (c.img_name + ".ppm")).read_bytes()
        assert mine.startswith(b"P6\n400 304\n255\n")
        assert hashlib.sha256(mine).digest() == hashlib.sha256(theirs[c.img_name]).digest(), c.img_name


def test_view_batch_views_match_oracle(ops, oracle_lib):
    """Views of the 64-view workload (a circle of cameras at 15 degrees elevation around one scene) at reduced size:
    the views a rank renders one after the other with one set of buffers are each the oracle's image of that view."""
    from flashgs_b200 import parallel
    from flashgs_b200.rasterizer import DeviceScene, Rasterizer, TorchCamera
    w = scenes.WORKLOADS["C5"]
    sc = scenes.make_scene(60000, w.clusters, w.log_scale, seed=w.seed)
    all_cams = scenes.make_cameras(w)
    assert len(all_cams) == 64
    mine = parallel.views_of_rank(len(all_cams), 8, 3)       # the views of rank 3 of 8
    assert mine == list(range(3, 64, 8))
    ds = DeviceScene(sc, DEV)
    ras = Rasterizer(ds, 1 << 22, 1 << 14)
    img = torch.zeros((270, 480, 3), device=DEV, dtype=torch.int8)
    for v in mine[:3]:
        full = all_cams[v]
        cam = scenes.look_at_camera(480, 270, w.radius, w.hfov_deg, w.azimuth_deg + 360.0 * v / w.views, w.elevation_deg, cam_id=v)
        assert np.allclose(cam.position, full.position) and np.allclose(cam.rotation, full.rotation)
        ras.forward(ds, TorchCamera(cam), torch.zeros(3), out_color=img)
        want = oracle_lib.render_frame(sc, cam, floats=False)
        assert ras.num_rendered == int(want["counters"][3])
        d = np.abs(img.cpu().numpy().view(np.uint8).astype(int) - want["u8"].astype(int))
        assert d.max() <= 1 and (d > 0).mean() <= 1e-3
    assert ops.device_status() == 0


def test_sort_from_preprocess_tile_counts(ops, oracle_lib):
    """preprocess counts the pairs per tile while it emits them; the sort given that table skips its own counting pass
    and gives the same bytes. A table that does not belong to the pair list is detected on the device: nothing is
    moved, the status word says so, nothing outside the buffers is touched."""
    from flashgs_b200 import _lib
    w, sc, cams = scenes.make_workload("C1", 50000)
    cam = cams[0]
    a = Frame(ops, sc, cam, floats=False)
    b = Frame(ops, sc, cam, floats=False, cull="bounds")
    assert a.R == b.R
    assert (a.np("ks", a.R) == b.np("ks", b.R)).all() and (a.np("vs", a.R) == b.np("vs", b.R)).all()
    assert (a.np("img") == b.np("img")).all()            # the same pair set -> byte for byte the same image
    gx, gy = scenes.tile_grid(cam.width, cam.height)
    counts = b.counts.cpu().numpy()
    want = np.bincount((b.np("ku", b.R) >> np.uint64(32)).astype(np.int64), minlength=65536)
    assert (counts == want).all() and counts[gx * gy:].sum() == 0
    # strips count their own pairs only
    c = Frame(ops, sc, cam, rows=(10, 20), cull="bounds")
    want = np.bincount((c.np("ku", c.R) >> np.uint64(32)).astype(np.int64), minlength=65536)
    assert (c.counts.cpu().numpy() == want).all()
    d = np.abs(a.np("img")[160:320].astype(int) - c.np("img")[160:320].astype(int))
    assert d.max() <= 1 and (d > 0).mean() <= 1e-5
    # a table of another frame: refused on the device
    assert ops.device_status() == 0
    guard_k = torch.full((a.R + 64,), -7, device=DEV, dtype=torch.int64)
    guard_v = torch.full((a.R + 64,), -7, device=DEV, dtype=torch.int32)
    ops.sort_gaussian(a.R, cam.width, cam.height, 16, 16, a.temp, a.ku, a.vu, guard_k[: a.R], guard_v[: a.R], tile_counts=c.counts)
    torch.cuda.synchronize()
    assert ops.device_status() & _lib.ERR_BAD_ARG
    assert (guard_k[a.R:] == -7).all() and (guard_v[a.R:] == -7).all()
    assert ops.device_status() == 0


def test_tile_order_changes_nothing_but_the_time(ops, oracle_lib):
    """The blend may be told in which order to take the tiles up (heaviest first shortens a launch's tail). Whatever the
    order, the image is the same bytes, the per-tile consumed counts are the oracle's, and an entry that is not a tile
    of the rendered rows is ignored."""
    w, sc, cams = scenes.make_workload("C1", 40000)
    cam = cams[0]
    f = Frame(ops, sc, cam)                       # float outputs and consumed counts through the general kernel
    o = oracle_lib.render_frame(sc, cam)
    gx, gy = scenes.tile_grid(cam.width, cam.height)
    T = gx * gy
    bg = torch.zeros(3)
    rng = np.random.default_rng(4)

    def render(order=None, rows=(0, -1), consumed=None):
        img = torch.full((cam.height, cam.width, 3), 0x33, device=DEV, dtype=torch.uint8)
        ops.render_16x16(f.R, cam.width, cam.height, f.xy, f.rd, f.co, f.ks, f.vs, f.ranges, bg, img,
                         tile_order=order, consumed=consumed) if rows == (0, -1) else \
            ops.render_ex(16, 16, f.R, cam.width, cam.height, f.xy, f.rd, f.co, f.ks, f.vs, f.ranges, bg, out_color=img,
                          tile_row_begin=rows[0], tile_row_end=rows[1], tile_order=order, consumed=consumed)
        torch.cuda.synchronize()
        return img.cpu().numpy()

    natural = render()
    d = np.abs(natural.astype(int) - f.np("img").astype(int))      # the kernel with float outputs beside it
    assert d.max() <= 1 and (d > 0).mean() <= 1e-5
    consumed = torch.full((T,), -1, device=DEV, dtype=torch.int32)
    shuffled = render(order=_t(rng.permutation(T).astype(np.int32)), consumed=consumed)
    assert (shuffled == natural).all()
    assert (consumed.cpu().numpy() == f.np("consumed")).all()
    assert (consumed.cpu().numpy() == o["consumed"]).mean() >= 0.999
    # heaviest first, as the frame loop uses it
    order = ops.tile_order_from(consumed, cam.width, cam.height)
    assert order.dtype == torch.int32 and sorted(order.tolist()) == list(range(T))
    c = consumed.cpu().numpy()[order.cpu().numpy()]
    assert (c[1:] <= c[:-1]).all()
    assert (render(order=order) == natural).all()
    # a strip with its own order; entries outside the strip (and negative ones) are ignored, their slots render nothing
    rows = (gy // 4, gy // 2)
    strip_order = ops.tile_order_from(consumed, cam.width, cam.height, 16, 16, rows[0], rows[1])
    assert strip_order.numel() == (rows[1] - rows[0]) * gx
    strip = render(order=strip_order, rows=rows)
    y0, y1 = rows[0] * 16, rows[1] * 16
    assert (strip[y0:y1] == natural[y0:y1]).all() and (strip[:y0] == 0x33).all() and (strip[y1:] == 0x33).all()
    bad = strip_order.clone()
    bad[0], bad[1], bad[2] = 0, T + 5, -3          # a tile of another strip, a tile beyond the grid, a negative entry
    part = render(order=bad, rows=rows)
    assert (part[:y0] == 0x33).all() and (part[y1:] == 0x33).all()
    skipped = strip_order[:3].cpu().numpy()
    for t in range(T):
        ty, tx = divmod(t, gx)
        if not (rows[0] <= ty < rows[1]):
            continue
        tile = part[ty * 16:(ty + 1) * 16, tx * 16:(tx + 1) * 16]
        if t in skipped:
            assert (tile == 0x33).all()
        else:
            assert (tile == natural[ty * 16:(ty + 1) * 16, tx * 16:(tx + 1) * 16]).all()
    with pytest.raises(RuntimeError):
        render(order=strip_order[:5], rows=rows)          # too short for the rendered rows
    # the frame loop: the order appears after a few frames of one view and leaves the image alone
    from flashgs_b200.rasterizer import DeviceScene, Rasterizer, TorchCamera
    ds = DeviceScene(sc, DEV)
    ras = Rasterizer(ds, 1 << 21, 1 << 12)
    ras.order_refresh = 2
    imgs = [ras.forward(ds, TorchCamera(cam), bg).cpu().numpy().view(np.uint8) for _ in range(5)]
    assert ras._order is not None
    for im in imgs:
        assert (im == natural).all()
    assert ops.device_status() == 0


def test_chained_launches_change_nothing(ops):
    """The kernels of a frame are launched so that each one's blocks are resident and waiting when the one before it ends
    (programmatic dependent launch). Two views are rendered alternately, so every frame overwrites the other view's
    buffers: each frame's sorted lists and image must be the bytes of that view's first frame, and the bytes of the same
    frames rendered with plain launches, through the operator calls and through the single-call frame."""
    from flashgs_b200 import _lib
    from flashgs_b200.rasterizer import DeviceScene, Rasterizer, TorchCamera
    w = scenes.WORKLOADS["C4"]
    sc = scenes.make_scene(250000, w.clusters, w.log_scale, seed=11)
    cams = [scenes.look_at_camera(1280, 720, w.radius, w.hfov_deg, w.azimuth_deg + a, w.elevation_deg) for a in (0.0, 25.0)]
    ds = DeviceScene(sc, DEV)
    bg = torch.tensor([0.0, 0.1, 0.2])
    L = _lib.load()
    seen = {}
    try:
        for chained in (1, 0, 1):
            L.fgs_debug_chained_launches(chained)
            ras = Rasterizer(ds, 1 << 23, 1 << 14)
            for frame in range(24):
                v = frame & 1
                fused = (frame >> 1) & 1
                img = (ras.forward_fused if fused else ras.forward)(ds, TorchCamera(cams[v]), bg)
                R = int(ras.curr_offset.cpu()[0])
                got = (R, ras.gaussian_keys_sorted[:R].clone(), ras.gaussian_values_sorted[:R].clone(), img.clone())
                if v not in seen:
                    seen[v] = got
                    assert R > 100000
                    continue
                want = seen[v]
                assert got[0] == want[0], (chained, frame)
                for a, b in zip(got[1:], want[1:]):
                    assert bool((a == b).all()), (chained, frame, fused)
            del ras
        assert ops.device_status() == 0
    finally:
        L.fgs_debug_chained_launches(1)


def test_two_frames_in_flight(ops):
    """Two rasterizers on two streams, the next frame's ``begin`` queued before this frame's ``finish``: every frame
    is the bytes of the same view rendered alone."""
    from flashgs_b200.rasterizer import DeviceScene, Rasterizer, TorchCamera
    w = scenes.WORKLOADS["C4"]
    sc = scenes.make_scene(200000, w.clusters, w.log_scale, seed=3)
    cams = [TorchCamera(scenes.look_at_camera(1280, 720, w.radius, w.hfov_deg, w.azimuth_deg + 20.0 * i, w.elevation_deg)) for i in range(5)]
    ds = DeviceScene(sc, DEV)
    bg = torch.tensor([0.3, 0.2, 0.1])
    alone = Rasterizer(ds, 1 << 23, 1 << 14)
    want = [alone.forward(ds, c, bg).clone() for c in cams]
    counts = []
    for c in cams:
        alone.forward(ds, c, bg)
        counts.append(alone.num_rendered)
    slots = [(Rasterizer(ds, 1 << 23, 1 << 14), torch.cuda.Stream()), (Rasterizer(ds, 1 << 23, 1 << 14), torch.cuda.Stream())]
    torch.cuda.synchronize()
    frames = [k % len(cams) for k in range(12)]
    got = []
    with torch.cuda.stream(slots[0][1]):
        slots[0][0].begin(ds, cams[frames[0]])
    for k, v in enumerate(frames):
        r, s = slots[k & 1]
        if k + 1 < len(frames):
            rn, sn = slots[(k + 1) & 1]
            with torch.cuda.stream(sn):
                rn.begin(ds, cams[frames[k + 1]])
        with torch.cuda.stream(s):
            got.append((v, r.finish(ds, cams[v], bg), r.num_rendered))
    torch.cuda.synchronize()
    for v, img, n in got:
        assert n == counts[v]
        assert bool((img == want[v]).all()), v
    assert ops.device_status() == 0
