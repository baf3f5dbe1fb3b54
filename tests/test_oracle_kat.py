"""Known-answer tests that pin the CPU oracle to the reference's semantics.

The reference has no tests or golden vectors, so each expected value here is derived by
hand from the cited reference lines (csrc/cuda_rasterizer/*.cu).
"""
import numpy as np
import pytest

from flashgs_b200 import scenes
from helpers import f2u, identity_camera, make_scene

C0 = 0.28209479177387814


@pytest.fixture(scope="module")
def orc(oracle_lib):
    return oracle_lib


def test_bit_length_and_sort_width(orc):
    # sort.cu:9-24 is int.bit_length; sort.cu:39 sorts bits [0, 32 + bit_length(tiles))
    L = orc.lib()
    for n in list(range(1, 5000)) + [2 ** k + d for k in range(12, 21) for d in (-1, 0, 1)]:
        assert L.fgso_higher_msb(n) == int(n).bit_length()
    want = {"C1": 44, "C2": 45, "C3": 47, "C4": 47, "C5": 46}
    for name, bits in want.items():
        w = scenes.WORKLOADS[name]
        assert scenes.sort_end_bit(w.width, w.height) == bits


def test_key_packing_and_float_order(orc):
    # preprocess.cu:327-329,399-401: key = (ty*grid.x + tx) << 32 | float_bits(depth)
    cam = identity_camera(65, 65, 32.0)
    # pixel = 32 * x/z + 32 = 40: well inside tile (2,2), the splat reaches less than 2 pixels
    sc = make_scene([[0.625, 0.625, 2.5]], 0.01, [0.9], dc=[[1, 1, 1]])
    pre = orc.preprocess(sc, cam)
    gx, _ = scenes.tile_grid(65, 65)
    assert pre["keys"].size == 1
    assert pre["xy"][0].tolist() == [40.0, 40.0]
    tile = (40 // 16) * gx + 40 // 16
    assert int(pre["keys"][0]) == (tile << 32) | int(f2u(2.5))
    assert int(pre["values"][0]) == 0
    z = np.sort(np.random.default_rng(0).uniform(0.2, 100.0, 1000).astype(np.float32))
    assert (np.diff(f2u(z).astype(np.int64)) >= 0).all()   # positive floats order like their bit patterns


def test_tile_ranges_hand_list(orc):
    # render.cu:9-31 + memset at 557: tiles without pairs stay (0,0)
    tiles = [1, 1, 1, 4, 6, 6]
    keys = np.array([(t << 32) | (100 + i) for i, t in enumerate(tiles)], np.uint64)
    r = orc.tile_ranges(keys, 8)
    want = np.zeros((8, 2), np.int32)
    want[1], want[4], want[6] = (0, 3), (3, 4), (4, 6)
    assert (r == want).all()
    assert (orc.tile_ranges(np.zeros(0, np.uint64), 5) == 0).all()


def test_cull_boundaries(orc):
    # preprocess.cu:288: z <= 0.2 culled; preprocess.cu:291: 255*opacity < 1 culled
    cam = identity_camera()
    z_cull = np.float32(0.2)
    z_keep = np.nextafter(z_cull, np.float32(1.0))
    op_lo = np.float32(1.0) / np.float32(255.0)
    while np.float32(255.0) * op_lo >= np.float32(1.0):
        op_lo = np.nextafter(op_lo, np.float32(0.0))
    op_hi = np.nextafter(op_lo, np.float32(1.0))
    assert np.float32(255.0) * op_hi >= np.float32(1.0)
    q = np.float32(0.25)   # x = y = z/4 projects to pixel (40, 40), inside one tile
    sc = make_scene([[q * z_cull, q * z_cull, z_cull], [q * z_keep, q * z_keep, z_keep], [q, q, 1.0], [q, q, 1.0]],
                    0.001, [0.9, 0.9, op_lo, op_hi])
    pre = orc.preprocess(sc, cam)
    assert sorted(pre["values"].tolist()) == [1, 3]
    assert pre["counters"].tolist() == [3, 2, 2, 2]     # P1, P2, V, R


def test_dc_only_colour(orc):
    # preprocess.cu:156,181-183: rgb = max(0, 0.5 + C0*dc), no upper clamp
    cam = identity_camera()
    dc = np.array([[1.0, -3.0, 4.0]], np.float32)
    sc = make_scene([[0.3, -0.2, 3.0]], 0.02, [0.8], dc=dc)
    pre = orc.preprocess(sc, cam)
    want = np.maximum(0.0, np.float32(0.5) + np.float32(C0) * dc[0])
    np.testing.assert_allclose(pre["rgb_depth"][0, :3], want, rtol=0, atol=1e-6)
    assert pre["rgb_depth"][0, 1] == 0.0 and pre["rgb_depth"][0, 2] > 1.0
    assert pre["rgb_depth"][0, 3] == np.float32(3.0)


def test_single_gaussian_centre_pixel(orc):
    # render.cu:40-52 with preprocess.cu:414: at the centre d = 0, alpha = 2^log2(opacity) = opacity
    cam = identity_camera(65, 65, 32.0)
    op = 0.75
    dc = [[1.0, 0.5, 0.0]]
    sc = make_scene([[0, 0, 1.0]], 0.05, [op], dc=dc)
    out = orc.render_frame(sc, cam)
    rgb = np.maximum(0.0, 0.5 + C0 * np.array(dc[0]))
    assert out["xy"][0].tolist() == [32.0, 32.0]
    np.testing.assert_allclose(out["alpha"][32, 32], op, atol=2e-7)
    np.testing.assert_allclose(out["rgb"][32, 32], rgb * op, atol=1e-6)
    np.testing.assert_allclose(out["depth"][32, 32], 1.0 * op, atol=1e-6)
    assert out["u8"][32, 32].tolist() == [int(v * op * 255.0) for v in rgb]
    # conic of an isotropic splat on the axis: 1 / (sigma^2 f^2 + 0.3) (preprocess.cu:140-141,303-305)
    c = 1.0 / (0.05 ** 2 * 32.0 ** 2 + 0.3)
    log2e = 1.4426950216293334961
    np.testing.assert_allclose(out["conic_opacity"][0], [-0.5 * log2e * c, 0.0, -0.5 * log2e * c, np.log2(op)], rtol=2e-6, atol=1e-7)
    # one pixel to the right: alpha = op * exp(-0.5 c)
    np.testing.assert_allclose(out["alpha"][32, 33], op * np.exp(-0.5 * c), rtol=1e-5)


def test_front_to_back_and_pair_stop_rule(orc):
    # render.cu:315,394-407: the tile stops after a PAIR once all its pixels have T < 1e-4
    cam = identity_camera(16, 16, 8.0)   # one tile
    big = 30.0                            # sigma in world units: alpha ~ opacity over the whole tile
    pos = [[0, 0, 1.0 + 0.5 * i] for i in range(5)]
    dcs = [[2, 0, 0], [0, 2, 0], [0, 0, 2], [2, 2, 0], [0, 2, 2]]
    sc = make_scene(pos, big, [0.5, 0.5, 0.995, 0.995, 0.9], dc=dcs)
    out = orc.render_frame(sc, cam)
    assert out["values_sorted"].tolist() == [0, 1, 2, 3, 4]        # depth order
    assert out["consumed"].tolist() == [4]                          # stops after the second pair, splat 4 unused
    a = out["alpha"][8, 8]
    assert a > 1 - 1e-4
    # red channel, front to back: colours r0, 0.5, 0.5, r0 with alphas 0.5, 0.5, 0.995, 0.995
    r0 = 0.5 + C0 * 2
    want = r0 * 0.5 + 0.5 * 0.5 * 0.5 + 0.5 * 0.995 * 0.25 + r0 * 0.995 * 0.25 * 0.005
    assert abs(out["rgb"][8, 8, 0] - want) < 2e-3
    # with the 3rd splat made transparent the tile never saturates inside a pair boundary before the list ends
    sc2 = make_scene(pos, big, [0.5, 0.5, 0.5, 0.5, 0.5], dc=dcs)
    assert orc.render_frame(sc2, cam)["consumed"].tolist() == [5]
    # two opaque splats first: stop right after the first pair
    sc3 = make_scene(pos, big, [0.995, 0.995, 0.9, 0.9, 0.9], dc=dcs)
    assert orc.render_frame(sc3, cam)["consumed"].tolist() == [2]


def _tiles_of(orc, cam, sc):
    pre = orc.preprocess(sc, cam)
    return sorted((pre["keys"] >> np.uint64(32)).astype(int).tolist())


def test_exact_tile_intersection(orc):
    # preprocess.cu:187-241: iso-ellipse conic.x dx^2 + 2 conic.y dx dy + conic.z dy^2 <= 2*power with
    # power = ln(256*opacity); axis-aligned, on the optical axis the 2D covariance is sigma_px^2 + 0.3.
    W = 64
    f = 32.0
    cam = identity_camera(W, W, f)
    gx, _ = scenes.tile_grid(W, W)
    op = 1.0
    reach = lambda s2: np.sqrt(2.0 * np.log(256.0 * op) * s2)   # noqa: E731  half-axis of the iso-ellipse in pixels
    # centre at pixel (8, 8) of tile (0,0): x_ndc such that pix = 8 -> x/z = (8 - 31.5)/32
    x = (8.0 - 31.5) / f
    # tile (1,0) starts at pixel x = 16: touched iff reach >= 8
    for sig_px, hit in ((2.30, False), (2.45, True)):
        s2 = sig_px ** 2 + 0.3
        assert (reach(s2) >= 8.0) == hit
        sc = make_scene([[x, x, 1.0]], [[sig_px / f, 0.3 / f, 0.3 / f]], [op])
        # the Jacobian's off-axis term adds a little x-variance; it is far below the margins chosen here
        tiles = _tiles_of(orc, cam, sc)
        assert (1 in tiles) == hit, (sig_px, tiles)
        assert 0 in tiles and gx not in tiles and gx + 1 not in tiles
    # corner: a round splat reaching the corner pixel (16,16) of tile (1,1): distance sqrt(128) = 11.31
    for sig_px, hit in ((3.2, False), (3.6, True)):
        s2 = sig_px ** 2 + 0.3
        assert (reach(s2) >= np.sqrt(128.0)) == hit
        # flat along z so that the off-axis Jacobian term adds no screen-space variance
        sc = make_scene([[x, x, 1.0]], [[sig_px / f, sig_px / f, 0.01 / f]], [op])
        tiles = _tiles_of(orc, cam, sc)
        assert ((gx + 1) in tiles) == hit, (sig_px, tiles)
        assert 1 in tiles and gx in tiles     # the edge-adjacent tiles are reached in both cases


def test_partial_tiles_stay_inside_image(orc):
    # width/height not multiples of the tile: every pixel written, nothing else touched
    cam = identity_camera(37, 21, 20.0)
    sc = make_scene([[0, 0, 1.0], [0.5, 0.2, 2.0]], 0.2, [0.9, 0.6], dc=[[1, 1, 1], [0, 1, 0]])
    out = orc.render_frame(sc, cam, bg=(0.25, 0.5, 0.75))
    assert out["u8"].shape == (21, 37, 3)
    assert out["u8"][20, 36].tolist() != [0, 0, 0]            # background reaches the last pixel
    far = out["u8"][0, 0].tolist()
    assert far == [int(0.25 * 255), int(0.5 * 255), int(0.75 * 255)] or max(abs(np.array(far) - [63, 127, 191])) <= 40


def test_strip_union_equals_frame(orc):
    w, sc, cams = scenes.make_workload("C1", 20000)
    cam = cams[0]
    full = orc.render_frame(sc, cam)
    gy = scenes.tile_grid(cam.width, cam.height)[1]
    keys, vals = [], []
    img = np.zeros_like(full["u8"])
    for rows in ((0, 13), (13, 30), (30, gy)):
        part = orc.render_frame(sc, cam, rows=rows)
        keys.append(part["keys"]); vals.append(part["values"])
        img[rows[0] * 16: rows[1] * 16] = part["u8"][rows[0] * 16: rows[1] * 16]
    from helpers import canonical_pairs
    ka, va = canonical_pairs(np.concatenate(keys), np.concatenate(vals))
    kb, vb = canonical_pairs(full["keys"], full["values"])
    assert (ka == kb).all() and (va == vb).all()
    assert (img == full["u8"]).all()
