"""Golden vectors recorded from the reference's own CUDA build (tests/golden/make_golden.py).

CPU part: the oracle reproduces them (this is what pins the oracle to the real reference).
GPU part: the sm_100a kernels reproduce them through the C ABI.
"""
import glob
import json
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden  # noqa: E402

from helpers import canonical_sorted_values, psnr_u8  # noqa: E402

FIXTURES = sorted(glob.glob(os.path.join(HERE, "golden", "ref_*.npz")))


def _load(path):
    g = np.load(path)
    spec = json.loads(str(g["spec"]))
    sc, cam = make_golden.build_inputs(spec)
    return g, sc, cam


def _compare(g, R, keys_unsorted, vals_unsorted, ks, vs, ranges, xy, rd, co, img, exact_colour):
    assert R == int(g["num_rendered"])
    assert make_golden.pair_checksum(keys_unsorted, vals_unsorted) == int(g["pair_checksum"])
    assert (canonical_sorted_values(ks, vs) == g["values_sorted"]).all()
    assert make_golden.bits_checksum((ks & np.uint64(0xFFFFFFFF)).astype(np.uint32)) == int(g["depth_bits_sorted_crc"])
    assert (ranges == g["ranges"]).all()
    vis, s = g["visible"], g["sample"]
    assert (np.unique(vals_unsorted) == vis).all()
    assert make_golden.bits_checksum(xy[vis]) == int(g["xy_crc"])
    assert (xy[s].view(np.uint32) == g["xy"].view(np.uint32)).all()
    assert (co[s][:, :3].view(np.uint32) == g["conic_opacity"][:, :3].view(np.uint32)).all()
    assert (rd[s][:, 3].view(np.uint32) == g["rgb_depth"][:, 3].view(np.uint32)).all()
    if exact_colour:
        assert make_golden.bits_checksum(rd[vis]) == int(g["rd_crc"])
        assert make_golden.bits_checksum(co[vis]) == int(g["co_crc"])
    else:   # the oracle uses libm where the GPU uses approximate instructions
        np.testing.assert_allclose(co[s][:, 3], g["conic_opacity"][:, 3], rtol=0, atol=2e-6)
        np.testing.assert_allclose(rd[s][:, :3], g["rgb_depth"][:, :3], rtol=0, atol=2e-6)
    d = np.abs(img.astype(int) - g["image"].astype(int))
    assert d.max() <= 1 and (d > 0).mean() <= 1e-3
    assert psnr_u8(img, g["image"]) > 60.0


def test_fixtures_exist():
    assert len(FIXTURES) >= 2, "golden vectors missing: run tests/golden/make_golden.py on a GPU box"


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p) for p in FIXTURES])
def test_oracle_reproduces_reference(path, oracle_lib):
    g, sc, cam = _load(path)
    o = oracle_lib.render_frame(sc, cam, floats=False)
    _compare(g, int(o["counters"][3]), o["keys"], o["values"], o["keys_sorted"], o["values_sorted"], o["ranges"],
             o["xy"], o["rgb_depth"], o["conic_opacity"], o["u8"], exact_colour=False)


@pytest.mark.gpu
@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p) for p in FIXTURES])
def test_kernels_reproduce_reference(path):
    from flashgs_b200 import ops
    from test_gpu_parity import Frame
    g, sc, cam = _load(path)
    f = Frame(ops, sc, cam, floats=False)
    R = f.R
    _compare(g, R, f.np("ku", R), f.np("vu", R), f.np("ks", R), f.np("vs", R), f.np("ranges"),
             f.np("xy"), f.np("rd"), f.np("co"), f.np("img"), exact_colour=True)
