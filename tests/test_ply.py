"""Scene loader parity (CPU): bit-identical to the reference's loadPly (csrc/pybind.cpp:58-120)."""
import json
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_ply_golden  # noqa: E402

from flashgs_b200 import ply  # noqa: E402


def test_matches_golden_from_reference(tmp_path):
    g = json.load(open(os.path.join(HERE, "golden", "ply_golden.json")))
    path = str(tmp_path / "model.ply")
    make_ply_golden.write_model(path)
    n, pos, shs, opa, cov = ply.load_ply(path)
    assert n == g["n"]
    for name, t in (("pos", pos), ("shs", shs), ("opacity", opa), ("cov3d", cov)):
        assert make_ply_golden.checksum(t) == g[name], name
        k = len(g["head"][name])
        assert t[:k].numpy().view(np.uint32).tolist() == g["head"][name]
    assert pos.dtype == torch.float32 and not pos.is_cuda and tuple(shs.shape) == (n, 48) and tuple(cov.shape) == (n, 6)


def test_matches_reference_loader_directly(tmp_path):
    from oracle import ref
    m = ref.load() if ref.available() else None
    if m is None:
        pytest.skip("reference build not present")
    rng = np.random.default_rng(5)
    n = 3000
    path = str(tmp_path / "m.ply")
    ply.save_ply(path, rng.normal(size=(n, 3)), rng.normal(size=(n, 3)), rng.normal(size=(n, 45)),
                 rng.normal(size=n) * 3, rng.normal(size=(n, 3)) - 3, rng.normal(size=(n, 4)))
    mine, theirs = ply.load_ply(path), m.ops.loadPly(path)
    assert mine[0] == theirs[0] == n
    for a, b in zip(mine[1:], theirs[1:]):
        assert (a.view(torch.int32) == b.view(torch.int32)).all()


def test_sh_layout_and_activations(tmp_path):
    # one vertex with recognisable values: f_rest is channel-major in the file, [coef][rgb] in the output
    path = str(tmp_path / "one.ply")
    f_rest = np.arange(45, dtype=np.float32).reshape(1, 45) + 100.0
    ply.save_ply(path, [[1, 2, 3]], [[10, 11, 12]], f_rest, [0.0], [[0.0, 0.0, 0.0]], [[2.0, 0.0, 0.0, 0.0]])
    n, pos, shs, opa, cov = ply.load_ply(path)
    assert n == 1 and pos[0].tolist() == [1, 2, 3]
    sh = shs[0].view(16, 3)
    assert sh[0].tolist() == [10, 11, 12]
    for j in range(1, 16):
        assert sh[j].tolist() == [100.0 + (j - 1), 100.0 + 15 + (j - 1), 100.0 + 30 + (j - 1)]
    assert opa[0].item() == 0.5                                   # sigmoid(0)
    assert cov[0].tolist() == [1.0, 0.0, 0.0, 1.0, 0.0, 1.0]       # unit scales, identity rotation (quaternion normalised)


def test_errors(tmp_path):
    with pytest.raises(RuntimeError):
        ply.load_ply(str(tmp_path / "missing.ply"))
    bad = tmp_path / "bad.ply"
    bad.write_bytes(b"ply\nformat binary_little_endian 1.0\nelement vertex 0\nend_header\n")
    with pytest.raises(RuntimeError):
        ply.load_ply(str(bad))
    trunc = tmp_path / "trunc.ply"
    trunc.write_bytes(b"ply\nelement vertex 5\nend_header\n" + b"\0" * 100)
    with pytest.raises(RuntimeError):
        ply.load_ply(str(trunc))
