"""Records what the REFERENCE's own loadPly returns for a seeded synthetic PLY (CPU only, needs oracle/_ref).

Run where the reference build is present:  python tests/golden/make_ply_golden.py
Writes tests/golden/ply_golden.json: order-independent checksums of the bit patterns of the four arrays
plus the first records in full. The test regenerates the PLY from the same seed.
"""
import json
import os
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from flashgs_b200 import ply  # noqa: E402

SEED, N = 1234, 20000


def write_model(path):
    rng = np.random.default_rng(SEED)
    ply.save_ply(path, rng.normal(size=(N, 3)) * 3.0, rng.normal(size=(N, 3)), rng.normal(size=(N, 45)) * 0.1,
                 rng.normal(size=N) * 2.0, rng.normal(size=(N, 3)) - 4.0, rng.normal(size=(N, 4)))


def checksum(t):
    return int(np.ascontiguousarray(t.numpy()).view(np.uint32).astype(np.uint64).sum(dtype=np.uint64))


if __name__ == "__main__":
    from oracle import ref
    m = ref.load()
    if m is None:
        sys.exit("the reference build (oracle/_ref) is not available")
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "model.ply")
        write_model(path)
        n, pos, shs, opa, cov = m.ops.loadPly(path)
    out = dict(seed=SEED, n=int(n), pos=checksum(pos), shs=checksum(shs), opacity=checksum(opa), cov3d=checksum(cov),
               head=dict(pos=pos[:4].numpy().view(np.uint32).tolist(), shs=shs[:2].numpy().view(np.uint32).tolist(),
                         opacity=opa[:8].numpy().view(np.uint32).tolist(), cov3d=cov[:4].numpy().view(np.uint32).tolist()))
    json.dump(out, open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "ply_golden.json"), "w"))
    print("recorded", out["n"])
