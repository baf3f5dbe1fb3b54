"""Shared helpers of the test-suite: tiny hand-made scenes and list comparison."""
from __future__ import annotations

import numpy as np

from flashgs_b200.scenes import Camera, Scene


def identity_camera(width=65, height=65, focal=32.0):
    """Camera at the origin looking down +z with +y down: p_view == p exactly."""
    return Camera(width=width, height=height, position=np.zeros(3, np.float32),
                  rotation=np.eye(3, dtype=np.float32), focal_x=float(focal), focal_y=float(focal))


def make_scene(positions, sigmas, opacities, dc=None, rest=None):
    """Isotropic (sigma scalar) or axis-aligned (sigma triple) Gaussians with a DC-only colour by default."""
    pos = np.asarray(positions, np.float32).reshape(-1, 3)
    P = pos.shape[0]
    s = np.asarray(sigmas, np.float32)
    if s.ndim == 0:
        s = np.full((P, 3), float(s), np.float32)
    elif s.ndim == 1 and s.shape[0] == P and P != 3:
        s = np.repeat(s[:, None], 3, axis=1)
    s = s.reshape(P, 3)
    cov = np.zeros((P, 6), np.float32)
    cov[:, 0], cov[:, 3], cov[:, 5] = s[:, 0] ** 2, s[:, 1] ** 2, s[:, 2] ** 2
    shs = np.zeros((P, 16, 3), np.float32)
    if dc is not None:
        shs[:, 0, :] = np.asarray(dc, np.float32).reshape(-1, 3)
    if rest is not None:
        shs[:, 1:, :] = rest
    return Scene(position=np.ascontiguousarray(pos), shs=np.ascontiguousarray(shs.reshape(P, 48)),
                 opacity=np.ascontiguousarray(np.asarray(opacities, np.float32).reshape(P)), cov3d=cov)


def canonical_pairs(keys, values):
    """Pairs ordered by (key, value): the order-free form of an unsorted pair list."""
    keys = np.asarray(keys, np.uint64)
    values = np.asarray(values, np.uint32)
    o = np.lexsort((values, keys))
    return keys[o], values[o]


def canonical_sorted_values(keys_sorted, values_sorted):
    """Values of a sorted list with every run of equal keys ordered by value.

    The reference's order inside a run of identical 64-bit keys is the arrival order of
    its atomics, so two correct runs may differ there; this is the comparable form.
    """
    keys_sorted = np.asarray(keys_sorted, np.uint64)
    values_sorted = np.asarray(values_sorted, np.uint32)
    o = np.lexsort((values_sorted, keys_sorted))
    assert (keys_sorted[o] == keys_sorted).all(), "keys are not sorted"
    return values_sorted[o]


def psnr_u8(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    mse = ((a - b) ** 2).mean()
    return 99.0 if mse == 0 else 10.0 * np.log10(255.0 ** 2 / mse)


def f2u(x):
    return np.asarray(x, np.float32).view(np.uint32)
