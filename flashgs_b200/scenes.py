"""Seeded synthetic scenes and cameras for the five benchmark workloads.

The pre-trained scenes the reference's README points to (README.md:21,
example.py:152) are not redistributable with this repository, so every test
and benchmark renders seeded synthetic Gaussians whose shapes and value
distributions follow the workload descriptions: a mixture of isotropic
clusters plus a uniform background, log-normal scales, random rotations,
logit-normal opacities and degree-3 spherical harmonics.

Everything here is host-side numpy (PCG64 + ziggurat normals, which are
bit-reproducible across machines) so that a scene generated on one box is
byte-identical to the same scene generated on another.

Input conventions (they are the reference's):
  * ``position [P,3]``, ``shs [P,48]`` laid out ``[coef][rgb]``, ``opacity [P]``
    already passed through the sigmoid, ``cov3d [P,6]`` in the order
    xx, xy, xz, yy, yz, zz built the way ``computeCov3D`` does
    (csrc/pybind.cpp:22-56): quaternion (w,x,y,z) -> R, M = S*R, Sigma = M^T*M.
  * camera ``rotation [3,3]`` is camera-to-world, row-major, with columns
    [right | down | forward]; the rasterizer computes
    ``p_view = rotation^T (p - position)`` (csrc/cuda_rasterizer/preprocess.cu:420-427,
    csrc/pybind.cpp:140-143).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np


@dataclass
class Scene:
    """Host-side Gaussian buffers (fp32, C-contiguous), SoA like the reference's Scene (example.py:10-27)."""

    position: np.ndarray  # [P,3]
    shs: np.ndarray  # [P,48]
    opacity: np.ndarray  # [P]
    cov3d: np.ndarray  # [P,6]

    @property
    def num_vertex(self) -> int:
        return int(self.opacity.shape[0])


@dataclass
class Camera:
    """Pinhole camera in the reference's JSON convention (example.py:30-41)."""

    width: int
    height: int
    position: np.ndarray  # [3] fp32
    rotation: np.ndarray  # [3,3] fp32, camera-to-world, row-major
    focal_x: float
    focal_y: float
    zFar: float = 100.0
    zNear: float = 0.01
    id: int = 0
    img_name: str = "view0"


@dataclass
class Workload:
    """One benchmark workload: scene parameters plus its camera(s)."""

    name: str
    num_gaussians: int
    clusters: int
    width: int
    height: int
    radius: float
    hfov_deg: float
    log_scale: tuple  # ((mu, sigma), (mu, sigma), (mu, sigma)) per axis
    views: int = 1
    elevation_deg: float = 17.0
    azimuth_deg: float = 34.0
    seed: int = 0
    notes: str = ""
    extra: dict = field(default_factory=dict)


_ISO = lambda mu, sd: ((mu, sd), (mu, sd), (mu, sd))  # noqa: E731

# The five workloads. C3/C4 do not state a camera; they reuse C2's (radius 12,
# 50 degree horizontal field of view). C5 does not state a field of view; it
# uses 50 degrees as well. Both assumptions are repeated in every report.
WORKLOADS = {
    "C1": Workload("C1", 100_000, 64, 800, 800, 15.0, 60.0, _ISO(-4.5, 0.8),
                   notes="100k Gaussians, 800x800, oracle-sized"),
    "C2": Workload("C2", 1_000_000, 64, 1920, 1080, 12.0, 50.0, _ISO(-4.5, 0.8),
                   notes="1M Gaussians, 1080p (last tile row partial)"),
    "C3": Workload("C3", 3_000_000, 256, 3840, 2160, 12.0, 50.0, _ISO(-4.0, 1.0),
                   notes="3M Gaussians, 4K, dense tiles"),
    "C4": Workload("C4", 6_000_000, 256, 3840, 2160, 12.0, 50.0,
                   ((-2.5, 0.5), (-5.5, 0.5), (-5.5, 0.5)),
                   notes="6M needle-like Gaussians, 4K (headline)"),
    "C5": Workload("C5", 10_000_000, 64, 2560, 1440, 14.0, 50.0, _ISO(-4.5, 0.8),
                   views=64, elevation_deg=15.0, azimuth_deg=0.0,
                   notes="10M Gaussians, 64 views on a circle, 1440p"),
}


def quat_scale_to_cov3d(scale: np.ndarray, quat: np.ndarray) -> np.ndarray:
    """Upper-triangular 3D covariance from per-axis scales and unit quaternions.

    Restates ``computeCov3D`` (csrc/pybind.cpp:22-56) in fp32, one rounding per
    operation (the reference runs this on the host without FMA contraction):
    the nine scalars handed to GLM's mat3 constructor are its *columns*, so
    ``R[c][r]`` below is GLM's indexing; ``M = S * R`` scales row r of every
    column by ``s[r]``; ``Sigma = transpose(M) * M``.
    """
    f = np.float32
    s = scale.astype(f)
    r, x, y, z = (quat[:, i].astype(f) for i in range(4))
    one, two = f(1.0), f(2.0)
    # GLM columns R[c] = (R[c][0], R[c][1], R[c][2])
    R = [
        [one - two * (y * y + z * z), two * (x * y - r * z), two * (x * z + r * y)],
        [two * (x * y + r * z), one - two * (x * x + z * z), two * (y * z - r * x)],
        [two * (x * z - r * y), two * (y * z + r * x), one - two * (x * x + y * y)],
    ]
    # M = S * R with S diagonal: M[c][r] = s[r] * R[c][r]. GLM's mat3*mat3 adds the
    # two zero products too; adding +-0 does not change a finite value.
    M = [[s[:, rr] * R[c][rr] for rr in range(3)] for c in range(3)]
    # Sigma = transpose(M) * M: Sigma[c][r] = sum_k Mt[k][r] * M[c][k], Mt[k][r] = M[r][k]
    def sig(c, rr):
        return (M[rr][0] * M[c][0] + M[rr][1] * M[c][1]) + M[rr][2] * M[c][2]

    cov = np.stack([sig(0, 0), sig(0, 1), sig(0, 2), sig(1, 1), sig(1, 2), sig(2, 2)], axis=1)
    return np.ascontiguousarray(cov.astype(f))


def make_scene(num_gaussians: int, clusters: int, log_scale, seed: int = 0,
               opacity_logit_sigma: float = 2.0) -> Scene:
    """Mixture-of-clusters scene with the stated distributions (fp32 SoA)."""
    rng = np.random.default_rng(seed)
    P = int(num_gaussians)
    f = np.float32
    centres = rng.uniform(-8.0, 8.0, size=(clusters, 3)).astype(f)
    n_bg = P // 10
    n_cl = P - n_bg
    which = rng.integers(0, clusters, size=n_cl)
    pos = np.empty((P, 3), dtype=f)
    pos[:n_cl] = centres[which] + rng.standard_normal(size=(n_cl, 3), dtype=f)
    pos[n_cl:] = rng.uniform(-10.0, 10.0, size=(n_bg, 3)).astype(f)
    perm = rng.permutation(P)  # background interleaved with clusters
    pos = np.ascontiguousarray(pos[perm])

    logs = np.empty((P, 3), dtype=f)
    for a, (mu, sd) in enumerate(log_scale):
        logs[:, a] = f(mu) + f(sd) * rng.standard_normal(size=P, dtype=f)
    scale = np.exp(logs).astype(f)

    q = rng.standard_normal(size=(P, 4), dtype=f)
    q /= np.sqrt((q * q).sum(axis=1, keepdims=True)).astype(f)

    logit = f(opacity_logit_sigma) * rng.standard_normal(size=P, dtype=f)
    opacity = (f(1.0) / (f(1.0) + np.exp(-logit))).astype(f)

    shs = np.empty((P, 16, 3), dtype=f)
    shs[:, 0, :] = f(0.5) * rng.standard_normal(size=(P, 3), dtype=f)
    shs[:, 1:, :] = f(0.05) * rng.standard_normal(size=(P, 15, 3), dtype=f)

    cov3d = quat_scale_to_cov3d(scale, q)
    return Scene(position=pos, shs=np.ascontiguousarray(shs.reshape(P, 48)),
                 opacity=np.ascontiguousarray(opacity), cov3d=cov3d)


def look_at_camera(width: int, height: int, radius: float, hfov_deg: float,
                   azimuth_deg: float, elevation_deg: float, cam_id: int = 0) -> Camera:
    """Camera on a sphere of ``radius`` looking at the origin, +y of the world pointing down."""
    az, el = math.radians(azimuth_deg), math.radians(elevation_deg)
    pos = np.array([radius * math.cos(el) * math.sin(az),
                    -radius * math.sin(el),
                    -radius * math.cos(el) * math.cos(az)], dtype=np.float64)
    fwd = -pos / np.linalg.norm(pos)
    world_down = np.array([0.0, 1.0, 0.0])
    right = np.cross(world_down, fwd)
    right /= np.linalg.norm(right)
    down = np.cross(fwd, right)
    rot = np.stack([right, down, fwd], axis=1)  # columns = camera axes in world space
    fx = width / (2.0 * math.tan(math.radians(hfov_deg) / 2.0))
    return Camera(width=width, height=height,
                  position=pos.astype(np.float32),
                  rotation=np.ascontiguousarray(rot.astype(np.float32)),
                  focal_x=float(np.float32(fx)), focal_y=float(np.float32(fx)),
                  id=cam_id, img_name="view%03d" % cam_id)


def make_cameras(w: Workload) -> list:
    if w.views == 1:
        return [look_at_camera(w.width, w.height, w.radius, w.hfov_deg, w.azimuth_deg, w.elevation_deg)]
    return [look_at_camera(w.width, w.height, w.radius, w.hfov_deg,
                           w.azimuth_deg + 360.0 * i / w.views, w.elevation_deg, cam_id=i)
            for i in range(w.views)]


def make_workload(name: str, num_gaussians: int | None = None):
    """Return ``(workload, scene, cameras)``; ``num_gaussians`` overrides the size (tests use small copies)."""
    w = WORKLOADS[name]
    n = w.num_gaussians if num_gaussians is None else int(num_gaussians)
    scene = make_scene(n, w.clusters, w.log_scale, seed=w.seed)
    return w, scene, make_cameras(w)


def tile_grid(width: int, height: int, block_x: int = 16, block_y: int = 16):
    """Tile grid of the reference launchers (preprocess.cu:461, render.cu:556)."""
    return (width + block_x - 1) // block_x, (height + block_y - 1) // block_y


def sort_end_bit(width: int, height: int, block_x: int = 16, block_y: int = 16) -> int:
    """Number of low key bits the sort orders on: 32 + bit_length(#tiles) (sort.cu:9-24,39)."""
    gx, gy = tile_grid(width, height, block_x, block_y)
    return 32 + int(gx * gy).bit_length()
