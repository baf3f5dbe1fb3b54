"""Render every camera of a trained model directory, like the reference's example script.

    python -m flashgs_b200.render_scene <model_path> [--perf]

Same inputs and outputs as ``render_scene`` of the reference (example.py:105-144): the model directory holds
``point_cloud/iteration_30000/point_cloud.ply`` and ``cameras.json`` (a list of objects with ``id``, ``img_name``,
``width``, ``height``, ``position`` [3], ``rotation`` [3][3] camera-to-world, ``fx``, ``fy``; example.py:30-41);
one binary PPM per camera is written to ``<model_path>/test_out/<img_name>.ppm``. With ``--perf`` each camera is
rendered 10 more times and the mean frame time is printed (example.py:130-141).
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch

from . import ops
from .rasterizer import Rasterizer, save_ppm


class Scene:
    """Device-resident Gaussians loaded from a PLY (example.py:10-27)."""

    def __init__(self, device):
        self.device = device
        self.num_vertex = 0
        self.position = self.shs = self.opacity = self.cov3d = None

    def loadPly(self, scene_path: str) -> None:
        self.num_vertex, pos, shs, opa, cov = ops.loadPly(scene_path)
        print("num_vertex = %d" % self.num_vertex)
        self.position, self.shs = pos.to(self.device), shs.to(self.device)
        self.opacity, self.cov3d = opa.to(self.device), cov.to(self.device)


class Camera:
    """example.py:30-41."""

    def __init__(self, camera_json: dict):
        self.id = camera_json["id"]
        self.img_name = camera_json["img_name"]
        self.width, self.height = camera_json["width"], camera_json["height"]
        self.position = torch.tensor(camera_json["position"], dtype=torch.float32)
        self.rotation = torch.tensor(camera_json["rotation"], dtype=torch.float32)
        self.focal_x, self.focal_y = camera_json["fx"], camera_json["fy"]
        self.zFar, self.zNear = 100.0, 0.01


def render_scene(model_path: str, test_performance: bool = False, device: str = "cuda:0",
                 max_num_rendered: int = 2 ** 27, max_num_tiles: int = 2 ** 20):
    scene_path = os.path.join(model_path, "point_cloud", "iteration_30000", "point_cloud.ply")
    camera_path = os.path.join(model_path, "cameras.json")
    dev = torch.device(device)
    bg_color = torch.zeros(3, dtype=torch.float32)
    scene = Scene(dev)
    scene.loadPly(scene_path)
    with open(camera_path) as f:
        cameras_json = json.load(f)
    image_dir = os.path.join(model_path, "test_out")
    os.makedirs(image_dir, exist_ok=True)
    rasterizer = Rasterizer(scene, max_num_rendered, max_num_tiles)
    times = {}
    for camera_json in cameras_json:
        camera = Camera(camera_json)
        print("image name = %s" % camera.img_name)
        image = rasterizer.forward(scene, camera, bg_color)
        if test_performance:
            n = 10
            torch.cuda.synchronize()
            t0 = time.time()
            for _ in range(n):
                image = rasterizer.forward(scene, camera, bg_color)
            torch.cuda.synchronize()
            t1 = time.time()
            times[camera.img_name] = (t1 - t0) / n * 1000
            print("elapsed time = %f ms" % times[camera.img_name])
            print("fps = %f" % (n / (t1 - t0)))
        save_ppm(image, os.path.join(image_dir, "%s.ppm" % camera.img_name))
    return times


def camera_to_json(cam) -> dict:
    """The cameras.json entry of a ``flashgs_b200.scenes.Camera``."""
    return dict(id=cam.id, img_name=cam.img_name, width=cam.width, height=cam.height,
                position=[float(v) for v in cam.position], rotation=[[float(v) for v in row] for row in cam.rotation],
                fx=cam.focal_x, fy=cam.focal_y)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("model_path")
    ap.add_argument("--perf", action="store_true")
    a = ap.parse_args()
    render_scene(a.model_path, a.perf)
