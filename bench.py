#!/usr/bin/env python
"""Benchmark of the forward raster path: 4K frames per second at 6 M Gaussians.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C4] [--impl ours|reference|port]

A step is one frame of the workload: preprocess -> pair-count readback -> sort -> tile ranges ->
blend, through the reference's operator API (the call sequence of example.py:67-94). With N > 1
(launched by torchrun, one rank per GPU) the frame is split into N strips of tile rows, every rank
holding the whole scene; there is no collective inside the frame, device-timed or end to end.

One JSON line is printed by rank 0:
  value     frames/s with the scene resident in HBM, timed with CUDA events over the K steps
            (max over ranks);
  e2e       frames/s through the public operator API including, every step, the camera handed
            over from pinned host memory and the finished 8-bit image copied to pinned host
            memory (N > 1: every rank copies its own strip into one host image that all ranks
            share, over its own PCIe link); both arms use the same harness: two output buffers and a
            copy stream, so that the copy of frame k overlaps frame k+1, with the figure of the
            serial form (copy, wait, next frame) beside it;
  roofline  the frame's longest kernel against the roofline that bounds it (blend: FP32 pipe;
            everything else: HBM); `roofline_hbm` the longest HBM-bound kernel; `kernels` every
            kernel of the frame with its fraction of the measured copy bandwidth and of 8 TB/s;
            `roofline_frame` the sum of the stages' minimum times over the measured step;
  positional_frame  the same frame with preprocess and sort_gaussian given the reference's positional arguments only
            (`config.preprocess_call` names the extension keywords the timed frame uses);
  cpu_baseline  the OpenMP restatement of the same pipeline on the host cores (N = 1 only);
  view_batch    the 64-view workload (C5) dealt out to the GPUs, views/s and per-view latency.

--impl reference times the reference's own CUDA build (compiled unmodified from its sources into
oracle/_ref) through the same loop -- that process never loads this repository's library;
--impl port times the OpenMP restatement alone. The synthetic scene stands in for the
pre-trained scenes the reference's README points to.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
SPEC_HBM_GBS = 8000.0
SM_COUNT, FP32_LANES_PER_SM, MUFU_LANES_PER_SM = 148, 128, 16
# DRAM bytes per unit measured by ncu (dram__bytes_read.sum + dram__bytes_write.sum of one launch) on a
# 1.5 M-Gaussian case of the same distribution (profiles/*_C4dist_1p5M_4K.txt); traffic grows in proportion
# to the unit, so the full-size figure is this times the launch's units. None: no capture of that kernel.
NCU_DRAM_BYTES_PER_UNIT = {
    "preprocess_kernel": (290.5e6 / 1.5e6, "P"),      # per Gaussian of the scene (kernel on the index list)
    "strip_cull_kernel": (24.0e6 / 1.5e6, "P"),       # the prepared 16-byte records
    "blend_kernel": (115.0e6 / 7.161e6, "S"),         # per blended pair
    "local_sort_kernel": (132.3e6 / 7.349e6, "R"),    # per pair
    "multisplit_kernel": (127.9e6 / 7.349e6, "R"),    # per pair and pass; the small case's output partly stays in L2 (a lower bound)
    "tile_hist_kernel": (59.0e6 / 7.349e6, "R"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                       "-lms", "20", "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def mark(self):
        """Start of the timed region: samples written from here on are the ones that count."""
        try:
            self.mark_at = os.path.getsize(self.f.name)
        except OSError:
            self.mark_at = 0

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.p is None:
            return out
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        text = open(self.f.name).read()
        os.unlink(self.f.name)
        parse = lambda t: [r.strip().split(", ") for r in t.strip().splitlines() if r.strip()]  # noqa: E731
        rows = parse(text[getattr(self, "mark_at", 0):])
        if len([r for r in rows if len(r) >= 8]) < 2:
            # a timed region shorter than two sampling periods: take the warm-up's samples (same load) as well
            rows = parse(text)
            out["window"] = "warm-up and timed region"
        sm, reasons = [], set()
        for r in rows:
            if len(r) < 8:
                continue
            try:
                sm.append(float(r[1]))
                out["sm_max_mhz"] = float(r[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        if sm:
            out["sm_mhz"] = float(np.median(sm))
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def run_port(args, scene, cam, bg=(0.0, 0.0, 0.0)):
    """The OpenMP restatement on the host cores, on a bounded sample: a band of tile rows of the frame."""
    from oracle import oracle
    gx, gy = tile_grid(cam)
    band = max(1, int(round(gy * args.cpu_sample)))
    rows = ((gy - band) // 2, (gy - band) // 2 + band)
    t0 = time.perf_counter()
    out = oracle.render_frame(scene, cam, bg=bg, rows=rows, floats=False)
    dt = time.perf_counter() - t0
    frac = band / gy
    return dict(value=frac / dt, unit="frames/s", cores=oracle.max_threads(), kind="port",
                sample="tile rows %d-%d of %d (%.0f%% of one frame, %d of its pairs) in %.2f s, scaled by rows"
                       % (rows[0], rows[1], gy, 100 * frac, int(out["counters"][3]), dt))


def tile_grid(cam, block=16):
    return (cam.width + block - 1) // block, (cam.height + block - 1) // block


def view_batch(args, ops, scene, cams, rank, local_rank, world, dist):
    """Independent views of one scene dealt out to the GPUs (scene replicated, no traffic between GPUs): one pass over
    all views; views per second over all GPUs and the time of one view on its GPU. Returns the record on every rank
    (complete on rank 0)."""
    import torch
    from flashgs_b200 import parallel
    from flashgs_b200.rasterizer import DeviceScene, Rasterizer, TorchCamera
    dev = torch.device("cuda", local_rank)
    ds = DeviceScene(scene, dev)
    mine = [TorchCamera(cams[i]) for i in parallel.views_of_rank(len(cams), world, rank)]
    ras = Rasterizer(ds, 1 << 26 if scene.num_vertex > 2_000_000 else 1 << 24, 1 << 20, ops=ops)
    bg = torch.zeros(3, dtype=torch.float32)
    img = torch.zeros((cams[0].height, cams[0].width, 3), device=dev, dtype=torch.int8)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    passes = max(1, args.view_passes)
    for tc in mine[: max(1, min(len(mine), 3))]:
        ras.forward(ds, tc, bg, out_color=img)
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in mine] for _ in range(passes)]
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for k in range(passes):
        for i, tc in enumerate(mine):
            ev[k][i][0].record()
            ras.forward(ds, tc, bg, out_color=img)
            ev[k][i][1].record()
    b.record()
    barrier()
    total_ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t[0])
    lat = np.array([e[0].elapsed_time(e[1]) for row in ev for e in row])
    status = ops.device_status() if hasattr(ops, "device_status") else 0
    del ras, ds
    torch.cuda.empty_cache()
    return {"workload": "C5: %d views of %d Gaussians at %dx%d, %d views per GPU, scene replicated, no traffic between GPUs"
                        % (len(cams), scene.num_vertex, cams[0].width, cams[0].height, len(mine)),
            "value": passes * len(cams) / (total_ms * 1e-3), "unit": "views/s", "n_gpus": world, "passes": passes,
            "ms_per_pass": total_ms / passes,
            "view_latency_ms": {"median": float(np.median(lat)), "max": float(lat.max()), "rank": 0},
            "device_status": status}


def main():
    # Libraries (NCCL's version banner, for one) write to stdout; the contract is ONE JSON line there. Everything
    # but that line is sent to stderr: fd 1 is pointed at stderr and the line goes to a saved copy of the real stdout.
    sys.stdout.flush()
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    emit = lambda obj: (real_stdout.write(json.dumps(obj) + "\n"), real_stdout.flush())  # noqa: E731
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="C4")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "port"])
    ap.add_argument("--gaussians", type=int, default=None, help="override the workload's Gaussian count (profiling aid)")
    ap.add_argument("--cpu-sample", type=float, default=1.0, help="fraction of the frame's tile rows the CPU baseline renders")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-view-batch", action="store_true", help="skip the 64-view workload (C5) that the default run adds")
    ap.add_argument("--view-batch", action="store_true",
                    help="only the view batch: all views of the workload (C5: 64), dealt out to the ranks")
    ap.add_argument("--view-passes", type=int, default=2)
    ap.add_argument("--view-gaussians", type=int, default=None, help="override the view batch's Gaussian count")
    ap.add_argument("--no-chained-launches", action="store_true",
                    help="plain kernel launches instead of programmatic dependent launches")
    ap.add_argument("--no-tile-order", action="store_true",
                    help="the blend takes the tiles up in row-major order instead of heaviest first")
    ap.add_argument("--no-tile-counts", action="store_true",
                    help="the sort counts the pairs per tile itself (one more pass over the keys) instead of taking preprocess's table")
    ap.add_argument("--no-scene-bounds", action="store_true",
                    help="the index list of the Gaussians that reach the image is found from the scene arrays (40 bytes per "
                         "Gaussian) instead of from records prepared once per scene (16 bytes)")
    ap.add_argument("--no-cull-scratch", action="store_true",
                    help="call preprocess with the reference's positional arguments only (no scratch for its index list)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, local_rank, world = dist_env()

    from flashgs_b200 import scenes
    if args.view_batch and args.workload == "C4":
        args.workload = "C5"
    wl, scene, cams = scenes.make_workload(args.workload, args.gaussians)
    cam = cams[0]
    config = {"workload": "%s: %s" % (wl.name, wl.notes), "gaussians": scene.num_vertex,
              "image": "%dx%d" % (cam.width, cam.height), "tile": "16x16",
              "camera": "radius %.0f, %.0f deg horizontal FoV%s" % (
                  wl.radius, wl.hfov_deg,
                  " (the workload states no camera; the 1080p workload's is used)" if wl.name in ("C3", "C4") else
                  (" (the workload states no field of view; 50 deg is used)" if wl.name == "C5" else "")),
              "partition": "whole frame" if world == 1 else "%d strips of tile rows, scene replicated" % world,
              "l2": ("inputs (%.2f GB scene) larger than L2" if scene.num_vertex * 232 > 126e6 else
                     "inputs (%.2f GB scene) fit in L2 and L2 is not flushed: not the headline workload") % (scene.num_vertex * 232 / 1e9)}

    if args.impl == "port":
        if rank == 0:
            b = run_port(args, scene, cam)
            emit(({"impl": "port", "metric": "4K frames/sec at 6M Gaussians", "value": b["value"], "unit": "frames/s",
                   "n_gpus": 0, "steps": 1, "warmup": 0, "ms_per_step": 1000.0 / b["value"],
                   "higher_is_better": True, "dtype": "f32", "data": "synthetic", "config": config,
                   "cpu_baseline": b}))
        return

    if args.impl == "reference" and rank != 0:
        return    # the reference is single-GPU: rank 0 alone runs it

    import torch
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    use_dist = world > 1 and args.impl == "ours"
    dist = None
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    # None of these imports loads this repository's shared library: the rasterizer takes the operator module as a
    # parameter, and the reference arm hands it the reference's.
    from flashgs_b200.rasterizer import DeviceScene, Rasterizer, TorchCamera
    from flashgs_b200 import parallel

    ours = args.impl == "ours"
    if ours:
        from flashgs_b200 import ops
    else:
        from oracle import ref
        mod = ref.load()
        if mod is None:
            emit({"impl": "reference", "unavailable": "oracle/_ref (the reference's CUDA build) is not present"})
            return
        ops = mod.ops

    if args.view_batch:
        vb = view_batch(args, ops, scene, cams, rank, local_rank, world, dist)
        if rank == 0:
            emit({"metric": "views/sec, %d views of %d Gaussians at %dx%d" % (len(cams), scene.num_vertex, cam.width, cam.height),
                  "value": vb["value"], "unit": "views/s", "n_gpus": world, "steps": vb["passes"], "warmup": 1,
                  "ms_per_step": vb["ms_per_pass"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                  "dtype": "f32", "data": "synthetic", "config": dict(config, partition=vb["workload"]),
                  "view_latency_ms": vb["view_latency_ms"], "gpu_launches": 13 * vb["passes"] * len(cams) // world,
                  "impl": args.impl})
        if use_dist:
            dist.destroy_process_group()
        return

    ds = DeviceScene(scene, dev)
    tc = TorchCamera(cam)
    bg = torch.zeros(3, dtype=torch.float32)
    gx, gy = tile_grid(cam)
    cap = 1 << 26 if scene.num_vertex > 2_000_000 else 1 << 24
    ras = Rasterizer(ds, cap, 1 << 20, ops=ops)
    if args.no_cull_scratch:
        ras.cull_scratch = ras.scene_bounds = None
    if args.no_scene_bounds:
        ras.scene_bounds = None
    if args.no_tile_counts or not ours:
        ras.tile_counts = None
    use_scratch = ours and ras.cull_scratch is not None
    use_bounds = use_scratch and ras.scene_bounds is not None
    use_counts = ours and ras.tile_counts is not None
    if args.no_tile_order or not ours:
        ras.order_refresh = 0
    use_order = ours and ras.order_refresh > 0
    if ours:
        from flashgs_b200 import _lib as _fgs_lib
        _fgs_lib.load().fgs_debug_chained_launches(0 if args.no_chained_launches else 1)
        config["launches"] = ("plain" if args.no_chained_launches else
                              "programmatic dependent launch: a kernel's blocks are resident and waiting when the kernel before it ends")
    config["preprocess_call"] = ("the reference's positional arguments plus cull_scratch= (the idle head of the sort's "
                                 "scratch, for the index list of the Gaussians that reach the image)"
                                 + (" and scene_bounds= (16-byte records prepared once per scene, outside the timed region, "
                                    "from which that list is found)" if use_bounds else "")
                                 + (" and tile_counts= (preprocess counts the pairs per tile as it emits them; sort_gaussian is "
                                    "given the table and does not count them again)" if use_counts else "")
                                 + "; stages.preprocess.preprocess_plain_call_ms is the call without them") if use_scratch else \
        "the reference's positional arguments only"
    if use_order:
        config["render_call"] = ("the reference's positional arguments plus consumed= and tile_order=: the blend records what it "
                                 "consumed per tile, and every %d frames that record becomes the order in which the tiles are taken "
                                 "up, heaviest first (the refresh, a sort of the tile counts, is inside the timed region)" % ras.order_refresh)
    H, W = cam.height, cam.width
    PAD = 32   # spare rows: the reference writes past ragged images
    out_img = torch.zeros((H + PAD, W, 3), device=dev, dtype=torch.int8)
    P = scene.num_vertex

    def stage_pre(rows=None, scratch=True):
        ras.curr_offset.fill_(0)
        extra = {} if rows is None else dict(tile_row_begin=rows[0], tile_row_end=rows[1])
        if not scratch:   # the reference's positional call (plus the strip's rows)
            return ops.preprocess(ds.position, ds.shs, ds.opacity, ds.cov3d, W, H, 16, 16, tc.position, tc.rotation,
                                  tc.focal_x, tc.focal_y, tc.zFar, tc.zNear, ras.points_xy, ras.rgb_depth, ras.conic_opacity,
                                  ras.gaussian_keys_unsorted, ras.gaussian_values_unsorted, ras.curr_offset, **extra)
        if use_scratch and scratch:
            extra["cull_scratch"] = ras.cull_scratch   # the head of the sort's scratch, idle at this point
            if use_bounds:
                extra["scene_bounds"] = ras.scene_bounds
        if use_counts:
            extra["tile_counts"] = ras.tile_counts
        ops.preprocess(ds.position, ds.shs, ds.opacity, ds.cov3d, W, H, 16, 16, tc.position, tc.rotation,
                       tc.focal_x, tc.focal_y, tc.zFar, tc.zNear, ras.points_xy, ras.rgb_depth, ras.conic_opacity,
                       ras.gaussian_keys_unsorted, ras.gaussian_values_unsorted, ras.curr_offset, **extra)

    def stage_sort(n):
        extra = {"tile_counts": ras.tile_counts} if use_counts else {}
        ops.sort_gaussian(n, W, H, 16, 16, ras.list_sorting_space, ras.gaussian_keys_unsorted, ras.gaussian_values_unsorted,
                          ras.gaussian_keys_sorted, ras.gaussian_values_sorted, **extra)

    def stage_render(n, rows=None, img=None, plain=False):
        img = out_img if img is None else img
        extra = ras._tile_order_arguments(tc, rows) if use_order and not plain else {}
        if rows is None:
            ops.render_16x16(n, W, H, ras.points_xy, ras.rgb_depth, ras.conic_opacity, ras.gaussian_keys_sorted,
                             ras.gaussian_values_sorted, ras.ranges, bg, img, **extra)
        else:
            ops.render_ex(16, 16, n, W, H, ras.points_xy, ras.rgb_depth, ras.conic_opacity, ras.gaussian_keys_sorted,
                          ras.gaussian_values_sorted, ras.ranges, bg, out_color=img, tile_row_begin=rows[0], tile_row_end=rows[1], **extra)

    # the pair count comes back through pinned memory (what `.cpu()` does in example.py:79, without its allocation)
    count_host = torch.zeros(1, dtype=torch.int32).pin_memory()

    def read_count():
        count_host.copy_(ras.curr_offset, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return int(count_host[0])

    def frame(rows, img=None):
        stage_pre(rows)
        n = read_count()
        stage_sort(n)
        stage_render(n, rows, img)
        return n

    def barrier():
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if not use_dist:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    def all_ranks(values):
        """[world, len(values)] array of every rank's values."""
        if not use_dist:
            return np.array([values], dtype=np.float64)
        t = torch.tensor(values, device=dev, dtype=torch.float64)
        out = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(out, t)
        return np.array([o.cpu().numpy() for o in out])

    # ---- calibration frame: pair counts per tile, the reference's guard, consumed pairs per tile row ----
    stage_pre()
    R_full = read_count()
    if R_full >= cap:
        raise RuntimeError("pair buffer too small: %d pairs" % R_full)
    stage_sort(R_full)
    torch.cuda.synchronize()
    tile_counts = torch.bincount(ras.gaussian_keys_sorted[:R_full] >> 32, minlength=gx * gy)
    if not ours and int(((tile_counts > 0) & (tile_counts < 3)).sum()) > 0:
        emit({"impl": "reference", "unavailable": "frame has tiles with one or two splats, for which the "
              "reference's blend kernel reads an uninitialised register (render.cu:268-306); not run"})
        return
    row_pairs = tile_counts.view(gy, gx).sum(dim=1).double().cpu().numpy()
    all_rows, rows, balance = [(0, gy)], None, None
    if use_dist:
        # Strips are balanced on what a rank's frame costs: preprocess and sort follow the pairs R of its rows, the
        # blend follows the pairs it actually consumes, S (early termination), which is distributed differently.
        consumed_all = torch.zeros(gx * gy, device=dev, dtype=torch.int32)
        ops.render_ex(16, 16, R_full, W, H, ras.points_xy, ras.rgb_depth, ras.conic_opacity, ras.gaussian_keys_sorted,
                      ras.gaussian_values_sorted, ras.ranges, bg, out_color=out_img, consumed=consumed_all)
        row_consumed = consumed_all.view(gy, gx).sum(dim=1).double().cpu().numpy()
        t3 = []
        for _ in range(3):
            e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            e[0].record(); stage_pre(); e[1].record(); n = read_count(); stage_sort(n); e[2].record(); stage_render(n); e[3].record()
            torch.cuda.synchronize()
            t3.append([e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2]), e[2].elapsed_time(e[3])])
        t_pre, t_sort, t_blend = np.median(np.array(t3), axis=0)
        w_pairs = (t_pre + t_sort) / max(R_full, 1)
        w_consumed = t_blend / max(float(row_consumed.sum()), 1.0)
        cost = w_pairs * row_pairs + w_consumed * row_consumed
        cost = all_ranks(cost.tolist()).mean(axis=0)     # every rank must cut the same strips
        all_rows = parallel.balanced_strip_rows(cost.tolist(), world)
        rows = all_rows[rank]
        # two rounds of feedback: rows of a rank that ran long are made dearer
        for _ in range(2):
            for _ in range(3):
                frame(rows)
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(5):
                frame(rows)
            b.record()
            torch.cuda.synchronize()
            t_rank = all_ranks([a.elapsed_time(b) / 5])[:, 0]
            for r, (y0, y1) in enumerate(all_rows):
                cost[y0:y1] *= (t_rank[r] / t_rank.mean()) ** 0.7
            all_rows = parallel.balanced_strip_rows(cost.tolist(), world)
            rows = all_rows[rank]
        balance = {"strip_rows": [list(r) for r in all_rows], "on": "pairs per tile row (preprocess, sort) and consumed pairs "
                   "per tile row (blend), weighted by the whole frame's stage times, then two rounds of feedback from the ranks' frame times"}

    # counters of the byte model (all from the device); the view row is built here in numpy, from the camera
    fwd = torch.from_numpy(np.ascontiguousarray(cam.rotation[:, 2].astype(np.float32))).to(dev)
    z_view = (ds.position - torch.from_numpy(cam.position.astype(np.float32)).to(dev)) @ fwd
    P1 = int((z_view > 0.2).sum())
    P2 = int(((z_view > 0.2) & (255.0 * ds.opacity >= 1.0)).sum())
    del z_view

    R = frame(rows)
    torch.cuda.synchronize()
    V = int(torch.unique(ras.gaussian_values_unsorted[:R]).numel())
    Tn = gx * gy if rows is None else (rows[1] - rows[0]) * gx
    S = None
    if ours:
        consumed = torch.zeros(gx * gy, device=dev, dtype=torch.int32)
        r = rows or (0, -1)
        ops.render_ex(16, 16, R, W, H, ras.points_xy, ras.rgb_depth, ras.conic_opacity, ras.gaussian_keys_sorted,
                      ras.gaussian_values_sorted, ras.ranges, bg, out_color=out_img, consumed=consumed,
                      tile_row_begin=r[0], tile_row_end=r[1])
        S = int(consumed.sum())
    y_span = (0, H) if rows is None else parallel.strip_pixel_rows(rows, 16, H)
    pix = W * (y_span[1] - y_span[0])

    # ---- device-resident throughput ----
    sampler = ClockSampler(local_rank)
    # No collector pauses inside timed regions (both arms): a frame is under two milliseconds, and the host reads the
    # pair count back once per frame, so a pause of the interpreter is a pause of the GPU.
    import gc
    gc.collect()
    gc.disable()
    sampler.start()   # before the warm-up: the tool needs a moment before its first sample
    t_warm = time.perf_counter()
    for _ in range(args.warmup):
        frame(rows)
    while time.perf_counter() - t_warm < 0.3:   # keep the GPU under the same load until the sampler is running
        frame(rows)
    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(K)]
    barrier()
    sampler.mark()
    e_begin, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_begin.record()
    for k in range(K):
        e = ev[k]
        e[0].record(); stage_pre(rows); e[1].record()
        n = read_count()
        e[2].record(); stage_sort(n); e[3].record(); stage_render(n, rows); e[4].record()
    e_end.record()
    barrier()
    clocks = sampler.stop()
    local_ms = e_begin.elapsed_time(e_end)
    total_ms = max_over_ranks(local_ms)
    st_ms = np.array([[e[0].elapsed_time(e[1]), e[2].elapsed_time(e[3]), e[3].elapsed_time(e[4])] for e in ev])
    pre_ms, sort_ms, render_ms = [float(x) for x in np.median(st_ms, axis=0)]
    ms_per_step = total_ms / K
    value = 1000.0 / ms_per_step
    # what a rank's step spends outside its kernels: launches, the read-back of the pair count, gaps
    host_ms = max(0.0, local_ms / K - (pre_ms + sort_ms + render_ms))
    per_rank = all_ranks([pre_ms, sort_ms, render_ms, host_ms, local_ms / K, float(R), float(S or 0)])

    # ---- the single-call frame (no host read-back of the pair count), plain launches and as a CUDA graph ----
    fused = None
    if ours:
        def timed(fn):
            for _ in range(args.warmup):
                fn()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(K):
                fn()
            b.record()
            barrier()
            return max_over_ranks(a.elapsed_time(b)) / K
        fused_ms = timed(lambda: ras.forward_fused(ds, tc, bg, out_color=out_img, rows=rows))
        fused = {"ms_per_step": fused_ms, "value": 1000.0 / fused_ms, "unit": "frames/s",
                 "note": "fgs_render_frame: whole frame in one C-ABI call, pair count stays on the device"}
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                ras.forward_fused(ds, tc, bg, out_color=out_img, rows=rows)
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            refresh, ras.order_refresh = ras.order_refresh, (1 << 30 if use_order else 0)   # the captured frame keeps the
            try:                                                                           # tile order it has, no refresh inside
                with torch.cuda.graph(graph):
                    ras.forward_fused(ds, tc, bg, out_color=out_img, rows=rows)
            finally:
                ras.order_refresh = refresh
            graph_ms = timed(graph.replay)
            fused["graph_ms_per_step"] = graph_ms
            fused["graph_value"] = 1000.0 / graph_ms
        except Exception as exc:
            fused["graph_error"] = repr(exc)[:200]

    # ---- the same frame through the reference's positional arguments only (no extension keyword at all) ----
    positional = None
    if ours and (use_scratch or use_counts or use_order):
        def positional_frame():
            stage_pre(rows, scratch=False)
            n = read_count()
            ops.sort_gaussian(n, W, H, 16, 16, ras.list_sorting_space, ras.gaussian_keys_unsorted, ras.gaussian_values_unsorted,
                              ras.gaussian_keys_sorted, ras.gaussian_values_sorted)
            stage_render(n, rows, plain=True)
        pos_ms = timed(positional_frame)
        positional = {"ms_per_step": pos_ms, "value": 1000.0 / pos_ms, "unit": "frames/s",
                      "note": "preprocess, sort_gaussian and render_16x16 called with the reference's positional arguments only"
                              + ("" if rows is None else " (plus the strip's tile rows)")}

    # ---- per-kernel times (CUDA events around every launch, through the library's measurement entry points) ----
    peak, peak_src = measured_peaks()
    f_sm = (clocks.get("sm_mhz") or 1965.0) * 1e6
    stages, kernels, roofline, roofline_hbm, roofline_frame = {}, [], None, None, None
    kind = []
    if ours:
        import ctypes as C
        from flashgs_b200 import _lib
        L = _lib.load()
        stream = torch.cuda.current_stream().cuda_stream
        # preprocess: index-list kernel and main kernel
        ms2 = (C.c_float * 2)()
        pre_k = []
        r0, r1 = rows or (0, -1)
        for _ in range(5):
            ras.curr_offset.fill_(0)
            st = L.fgs_preprocess_profile(P, ds.position.data_ptr(), ds.shs.data_ptr(), ds.opacity.data_ptr(), ds.cov3d.data_ptr(),
                                          W, H, 16, 16, tc.position.data_ptr(), tc.rotation.data_ptr(),
                                          tc.focal_x, tc.focal_y, tc.zFar, tc.zNear, r0, r1,
                                          ras.points_xy.data_ptr(), ras.rgb_depth.data_ptr(), ras.conic_opacity.data_ptr(),
                                          ras.gaussian_keys_unsorted.data_ptr(), ras.gaussian_values_unsorted.data_ptr(), cap,
                                          ras.curr_offset.data_ptr(),
                                          ras.cull_scratch.data_ptr() if use_scratch else None,
                                          ras.cull_scratch.numel() if use_scratch else 0,
                                          ras.scene_bounds.data_ptr() if use_bounds else None,
                                          ras.tile_counts.data_ptr() if use_counts else None, stream, ms2)
            _lib.check("fgs_preprocess_profile", st)
            pre_k.append([ms2[0], ms2[1]])
        cull_ms, main_ms = [float(x) for x in np.median(np.array(pre_k), axis=0)]
        listed = int(ras.cull_scratch[0]) if use_scratch else P
        plain_ms = None
        if use_scratch:
            t = []
            for _ in range(5):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); stage_pre(rows, scratch=False); b.record(); torch.cuda.synchronize()
                t.append(a.elapsed_time(b))
            plain_ms = float(np.median(t))
        # sort: every launch
        CAPN = 32
        ms = (C.c_float * CAPN)()
        kinds = (C.c_int * CAPN)()
        nl = C.c_int(0)
        per = []
        for _ in range(5):
            stage_pre(rows)
            n = read_count()
            st = L.fgs_sort_pairs_profile(n, W, H, 16, 16, ras.list_sorting_space.data_ptr(), ras.list_sorting_space.numel(),
                                          ras.gaussian_keys_unsorted.data_ptr(), ras.gaussian_values_unsorted.data_ptr(),
                                          ras.gaussian_keys_sorted.data_ptr(), ras.gaussian_values_sorted.data_ptr(),
                                          ras.tile_counts.data_ptr() if use_counts else None, stream, ms, kinds, CAPN, C.byref(nl))
            _lib.check("fgs_sort_pairs_profile", st)
            per.append([ms[i] for i in range(nl.value)])
        per = np.median(np.array(per), axis=0) if nl.value else np.zeros(0)
        kind = [kinds[i] for i in range(nl.value)]
        by_kind = lambda k: [float(per[i]) for i in range(len(kind)) if kind[i] == k]  # noqa: E731
        # tile ranges alone; the blend is the render op minus it
        t = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            L.fgs_tile_ranges(R, gx * gy, ras.gaussian_keys_sorted.data_ptr(), ras.ranges.data_ptr(), stream)
            b.record(); torch.cuda.synchronize()
            t.append(a.elapsed_time(b))
        ranges_ms = float(np.median(t))
        blend_ms = max(render_ms - ranges_ms, 1e-6)
        pairs_px = (S or 0) * 256

        def hbm(name, t_ms, launches, bytes_per_launch, note=None):
            gbs = bytes_per_launch / (t_ms * 1e-3) / 1e9 if t_ms > 0 else 0.0
            k = {"kernel": name, "ms": t_ms, "launches": launches, "bound": "hbm", "algorithmic_bytes_per_launch": bytes_per_launch,
                 "gbs": gbs, "frac_of_measured": gbs / peak, "frac_of_8tbs": gbs / SPEC_HBM_GBS}
            if note:
                k["note"] = note
            kernels.append(k)
            return k

        bytes_cull = (16 * P if use_bounds else 12 * P + 4 * P1 + 24 * P2) + 4 * listed
        bytes_main = (4 + 40) * listed + 192 * V + 40 * V + 12 * R if use_scratch else 12 * P + 4 * P1 + 24 * P2 + 232 * V + 12 * R
        if use_scratch:
            hbm("strip_cull_kernel", cull_ms, 1, bytes_cull)
        hbm("preprocess_kernel", main_ms, 1, bytes_main)
        names = {0: "tile_hist_kernel", 1: "multisplit_kernel", 2: "tile_scan_kernel", 3: "local_sort_kernel + long_list_kernel"}
        hist_ms, pass_ms, seg_ms, tile_sort_ms = sum(by_kind(0)), by_kind(1), sum(by_kind(2)), sum(by_kind(3))
        if by_kind(0):
            hbm(names[0], hist_ms, len(by_kind(0)), 8 * R)
        mean_pass = float(np.mean(pass_ms)) if pass_ms else 0.0
        hbm(names[1], mean_pass, len(pass_ms), 24 * R, "mean of the passes: " + ", ".join("%.3f" % x for x in pass_ms))
        hbm(names[2], seg_ms, len(by_kind(2)), 16 * 32768, "one block; bound by its own latency, not by HBM")
        k_local = hbm(names[3], tile_sort_ms, len(by_kind(3)), 24 * R, "all four launches (three list-length classes and the long lists) as one: "
                      + ", ".join("%.3f" % x for x in by_kind(3)))
        k_local["lumped"] = True
        hbm("tile_ranges_kernel", ranges_ms, 1, 8 * Tn, "binary searches: 2 log2(R) cached reads per tile")
        fp32_peak = SM_COUNT * FP32_LANES_PER_SM * f_sm
        t_min_13 = 13 * pairs_px / fp32_peak * 1e3
        t_min_own = max(10 * pairs_px / fp32_peak, pairs_px / (SM_COUNT * MUFU_LANES_PER_SM * f_sm)) * 1e3
        blend = {"kernel": "blend_kernel", "ms": blend_ms, "launches": 1, "bound": "fp32",
                 "achieved": 13 * pairs_px / (blend_ms * 1e-3) / 1e9, "peak": fp32_peak / 1e9, "unit": "G FP32 lane-instructions/s",
                 "frac": t_min_13 / blend_ms,
                 "formula": "13 FP32 instructions per (pixel, splat) pair x S x 256 pixels / time, against 148 SMs x 128 lanes x the sampled SM clock",
                 "sm_mhz": f_sm / 1e6, "pixel_splat_pairs": pairs_px,
                 "own_floor": {"ms": t_min_own, "frac": t_min_own / blend_ms,
                               "formula": "this kernel's own count: per lane and splat 4 per-column, 2 per-row and 7 per-pixel-pair packed operations, "
                                          "40 for 8 pixels = 10 FP32 lane-instructions per pair, and 1 ex2: max(10 pairs / FP32 lanes, pairs / 16 SFU lanes per SM)"},
                 "algorithmic_bytes_per_launch": 8 * Tn + 44 * (S or 0) + 3 * pix}
        kernels.append(blend)
        longest = max(kernels, key=lambda k: max(by_kind(3) or [0.0]) if k.get("lumped") else k["ms"])   # by single launch
        hbm_longest = max([k for k in kernels if k["bound"] == "hbm"], key=lambda k: k["ms"] * k["launches"])

        def traffic_of(k):
            per_unit = NCU_DRAM_BYTES_PER_UNIT.get(k["kernel"].split(" ")[0])
            if per_unit is None:
                return None, None
            units = {"R": R, "P": P, "S": S or 0}[per_unit[1]]
            return per_unit[0] * units, "ncu capture of a smaller case scaled by %s" % per_unit[1]

        def as_roofline(k):
            tr, src = traffic_of(k)
            if k["bound"] == "hbm":
                return {"kernel": k["kernel"], "bound": "hbm", "achieved": k["gbs"], "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                        "frac": k["frac_of_measured"], "frac_of_8tbs": k["frac_of_8tbs"], "traffic": tr, "traffic_source": src,
                        "algorithmic_bytes_per_launch": k["algorithmic_bytes_per_launch"], "launch_ms": k["ms"], "launches_per_frame": k["launches"]}
            return {"kernel": k["kernel"], "bound": "fp32", "achieved": k["achieved"], "peak": k["peak"], "peak_source": "148 SMs x 128 FP32 lanes x sampled SM clock",
                    "unit": k["unit"], "frac": k["frac"], "own_floor": k["own_floor"], "traffic": tr, "traffic_source": src,
                    "algorithmic_bytes_per_launch": k["algorithmic_bytes_per_launch"], "launch_ms": k["ms"], "launches_per_frame": 1}

        roofline = as_roofline(longest)
        roofline_hbm = as_roofline(hbm_longest)
        bytes_pre = 12 * P + 4 * P1 + 24 * P2 + 192 * V + 40 * V + 12 * R
        t_min = {"preprocess": bytes_pre / (peak * 1e9) * 1e3, "sort": 24 * R / (peak * 1e9) * 1e3,
                 "ranges": (8 * R + 8 * Tn) / (peak * 1e9) * 1e3, "blend": t_min_13}
        roofline_frame = {"t_min_ms": t_min, "sum_ms": sum(t_min.values()), "frac": sum(t_min.values()) / (local_ms / K),
                          "fps_at_roofline": 1000.0 / sum(t_min.values()),
                          "note": "HBM stages at the measured copy bandwidth, blend at 13 FP32 instructions per pair; this rank's step"}
        stages = {"preprocess": {"ms": pre_ms, "launches": 2 if use_scratch else 1, "bytes": bytes_pre,
                                 "gbs": bytes_pre / (pre_ms * 1e-3) / 1e9, "listed_gaussians": listed, "preprocess_plain_call_ms": plain_ms},
                  "sort": {"ms": sort_ms, "launches": len(kind), "bytes_compulsory": 24 * R, "gbs": 24 * R / (sort_ms * 1e-3) / 1e9},
                  "ranges_blend": {"ms": render_ms, "launches": 2, "ranges_ms": ranges_ms, "blend_ms": blend_ms}}
        for s in ("preprocess", "sort"):
            stages[s]["frac_of_measured"] = stages[s]["gbs"] / peak
            stages[s]["frac_of_8tbs"] = stages[s]["gbs"] / SPEC_HBM_GBS

    # ---- end to end through the operator API: camera from pinned host memory, image to pinned host memory ----
    e2e = None
    if not args.no_e2e:
        cam_pinned = torch.cat([tc.position.flatten(), tc.rotation.flatten()]).pin_memory()
        copy_stream = torch.cuda.Stream(device=dev)
        bufs = [out_img, torch.zeros_like(out_img)]
        done = [torch.cuda.Event() for _ in range(2)]
        host = None
        if use_dist:
            host = parallel.HostFrames(2, H, W, dst=0)
            host_imgs = host.images
        else:
            host_imgs = [torch.empty((H, W, 3), dtype=torch.int8).pin_memory() for _ in range(2)]
        y0, y1 = y_span

        def camera_from_host():
            tc.position = cam_pinned[:3].clone()
            tc.rotation = cam_pinned[3:].view(3, 3).clone()

        def e2e_overlapped(k):
            """Frame k into device buffer k % 2; its rows go to host image k % 2 on the copy stream while frame k+1 runs."""
            b = k % 2
            camera_from_host()
            done[b].synchronize()                    # the copy of frame k-2 out of this device buffer is over
            if host is not None:
                host.wait_consumed(k - 2)            # and the consumer has released host image k % 2
            frame(rows, bufs[b])
            ready = torch.cuda.Event()
            ready.record()
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(ready)
                host_imgs[b][y0:y1].copy_(bufs[b][y0:y1], non_blocking=True)
                done[b].record(copy_stream)
            if host is not None and k >= 1:
                done[(k - 1) % 2].synchronize()      # frame k-1: this rank's strip is in host memory
                host.publish(k - 1)
                if rank == 0:
                    host.wait_produced(k - 1)        # ... and so is everybody's: the frame is complete on the host
                    host.consume(k - 1)

        def e2e_flush(k_last):
            done[k_last % 2].synchronize()
            if host is not None:
                host.publish(k_last)
                if rank == 0:
                    host.wait_produced(k_last)
                    host.consume(k_last)

        def e2e_serial(k):
            camera_from_host()
            frame(rows, bufs[0])
            host_imgs[0][y0:y1].copy_(bufs[0][y0:y1], non_blocking=True)     # what image.cpu() does in example.py:98
            torch.cuda.current_stream().synchronize()

        def run(step, flush, first):
            barrier()
            t0 = time.perf_counter()
            for k in range(first, first + K):
                step(k)
            if flush:
                flush(first + K - 1)
            torch.cuda.synchronize()
            wall = (time.perf_counter() - t0) * 1e3
            barrier()
            return max_over_ranks(wall) / K

        for k in range(args.warmup):
            e2e_overlapped(k)
        e2e_flush(args.warmup - 1)
        e2e_ms = run(e2e_overlapped, e2e_flush, args.warmup)
        serial_ms = None
        if not use_dist:
            for k in range(2):
                e2e_serial(k)
            serial_ms = run(e2e_serial, None, 0)
        pinned = bool(host_imgs[0].is_pinned())
        e2e = {"value": 1000.0 / e2e_ms, "unit": "frames/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": 12 * 4 + 188, "d2h_bytes_per_step": pix * 3 + 4,
               "host_image_pinned": pinned,
               "note": "camera (12 floats) read from pinned host memory and handed to the kernel as a parameter block; "
                       "8-bit image copied to pinned host memory every frame; two output buffers and a copy stream in BOTH arms "
                       "(harness code around caller-owned buffers): the copy of frame k overlaps frame k+1"
                       + ("; every rank copies the pixel rows of its own strip into one host image shared by all ranks "
                          "(POSIX shared memory, page-locked in every rank): N PCIe links carry 1/N of the image each; "
                          "d2h_bytes_per_step is this rank's share" if use_dist else "")}
        if serial_ms is not None:
            e2e["serial"] = {"value": 1000.0 / serial_ms, "ms_per_step": serial_ms,
                             "note": "copy, wait, next frame -- what example.py does (image.cpu())"}
        if host is not None:
            # the frame assembled on the host against the same frame's strips gathered with NCCL
            frame(rows, bufs[0])
            full = parallel.gather_strips(bufs[0][:H], all_rows, 16, H, dst=0)
            host_imgs[0][y0:y1].copy_(bufs[0][y0:y1])
            torch.cuda.synchronize()
            dist.barrier()
            if rank == 0:
                same = bool((full.cpu() == host_imgs[0]).all())
                e2e["host_frame_check"] = "identical to the NCCL-gathered strips" if same else "MISMATCH against the NCCL-gathered strips"
            dist.barrier()
            host_imgs = None
            host.close()

    status = ops.device_status() if ours else 0
    # preprocess (+ its index-list kernel when it is given scratch), tile ranges, blend + the sort's kernels
    launches_per_frame = 3 + (1 if use_scratch else 0) + (len(kind) if ours else 0)

    # ---- the 64-view workload, dealt out to the GPUs ----
    vb = None
    if ours and not args.no_view_batch and wl.name == "C4" and args.gaussians is None:
        try:
            del ras, ds
            torch.cuda.empty_cache()
            w5, scene5, cams5 = scenes.make_workload("C5", args.view_gaussians)
            vb = view_batch(args, ops, scene5, cams5, rank, local_rank, world, dist)
        except Exception as exc:
            vb = {"error": repr(exc)[:300]}

    cpu_baseline = None
    if ours and rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            cpu_baseline = run_port(args, scene, cam)
        except Exception as exc:   # the oracle is a checker; the bench line survives without it
            cpu_baseline = {"value": None, "unit": "frames/s", "cores": 0, "kind": "port", "sample": "failed: %r" % (exc,)}

    if rank == 0:
        names5 = ["preprocess", "sort", "ranges_blend", "host", "step"]
        line = {
            "metric": "4K frames/sec at 6M Gaussians", "value": value, "unit": "frames/s", "n_gpus": world if ours else 1,
            "steps": K, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
            "clocks": clocks, "e2e": e2e,
            "gpu_launches": (launches_per_frame * K) if ours else 0,
            "stage_ms": {"preprocess": pre_ms, "sort": sort_ms, "ranges_blend": render_ms, "host": host_ms},
            "counters": {"P": P, "P1": P1, "P2": P2, "V": V, "R": R, "S": S, "tiles": Tn},
            "device_status": status,
        }
        if use_dist:
            mx = per_rank[:, :5].max(axis=0)
            line["per_rank"] = {"stage_ms_max": dict(zip(names5, [float(x) for x in mx])),
                                "stage_ms_min": dict(zip(names5, [float(x) for x in per_rank[:, :5].min(axis=0)])),
                                "step_ms": [float(x) for x in per_rank[:, 4]],
                                "pairs": [int(x) for x in per_rank[:, 5]], "consumed_pairs": [int(x) for x in per_rank[:, 6]],
                                "limiter": names5[int(np.argmax(mx[:4]))],
                                "note": "the stage whose maximum over the ranks is largest; 'host' is a rank's step minus its kernels "
                                        "(launches, the read-back of the pair count)"}
            line["strip_balance"] = balance
        if ours:
            line["fused_frame"] = fused
            line["positional_frame"] = positional
            line["roofline"] = roofline
            line["roofline_hbm"] = roofline_hbm
            line["roofline_frame"] = roofline_frame
            line["kernels"] = kernels
            line["stages"] = stages
            line["cpu_baseline"] = cpu_baseline
            line["view_batch"] = vb
        else:
            line["impl"] = "reference"
            line["gpu_launches"] = 0
            line["cpu_baseline"] = {"value": value, "unit": "frames/s", "cores": 0, "kind": "reference",
                                    "sample": "the reference has no CPU path: this arm is its own CUDA build "
                                              "(compiled unmodified, -O1 as its setup.py asks) on one B200, whole frames"}
        emit(line)
    if use_dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
