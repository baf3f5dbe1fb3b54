#!/usr/bin/env python
"""Benchmark of the forward raster path: 4K frames per second at 6 M Gaussians.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C4] [--impl ours|reference|port]

A step is one frame of the workload: preprocess -> pair-count readback -> sort -> tile ranges ->
blend, through the reference's operator API (the call sequence of example.py:67-94). With N > 1
(launched by torchrun, one rank per GPU) the frame is split into N strips of tile rows, every rank
holding the whole scene; there is no collective inside the device-timed frame, and the end-to-end
figure adds one NCCL gather of the strips plus the copy of the image to pinned host memory.

One JSON line is printed by rank 0:
  value     frames/s with the scene resident in HBM, timed with CUDA events over the K steps
            (max over ranks);
  e2e       frames/s through the public operator API including, every step, the camera handed
            over from pinned host memory and the finished 8-bit image copied back to pinned host
            memory (for N > 1 after the strip gather);
  roofline  the dominant kernel's achieved algorithmic bytes/s against the measured HBM copy
            bandwidth of this machine pool; `stages` lists every stage the same way;
  cpu_baseline  the OpenMP restatement of the same pipeline on the host cores (N = 1 only).

--impl reference times the reference's own CUDA build (compiled unmodified from its sources into
oracle/_ref) through the same loop; --impl port times the OpenMP restatement alone. The
synthetic scene stands in for the pre-trained scenes the reference's README points to.
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
# DRAM bytes per unit measured by ncu (dram__bytes_read.sum + dram__bytes_write.sum of one launch) on a
# 1.5 M-Gaussian case of the same distribution (profiles/*_C4dist_1p5M_4K.txt); traffic grows in proportion
# to the unit, so the full-size figure is this times the launch's units.
NCU_DRAM_BYTES_PER_UNIT = {
    "onesweep_kernel": (128.6e6 / 7.349e6, "R"),      # per pair and pass
    "preprocess_kernel": ((287.9e6 + 60.2e6) / 1.5e6, "P"),   # per Gaussian: the kernel on the index list + the cull kernel
    "blend_kernel": (117.3e6 / 7.161e6, "S"),         # per blended pair
    "local_sort_kernel": (133.3e6 / 7.349e6, "R"),    # per pair
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
                                       "-lms", "25", "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
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


def run_view_batch(args, emit, wl, scene, cams, config, rank, local_rank, world):
    """Independent views of one scene dealt out to the GPUs (scene replicated, no traffic between GPUs): a step is one
    pass over all views; value = views per second over all GPUs; latency = time of one view on its GPU."""
    import torch
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from flashgs_b200 import ops
    from flashgs_b200.rasterizer import DeviceScene, Rasterizer, TorchCamera
    ds = DeviceScene(scene, dev)
    from flashgs_b200 import parallel
    mine = [TorchCamera(cams[i]) for i in parallel.views_of_rank(len(cams), world, rank)]
    ras = Rasterizer(ds, 1 << 26 if scene.num_vertex > 2_000_000 else 1 << 24, 1 << 20, ops=ops)
    bg = torch.zeros(3, dtype=torch.float32)
    img = torch.zeros((cams[0].height, cams[0].width, 3), device=dev, dtype=torch.int8)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(1, args.warmup // 3)):
        for tc in mine:
            ras.forward(ds, tc, bg, out_color=img)
    K = max(1, args.steps // 10)
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in mine] for _ in range(K)]
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    sampler.mark()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for k in range(K):
        for i, tc in enumerate(mine):
            ev[k][i][0].record()
            ras.forward(ds, tc, bg, out_color=img)
            ev[k][i][1].record()
    b.record()
    barrier()
    clocks = sampler.stop()
    total_ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t[0])
    lat = np.array([e[0].elapsed_time(e[1]) for row in ev for e in row])
    if rank == 0:
        emit({"metric": "views/sec, %d views of %d Gaussians at %dx%d" % (len(cams), scene.num_vertex, cams[0].width, cams[0].height),
              "value": K * len(cams) / (total_ms * 1e-3), "unit": "views/s", "n_gpus": world, "steps": K, "warmup": max(1, args.warmup // 3),
              "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
              "data": "synthetic", "config": dict(config, partition="%d views per GPU, scene replicated, no traffic between GPUs" % len(mine)),
              "view_latency_ms": {"median": float(np.median(lat)), "max": float(lat.max())}, "clocks": clocks,
              "gpu_launches": 13 * K * len(mine)})
    if world > 1:
        dist.destroy_process_group()


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
    ap.add_argument("--view-batch", action="store_true",
                    help="render all views of the workload (C5: 64), dealt out to the ranks; a step is one pass over them")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, local_rank, world = dist_env()

    from flashgs_b200 import scenes
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

    if args.view_batch:
        return run_view_batch(args, emit, wl, scene, cams, config, rank, local_rank, world)

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
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from flashgs_b200.rasterizer import DeviceScene, Rasterizer, TorchCamera
    from flashgs_b200 import parallel

    if args.impl == "reference":
        from oracle import ref
        mod = ref.load()
        if mod is None:
            emit({"impl": "reference", "unavailable": "oracle/_ref (the reference's CUDA build) is not present"})
            return
        ops = mod.ops
    else:
        from flashgs_b200 import ops

    ds = DeviceScene(scene, dev)
    tc = TorchCamera(cam)
    bg = torch.zeros(3, dtype=torch.float32)
    gx, gy = tile_grid(cam)
    cap = 1 << 26 if scene.num_vertex > 2_000_000 else 1 << 24
    ras = Rasterizer(ds, cap, 1 << 20, ops=ops)
    H, W = cam.height, cam.width
    out_img = torch.zeros((H + 32, W, 3), device=dev, dtype=torch.int8)   # spare rows: the reference writes past ragged images

    # ---- one calibration frame: pair counts per tile row (strip balancing), counters for the byte model ----
    def stage_pre(rows=None):
        ras.curr_offset.fill_(0)
        extra = {} if rows is None else dict(tile_row_begin=rows[0], tile_row_end=rows[1])
        if args.impl == "ours" and ras.cull_scratch is not None:
            extra["cull_scratch"] = ras.cull_scratch   # the head of the sort's scratch, idle at this point
        ops.preprocess(ds.position, ds.shs, ds.opacity, ds.cov3d, W, H, 16, 16, tc.position, tc.rotation,
                       tc.focal_x, tc.focal_y, tc.zFar, tc.zNear, ras.points_xy, ras.rgb_depth, ras.conic_opacity,
                       ras.gaussian_keys_unsorted, ras.gaussian_values_unsorted, ras.curr_offset, **extra)

    def stage_sort(n):
        ops.sort_gaussian(n, W, H, 16, 16, ras.list_sorting_space, ras.gaussian_keys_unsorted, ras.gaussian_values_unsorted,
                          ras.gaussian_keys_sorted, ras.gaussian_values_sorted)

    def stage_render(n, rows=None):
        if rows is None:
            ops.render_16x16(n, W, H, ras.points_xy, ras.rgb_depth, ras.conic_opacity, ras.gaussian_keys_sorted,
                             ras.gaussian_values_sorted, ras.ranges, bg, out_img)
        else:
            ops.render_ex(16, 16, n, W, H, ras.points_xy, ras.rgb_depth, ras.conic_opacity, ras.gaussian_keys_sorted,
                          ras.gaussian_values_sorted, ras.ranges, bg, out_color=out_img, tile_row_begin=rows[0], tile_row_end=rows[1])

    stage_pre()
    R_full = int(ras.curr_offset.cpu()[0])
    if R_full >= cap:
        raise RuntimeError("pair buffer too small: %d pairs" % R_full)
    stage_sort(R_full)
    torch.cuda.synchronize()
    tile_counts = torch.bincount(ras.gaussian_keys_sorted[:R_full] >> 32, minlength=gx * gy)
    if args.impl == "reference" and int(((tile_counts > 0) & (tile_counts < 3)).sum()) > 0:
        emit({"impl": "reference", "unavailable": "frame has tiles with one or two splats, for which the "
              "reference's blend kernel reads an uninitialised register (render.cu:268-306); not run"})
        return
    row_cost = tile_counts.view(gy, gx).sum(dim=1).double().cpu().tolist()
    all_rows = parallel.balanced_strip_rows(row_cost, world) if use_dist else [(0, gy)]
    rows = all_rows[rank] if use_dist else None

    # counters of the byte model (all from the device)
    view = np.zeros(16, np.float32)
    proj = np.zeros(16, np.float32)
    from flashgs_b200 import _lib
    _lib.load().fgs_view_proj_matrices(W, H, tc.position.numpy().ctypes.data, tc.rotation.numpy().ctypes.data,
                                       tc.focal_x, tc.focal_y, tc.zFar, tc.zNear, view.ctypes.data, proj.ctypes.data)
    vm = torch.from_numpy(view.reshape(4, 4).T.copy()).to(dev)
    z_view = ds.position @ vm[2, :3] + vm[2, 3]
    P = scene.num_vertex
    P1 = int((z_view > 0.2).sum())
    P2 = int(((z_view > 0.2) & (255.0 * ds.opacity >= 1.0)).sum())
    del z_view

    def frame(rows):
        stage_pre(rows)
        n = int(ras.curr_offset.cpu()[0])
        stage_sort(n)
        stage_render(n, rows)
        return n

    R = frame(rows)
    torch.cuda.synchronize()
    V = int(torch.unique(ras.gaussian_values_unsorted[:R]).numel())
    Tn = gx * gy if rows is None else (rows[1] - rows[0]) * gx
    S = None
    if args.impl == "ours":
        consumed = torch.zeros(gx * gy, device=dev, dtype=torch.int32)
        r = rows or (0, -1)
        ops.render_ex(16, 16, R, W, H, ras.points_xy, ras.rgb_depth, ras.conic_opacity, ras.gaussian_keys_sorted,
                      ras.gaussian_values_sorted, ras.ranges, bg, out_color=out_img, consumed=consumed,
                      tile_row_begin=r[0], tile_row_end=r[1])
        S = int(consumed.sum())
    pix = W * (H if rows is None else (parallel.strip_pixel_rows(rows, 16, H)[1] - parallel.strip_pixel_rows(rows, 16, H)[0]))
    bytes_pre = 12 * P + 4 * P1 + 24 * P2 + 192 * V + 40 * V + 12 * R
    bytes_sort_pass = 24 * R
    bytes_hist = 8 * R
    bytes_render = 8 * R + 8 * Tn + 8 * Tn + 44 * (S if S is not None else R) + 3 * pix

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

    # ---- device-resident throughput ----
    sampler = ClockSampler(local_rank)
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
        n = int(ras.curr_offset.cpu()[0])
        e[2].record(); stage_sort(n); e[3].record(); stage_render(n, rows); e[4].record()
    e_end.record()
    barrier()
    clocks = sampler.stop()
    total_ms = max_over_ranks(e_begin.elapsed_time(e_end))
    st_ms = np.array([[e[0].elapsed_time(e[1]), e[2].elapsed_time(e[3]), e[3].elapsed_time(e[4])] for e in ev])
    pre_ms, sort_ms, render_ms = [float(x) for x in np.median(st_ms, axis=0)]
    ms_per_step = total_ms / K
    value = 1000.0 / ms_per_step

    # ---- the single-call frame (no host read-back of the pair count), plain launches and as a CUDA graph ----
    fused = None
    if args.impl == "ours":
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
            with torch.cuda.graph(graph):
                ras.forward_fused(ds, tc, bg, out_color=out_img, rows=rows)
            graph_ms = timed(graph.replay)
            fused["graph_ms_per_step"] = graph_ms
            fused["graph_value"] = 1000.0 / graph_ms
        except Exception as exc:
            fused["graph_error"] = repr(exc)[:200]

    # ---- per-launch times of the sort (its passes are separate launches inside one op) ----
    peak, peak_src = measured_peaks()
    stages = {}
    roofline = None
    kind = []
    if args.impl == "ours":
        L = _lib.load()
        import ctypes as C
        CAPN = 32
        ms = (C.c_float * CAPN)()
        kinds = (C.c_int * CAPN)()
        nl = C.c_int(0)
        per = []
        for _ in range(5):
            stage_pre(rows)
            n = int(ras.curr_offset.cpu()[0])
            st = L.fgs_sort_pairs_profile(n, W, H, 16, 16, ras.list_sorting_space.data_ptr(), ras.list_sorting_space.numel(),
                                          ras.gaussian_keys_unsorted.data_ptr(), ras.gaussian_values_unsorted.data_ptr(),
                                          ras.gaussian_keys_sorted.data_ptr(), ras.gaussian_values_sorted.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream, ms, kinds, CAPN, C.byref(nl))
            _lib.check("fgs_sort_pairs_profile", st)
            per.append([ms[i] for i in range(nl.value)])
        per = np.median(np.array(per), axis=0) if nl.value else np.zeros(0)
        kind = [kinds[i] for i in range(nl.value)]
        by_kind = lambda k: [float(per[i]) for i in range(len(kind)) if kind[i] == k]  # noqa: E731
        hist_ms = sum(by_kind(0))
        pass_ms = by_kind(1)
        seg_ms, local_ms = sum(by_kind(2)), sum(by_kind(3))
        gbs = lambda b, t: b / (t * 1e-3) / 1e9 if t > 0 else 0.0  # noqa: E731
        mean_pass = float(np.mean(pass_ms)) if pass_ms else 0.0
        stages = {
            "preprocess": {"ms": pre_ms, "launches": 2 if (args.impl == "ours" and ras.cull_scratch is not None) else 1,
                           "bytes": bytes_pre, "gbs": gbs(bytes_pre, pre_ms)},
            "sort_histogram": {"ms": hist_ms, "launches": 1, "bytes": bytes_hist, "gbs": gbs(bytes_hist, hist_ms)},
            "sort_digit_pass": {"ms": mean_pass, "launches": len(pass_ms), "bytes": bytes_sort_pass, "gbs": gbs(bytes_sort_pass, mean_pass)},
            "sort_tile_segments": {"ms": seg_ms, "launches": len(by_kind(2))},
            "sort_tile_local": {"ms": local_ms, "launches": len(by_kind(3)), "bytes": bytes_sort_pass, "gbs": gbs(bytes_sort_pass, local_ms)},
            "sort_total": {"ms": sort_ms, "bytes_compulsory": 24 * R},
            "ranges_blend": {"ms": render_ms, "launches": 2, "bytes": bytes_render, "gbs": gbs(bytes_render, render_ms),
                             "pixel_splat_pairs": None if S is None else S * 256},
        }
        for s in stages.values():
            if "gbs" in s:
                s["frac"] = s["gbs"] / peak
        # the dominant HBM-bound kernel: the one with the largest total time per frame. blend_kernel takes as long
        # but is bound by the FP32 pipe (FMA pipe 73 % busy under ncu, DRAM 2 %), for which the schema has no roofline;
        # its rate is in stages["ranges_blend"].
        cand = {"preprocess": pre_ms, "sort_digit_pass": mean_pass * len(pass_ms), "sort_tile_local": local_ms}
        dom = max(cand, key=cand.get)
        d = stages[dom]
        roofline = {"kernel": {"preprocess": "preprocess_kernel", "sort_digit_pass": "onesweep_kernel",
                               "sort_tile_local": "local_sort_kernel", "ranges_blend": "blend_kernel"}[dom],
                    "bound": "hbm", "achieved": d["gbs"], "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                    "frac": d["gbs"] / peak, "traffic": None, "traffic_source": None,
                    "algorithmic_bytes_per_launch": d["bytes"], "launch_ms": d["ms"], "launches_per_frame": d["launches"],
                    "note": "blend_kernel (%.3f ms) is FP32-pipe bound, not HBM or tensor: see stages.ranges_blend" % render_ms}

    if roofline is not None:
        per, unit = NCU_DRAM_BYTES_PER_UNIT[roofline["kernel"]]
        roofline["traffic"] = per * {"R": R, "P": P, "S": S or 0}[unit]
        roofline["traffic_source"] = "ncu capture of a smaller case scaled by %s" % unit

    # ---- end to end through the operator API: camera from pinned host memory, image to pinned host memory ----
    e2e = None
    if not args.no_e2e:
        cam_pinned = torch.cat([tc.position.flatten(), tc.rotation.flatten()]).pin_memory()
        host_img = torch.empty((H, W, 3), dtype=torch.int8).pin_memory()
        copy_stream = torch.cuda.Stream(device=dev)
        done = [torch.cuda.Event() for _ in range(2)]
        keep = [None, None]
        bufs = [out_img, torch.zeros_like(out_img)] if args.impl == "ours" else [out_img, out_img]
        # Several GPUs: the blend kernels store their strips straight into rank 0's frame buffer (peer memory over
        # NVLink) when the symmetric-memory mapping can be set up; otherwise the strips are gathered with NCCL.
        peer = None
        if use_dist and os.environ.get("FLASHGS_PEER_FRAMES", "1") != "0":
            try:
                peer = parallel.PeerFrames(2, H, W, dev, dst=0)
            except Exception as exc:
                print("peer frame buffers unavailable (%r): gathering strips with NCCL" % (exc,), file=sys.stderr)
                peer = None
            ok = torch.tensor([1 if peer is not None else 0], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok[0]) == 0:
                peer = None

        def e2e_frame(k):
            # the camera of this step comes from pinned host memory
            tc.position = cam_pinned[:3].clone()
            tc.rotation = cam_pinned[3:].view(3, 3).clone()
            nonlocal out_img
            if args.impl == "ours" and not use_dist:
                # the copy of frame k overlaps the kernels of frame k+1: two output buffers
                done[k % 2].synchronize()
                out_img = bufs[k % 2]
            if peer is not None:
                out_img = peer.frames[k % 2]          # rank 0's buffer, mapped here
            frame(rows)
            if peer is not None:
                # Frame k+1 will be written into the buffer of frame k-1: rank 0 joins the barrier only when that
                # buffer's copy to the host is over, so nobody overwrites it early.
                if rank == 0:
                    torch.cuda.current_stream().wait_event(done[(k - 1) % 2])
                peer.barrier()                        # every strip of frame k has landed in rank 0's buffer
                if rank == 0:
                    ready = torch.cuda.Event()
                    ready.record()
                    with torch.cuda.stream(copy_stream):
                        copy_stream.wait_event(ready)
                        host_img.copy_(peer.frames[k % 2], non_blocking=True)
                        done[k % 2].record(copy_stream)
            elif use_dist:
                # strips -> rank 0 over NCCL, then the copy to the host overlaps the next frame like on one GPU
                done[k % 2].synchronize()
                full = parallel.gather_strips(out_img[:H], all_rows, 16, H, dst=0)
                if rank == 0:
                    keep[k % 2] = full
                    ready = torch.cuda.Event()
                    ready.record()
                    with torch.cuda.stream(copy_stream):
                        copy_stream.wait_event(ready)
                        host_img.copy_(full, non_blocking=True)
                        done[k % 2].record(copy_stream)
            elif args.impl == "ours":
                ready = torch.cuda.Event()
                ready.record()
                with torch.cuda.stream(copy_stream):
                    copy_stream.wait_event(ready)
                    host_img.copy_(out_img[:H], non_blocking=True)
                    done[k % 2].record(copy_stream)
            else:
                host_img.copy_(out_img[:H], non_blocking=True)     # what image.cpu() does in example.py:98
                torch.cuda.current_stream().synchronize()

        for k in range(args.warmup):
            e2e_frame(k)
        barrier()
        t0 = time.perf_counter()
        e_b, e_e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e_b.record()
        for k in range(K):
            e2e_frame(k)
        copy_stream.synchronize()
        e_e.record()
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
        dev_ms = max_over_ranks(max(e_b.elapsed_time(e_e), 0.0))
        e2e_ms = max(max_over_ranks(wall_ms), dev_ms) / K
        e2e = {"value": 1000.0 / e2e_ms, "unit": "frames/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": 12 * 4 + 188, "d2h_bytes_per_step": H * W * 3 + 4,
               "note": "camera (12 floats) read from pinned host memory and handed to the kernel as a parameter block; "
                       "8-bit image copied to pinned host memory every frame"
                       + ("; copy of frame k overlaps frame k+1" if args.impl == "ours" else "")
                       + ("; the blend kernels store their strips straight into rank 0's frame buffer (peer memory over "
                          "NVLink), one device-side barrier per frame" if peer is not None else
                          ("; strips gathered on rank 0 with one NCCL gather per frame" if use_dist else ""))}
        out_img = bufs[0]
        if peer is not None:
            # the image assembled through peer stores against the same frame's strips gathered with NCCL
            frame(rows)
            full = parallel.gather_strips(out_img[:H], all_rows, 16, H, dst=0)
            torch.cuda.synchronize()
            if rank == 0:
                same = bool((full.cpu() == host_img).all())
                e2e["peer_frames_check"] = "identical to the NCCL-gathered strips" if same else "MISMATCH against the NCCL-gathered strips"
                if not same:
                    raise RuntimeError("peer frame buffers: image differs from the gathered strips")

    status = ops.device_status() if args.impl == "ours" else 0
    # preprocess (+ its cull kernel when it is given scratch), tile ranges, blend + the sort's kernels
    launches_per_frame = 3 + (1 if ras.cull_scratch is not None else 0) + (len(kind) if args.impl == "ours" else 0)

    cpu_baseline = None
    if args.impl == "ours" and rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            cpu_baseline = run_port(args, scene, cam)
        except Exception as exc:   # the oracle is a checker; the bench line survives without it
            cpu_baseline = {"value": None, "unit": "frames/s", "cores": 0, "kind": "port", "sample": "failed: %r" % (exc,)}

    if rank == 0:
        line = {
            "metric": "4K frames/sec at 6M Gaussians", "value": value, "unit": "frames/s", "n_gpus": world if args.impl == "ours" else 1,
            "steps": K, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
            "clocks": clocks, "e2e": e2e,
            "gpu_launches": (launches_per_frame * K) if args.impl == "ours" else 0,
            "stage_ms": {"preprocess": pre_ms, "sort": sort_ms, "ranges_blend": render_ms},
            "counters": {"P": P, "P1": P1, "P2": P2, "V": V, "R": R, "S": S, "tiles": Tn},
            "device_status": status,
        }
        if args.impl == "ours":
            line["fused_frame"] = fused
            line["roofline"] = roofline
            line["stages"] = stages
            line["cpu_baseline"] = cpu_baseline
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
