"""Single-layer benchmark: int8 (or fp16) SubMConv3d 3x3x3 with the fused
bias + ReLU + requant epilogue, through the kernel-level C ABI.

    python -m lidar_ai_solution_b200.layer_bench --channels 16 32 64 128 \
        --voxels 10000 50000 120000 200000 [--fp16] [--reps 20] [--grid 41 1440 1440]

For every (C, N) it builds the coordinate hash and the SubM map once, then
times the convolution launch with CUDA events, an L2 flush (a 256 MB write)
before each launch, and prints one JSON line per case: microseconds,
algorithmic bytes and useful ops of the launch, achieved GB/s and TOPS, and the
fraction of the measured HBM copy bandwidth (MEASURED_PEAKS.json when present).
The rulebook kernels are timed the same way.  This is the per-layer view the
reference's `infer --profiling` gives for a whole model.

    python -m lidar_ai_solution_b200.layer_bench --voxelizer 100000 200000 300000 [--fp16]

times the voxelizer on raw sweeps of that many points instead.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

from . import ops, scenes

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _peak_gbs():
    try:
        return float(json.load(open(os.path.join(_ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except (OSError, ValueError, KeyError):
        return 6650.0, "fallback"


def _time(fn, reps, flush):
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    total = 0.0
    for i in range(reps):
        if flush is not None:
            flush.fill_(i & 0xFF)
        start.record()
        fn()
        end.record()
        end.synchronize()
        total += start.elapsed_time(end)
    return total / reps * 1000.0  # microseconds


def run_case(c, n, grid, fp16, reps, flush, seed=0):
    rng = np.random.default_rng(seed)
    coords = torch.from_numpy(scenes.make_coords(n, grid, seed)).cuda()
    n_ptr, st = ops.device_count(n), ops.new_status()
    table = ops.hash_build(coords, n_ptr, grid, status=st)
    m = ops.subm_map(coords, n_ptr, grid, table, status=st)
    torch.cuda.synchronize()
    w = (rng.standard_normal((c, 27, c)) * np.sqrt(2.0 / (27 * c))).astype(np.float32)
    bias = (rng.standard_normal(c) * 0.1).astype(np.float32)
    if fp16:
        x = torch.from_numpy(rng.standard_normal((n, c)).astype(np.float16)).cuda()
        wts = ops.ConvWeights(w.astype(np.float16), ops.F16, None, bias)
        es, out_kind = 2, ops.F16
    else:
        x = torch.from_numpy(rng.integers(-127, 128, (n, c)).astype(np.int8)).cuda()
        amax = np.abs(w).reshape(c, -1).max(1)
        wq = np.clip(np.rint(w * (127.0 / amax)[:, None, None]), -127, 127).astype(np.int8)
        wts = ops.ConvWeights(wq, ops.I8, (amax / 127.0 * 0.02).astype(np.float32), bias)
        es, out_kind = 1, ops.I8
    out = torch.empty((n, c), dtype=torch.int8 if out_kind == ops.I8 else torch.float16,
                      device="cuda")

    def conv():
        ops.conv_forward(x, m, n_ptr, wts, act=ops.ACT_RELU, out_kind=out_kind, inv_out_scale=8.0,
                         status=st, out=out)

    conv()
    torch.cuda.synchronize()
    if int(st.cpu()[0]):
        raise RuntimeError("device status %s" % st.cpu().tolist())
    us = _time(conv, reps, flush)
    us_hash = _time(lambda: ops.hash_build(coords, n_ptr, grid), max(1, reps // 4), flush)
    us_map = _time(lambda: ops.subm_map(coords, n_ptr, grid, table), max(1, reps // 4), flush)
    pairs = int((m >= 0).sum().item())
    nbytes = n * c * es * 2 + 27 * c * c * es + c * 8 + 4 * 27 * n
    opsn = 2 * pairs * c * c
    peak, src = _peak_gbs()
    return {"channels": c, "voxels": n, "dtype": "fp16" if fp16 else "int8", "pairs": pairs,
            "conv_us": us, "algorithmic_bytes": nbytes, "useful_ops": opsn,
            "achieved_gbs": nbytes / us / 1e3, "achieved_tops": opsn / us / 1e6,
            "hbm_frac": nbytes / us / 1e3 / peak, "hbm_peak_gbs": peak, "peak_source": src,
            "hash_us": us_hash, "subm_map_us": us_map,
            "map_gbs": (16 * n + 4 * 27 * n) / us_map / 1e3}


def run_voxelizer(n_points, fp16, reps, flush, seed=0):
    """One raw sweep through the voxelizer (CenterPoint ranges: 1440x1440x40 voxels of
    0.075 x 0.075 x 0.2 m, at most 10 points per voxel, 160 000 voxels)."""
    pts = scenes.make_points(n_points, seed)
    if fp16:
        pts = pts.astype(np.float16)
    dev = torch.from_numpy(pts).cuda()
    params = ops.voxel_params(scenes.CENTERPOINT_RANGE, scenes.CENTERPOINT_VOXEL, (1440, 1440, 40),
                              5, 1 if fp16 else 0, 10, 160000, 0)
    st = ops.new_status()
    lib = ops.cabi.lib()
    import ctypes as C
    ws = torch.empty(max(256, lib.spconvb_voxelize_workspace_bytes(C.byref(params), n_points)),
                     dtype=torch.uint8, device="cuda")
    feat = torch.zeros((160000, 5), dtype=torch.float16, device="cuda")
    idx = torch.zeros((160000, 4), dtype=torch.int32, device="cuda")
    n_ptr = torch.zeros(1, dtype=torch.int32, device="cuda")

    def vox():
        ops.cabi.check(lib.spconvb_voxelize(
            C.byref(params), C.c_void_p(dev.data_ptr()), n_points, C.c_void_p(ws.data_ptr()),
            C.c_void_p(feat.data_ptr()), C.c_void_p(idx.data_ptr()), C.c_void_p(n_ptr.data_ptr()),
            C.c_void_p(st.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream)),
            "voxelize")

    vox()
    torch.cuda.synchronize()
    n = int(n_ptr.item())
    us = _time(vox, reps, flush)
    nbytes = n_points * 5 * (2 if fp16 else 4) + n * (5 * 2 + 16)
    peak, src = _peak_gbs()
    return {"kernel": "voxelize", "points": n_points, "points_dtype": "fp16" if fp16 else "fp32",
            "voxels": n, "us": us, "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / us / 1e3,
            "hbm_frac": nbytes / us / 1e3 / peak, "hbm_peak_gbs": peak, "peak_source": src,
            "points_per_s": n_points / us * 1e6}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--channels", type=int, nargs="+", default=[16, 32, 64, 128])
    ap.add_argument("--voxels", type=int, nargs="+", default=[10000, 50000, 120000, 200000])
    ap.add_argument("--grid", type=int, nargs=3, default=list(scenes.CENTERPOINT_GRID_ZYX))
    ap.add_argument("--fp16", action="store_true")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--voxelizer", type=int, nargs="*", default=None, metavar="POINTS",
                    help="time the voxelizer on sweeps of this many points instead")
    args = ap.parse_args()
    flush = None if args.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    if args.voxelizer is not None:
        for n in (args.voxelizer or [100000, 200000, 300000]):
            print(json.dumps(run_voxelizer(n, args.fp16, args.reps, flush)), flush=True)
        return
    for c in args.channels:
        for n in args.voxels:
            print(json.dumps(run_case(c, n, tuple(args.grid), args.fp16, args.reps, flush)),
                  flush=True)


if __name__ == "__main__":
    main()
