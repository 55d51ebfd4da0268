#!/usr/bin/env python
"""Throughput of the CenterPoint SCN int8 backbone (frames/s) on 1-8 B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W    # CPU restatement, host cores

A step is one pass of the hot path (rulebooks, 21 convolutions with fused
epilogues, dense BEV scatter) over a set of independent synthetic frames:
per GPU, `--frames` frames of ~120 k active voxels in the 41x1440x1440 grid,
every frame from its own seed.  Frames are independent, so ranks share nothing:
no collective runs inside the timed region, scaling is weak (per-GPU work fixed).
`--batch` frames go through one engine call (the index tensor's batch column tells
them apart), so that a layer's tiles of several frames share one kernel launch.

`value`  inputs resident in HBM, one CUDA graph per batch spread over
         `--replicas` engine replicas (streams) per GPU, timed with CUDA events;
`e2e`    the same through the engine C ABI with HOST buffers: every frame's pinned
         features, indices and the row count copied in, the dense fp16 BEV tensors
         copied out, all inside the timed region.
Rank 0 prints one JSON line.  Beside the headline it carries, as extra keys that
each cost a few seconds: the roofline of the convolution kernel (per-launch CUDA
events, cold L2), the CPU baselines, the voxelizer and a run from raw points, the
reference's own sample frame, and the fixed 64-frame mixed-size set sharded over
the ranks.

Other measurements (not the headline):
    python bench.py --workload layer_sweep [--fp16]   # one SubM 3x3x3 layer, C x N sweep
    python bench.py --workload voxelizer              # the voxelizer alone
    python bench.py --workload frame_once [--batch B] # one voxelizer call and one eager engine call
                                                      # inside a cudaProfilerStart/Stop range (for
                                                      # `ncu --profile-from-start off`)
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GRID = (41, 1440, 1440)
VOXELS = 120000
# The synthetic scenes are less clustered than real sweeps: a 120 k-voxel frame has ~235 k
# active voxels after the first stride-2 conv, above the exporters' default bound of 200 000.
OUTPUT_BOUND = 300000
WORKLOAD = "centerpoint_scn_int8 full backbone, 41x1440x1440 grid, ~120k active voxels/frame"


def _env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def host_threads():
    return len(os.sched_getaffinity(0))


def peak_hbm():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except (OSError, ValueError, KeyError):
        return 6650.0, "fallback"


# ------------------------------------------------------------------ clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(np.max(mx)) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


# -------------------------------------------------------------- frame data
def make_frames(count, seed0, voxels=VOXELS):
    from lidar_ai_solution_b200 import scenes
    frames = []
    for i in range(count):
        coords = scenes.make_coords(voxels, GRID, seed0 + i)
        feats = scenes.make_point_features(coords, seed0 + i)
        frames.append((feats, coords))
    return frames


# Workloads: the default is the one the headline metric is quoted on; the others are the
# remaining benchmark configurations, selectable for extra measurements.
WORKLOADS = {
    "centerpoint_int8": dict(kind="centerpoint", precision="int8", voxels=(VOXELS, VOXELS),
                             bound=OUTPUT_BOUND, name=WORKLOAD),
    "centerpoint_int8_mixed": dict(
        kind="centerpoint", precision="int8", voxels=(60000, 200000), bound=520000,
        name="centerpoint_scn_int8 full backbone, 41x1440x1440 grid, voxel counts U[60k,200k]"),
    "centerpoint_int8_fixture": dict(
        kind="centerpoint", precision="int8", voxels=(79745, 79745), bound=OUTPUT_BOUND,
        fixture="centerpoint_zyx",
        name="centerpoint_scn_int8 full backbone, the reference's 79 745-voxel sample frame "
             "(coordinates from tests/golden/fixture_coords.npz, synthetic features)"),
    "bevfusion_fp16": dict(
        kind="bevfusion", precision="fp16", voxels=(VOXELS, VOXELS), bound=OUTPUT_BOUND,
        name="bevfusion lidar SparseEncoder fp16, 41x1440x1440 grid, ~120k active voxels/frame"),
}


def workload_frame(spec, seed):
    """(features, coords) of one frame of a workload."""
    if "fixture" in spec:
        from lidar_ai_solution_b200 import scenes
        zyx = np.load(os.path.join(ROOT, "tests", "golden", "fixture_coords.npz"))[spec["fixture"]]
        coords = np.zeros((len(zyx), 4), np.int32)
        coords[:, 1:] = zyx
        return scenes.make_point_features(coords, seed), coords
    return make_frames(1, seed, frame_voxels(spec, seed))[0]


def frame_voxels(spec, seed):
    lo, hi = spec["voxels"]
    return lo if lo == hi else int(np.random.default_rng(seed).integers(lo, hi + 1))


_RANGES = {}


def build_model(torch, spec):
    """Random-init backbone; for int8, activation ranges from absmax on the seed-0 frame
    (computed once per backbone kind, whatever the output bound)."""
    from lidar_ai_solution_b200 import engine, models, scenes
    model = models.scn_backbone(spec["kind"], seed=0, grid_zyx=GRID, output_bound=spec["bound"])
    if spec["precision"] != "int8":
        return model
    if spec["kind"] not in _RANGES:
        coords = scenes.make_coords(VOXELS, GRID, 0)
        feats = scenes.make_point_features(coords, 0)
        _RANGES[spec["kind"]] = engine.calibrate(model, torch.from_numpy(feats).cuda(),
                                                 torch.from_numpy(coords).cuda(), GRID)
    return models.quantize(model, _RANGES[spec["kind"]])


def save_model(qm):
    from lidar_ai_solution_b200 import onnx_writer
    path = os.path.join(tempfile.mkdtemp(prefix="scn_bench_"), "model.scn.onnx")
    onnx_writer.save(qm, path)
    return path


# ------------------------------------------------- algorithmic work per step
def step_work(line, rows_of, pairs_of, dense_elems):
    """(ops, bytes) of one engine step from its describe line (the per-unit
    figures of the roofline: useful MACs only, every tensor touched once)."""
    f = line.split()
    kind, kv = f[0], dict(x.split("=") for x in f[2:])
    cin, cout, kvol = int(kv["cin"]), int(kv["cout"]), int(kv["kvol"])
    n_in, n_out = rows_of(int(kv["in_cs"])), rows_of(int(kv["out_cs"]))
    s_in = 1 if kv["in"] == "i8" else 2
    s_out = 1 if kv["out"] == "i8" else 2
    if kind == "conv":
        p = pairs_of(int(kv["rule"]))
        b = n_in * cin * s_in + n_out * cout * s_out + kvol * cin * cout * s_in + cout * 8 \
            + 4 * kvol * n_out
        if kv["res"] == "1":
            b += n_out * cout * s_out
        return 2 * p * cin * cout, b
    if kind in ("hash",):
        return 0, 16 * n_in
    if kind == "subm_map":
        return 0, 16 * n_in + 4 * kvol * n_in
    if kind == "down_map":
        return 0, 16 * n_in + 16 * n_out + 4 * kvol * n_out
    if kind == "add":
        return 0, n_out * cout * (2 * s_in + s_out)
    if kind == "relu":
        return 0, n_out * cout * (s_in + s_out)
    if kind == "convert":
        return 0, n_in * (cin * s_in + cout * s_out)
    if kind == "dense":
        return 0, n_in * cout * s_in + 16 * n_in + dense_elems * 2
    return 0, 0


# DRAM bytes (read + write) per algorithmic byte of a convolution launch, by the row width
# of its input in bytes: from one ncu counter pass over every launch of a batch of 4 frames
# of this workload (`--workload frame_once --batch 4`; dram__bytes_read.sum +
# dram__bytes_write.sum of the launches of a width over their algorithmic bytes; 0.92 over
# all 21).  A frame's traffic is these ratios weighted by each layer's bytes.
CONV_DRAM_RATIO = {16: 0.91, 32: 0.93, 64: 0.96, 128: 0.79, 256: 0.79}


# ------------------------------------------------------------ reference arm
def run_reference(args, rank, world):
    """The CPU restatement of the path (oracle/, OpenMP over all host threads) on the
    same workload; a step is one frame."""
    if rank != 0:
        return
    from lidar_ai_solution_b200 import models, scenes
    from oracle import graph_oracle, oracle as orc
    # launchers such as torch.distributed.run export OMP_NUM_THREADS=1
    cores = orc.set_num_threads(host_threads())
    spec = WORKLOADS[args.workload]
    qm = models.scn_backbone(spec["kind"], seed=0, grid_zyx=GRID, output_bound=spec["bound"])
    if spec["precision"] == "int8":
        coords = scenes.make_coords(VOXELS, GRID, 0)
        feats = scenes.make_point_features(coords, 0)
        # calibration on the CPU: fp16 run of the seed frame, absmax per tensor
        _, T = graph_oracle.run(qm, feats, coords, GRID, "fp16")
        ranges = {k: float(np.abs(v["feat"].astype(np.float32)).max()) for k, v in T.items()}
        qm = models.quantize(qm, ranges)
    steps = max(1, min(args.steps, 6))
    warm = max(0, min(args.warmup, 1))
    frames = [workload_frame(spec, s) for s in range(1, 1 + steps + warm)]
    for f, c in frames[:warm]:
        graph_oracle.run(qm, f, c, GRID, spec["precision"])
    t0 = time.perf_counter()
    for f, c in frames[warm:]:
        graph_oracle.run(qm, f, c, GRID, spec["precision"])
    dt = time.perf_counter() - t0
    voxels = float(np.mean([len(f) for f, _ in frames[warm:]]))
    fps = steps / dt
    line = {
        "impl": "reference",
        "metric": "%s_scn_%s_frames_per_s" % (spec["kind"], spec["precision"]), "value": fps,
        "unit": "frames/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "ms_per_step": 1000.0 * dt / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": spec["precision"], "data": "synthetic",
        "config": {"workload": spec["name"], "frames_per_step": 1, "voxels_per_frame": voxels},
        "cpu_baseline": {"value": fps, "unit": "frames/s", "cores": cores, "kind": "port",
                         "sample": "%d frames, one per step, %d host threads (OpenMP)"
                                   % (steps, cores)},
        "e2e": {"value": fps, "unit": "frames/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "active_voxels_per_s": fps * voxels,
    }
    print(json.dumps(line), flush=True)


def bind_to_gpu_cpus(index):
    """One process per GPU: run it (and first-touch its pinned buffers) on the CPUs NVML lists
    as local to that GPU, so that eight ranks' host copies do not all cross to one socket.
    Best effort: any failure leaves the affinity as it was."""
    try:
        import pynvml
        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            index = int(visible.split(",")[index])
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
        pynvml.nvmlShutdown()
    except Exception:
        pass


# ------------------------------------------------------------------ GPU arm
class Pipeline:
    """`replicas` engine replicas on their own streams; the frames go through them in
    batches of `batch` frames, one CUDA graph per batch (row count read on the device)."""

    def __init__(self, torch, dev, onnx_path, precision, frames, batch, replicas, dist=None):
        from lidar_ai_solution_b200 import cabi, engine
        self.torch, self.dev, self.dist = torch, dev, dist
        self.lib = cabi.lib()
        self.cabi = cabi
        self.frames = frames
        self.B = max(1, batch)
        self.groups = [list(range(i, min(i + self.B, len(frames))))
                       for i in range(0, len(frames), self.B)]
        self.R = max(1, min(replicas, len(self.groups)))
        self.streams = [torch.cuda.Stream(device=dev) for _ in range(self.R)]
        self.engines = [engine.Engine.from_onnx(onnx_path, precision, 0, 0, dev)
                        for _ in range(self.R)]
        for e in self.engines:
            e.prepare(GRID, self.B)
        # host side: one pinned buffer pair per frame, the batch column = place in its batch
        self.host_f, self.host_c, self.host_n = [], [], []
        self.dev_f, self.dev_c, self.dev_n, self.offsets = [], [], [], []
        for g in self.groups:
            off, offs = 0, []
            for b, i in enumerate(g):
                f, c = frames[i]
                c = c.copy()
                c[:, 0] = b
                self.host_f.append(torch.from_numpy(f).pin_memory())
                self.host_c.append(torch.from_numpy(c).pin_memory())
                offs.append(off)
                off += len(f)
            self.offsets.append(offs)
            self.host_n.append(torch.tensor([off], dtype=torch.int32).pin_memory())
            self.dev_f.append(torch.empty((off, frames[g[0]][0].shape[1]), dtype=torch.float16,
                                          device=dev))
            self.dev_c.append(torch.empty((off, 4), dtype=torch.int32, device=dev))
            self.dev_n.append(torch.empty(1, dtype=torch.int32, device=dev))
        for gi in range(len(self.groups)):
            self._copy_in(gi, blocking=True)
        _, nbytes = self.engines[0].output_ptr(0)
        self.out_bytes_per_frame = nbytes // self.B
        self.host_out = [torch.empty(nbytes // 2, dtype=torch.float16).pin_memory()
                         for _ in range(self.R)]
        self.graphs = []
        for gi in range(len(self.groups)):
            e, st = self.engines[gi % self.R], self.streams[gi % self.R]
            with torch.cuda.stream(st):
                e.forward_dds(self.dev_f[gi], self.dev_c[gi], self.dev_n[gi], GRID, batch=self.B,
                              stream=st)
                st.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    e.forward_dds(self.dev_f[gi], self.dev_c[gi], self.dev_n[gi], GRID,
                                  batch=self.B, stream=st)
            self.graphs.append(g)
        torch.cuda.synchronize()
        self.check_status("warm-up")
        self.launches_per_step = sum(self.engines[gi % self.R].last_launches()
                                     for gi in range(len(self.groups)))
        self.main = torch.cuda.Stream(device=dev)

    def _copy_in(self, gi, blocking=False):
        k = sum(len(g) for g in self.groups[:gi])
        for b, off in enumerate(self.offsets[gi]):
            n = self.host_f[k + b].shape[0]
            self.dev_f[gi][off:off + n].copy_(self.host_f[k + b], non_blocking=not blocking)
            self.dev_c[gi][off:off + n].copy_(self.host_c[k + b], non_blocking=not blocking)
        self.dev_n[gi].copy_(self.host_n[gi], non_blocking=not blocking)

    def check_status(self, when):
        for e in self.engines:
            st = e.status()
            if st[0]:
                raise RuntimeError("device status %s after %s" % (st, when))

    def h2d_bytes(self):
        return sum(f.numel() * 2 for f in self.host_f) + sum(c.numel() * 4 for c in self.host_c) \
            + 4 * len(self.groups)

    def d2h_bytes(self):
        return self.out_bytes_per_frame * len(self.frames)

    def one_step(self, e2e, compute=True):
        torch = self.torch
        for gi in range(len(self.groups)):
            st = self.streams[gi % self.R]
            with torch.cuda.stream(st):
                if e2e:
                    self._copy_in(gi)
                if compute:
                    self.graphs[gi].replay()
                if e2e:
                    p, _ = self.engines[gi % self.R].output_ptr(0)
                    nb = self.out_bytes_per_frame * len(self.groups[gi])
                    self.cabi.check(self.lib.spconvb_copy_async(
                        self.host_out[gi % self.R].data_ptr(), p, nb, 1, st.cuda_stream))

    def timed(self, steps, warm, e2e, compute=True):
        """(max over ranks of the elapsed device ms, frames done by all ranks)."""
        from lidar_ai_solution_b200 import sharding
        torch, dist = self.torch, self.dist
        for _ in range(warm):
            self.one_step(e2e, compute)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(self.main):
            start.record(self.main)
        for st in self.streams:
            st.wait_event(start)
        for _ in range(steps):
            self.one_step(e2e, compute)
        for st in self.streams:
            ev = torch.cuda.Event()
            ev.record(st)
            self.main.wait_event(ev)
        with torch.cuda.stream(self.main):
            end.record(self.main)
        torch.cuda.synchronize()
        ms, frames_done = sharding.aggregate(start.elapsed_time(end), len(self.frames) * steps,
                                             dist, self.dev)
        if dist is not None:
            dist.barrier()
        return ms, frames_done

    def close(self):
        self.graphs = []
        for e in self.engines:
            e.close()


def conv_roofline(torch, dev, onnx_path, precision, pipe, qm, profile_table=None):
    """Per-launch times of one batch (CUDA events on the launching stream, a 256 MB write
    between launches so that every launch starts with a cold L2) and the roofline of the
    convolution kernel from them."""
    from lidar_ai_solution_b200 import engine
    prof_engine = engine.Engine.from_onnx(onnx_path, precision, 0, 0, dev)
    prof_engine.prepare(GRID, pipe.B)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    feats, coords = pipe.dev_f[0], pipe.dev_c[0]
    nb = len(pipe.groups[0])
    prof_engine.forward(feats, coords, GRID, batch=pipe.B)
    torch.cuda.synchronize()
    prof = prof_engine.profile(feats, coords, GRID, batch=pipe.B, reps=5, flush=flush)
    rules = prof_engine.rules()
    pairs = [int((m[:, :n_out] >= 0).sum().item()) for m, n_out, _ in rules]
    dense_elems = int(np.prod(qm["outputs"][0][1])) * nb
    tot_ops = tot_bytes = 0
    conv_ops = conv_bytes = conv_ms = all_ms = traffic = 0.0
    n_conv = 0
    rows = []
    for ln, ms in prof:
        ops, nbytes = step_work(ln, prof_engine.coordset_rows, lambda r: pairs[r], dense_elems)
        rows.append((ln, ms, ops, nbytes))
        tot_ops += ops
        tot_bytes += nbytes
        all_ms += ms
        if ln.startswith("conv "):
            kv = dict(x.split("=") for x in ln.split()[2:])
            rb = int(kv["cin"]) * (1 if kv["in"] == "i8" else 2)
            rb = max(16, 1 << (rb - 1).bit_length())
            traffic += CONV_DRAM_RATIO.get(rb, 0.75) * nbytes
            conv_ops += ops
            conv_bytes += nbytes
            conv_ms += ms
            n_conv += 1
    peak, src = peak_hbm()
    achieved = conv_bytes / (conv_ms / 1000.0) / 1e9 if conv_ms > 0 else 0.0
    roof = {
        "bound": "hbm",
        "kernel": "conv_umma_kernel (the %d convolution launches of a batch of %d frames)"
                  % (n_conv, nb),
        "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
        "peak_source": src, "traffic": traffic / nb,
        "algorithmic_bytes_per_frame": conv_bytes / nb, "kernel_ms_per_frame": conv_ms / nb,
        "frames_per_launch": nb,
        "share_of_frame_kernel_time": conv_ms / all_ms if all_ms else None,
        "int8_tops_achieved": conv_ops / (conv_ms / 1000.0) / 1e12 if conv_ms else 0.0,
        "int8_tops_peak_nominal": 4500.0,
    }
    frame = {"algorithmic_bytes": tot_bytes / nb, "useful_int8_ops": tot_ops / nb,
             "serial_kernel_ms": all_ms / nb}
    if profile_table:
        # per step: time, algorithmic bytes and useful ops, the roofline time (the larger of
        # bytes / measured HBM copy bandwidth and ops / tensor peak: int8 at the nominal
        # 4 500 TOPS, fp16 at the measured bf16 cuBLAS rate) and the fraction of it achieved
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except (OSError, ValueError):
            peaks = {}
        tensor_i8 = 4500e12
        tensor_f16 = float(peaks.get("bf16_tflops", 1590.0)) * 1e12
        with open(profile_table, "w") as f:
            f.write("# one batch of %d frames; times are per launch\n" % nb)
            for ln, ms, ops, nbytes in rows:
                t_hbm = nbytes / (peak * 1e9)
                t_tc = ops / (tensor_i8 if " in=i8 " in ln else tensor_f16)
                bound_us = 1e6 * max(t_hbm, t_tc)
                f.write("%8.2f us  %8.3f MB  %8.3f GOP  %6.2f us %s  %5.3f  %s\n" % (
                    ms * 1000, nbytes / 1e6, ops / 1e9, bound_us,
                    "hbm" if t_hbm >= t_tc else "tc ", bound_us / (ms * 1000) if ms else 0.0, ln))
    prof_engine.close()
    return roof, frame


def voxelizer_case(torch, n_points, fp16, reps, flush, seed=0):
    """One raw sweep through the voxelizer (CenterPoint ranges: 1440x1440x40 voxels of
    0.075 x 0.075 x 0.2 m, at most 10 points per voxel, 160 000 voxels)."""
    from lidar_ai_solution_b200 import ops, scenes
    pts = scenes.make_points(n_points, seed)
    if fp16:
        pts = pts.astype(np.float16)
    dev = torch.from_numpy(pts).cuda()
    run, bufs = make_voxelizer(torch, n_points, fp16)
    run(dev)
    torch.cuda.synchronize()
    n = int(bufs["n"].item())
    us = time_launches(torch, lambda: run(dev), reps, flush)
    nbytes = n_points * 5 * (2 if fp16 else 4) + n * (5 * 2 + 16)
    peak, src = peak_hbm()
    return {"kernel": "voxelize", "points": n_points, "points_dtype": "fp16" if fp16 else "fp32",
            "voxels": n, "us": us, "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / us / 1e3,
            "hbm_frac": nbytes / us / 1e3 / peak, "hbm_peak_gbs": peak, "peak_source": src,
            "points_per_s": n_points / us * 1e6}


def make_voxelizer(torch, n_points, fp16, max_voxels=160000):
    """(run(points_dev), buffers): the voxelizer with its buffers allocated once."""
    from lidar_ai_solution_b200 import ops, scenes
    params = ops.voxel_params(scenes.CENTERPOINT_RANGE, scenes.CENTERPOINT_VOXEL, (1440, 1440, 40),
                              5, 1 if fp16 else 0, 10, max_voxels, 0)
    lib = ops.cabi.lib()
    st = ops.new_status()
    ws = torch.empty(max(256, lib.spconvb_voxelize_workspace_bytes(C.byref(params), n_points)),
                     dtype=torch.uint8, device="cuda")
    bufs = {"feat": torch.zeros((max_voxels, 5), dtype=torch.float16, device="cuda"),
            "idx": torch.zeros((max_voxels, 4), dtype=torch.int32, device="cuda"),
            "n": torch.zeros(1, dtype=torch.int32, device="cuda"), "status": st}

    def run(points_dev):
        ops.cabi.check(lib.spconvb_voxelize(
            C.byref(params), C.c_void_p(points_dev.data_ptr()), n_points, C.c_void_p(ws.data_ptr()),
            C.c_void_p(bufs["feat"].data_ptr()), C.c_void_p(bufs["idx"].data_ptr()),
            C.c_void_p(bufs["n"].data_ptr()), C.c_void_p(st.data_ptr()),
            C.c_void_p(torch.cuda.current_stream().cuda_stream)), "voxelize")
    return run, bufs


def time_launches(torch, fn, reps, flush):
    """Median microseconds of fn() over `reps` runs, an L2 flush (a 256 MB write) before each
    (the median, because a helper that allocates its result can stall one run on the host)."""
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    times = []
    for i in range(reps):
        if flush is not None:
            flush.fill_(i & 0xFF)
        start.record()
        fn()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end))
    return float(np.median(times)) * 1000.0


def from_points_leg(torch, dev, onnx_path, precision, steps):
    """H2D of a raw 140 000-point sweep -> voxelizer -> backbone -> D2H of the BEV tensor, one
    frame at a time on one stream (the call sequence of CenterPoint::doinfer up to the RPN)."""
    from lidar_ai_solution_b200 import cabi, engine, scenes
    n_points = 140000
    host_pts = torch.from_numpy(scenes.make_points(n_points, 7)).pin_memory()
    dev_pts = torch.empty_like(host_pts, device=dev)
    run, bufs = make_voxelizer(torch, n_points, False)
    e = engine.Engine.from_onnx(onnx_path, precision, 0, 0, dev)
    e.prepare(GRID, 1)
    p, nbytes = e.output_ptr(0)
    host_out = torch.empty(nbytes // 2, dtype=torch.float16).pin_memory()
    lib = cabi.lib()
    st = torch.cuda.current_stream()

    def frame():
        dev_pts.copy_(host_pts, non_blocking=True)
        run(dev_pts)
        e.forward_dds(bufs["feat"], bufs["idx"], bufs["n"], GRID, batch=1)
        cabi.check(lib.spconvb_copy_async(host_out.data_ptr(), p, nbytes, 1, st.cuda_stream))

    for _ in range(3):
        frame()
    torch.cuda.synchronize()
    status = e.status()
    if status[0] or int(bufs["status"][0].item()):
        raise RuntimeError("device status %s / %s in the from-points leg"
                           % (status, bufs["status"].tolist()))
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        frame()
    t1.record()
    t1.synchronize()
    ms = t0.elapsed_time(t1) / steps
    voxels = int(bufs["n"].item())
    e.close()
    return {"value": 1000.0 / ms, "unit": "frames/s", "ms_per_frame": ms, "points": n_points,
            "voxels": voxels, "h2d_bytes_per_step": host_pts.numel() * 4,
            "d2h_bytes_per_step": nbytes,
            "what": "pinned fp32 points -> voxelize -> backbone -> pinned BEV, one stream, "
                    "one frame in flight"}


def run_gpu(args, rank, world, local_rank):
    import torch
    from lidar_ai_solution_b200 import cabi, engine, sharding

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        bind_to_gpu_cpus(local_rank)  # before the pinned buffers are allocated
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    cabi.lib()  # fails loudly if the CUDA extension was not built

    spec = WORKLOADS[args.workload]
    precision = engine.PRECISION_INT8 if spec["precision"] == "int8" else engine.PRECISION_FP16
    qm = build_model(torch, spec)
    onnx_path = save_model(qm)
    legs = set(args.legs.split(",")) if args.legs else set()

    F = args.frames
    frames = [workload_frame(spec, s) for s in sharding.frame_seeds(rank, F)]
    pipe = Pipeline(torch, dev, onnx_path, precision, frames, args.batch, args.replicas, dist)

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_dev, total_frames = pipe.timed(args.steps, args.warmup, e2e=False)
    clocks = sampler.stop()
    ms_e2e, _ = pipe.timed(args.steps, args.warmup, e2e=True)
    pipe.check_status("the timed region")
    copy_only = None
    if world > 1 and "copy_only" in legs:
        # control: the same pinned copies with no compute, all ranks at once
        ms_copy, _ = pipe.timed(args.steps, 1, e2e=True, compute=False)
        per_rank = (pipe.h2d_bytes() + pipe.d2h_bytes()) * args.steps / (ms_copy / 1000.0) / 1e9
        copy_only = {"ms_per_step": ms_copy / args.steps, "gbs_per_rank": per_rank,
                     "frames_per_s_ceiling": total_frames / (ms_copy / 1000.0)}

    voxels_per_frame = float(np.mean([len(f) for f, _ in frames]))
    value = total_frames / (ms_dev / 1000.0)
    e2e_value = total_frames / (ms_e2e / 1000.0)

    line = {
        "metric": "%s_scn_%s_frames_per_s" % (spec["kind"], spec["precision"]), "value": value,
        "unit": "frames/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": spec["precision"], "data": "synthetic",
        "config": {"workload": spec["name"], "frames_per_gpu_per_step": F,
                   "frames_per_engine_call": pipe.B, "replicas_per_gpu": pipe.R,
                   "voxels_per_frame": voxels_per_frame,
                   "parallelism": "frames sharded, no collective",
                   "l2": "no flush: a step touches ~%d MB per GPU (> 126 MB L2)" % (F * 150)},
        "e2e": {"value": e2e_value, "unit": "frames/s", "h2d_bytes_per_step": pipe.h2d_bytes() * world,
                "d2h_bytes_per_step": pipe.d2h_bytes() * world, "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": pipe.launches_per_step * args.steps * world,
        "launches_per_frame": pipe.launches_per_step / float(F),
        "active_voxels_per_s": value * voxels_per_frame,
        "clocks": clocks,
    }
    if copy_only:
        line["copy_only"] = copy_only
        line["e2e"]["frac_of_copy_ceiling"] = e2e_value / copy_only["frames_per_s_ceiling"]

    if rank == 0:
        roof, frame = conv_roofline(torch, dev, onnx_path, precision, pipe, qm, args.profile_table)
        line["roofline"] = roof
        frame_s = (ms_dev / 1000.0) / (F * args.steps)
        peak = roof["peak"]
        frame.update({"achieved_gbs": frame["algorithmic_bytes"] / frame_s / 1e9,
                      "achieved_tops": frame["useful_int8_ops"] / frame_s / 1e12,
                      "hbm_frac_of_measured": frame["algorithmic_bytes"] / frame_s / 1e9 / peak})
        line["frame"] = frame
    pipe.close()

    # the same backbone with room for 520 000 rows per frame: frames of up to 200 k voxels
    # (and raw sweeps whose voxel count is not known in advance)
    onnx4 = None
    if legs & {"config4", "voxelizer"} and spec["kind"] == "centerpoint" and spec["precision"] == "int8":
        onnx4 = save_model(build_model(torch, WORKLOADS["centerpoint_int8_mixed"]))

    # ---- the fixed 64-frame set with mixed voxel counts, sharded over the ranks (strong scaling)
    if "config4" in legs and onnx4:
        spec4 = WORKLOADS["centerpoint_int8_mixed"]
        seeds = list(range(100, 164))
        counts = [frame_voxels(spec4, s) for s in seeds]
        mine = sharding.assign_frames(counts, world)[rank]
        frames4 = [workload_frame(spec4, seeds[i]) for i in mine]
        # the set is fixed, so a rank's share shrinks with N: keep every replica busy
        batch4 = max(1, min(args.batch, -(-len(frames4) // max(1, args.replicas))))
        p4 = Pipeline(torch, dev, onnx4, precision, frames4, batch4, args.replicas, dist)
        ms4, done4 = p4.timed(3, 1, e2e=False)
        ms4e, _ = p4.timed(3, 1, e2e=True)
        p4.check_status("the 64-frame set")
        load = float(sum(counts[i] for i in mine))
        loads = sharding.gather_floats(load, dist, dev)
        line["config4"] = {
            "workload": "64 frames, seeds 100..163, voxel counts U[60k,200k], assigned to ranks "
                        "longest-first (strong scaling: the set is fixed)",
            "value": done4 / (ms4 / 1000.0), "e2e": done4 / (ms4e / 1000.0), "unit": "frames/s",
            "active_voxels_per_s": float(sum(counts)) * 3 / (ms4 / 1000.0),
            "frames_total": done4 // 3, "ms_per_pass": ms4 / 3, "frames_per_engine_call": batch4,
            "rank_load_max_over_mean": max(loads) / (sum(loads) / len(loads))}
        p4.close()

    if rank == 0:
        # ---- the reference's own sample frame (real sweep geometry: a fifth of the work of a
        # synthetic frame of equal voxel count)
        if "real_frame" in legs and spec["kind"] == "centerpoint" and spec["precision"] == "int8" \
                and world == 1:
            specf = WORKLOADS["centerpoint_int8_fixture"]
            framesf = [workload_frame(specf, 2000 + i) for i in range(F)]
            pf = Pipeline(torch, dev, onnx_path, precision, framesf, args.batch, args.replicas)
            msf, donef = pf.timed(5, 3, e2e=False)
            msfe, _ = pf.timed(5, 3, e2e=True)
            pf.check_status("the sample-frame leg")
            rooff, _ = conv_roofline(torch, dev, onnx_path, precision, pf, qm)
            line["real_frame"] = {
                "workload": specf["name"], "value": donef / (msf / 1000.0),
                "e2e": donef / (msfe / 1000.0), "unit": "frames/s",
                "conv_frac_of_hbm": rooff["frac"], "conv_ms_per_frame": rooff["kernel_ms_per_frame"],
                "launches_per_frame": pf.launches_per_step / float(F)}
            pf.close()
        # ---- voxelizer alone, and the path from raw points
        if "voxelizer" in legs and world == 1 and onnx4:
            flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
            v = voxelizer_case(torch, 300000, False, 10, flush)
            line["voxelizer"] = {k: v[k] for k in ("points", "voxels", "us", "achieved_gbs",
                                                   "hbm_frac", "points_per_s")}
            del flush
            line["e2e_from_points"] = from_points_leg(torch, dev, onnx4, precision, 20)
        # ---- CPU baselines on the host cores of this box (bounded samples)
        if world == 1 and not args.no_cpu_baseline:
            from oracle import cpu_baseline_config0, graph_oracle, oracle as orc
            cores = orc.set_num_threads(host_threads())
            sample = frames[: max(1, min(args.cpu_frames, F))]
            graph_oracle.run(qm, sample[0][0][:2000], sample[0][1][:2000], GRID,
                             spec["precision"])  # warm
            t0 = time.perf_counter()
            for f, c in sample:
                graph_oracle.run(qm, f, c, GRID, spec["precision"])
            dt = time.perf_counter() - t0
            line["cpu_baseline"] = {
                "value": len(sample) / dt, "unit": "frames/s", "cores": cores, "kind": "port",
                "sample": "%d of the step's %d frames through the CPU oracle (OpenMP), %.1f s"
                          % (len(sample), F, dt)}
            c0 = cpu_baseline_config0.measure(3)
            line["cpu_baseline_config0"] = {
                "what": c0["config"], "oracle_ms": c0["oracle_ms"],
                "oracle_rulebook_ms": c0["oracle_rulebook_ms"], "oracle_threads": c0["oracle_threads"],
                "torch_cpu_conv_ms": c0["torch_cpu_conv_ms"], "torch_threads": c0["torch_threads"]}
        print(json.dumps(line), flush=True)

    if dist is not None:
        dist.destroy_process_group()


# --------------------------------------------------------- per-layer sweeps
def layer_case(torch, c, n, fp16, reps, flush, seed=0):
    """One SubMConv3d 3x3x3 layer, Cin = Cout = c, n voxels, fused bias + ReLU + requant,
    through the kernel-level C ABI: microseconds of the launch (L2 flushed before each), its
    algorithmic bytes and useful ops."""
    from lidar_ai_solution_b200 import ops, scenes
    rng = np.random.default_rng(seed)
    coords = torch.from_numpy(scenes.make_coords(n, GRID, seed)).cuda()
    n_ptr, st = ops.device_count(n), ops.new_status()
    table = ops.hash_build(coords, n_ptr, GRID, status=st)
    m = ops.subm_map(coords, n_ptr, GRID, table, status=st)
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
                         status=st, out=out, n_in_ptr=n_ptr)

    conv()
    torch.cuda.synchronize()
    if int(st.cpu()[0]):
        raise RuntimeError("device status %s" % st.cpu().tolist())
    us = time_launches(torch, conv, reps, flush)
    us_hash = time_launches(torch, lambda: ops.hash_build(coords, n_ptr, GRID), max(3, reps // 4),
                            flush)
    us_map = time_launches(torch, lambda: ops.subm_map(coords, n_ptr, GRID, table),
                           max(3, reps // 4), flush)
    pairs = int((m >= 0).sum().item())
    nbytes = n * c * es * 2 + 27 * c * c * es + c * 8 + 4 * 27 * n
    opsn = 2 * pairs * c * c
    peak, src = peak_hbm()
    return {"channels": c, "voxels": n, "dtype": "fp16" if fp16 else "int8", "pairs": pairs,
            "conv_us": us, "algorithmic_bytes": nbytes, "useful_ops": opsn,
            "achieved_gbs": nbytes / us / 1e3, "achieved_tops": opsn / us / 1e6,
            "hbm_frac": nbytes / us / 1e3 / peak, "hbm_peak_gbs": peak, "peak_source": src,
            "hash_us": us_hash, "subm_map_us": us_map,
            "map_gbs": (16 * n + 4 * 27 * n) / us_map / 1e3}


def run_frame_once(args):
    """Everything a frame launches, exactly once, between cudaProfilerStart and cudaProfilerStop:
    the voxelizer on a raw sweep, then one eager engine call on `--batch` synthetic frames."""
    import torch
    from lidar_ai_solution_b200 import cabi, engine, scenes
    cabi.lib()
    dev = torch.device("cuda", 0)
    spec = WORKLOADS["centerpoint_int8"]
    onnx_path = save_model(build_model(torch, spec))
    B = max(1, args.batch)
    frames = [workload_frame(spec, 1000 + i) for i in range(B)]
    feats = np.concatenate([f for f, _ in frames])
    coords = np.concatenate([np.concatenate([np.full((len(c), 1), b, np.int32), c[:, 1:]], 1)
                             for b, (_, c) in enumerate(frames)])
    df, dc = torch.from_numpy(feats).to(dev), torch.from_numpy(coords).to(dev)
    e = engine.Engine.from_onnx(onnx_path, engine.PRECISION_INT8, 0, 0, dev)
    e.forward(df, dc, GRID, batch=B)   # allocation and warm-up
    pts = torch.from_numpy(scenes.make_points(140000, 7)).to(dev)
    vox, bufs = make_voxelizer(torch, 140000, False)
    vox(pts)
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    vox(pts)
    e.forward(df, dc, GRID, batch=B)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(json.dumps({"workload": "frame_once", "frames": B, "launches": e.last_launches(),
                      "status": e.status(), "voxels_from_points": int(bufs["n"].item())}))
    e.close()


def run_sweeps(args):
    import torch
    from lidar_ai_solution_b200 import cabi
    cabi.lib()
    flush = None if args.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    if args.workload == "voxelizer":
        for n in args.points:
            print(json.dumps(voxelizer_case(torch, n, args.fp16, args.reps, flush)), flush=True)
        return
    for c in args.channels:
        for n in args.voxels:
            print(json.dumps(layer_case(torch, c, n, args.fp16, args.reps, flush)), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="centerpoint_int8",
                    choices=sorted(WORKLOADS) + ["layer_sweep", "voxelizer", "frame_once"])
    ap.add_argument("--frames", type=int, default=32, help="frames per GPU per step")
    ap.add_argument("--batch", type=int, default=8, help="frames per engine call")
    ap.add_argument("--replicas", type=int, default=4, help="engine replicas (streams) per GPU")
    ap.add_argument("--legs", default="config4,real_frame,voxelizer,copy_only",
                    help="extra measurements added to the line (comma separated; '' for none)")
    ap.add_argument("--cpu-frames", type=int, default=4, help="frames timed on the CPU oracle")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-table", default=None, help="write the per-step table here")
    # sweeps
    ap.add_argument("--channels", type=int, nargs="+", default=[16, 32, 64, 128])
    ap.add_argument("--voxels", type=int, nargs="+", default=[10000, 50000, 120000, 200000])
    ap.add_argument("--points", type=int, nargs="+", default=[100000, 200000, 300000])
    ap.add_argument("--fp16", action="store_true")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--no-flush", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    rank, world = _env_int("RANK", 0), _env_int("WORLD_SIZE", 1)
    local_rank = _env_int("LOCAL_RANK", 0)
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif args.workload in ("layer_sweep", "voxelizer"):
        run_sweeps(args)
    elif args.workload == "frame_once":
        run_frame_once(args)
    else:
        run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
