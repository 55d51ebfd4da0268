#!/usr/bin/env python
"""Throughput of the CenterPoint SCN int8 backbone (frames/s) on 1-8 B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W    # CPU restatement, host cores

A step is one pass of the hot path (rulebooks, 21 convolutions with fused
epilogues, dense BEV scatter) over a batch of independent synthetic frames:
per GPU, `--frames` frames of ~120 k active voxels in the 41x1440x1440 grid,
every frame from its own seed.  Frames are independent, so ranks share nothing:
no collective runs inside the timed region, scaling is weak (per-GPU work fixed).

`value`  inputs resident in HBM, one CUDA graph per frame spread over
         `--replicas` engine replicas (streams) per GPU, timed with CUDA events;
`e2e`    the same through the engine C ABI with HOST buffers: pinned features,
         indices and row count copied in, the dense fp16 BEV tensor copied out,
         all inside the timed region.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
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
                 "-lms", "100", "-i", str(self.gpu_index)],
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


def build_model(torch, spec):
    """Random-init backbone; for int8, activation ranges from absmax on the seed-0 frame."""
    from lidar_ai_solution_b200 import engine, models, scenes
    model = models.scn_backbone(spec["kind"], seed=0, grid_zyx=GRID, output_bound=spec["bound"])
    if spec["precision"] != "int8":
        return model
    coords = scenes.make_coords(VOXELS, GRID, 0)
    feats = scenes.make_point_features(coords, 0)
    ranges = engine.calibrate(model, torch.from_numpy(feats).cuda(),
                              torch.from_numpy(coords).cuda(), GRID)
    return models.quantize(model, ranges)


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


# ------------------------------------------------------------ reference arm
def run_reference(args, rank, world):
    """The CPU restatement of the path (oracle/, OpenMP over all host threads) on the
    same workload; a step is one frame."""
    if rank != 0:
        return
    from lidar_ai_solution_b200 import models, scenes
    from oracle import graph_oracle, oracle as orc
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
    cores = orc.num_threads()
    line = {
        "impl": "reference",
        "metric": "%s_scn_%s_frames_per_s" % (spec["kind"], spec["precision"]), "value": fps,
        "unit": "frames/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "ms_per_step": 1000.0 * dt / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": spec["precision"], "data": "synthetic",
        "config": {"workload": spec["name"], "frames_per_step": 1, "voxels_per_frame": voxels},
        "cpu_baseline": {"value": fps, "unit": "frames/s", "cores": cores, "kind": "port",
                         "sample": "%d frames, one per step, all host threads (OpenMP)" % steps},
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
def run_gpu(args, rank, world, local_rank):
    import torch
    from lidar_ai_solution_b200 import cabi, engine, onnx_writer, sharding

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
    tmp = tempfile.mkdtemp(prefix="scn_bench_")
    onnx_path = os.path.join(tmp, "model.scn.onnx")
    onnx_writer.save(qm, onnx_path)

    F, R = args.frames, max(1, min(args.replicas, args.frames))
    frames = [workload_frame(spec, s) for s in sharding.frame_seeds(rank, F)]
    streams = [torch.cuda.Stream(device=dev) for _ in range(R)]
    engines = [engine.Engine.from_onnx(onnx_path, precision, 0, 0, dev) for _ in range(R)]
    for e in engines:
        e.prepare(GRID)

    host_f = [torch.from_numpy(f).pin_memory() for f, _ in frames]
    host_c = [torch.from_numpy(c).pin_memory() for _, c in frames]
    host_n = [torch.tensor([len(f)], dtype=torch.int32).pin_memory() for f, _ in frames]
    dev_f = [t.to(dev) for t in host_f]
    dev_c = [t.to(dev) for t in host_c]
    dev_n = [t.to(dev) for t in host_n]
    out_ptr, out_bytes = engines[0].output_ptr(0)
    host_out = [torch.empty(out_bytes // 2, dtype=torch.float16).pin_memory() for _ in range(R)]
    lib = cabi.lib()

    # one CUDA graph per frame on its replica's stream (DDS row count in device memory)
    graphs = []
    for i in range(F):
        e, st = engines[i % R], streams[i % R]
        with torch.cuda.stream(st):
            e.forward_dds(dev_f[i], dev_c[i], dev_n[i], GRID, stream=st)
            st.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                e.forward_dds(dev_f[i], dev_c[i], dev_n[i], GRID, stream=st)
        graphs.append(g)
    torch.cuda.synchronize()
    for e in engines:
        st = e.status()
        if st[0]:
            raise RuntimeError("device status %s after warm-up" % st)
    launches_per_frame = engines[0].last_launches()

    main = torch.cuda.Stream(device=dev)

    def one_step(e2e):
        for i in range(F):
            st = streams[i % R]
            with torch.cuda.stream(st):
                if e2e:
                    dev_f[i].copy_(host_f[i], non_blocking=True)
                    dev_c[i].copy_(host_c[i], non_blocking=True)
                    dev_n[i].copy_(host_n[i], non_blocking=True)
                graphs[i].replay()
                if e2e:
                    e = engines[i % R]
                    p, nb = e.output_ptr(0)
                    cabi.check(lib.spconvb_copy_async(host_out[i % R].data_ptr(), p, nb, 1,
                                                      st.cuda_stream))

    def timed(steps, warm, e2e):
        for _ in range(warm):
            one_step(e2e)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(main):
            start.record(main)
        for st in streams:
            st.wait_event(start)
        for _ in range(steps):
            one_step(e2e)
        for st in streams:
            ev = torch.cuda.Event()
            ev.record(st)
            main.wait_event(ev)
        with torch.cuda.stream(main):
            end.record(main)
        torch.cuda.synchronize()
        ms, frames_done = sharding.aggregate(start.elapsed_time(end), F * steps, dist, dev)
        if dist is not None:
            dist.barrier()
        return ms, frames_done

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_dev, total_frames = timed(args.steps, args.warmup, e2e=False)
    clocks = sampler.stop()
    ms_e2e, _ = timed(args.steps, args.warmup, e2e=True)
    for e in engines:
        st = e.status()
        if st[0]:
            raise RuntimeError("device status %s after the timed region" % st)

    voxels_per_frame = float(np.mean([len(f) for f, _ in frames]))
    value = total_frames / (ms_dev / 1000.0)
    e2e_value = total_frames / (ms_e2e / 1000.0)
    h2d = sum(host_f[i].numel() * 2 + host_c[i].numel() * 4 + 4 for i in range(F))
    d2h = out_bytes * F

    line = {
        "metric": "%s_scn_%s_frames_per_s" % (spec["kind"], spec["precision"]), "value": value,
        "unit": "frames/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": spec["precision"], "data": "synthetic",
        "config": {"workload": spec["name"], "frames_per_gpu_per_step": F, "replicas_per_gpu": R,
                   "voxels_per_frame": voxels_per_frame, "parallelism": "frames sharded, no collective",
                   "l2": "no flush: a step touches ~%d MB per GPU (> 126 MB L2)" % (F * 150)},
        "e2e": {"value": e2e_value, "unit": "frames/s", "h2d_bytes_per_step": h2d * world,
                "d2h_bytes_per_step": d2h * world, "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": launches_per_frame * F * args.steps * world,
        "active_voxels_per_s": value * voxels_per_frame,
        "clocks": clocks,
    }

    if rank == 0:
        # ---- per-kernel times (cold L2) and the roofline of the dominant kernel
        prof_engine = engine.Engine.from_onnx(onnx_path, precision, 0, 0, dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        prof_engine.forward(dev_f[0], dev_c[0], GRID)
        torch.cuda.synchronize()
        prof = prof_engine.profile(dev_f[0], dev_c[0], GRID, reps=5, flush=flush)
        rules = prof_engine.rules()
        pairs = [int((m[:, :n_out] >= 0).sum().item()) for m, n_out, _ in rules]
        dense_elems = int(np.prod(qm["outputs"][0][1]))
        tot_ops = tot_bytes = 0
        conv_ops = conv_bytes = conv_ms = all_ms = 0.0
        n_conv = 0
        for ln, ms in prof:
            ops, nbytes = step_work(ln, prof_engine.coordset_rows, lambda r: pairs[r], dense_elems)
            tot_ops += ops
            tot_bytes += nbytes
            all_ms += ms
            if ln.startswith("conv "):
                conv_ops += ops
                conv_bytes += nbytes
                conv_ms += ms
                n_conv += 1
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except (OSError, ValueError):
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        achieved = conv_bytes / (conv_ms / 1000.0) / 1e9 if conv_ms > 0 else 0.0
        line["roofline"] = {
            "bound": "hbm",
            "kernel": "conv_umma_kernel (all %d convolution launches of a frame)" % n_conv,
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "peak_source": "measured" if "hbm_gbs" in peaks else "fallback",
            "traffic": CONV_DRAM_PER_ALGORITHMIC_BYTE * conv_bytes,
            "algorithmic_bytes_per_frame": conv_bytes, "kernel_ms_per_frame": conv_ms,
            "share_of_frame_kernel_time": conv_ms / all_ms if all_ms else None,
            "int8_tops_achieved": conv_ops / (conv_ms / 1000.0) / 1e12 if conv_ms else 0.0,
        }
        frame_s = (ms_dev / 1000.0) / (F * args.steps)
        line["frame"] = {"algorithmic_bytes": tot_bytes, "useful_int8_ops": tot_ops,
                         "achieved_gbs": tot_bytes / frame_s / 1e9 / 1.0,
                         "achieved_tops": tot_ops / frame_s / 1e12,
                         "hbm_frac_of_measured": tot_bytes / frame_s / 1e9 / peak,
                         "serial_kernel_ms": all_ms}
        if args.profile_table:
            # per step: time, algorithmic bytes and useful ops, the roofline time (the larger of
            # bytes / measured HBM copy bandwidth and ops / tensor peak: int8 at the nominal
            # 4 500 TOPS, fp16 at the measured bf16 cuBLAS rate) and the fraction of it achieved
            tensor_i8 = 4500e12
            tensor_f16 = float(peaks.get("bf16_tflops", 1590.0)) * 1e12
            with open(args.profile_table, "w") as f:
                for ln, ms in prof:
                    ops, nbytes = step_work(ln, prof_engine.coordset_rows, lambda r: pairs[r],
                                            dense_elems)
                    t_hbm = nbytes / (peak * 1e9)
                    t_tc = ops / (tensor_i8 if " in=i8 " in ln else tensor_f16)
                    bound_us = 1e6 * max(t_hbm, t_tc)
                    f.write("%8.2f us  %8.3f MB  %8.3f GOP  %6.2f us %s  %5.3f  %s\n" % (
                        ms * 1000, nbytes / 1e6, ops / 1e9, bound_us,
                        "hbm" if t_hbm >= t_tc else "tc ", bound_us / (ms * 1000) if ms else 0.0,
                        ln))
        prof_engine.close()

        # ---- CPU baseline on the host cores of this box (bounded sample)
        if world == 1 and not args.no_cpu_baseline:
            from oracle import graph_oracle, oracle as orc
            sample = frames[: max(1, min(args.cpu_frames, F))]
            graph_oracle.run(qm, sample[0][0][:2000], sample[0][1][:2000], GRID,
                             spec["precision"])  # warm
            t0 = time.perf_counter()
            for f, c in sample:
                graph_oracle.run(qm, f, c, GRID, spec["precision"])
            dt = time.perf_counter() - t0
            line["cpu_baseline"] = {
                "value": len(sample) / dt, "unit": "frames/s", "cores": orc.num_threads(),
                "kind": "port",
                "sample": "%d of the step's %d frames through the CPU oracle (OpenMP), %.1f s"
                          % (len(sample), F, dt)}
        print(json.dumps(line), flush=True)

    for e in engines:
        e.close()
    if dist is not None:
        dist.destroy_process_group()


# DRAM bytes (read + write) of the convolution launches per algorithmic byte.  ncu cannot
# capture the full frame within its size limits, so the frame's traffic is one captured
# launch (profiles/conv_umma_int8_c64_170k.md: dram read + write = 29.41 MB for 40.23 MB of
# algorithmic bytes; the output is still in L2 when the launch ends) scaled to the frame's
# algorithmic convolution bytes (704.4 MB on the default workload), traffic growing in
# proportion to rows.
CONV_DRAM_PER_ALGORITHMIC_BYTE = 0.731


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="centerpoint_int8", choices=sorted(WORKLOADS))
    ap.add_argument("--frames", type=int, default=16, help="frames per GPU per step")
    ap.add_argument("--replicas", type=int, default=4, help="engine replicas (streams) per GPU")
    ap.add_argument("--cpu-frames", type=int, default=4, help="frames timed on the CPU oracle")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-table", default=None, help="write the per-step table here")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    rank, world = _env_int("RANK", 0), _env_int("WORLD_SIZE", 1)
    local_rank = _env_int("LOCAL_RANK", 0)
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
