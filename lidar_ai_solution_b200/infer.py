"""Command-line inference with the options of the reference's `infer` tool
(libraries/3DSparseConvolution/src/infer.cpp:475-491, libspconv/example/infer.cpp:161-375).

    python -m lidar_ai_solution_b200.infer --onnx model.scn.onnx --feature f.tensor \\
        --indice i.tensor --grid_size 41,1440,1440 --int8 --cudagraph --dds --profiling

Tensor files use the reference's format (tensor_file.py).  Without real model files, a
random-init backbone and a synthetic frame can stand in:

    python -m lidar_ai_solution_b200.infer --synthetic centerpoint --voxels 120000 --int8 --profiling

Options that select between kernel generations in the reference (`--blackwell`,
`--sortmask`, `--auxiliary_stream`) are accepted and ignored: there is one code path here,
written for sm_100a.  `--search_best_perf` therefore only sweeps what exists: CUDA graph
on/off and the fixed launch size (which every kernel here ignores: grids are sized by the
SM count and stride over the rows, so its three proposals are expected to tie).
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile

import numpy as np
import torch

from . import cabi, engine, models, onnx_writer, scenes, tensor_file


def _flag(ap, name, default, text):
    ap.add_argument("--" + name, nargs="?", const="true", default=default, help=text,
                    type=lambda s: str(s).lower())


def parse_args(argv=None):
    ap = argparse.ArgumentParser(prog="infer", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--onnx", default="", help="ONNX file exported for spconv")
    ap.add_argument("--feature", default="", help="feature tensor file, fp16 [N, C]")
    ap.add_argument("--indice", default="", help="indice tensor file, int32 [N, 4]")
    ap.add_argument("--grid_size", default="", help="sparse grid size, e.g. 41,1440,1440")
    _flag(ap, "fp16", "true", "main precision fp16")
    _flag(ap, "int8", "false", "main precision int8 (wins over fp16)")
    _flag(ap, "sortmask", "false", "accepted, ignored")
    _flag(ap, "blackwell", "false", "accepted, ignored (always sm_100a kernels)")
    _flag(ap, "auxiliary_stream", "true", "build the rulebooks on a second stream inside the engine")
    _flag(ap, "cudagraph", "false", "capture the forward in a CUDA graph and replay it")
    ap.add_argument("--fixed_points", type=int, default=10000,
                    help="fixed launch size of all kernels (with cudagraph or dds)")
    _flag(ap, "profiling", "false", "measure latency and per-layer times")
    _flag(ap, "verbose", "false", "verbose engine log")
    _flag(ap, "dds", "false", "row count read on the device (data dependent shape)")
    _flag(ap, "stress", "false", "1000 forwards with a shrinking row count")
    _flag(ap, "search_best_perf", "false", "sweep cudagraph x fixed launch size")
    ap.add_argument("--synthetic", default="", choices=["", "centerpoint", "bevfusion"],
                    help="random-init backbone + synthetic frame instead of files")
    ap.add_argument("--voxels", type=int, default=120000, help="voxels of the synthetic frame")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--save_dir", default=".", help="where outputN_<name>.tensor files go")
    a = ap.parse_args(argv)
    for k in ("fp16", "int8", "sortmask", "blackwell", "auxiliary_stream", "cudagraph",
              "profiling", "verbose", "dds", "stress", "search_best_perf"):
        setattr(a, k, getattr(a, k) in ("true", "1", "yes"))
    return a


class Task:
    """What the reference calls InferenceTask: model path, inputs, switches."""

    def __init__(self, a):
        self.args = a
        self.tmp = None
        self.precision = engine.PRECISION_INT8 if a.int8 else engine.PRECISION_FP16
        if a.synthetic:
            grid = tuple(scenes.CENTERPOINT_GRID_ZYX)
            coords = scenes.make_coords(a.voxels, grid, a.seed)
            feats = scenes.make_point_features(coords, a.seed)
            model = models.scn_backbone(a.synthetic, seed=0, grid_zyx=grid,
                                        output_bound=max(300000, 3 * a.voxels))
            if a.int8:
                ranges = engine.calibrate(model, torch.from_numpy(feats).cuda(),
                                          torch.from_numpy(coords).cuda(), grid)
                model = models.quantize(model, ranges)
            self.tmp = tempfile.mkdtemp(prefix="infer_")
            self.onnx = os.path.join(self.tmp, a.synthetic + ".scn.onnx")
            onnx_writer.save(model, self.onnx)
            self.features, self.indices, self.grid = feats, coords, list(grid)
        else:
            missing = [k for k in ("onnx", "feature", "indice", "grid_size") if not getattr(a, k)]
            if missing:
                raise SystemExit("missing required option(s): " + ", ".join("--" + m for m in missing))
            if not os.path.exists(a.onnx):
                raise SystemExit("ONNX file does not exist: %s" % a.onnx)
            self.onnx = a.onnx
            self.features = np.array(tensor_file.load(a.feature))  # writable copies
            self.indices = np.array(tensor_file.load(a.indice))
            self.grid = [int(v) for v in a.grid_size.split(",")]
        if self.features.dtype != np.float16 or self.features.ndim != 2:
            raise SystemExit("features must be a float16 [N, C] tensor")
        if self.indices.dtype != np.int32 or self.indices.shape != (len(self.features), 4):
            raise SystemExit("indices must be an int32 [N, 4] tensor")
        if len(self.grid) != 3:
            raise SystemExit("grid_size needs three numbers")


def run_task(task, cudagraph, dds, fixed_points, profiling, stress=False, quiet=False):
    """One engine, one stream.  Returns the mean latency in ms when profiling."""
    a = task.args
    cabi.lib().spconvb_set_log_level(0 if a.verbose and not profiling else 1)
    dev = torch.device("cuda", torch.cuda.current_device())
    n = len(task.features)
    use_fixed = fixed_points if (cudagraph or dds) else 0
    flags = 0 if a.auxiliary_stream else engine.BUILD_SINGLE_STREAM
    eng = engine.Engine.from_onnx(task.onnx, task.precision, flags, use_fixed, dev)
    stream = torch.cuda.Stream(device=dev)  # "Please avoid using the default stream"
    f = torch.from_numpy(task.features).to(dev)
    c = torch.from_numpy(task.indices).to(dev)
    n_dev = torch.tensor([n], dtype=torch.int32, device=dev)
    latency = None
    with torch.cuda.stream(stream):
        def forward():
            if dds or cudagraph:
                eng.forward_dds(f, c, n_dev, task.grid, stream=stream)
            else:
                eng.forward(f, c, task.grid, stream=stream)

        forward()
        stream.synchronize()
        run = forward
        if cudagraph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                forward()
            run = g.replay
        if stress:
            rng = np.random.default_rng(0)
            real = n
            for i in range(1000):
                if real <= 0:
                    break
                if dds or cudagraph:
                    n_dev.fill_(real)
                    run()
                else:
                    eng.forward(f, c, task.grid, n=real, stream=stream)
                stream.synchronize()
                st = eng.status()
                if st[0]:
                    raise SystemExit("device status %s at stress iteration %d" % (st, i))
                if (i + 1) % 100 == 0:
                    print("Stress test: %d / 1000, num_inputs: %d" % (i + 1, real))
                real -= int(rng.integers(0, 200))
            print("Stress test done: %d forwards, last num_inputs: %d" % (i + 1, max(real, 0)))
        if profiling:
            for _ in range(5):
                run()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 20
            e0.record(stream)
            for _ in range(reps):
                run()
            e1.record(stream)
            e1.synchronize()
            latency = e0.elapsed_time(e1) / reps
            if not quiet:
                print("Latency: %.3f ms per forward (%d voxels, cudagraph %s, dds %s)" % (
                    latency, n, "yes" if cudagraph else "no", "yes" if dds else "no"))
                for line, ms in eng.profile(f, c, task.grid, reps=5, stream=stream):
                    print("  %8.2f us  %s" % (ms * 1000.0, line))
        stream.synchronize()
        st = eng.status()
        if st[0]:
            raise SystemExit("device status %s" % (st,))
        if not profiling and not stress and not quiet:
            for i in range(eng.num_outputs()):
                out = eng.output(i)
                name = os.path.join(a.save_dir, "output%d.tensor" % i)
                print("Save output[%d] %s %s to %s" % (i, list(out.shape), out.dtype, name))
                tensor_file.save(out.cpu().numpy(), name)
    eng.close()
    return latency


def search_best_perf(task):
    """infer.cpp:371-466 restated over the switches that exist here."""
    a = task.args
    n = len(task.features)
    print("Search the best performance configuration for the model: %s" % task.onnx)
    p2 = int(n * 0.2) // 256 * 256
    p3 = int(n * 0.6) // 256 * 256
    print("Proposed fixed launch points: %d, %d, %d" % (p2, p3, a.fixed_points))
    results = []
    for cudagraph in (True, False):
        for fixed in ((p2, p3, a.fixed_points) if cudagraph else (a.fixed_points,)):
            # a launch size below the real row count only makes sense when kernels stride
            lat = run_task(task, cudagraph, cudagraph, fixed, True, quiet=True)
            results.append((lat, cudagraph, fixed))
            print("  Cudagraph: %s, Fixed Launch Points: %d, Latency: %.3f ms" % (
                "yes" if cudagraph else "no", fixed, lat))
    results.sort()
    lat, cudagraph, fixed = results[0]
    print("\nBest configuration found: \n   Cudagraph: %s, Fixed Launch Points: %d, Latency: %.3f ms" % (
        "yes" if cudagraph else "no", fixed, lat))
    return results


def main(argv=None):
    a = parse_args(argv)
    cabi.lib()  # fails loudly if the CUDA extension was not built
    if not torch.cuda.is_available():
        raise SystemExit("infer needs a CUDA device")
    task = Task(a)
    if a.search_best_perf and a.profiling:
        print("Ignore the search_best_perf flag because --profiling is specified.")
        a.search_best_perf = False
    if (a.search_best_perf or a.profiling) and a.stress:
        print("Ignore the stress_test flag because --search_best_perf or --profiling is specified.")
        a.stress = False
    if a.search_best_perf:
        search_best_perf(task)
    else:
        run_task(task, a.cudagraph, a.dds, a.fixed_points, a.profiling, a.stress)
    return 0


if __name__ == "__main__":
    sys.exit(main())
