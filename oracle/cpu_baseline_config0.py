"""CPU baseline of benchmark configuration 0, timed two ways.  Test infrastructure, like the
rest of oracle/: nothing in the product path imports it.

Configuration 0: one SubMConv3d 3x3x3, Cin = Cout = 16, fp32, on 20 000 unique active voxels in
a 41x180x180 (z, y, x) grid (scenes.make_coords), features N(0, 1), Kaiming-normal weights,
zero bias; seeds 0..4, best of 5 after one warm-up, all host cores.

  (i)  the C/OpenMP oracle: rulebook (orc_subm_map) + convolution (orc_conv_f32);
  (ii) torch on the CPU, the per-offset gather -> GEMM -> scatter-add that the PyTorch sparse
       convolution packages run (index_select + mm + index_add_ per kernel offset, fp32), on
       the rulebook of (i).

    python oracle/cpu_baseline_config0.py

prints one JSON line with both times, the pair count, the thread counts and the largest
difference between the two results.
"""
from __future__ import annotations

import json
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from lidar_ai_solution_b200 import scenes  # noqa: E402
from oracle import oracle as orc  # noqa: E402

GRID = (41, 180, 180)
N, C = 20000, 16


def problem(seed):
    rng = np.random.default_rng(seed)
    coords = scenes.make_coords(N, GRID, seed)
    x = rng.standard_normal((N, C)).astype(np.float32)
    w = (rng.standard_normal((C, 27, C)) * np.sqrt(2.0 / (27 * C))).astype(np.float32)
    return coords, x, w


def run_oracle(coords, x, w):
    m, pairs = orc.subm_map(coords, GRID)
    return orc.conv_f32(x, m, N, w), m, pairs


def run_torch(torch, x, w, m):
    xt, out = torch.from_numpy(x), torch.zeros((N, C), dtype=torch.float32)
    for k in range(27):
        rows = torch.from_numpy(np.nonzero(m[k, :N] >= 0)[0])
        if rows.numel() == 0:
            continue
        src = torch.from_numpy(m[k, :N][rows.numpy()].astype(np.int64))
        out.index_add_(0, rows, xt.index_select(0, src) @ torch.from_numpy(w[:, k, :]).t())
    return out.numpy()


def measure(seeds=5):
    """Both timings as a dict (milliseconds, best of ``seeds`` seeds after a warm-up each)."""
    import torch
    orc.set_num_threads()
    torch.set_num_threads(len(os.sched_getaffinity(0)))
    best_c = best_t = best_map = float("inf")
    err = 0.0
    pairs = 0
    for seed in range(seeds):
        coords, x, w = problem(seed)
        run_oracle(coords, x, w)  # warm-up
        t0 = time.perf_counter()
        m, pairs = orc.subm_map(coords, GRID)
        t1 = time.perf_counter()
        y = orc.conv_f32(x, m, N, w)
        t2 = time.perf_counter()
        best_map, best_c = min(best_map, t1 - t0), min(best_c, t2 - t0)
        run_torch(torch, x, w, m)  # warm-up
        t0 = time.perf_counter()
        yt = run_torch(torch, x, w, m)
        best_t = min(best_t, time.perf_counter() - t0)
        err = max(err, float(np.abs(y - yt).max()))
    return {
        "config": "0: SubMConv3d 3x3x3, 16->16, fp32, 20000 voxels, 41x180x180",
        "pairs_last_seed": pairs,
        "oracle_ms": 1e3 * best_c, "oracle_rulebook_ms": 1e3 * best_map,
        "oracle_threads": orc.num_threads(),
        "torch_cpu_conv_ms": 1e3 * best_t, "torch_threads": torch.get_num_threads(),
        "host_cpus": os.cpu_count(), "max_abs_difference": err}


def main():
    print(json.dumps(measure()))


if __name__ == "__main__":
    main()
