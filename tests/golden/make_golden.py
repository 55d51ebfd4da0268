"""Regenerates the golden fixtures from the reference checkout (run where the
reference tree is mounted; the test-suite itself only reads the outputs).

usage: python tests/golden/make_golden.py /path/to/Lidar_AI_Solution

Outputs (next to this script)
  fixture_coords.npz     the voxel coordinates of the reference's two sample
                         frames (libraries/3DSparseConvolution/workspace/
                         centerpoint/in_indices_zyx.torch.int32.tensor and
                         workspace/bevfusion/infer.{zyx,xyz}.coors), stored as
                         uint16 (z, y, x) columns, plus the first 40 rows of the
                         fp16 CenterPoint features for the tensor-file reader
  fixture_counts.json    per-stage active-voxel and rulebook-pair counts of those
                         frames through the CenterPoint / BEVFusion stage chain
                         (SubM 3x3x3; down k3 s2 pads (1,1,1),(1,1,1),(0,1,1);
                         then k(3,1,1) s(2,1,1) p0), computed by the CPU oracle
  sweep_points.npz       every 8th point of the raw fp16 sweep
                         workspace/ff9eff4389a740848f9a56ad749a4ae8.bin
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import oracle as orc  # noqa: E402

STAGES = [((3, 3, 3), (2, 2, 2), (1, 1, 1)), ((3, 3, 3), (2, 2, 2), (1, 1, 1)),
          ((3, 3, 3), (2, 2, 2), (0, 1, 1)), ((3, 1, 1), (2, 1, 1), (0, 0, 0))]


def load_tensor(path):
    """Reader for the reference's tensor container (tool/tensor.py:51-69)."""
    codes = {1: np.int32, 2: np.float16, 3: np.float32, 4: np.int64, 5: np.uint64,
             6: np.uint32, 7: np.int8, 8: np.uint8}
    raw = open(path, "rb").read()
    magic, ndim, code = np.frombuffer(raw[:12], np.int32)
    assert magic == 0x33FF1101
    dims = np.frombuffer(raw[12:12 + 4 * ndim], np.int32)
    return np.frombuffer(raw[12 + 4 * ndim:], codes[int(code)]).reshape(dims)


def chain(coords, grid):
    rows = []
    for k, s, p in STAGES:
        _, pairs = orc.subm_map(coords, grid)
        oc, _, dpairs, og, n_out = orc.down_map(coords, grid, k, s, p)
        rows.append({"grid": list(grid), "n": int(len(coords)), "subm_pairs": pairs,
                     "down_n": int(n_out), "down_pairs": dpairs, "down_grid": og})
        coords, grid = oc, og
    return rows


def main(ref):
    ws = os.path.join(ref, "libraries/3DSparseConvolution/workspace")
    cp = load_tensor(os.path.join(ws, "centerpoint/in_indices_zyx.torch.int32.tensor"))
    cpf = load_tensor(os.path.join(ws, "centerpoint/in_features.torch.fp16.tensor"))
    bz = load_tensor(os.path.join(ws, "bevfusion/infer.zyx.coors"))
    bx = load_tensor(os.path.join(ws, "bevfusion/infer.xyz.coors"))
    assert (cp[:, 0] == 0).all() and (bz[:, 0] == 0).all()
    assert (bx[:, 1:] == bz[:, :0:-1]).all()
    np.savez_compressed(os.path.join(HERE, "fixture_coords.npz"),
                        centerpoint_zyx=cp[:, 1:].astype(np.uint16),
                        bevfusion_zyx=bz[:, 1:].astype(np.uint16),
                        centerpoint_feat_head=cpf[:40])
    counts = {"centerpoint": chain(cp, [41, 1440, 1440]),
              "bevfusion": chain(bz, [41, 1440, 1440])}
    with open(os.path.join(HERE, "fixture_counts.json"), "w") as f:
        json.dump(counts, f, indent=1)
    pts = np.fromfile(os.path.join(ws, "ff9eff4389a740848f9a56ad749a4ae8.bin"), np.float16)
    np.savez_compressed(os.path.join(HERE, "sweep_points.npz"), points=pts.reshape(-1, 5)[::8])
    # a small tensor file in the reference's container format (tool/tensor.py:24-48),
    # for the reader tests: int32 header (magic, ndim, dtype code), int32 dims, raw data
    head = np.array([0x33FF1101, 2, 2, 40, 5], np.int32).tobytes()
    open(os.path.join(HERE, "sample.tensor"), "wb").write(head + cpf[:40].tobytes())


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
