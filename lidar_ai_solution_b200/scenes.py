"""Seeded synthetic lidar scenes.

They stand in for nuScenes 10-sweep frames, whose voxel statistics the
reference logs in ``libraries/3DSparseConvolution/workspace/perf-int8.log``
(10.8 k - 135 k active voxels per frame, mean 82.5 k).  The spatial law is the
one the benchmark configurations state: 70 % of the voxels on a ground band
z in [2, 6] with radial density proportional to 1/r about the grid centre,
30 % inside random 8x4x4-voxel object boxes (50 boxes per 20 000 voxels).
"""
from __future__ import annotations

import numpy as np

CENTERPOINT_GRID_ZYX = (41, 1440, 1440)
CENTERPOINT_RANGE = (-54.0, -54.0, -5.0, 54.0, 54.0, 3.0)  # x0,y0,z0,x1,y1,z1
CENTERPOINT_VOXEL = (0.075, 0.075, 0.2)                     # vx,vy,vz


def _unique_keep_order(keys: np.ndarray) -> np.ndarray:
    _, first = np.unique(keys, return_index=True)
    return np.sort(first)


def make_coords(n: int, grid_zyx=CENTERPOINT_GRID_ZYX, seed: int = 0) -> np.ndarray:
    """``n`` unique voxel coordinates, int32 ``[n, 4] = (0, z, y, x)``, in random row order."""
    gz, gy, gx = (int(v) for v in grid_zyx)
    rng = np.random.default_rng(seed)
    if n <= 0:
        return np.zeros((0, 4), np.int32)
    cells = gz * gy * gx
    if n > cells:
        raise ValueError("more voxels than grid cells")
    if n > cells // 8:
        # too dense for the lidar law (tiny test grids): uniform without replacement
        keys = rng.permutation(cells)[:n].astype(np.int64)
        out = np.zeros((n, 4), np.int32)
        out[:, 3] = keys % gx
        out[:, 2] = (keys // gx) % gy
        out[:, 1] = keys // (gx * gy)
        return out

    n_boxes = max(1, int(round(50 * n / 20000)))
    bz, by, bx = min(4, gz), min(4, gy), min(8, gx)
    oz = rng.integers(0, gz - bz + 1, n_boxes)
    oy = rng.integers(0, gy - by + 1, n_boxes)
    ox = rng.integers(0, gx - bx + 1, n_boxes)

    want_box = int(round(0.3 * n))
    keys = np.zeros(0, np.int64)
    # object boxes: uniform inside a random box, duplicates rejected
    for _ in range(64):
        m = max(1024, 2 * want_box)
        b = rng.integers(0, n_boxes, m)
        z = oz[b] + rng.integers(0, bz, m)
        y = oy[b] + rng.integers(0, by, m)
        x = ox[b] + rng.integers(0, bx, m)
        keys = np.concatenate([keys, (z.astype(np.int64) * gy + y) * gx + x])
        keys = keys[_unique_keep_order(keys)]
        if len(keys) >= want_box:
            break
    # boxes overlap, so they may not hold 30 %; the ground band takes the rest
    keys = keys[: min(want_box, int(0.9 * len(keys)) if len(keys) < want_box else want_box)]

    z_lo, z_hi = min(2, gz - 1), min(6, gz - 1)
    radius = 0.5 * min(gy, gx)
    for _ in range(256):
        need = n - len(keys)
        if need <= 0:
            break
        m = max(1024, 2 * need)
        r = rng.random(m) * radius          # uniform r  <=>  areal density ~ 1/r
        t = rng.random(m) * (2.0 * np.pi)
        y = np.floor(gy / 2.0 + r * np.sin(t)).astype(np.int64)
        x = np.floor(gx / 2.0 + r * np.cos(t)).astype(np.int64)
        z = rng.integers(z_lo, z_hi + 1, m).astype(np.int64)
        ok = (y >= 0) & (y < gy) & (x >= 0) & (x < gx)
        keys = np.concatenate([keys, ((z * gy + y) * gx + x)[ok]])
        keys = keys[_unique_keep_order(keys)]
    keys = keys[:n]
    if len(keys) != n:
        raise RuntimeError("scene generator could not place all voxels")
    keys = keys[rng.permutation(n)]
    out = np.zeros((n, 4), np.int32)
    out[:, 3] = keys % gx
    out[:, 2] = (keys // gx) % gy
    out[:, 1] = keys // (gx * gy)
    return out


def make_point_features(coords_zyx: np.ndarray, seed: int = 0, voxel=CENTERPOINT_VOXEL,
                        prange=CENTERPOINT_RANGE) -> np.ndarray:
    """5 features per voxel as the CenterPoint voxelizer emits them: the mean
    x, y, z (metres) of the points inside, intensity U[0,1], time in {0,0.05..0.5}."""
    rng = np.random.default_rng(seed + 7919)
    n = len(coords_zyx)
    vx, vy, vz = voxel
    jit = rng.random((n, 3)) - 0.5
    f = np.empty((n, 5), np.float32)
    f[:, 0] = prange[0] + (coords_zyx[:, 3] + 0.5 + jit[:, 0]) * vx
    f[:, 1] = prange[1] + (coords_zyx[:, 2] + 0.5 + jit[:, 1]) * vy
    f[:, 2] = prange[2] + (coords_zyx[:, 1] + 0.5 + jit[:, 2]) * vz
    f[:, 3] = rng.random(n)
    f[:, 4] = rng.integers(0, 11, n) * 0.05
    return f.astype(np.float16)


def make_points(n_points: int, seed: int = 0, prange=CENTERPOINT_RANGE) -> np.ndarray:
    """A raw sweep for the voxelizer: fp32 ``[n, 5]`` (x, y, z, intensity, time).
    About 10 % of the points fall outside the range, as in the reference's
    sample sweep; points cluster so that some voxels hold more than 10."""
    rng = np.random.default_rng(seed + 104729)
    r = rng.random(n_points) ** 2 * 60.0
    t = rng.random(n_points) * 2 * np.pi
    p = np.empty((n_points, 5), np.float32)
    p[:, 0] = r * np.cos(t)
    p[:, 1] = r * np.sin(t)
    p[:, 2] = rng.normal(-1.5, 1.2, n_points)
    p[:, 3] = rng.random(n_points)
    p[:, 4] = rng.integers(0, 11, n_points) * 0.05
    return p


def make_centerpoint_heads(seed=0, H=180, W=180, mean_logit=-6.0, num_classes=(1, 2, 2, 1, 2, 2),
                           objects=60):
    """Synthetic outputs of the CenterPoint RPN + heads for one frame: per task a dict of fp16
    arrays ``reg [2,H,W] height [1,H,W] dim [3,H,W] rot [2,H,W] vel [2,H,W] hm [C,H,W]``.
    Heat maps are background noise around ``mean_logit`` plus ``objects`` Gaussian blobs per
    task, so that neighbouring cells propose overlapping boxes as a trained head does."""
    rng = np.random.default_rng(seed)
    yy, xx = np.mgrid[0:H, 0:W].astype(np.float32)
    heads = []
    for classes in num_classes:
        hm = rng.normal(mean_logit, 1.2, (classes, H, W)).astype(np.float32)
        for _ in range(objects):
            c = rng.integers(0, classes)
            cy, cx = rng.uniform(0, H), rng.uniform(0, W)
            hm[c] += rng.uniform(3.0, 9.0) * np.exp(-((yy - cy) ** 2 + (xx - cx) ** 2) / 3.0)
        head = {
            "hm": hm,
            "reg": rng.uniform(0.0, 1.0, (2, H, W)),
            "height": rng.normal(-1.0, 1.0, (1, H, W)),
            "dim": rng.normal(0.6, 0.35, (3, H, W)),
            "rot": rng.normal(0.0, 1.0, (2, H, W)),
            "vel": rng.normal(0.0, 2.0, (2, H, W)),
        }
        heads.append({k: np.ascontiguousarray(v, np.float16) for k, v in head.items()})
    return heads

