"""Shared builders of seeded test problems (numpy side)."""
import numpy as np

from lidar_ai_solution_b200 import scenes


def kaiming(rng, cout, kvol, cin):
    return (rng.standard_normal((cout, kvol, cin)) * np.sqrt(2.0 / (kvol * cin))).astype(np.float32)


def int8_problem(n, c_in, c_out, grid=(41, 180, 180), seed=0, kvol=27):
    """Config-1 style int8 layer: features N(0,1) quantised per tensor from absmax,
    Kaiming weights quantised per output channel, bias N(0, 0.1)."""
    from oracle import oracle as orc
    rng = np.random.default_rng(seed)
    coords = scenes.make_coords(n, grid, seed)
    x = rng.standard_normal((n, c_in)).astype(np.float32)
    dr_in = float(np.abs(x).max())
    xq = orc.quantize_f16(x.astype(np.float16), dr_in)
    w = kaiming(rng, c_out, kvol, c_in)
    amax = np.abs(w).reshape(c_out, -1).max(1).astype(np.float32)
    wq = orc.quantize_weights(w, amax)
    scale = (np.float32(dr_in) / np.float32(127.0)) * (amax / np.float32(127.0))
    bias = (rng.standard_normal(c_out) * 0.1).astype(np.float32)
    return dict(coords=coords, grid=list(grid), x=x, xq=xq, dr_in=dr_in, w=w, wq=wq,
                scale=scale.astype(np.float32), bias=bias)
