"""ctypes front-end of the CPU oracle (``oracle/spconv_oracle.c``, ``oracle/centerpoint_post_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, the smoke check and the
benchmark's ``cpu_baseline`` / ``--impl reference`` legs.  The shipped package
never imports this module.

Parity status: unpinned against the closed reference engine (no golden output
tensors exist); pinned against dense ``torch.nn.functional.conv3d`` and the
pair / voxel counts of the reference's input fixtures (see tests).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

ACT_NONE, ACT_RELU = 0, 1
KIND_F16, KIND_I8, KIND_F32 = 0, 1, 2


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` next to its source (gcc, OpenMP)."""
    so = os.path.join(_HERE, "liboracle.so")
    srcs = [os.path.join(_HERE, f) for f in ("spconv_oracle.c", "centerpoint_post_oracle.c")]
    if force or not os.path.exists(so) or \
            os.path.getmtime(so) < max(os.path.getmtime(f) for f in srcs):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return so


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        _LIB.orc_subm_map.restype = C.c_int64
        _LIB.orc_down_map.restype = C.c_int64
        _LIB.orc_rotated_iou.restype = C.c_float
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _i3(v):
    return (C.c_int * 3)(*[int(x) for x in v])


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int | None = None) -> int:
    """OpenMP threads for the calls that follow; default: every CPU this process may run on."""
    if n is None:
        n = len(os.sched_getaffinity(0))
    return int(lib().orc_set_num_threads(int(n)))


def out_grid(grid, ksize, stride, pad, dil):
    return [int(lib().orc_out_extent(int(g), int(k), int(s), int(p), int(d)))
            for g, k, s, p, d in zip(grid, ksize, stride, pad, dil)]


def count_duplicates(coords, grid) -> int:
    coords = np.ascontiguousarray(coords, np.int32)
    return int(lib().orc_count_duplicates(_p(coords), len(coords), _i3(grid)))


def subm_map(coords, grid, ksize=(3, 3, 3), dil=(1, 1, 1), cap=None):
    """Returns (map [KVOL, cap] int32, pairs)."""
    coords = np.ascontiguousarray(coords, np.int32)
    n = len(coords)
    cap = max(n, 1) if cap is None else cap
    kvol = int(np.prod(ksize))
    m = np.full((kvol, cap), -1, np.int32)
    pairs = lib().orc_subm_map(_p(coords), n, _i3(grid), _i3(ksize), _i3(dil), _p(m), cap)
    return m, int(pairs)


def down_map(coords, grid, ksize, stride, pad, dil=(1, 1, 1), cap=None):
    """Returns (out_coords [n_out,4], map [KVOL, cap], pairs, out_grid)."""
    coords = np.ascontiguousarray(coords, np.int32)
    n = len(coords)
    kvol = int(np.prod(ksize))
    if cap is None:
        cap = max(n * kvol, 1)
        cap = min(cap, max(1, int(np.prod(out_grid(grid, ksize, stride, pad, dil)))))
    oc = np.zeros((cap, 4), np.int32)
    m = np.full((kvol, cap), -1, np.int32)
    n_out = C.c_int(0)
    og = (C.c_int * 3)()
    pairs = lib().orc_down_map(_p(coords), n, _i3(grid), _i3(ksize), _i3(stride), _i3(pad),
                               _i3(dil), _p(oc), _p(m), cap, C.byref(n_out), og)
    return oc[: min(n_out.value, cap)], m, int(pairs), [int(x) for x in og], n_out.value


def conv_f32(x, m, n_out, w, bias=None, act=ACT_NONE):
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    cout, kvol, cin = w.shape[0], int(np.prod(w.shape[1:-1])), w.shape[-1]
    assert m.shape[0] == kvol and x.shape[1] == cin
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    out = np.empty((n_out, cout), np.float32)
    lib().orc_conv_f32(_p(x), _p(m), m.shape[1], n_out, kvol, cin, cout, _p(w), _p(b), act,
                       _p(out))
    return out


def quantize_weights(w, amax):
    w = np.ascontiguousarray(w, np.float32)
    amax = np.ascontiguousarray(amax, np.float32)
    q = np.empty(w.shape, np.int8)
    lib().orc_quantize_weights(_p(w), w.shape[0], int(np.prod(w.shape[1:])), _p(amax), _p(q))
    return q


def quantize_f16(x, dynamic_range):
    x = np.ascontiguousarray(x, np.float16)
    q = np.empty(x.shape, np.int8)
    inv = np.float32(127.0) / np.float32(dynamic_range)
    lib().orc_quantize_f16(_p(x), C.c_size_t(x.size), C.c_float(inv), _p(q))
    return q


def _out_array(n, cout, out_kind):
    return np.empty((n, cout), {KIND_F16: np.float16, KIND_I8: np.int8, KIND_F32: np.float32}[out_kind])


def conv_i8(xq, m, n_out, wq, scale, bias, act, out_kind, inv_out_scale=1.0):
    xq = np.ascontiguousarray(xq, np.int8)
    wq = np.ascontiguousarray(wq, np.int8)
    cout, kvol, cin = wq.shape[0], int(np.prod(wq.shape[1:-1])), wq.shape[-1]
    assert m.shape[0] == kvol and xq.shape[1] == cin
    scale = np.ascontiguousarray(scale, np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    out = _out_array(n_out, cout, out_kind)
    lib().orc_conv_i8(_p(xq), _p(m), m.shape[1], n_out, kvol, cin, cout, _p(wq), _p(scale),
                      _p(b), act, out_kind, C.c_float(inv_out_scale), _p(out))
    return out


def conv_f16(x, m, n_out, w, bias, act, out_kind, inv_out_scale=1.0):
    x = np.ascontiguousarray(x, np.float16)
    w = np.ascontiguousarray(w, np.float16)
    cout, kvol, cin = w.shape[0], int(np.prod(w.shape[1:-1])), w.shape[-1]
    assert m.shape[0] == kvol and x.shape[1] == cin
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    out = _out_array(n_out, cout, out_kind)
    lib().orc_conv_f16(_p(x), _p(m), m.shape[1], n_out, kvol, cin, cout, _p(w), _p(b), act,
                       out_kind, C.c_float(inv_out_scale), _p(out))
    return out


def _kind(a):
    return KIND_I8 if a.dtype == np.int8 else KIND_F16


def add(a, a_scale, b, b_scale, relu, out_kind, inv_out_scale=1.0):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    out = _out_array(a.shape[0], a.shape[1], out_kind)
    lib().orc_add(_p(a), _kind(a), C.c_float(a_scale), _p(b), _kind(b), C.c_float(b_scale),
                  C.c_size_t(a.size), int(relu), out_kind, C.c_float(inv_out_scale), _p(out))
    return out


def relu(x):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    lib().orc_relu(_p(x), _kind(x), C.c_size_t(x.size), _p(out))
    return out


def scatter_dense(feat, coords, grid, batch=1, in_scale=1.0, perm=None):
    feat = np.ascontiguousarray(feat)
    coords = np.ascontiguousarray(coords, np.int32)
    ch = feat.shape[1]
    g = [grid[p] for p in perm] if perm is not None else list(grid)
    out = np.empty((batch, ch, g[0], g[1], g[2]), np.float16)
    lib().orc_scatter_dense(_p(feat), _kind(feat), C.c_float(in_scale), _p(coords), len(coords),
                            ch, batch, _i3(grid), _i3(perm) if perm is not None else None,
                            _p(out))
    return out


def scatter_dense_i8(featq, coords, grid, batch=1, perm=None):
    """int8 rows scattered into a zero int8 [batch, C, g(p0), g(p1), g(p2)] tensor (rows outside
    the grid are dropped; coordinates are unique)."""
    featq = np.ascontiguousarray(featq, np.int8)
    coords = np.asarray(coords, np.int64)
    p = list(perm) if perm is not None else [0, 1, 2]
    g = [grid[a] for a in p]
    out = np.zeros((batch, featq.shape[1], g[0], g[1], g[2]), np.int8)
    sp = coords[:, 1:4][:, p]
    ok = (coords[:, 0] >= 0) & (coords[:, 0] < batch)
    for a in range(3):
        ok &= (sp[:, a] >= 0) & (sp[:, a] < g[a])
    b, s0, s1, s2 = coords[ok, 0], sp[ok, 0], sp[ok, 1], sp[ok, 2]
    out[b, :, s0, s1, s2] = featq[ok]
    return out


def dense_layout(dense, layout, channels):
    """Physical arrangement of a dense [N, C, D, H, W] tensor (or its [N, C*D, H, W] view) in
    one of the engine's TensorLayout values (engine.hpp:26): "NCHW" leaves it as it is,
    "NCHW32" is [N, ceil(C*D/32), H, W, 32] with zero padding, "NHWzC" is [N, H, W, D, C]."""
    if layout in ("NCHW", "", None):
        return dense
    n = dense.shape[0]
    h, w = dense.shape[-2], dense.shape[-1]
    merged = dense.reshape(n, -1, h, w)
    m = merged.shape[1]
    if layout == "NCHW32":
        mb = (m + 31) // 32
        pad = np.zeros((n, mb * 32, h, w), dense.dtype)
        pad[:, :m] = merged
        return np.ascontiguousarray(pad.reshape(n, mb, 32, h, w).transpose(0, 1, 3, 4, 2))
    if layout == "NHWzC":
        d = m // channels
        return np.ascontiguousarray(merged.reshape(n, channels, d, h, w).transpose(0, 3, 4, 2, 1))
    raise ValueError(layout)


def voxelize(points, range6, vsize, gridxyz, max_voxels=160000, max_pts=10, order=0):
    """points: [n, nfeat] float32 or float16.  Returns (features f16, coords i32, total)."""
    points = np.ascontiguousarray(points)
    kind = 1 if points.dtype == np.float16 else 0
    if kind == 0:
        points = points.astype(np.float32, copy=False)
    n, nfeat = points.shape
    feat = np.zeros((max_voxels, nfeat), np.float16)
    coords = np.zeros((max_voxels, 4), np.int32)
    r = (C.c_float * 6)(*[float(x) for x in range6])
    v = (C.c_float * 3)(*[float(x) for x in vsize])
    nv = lib().orc_voxelize(_p(points), kind, n, nfeat, r, v, _i3(gridxyz), max_voxels, max_pts,
                            order, _p(feat), _p(coords))
    m = min(nv, max_voxels)
    return feat[:m], coords[:m], int(nv)


# ---- CenterPoint head decode + NMS (oracle/centerpoint_post_oracle.c) -------------------
CP_DEFAULTS = dict(out_size_factor=8.0, voxel_size=(0.075, 0.075), pc_range=(-54.0, -54.0),
                   score_threshold=0.1, post_center_range=(-61.2, -61.2, -10.0, 61.2, 61.2, 10.0),
                   nms_iou_threshold=0.2, max_det=1000, nms_post_max=83)


def _f(vals):
    return (C.c_float * len(vals))(*[float(v) for v in vals])


def centerpoint_decode(head, params=None):
    """head: dict of fp16 arrays reg [2,H,W], height [1,H,W], dim [3,H,W], rot [2,H,W],
    vel [2,H,W], hm [C,H,W].  Returns (detections [n, 11] float32 ranked by score, cells)."""
    prm = dict(CP_DEFAULTS, **(params or {}))
    t = {k: np.ascontiguousarray(head[k], np.float16) for k in ("reg", "height", "dim", "rot",
                                                                 "vel", "hm")}
    c_hm, h, w = t["hm"].shape
    det = np.zeros((prm["max_det"], 11), np.float32)
    cells = np.zeros(prm["max_det"], np.int32)
    n = lib().orc_centerpoint_decode(
        h, w, c_hm, _p(t["reg"]), _p(t["height"]), _p(t["dim"]), _p(t["rot"]), _p(t["vel"]),
        _p(t["hm"]), _f(prm["post_center_range"]), C.c_float(prm["out_size_factor"]),
        _f(prm["voxel_size"]), _f(prm["pc_range"]), C.c_float(prm["score_threshold"]),
        int(prm["max_det"]), _p(det), _p(cells))
    return det[:n], cells[:n]


def centerpoint_nms(det, label_offset=0, params=None):
    """Greedy rotated NMS over ranked detections.  Returns (boxes [k, 11] as
    x y z w l h vx vy rt id score, kept indices, smallest |iou - threshold| evaluated)."""
    prm = dict(CP_DEFAULTS, **(params or {}))
    det = np.ascontiguousarray(det, np.float32)
    out = np.zeros((max(prm["nms_post_max"], 1), 11), np.float32)
    idx = np.zeros(max(prm["nms_post_max"], 1), np.int32)
    margin = C.c_float(0)
    k = lib().orc_centerpoint_nms(_p(det), len(det), C.c_float(prm["nms_iou_threshold"]),
                                  int(prm["nms_post_max"]), int(label_offset), _p(out), _p(idx),
                                  C.byref(margin))
    return out[:k], idx[:k], float(margin.value)


def rotated_iou(a, b):
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    return np.array([lib().orc_rotated_iou(_p(a[i]), _p(b[i])) for i in range(len(a))],
                    np.float32)

