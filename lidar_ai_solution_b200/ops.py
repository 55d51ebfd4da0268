"""Thin torch-tensor wrappers over the kernel-level C ABI.

torch is used only to own device memory and streams; every function here ends
in exactly one ``spconvb_*`` call on the current CUDA stream.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import cabi
from .cabi import ACT_NONE, ACT_RELU, F16, I8  # noqa: F401


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def kind_of(t: torch.Tensor) -> int:
    return I8 if t.dtype == torch.int8 else F16


def new_status(device="cuda"):
    return torch.zeros(4, dtype=torch.int32, device=device)


def device_count(n: int, device="cuda") -> torch.Tensor:
    """A row count in device memory (what kernels read instead of a host value)."""
    return torch.tensor([n], dtype=torch.int32, device=device)


def hash_build(coords, n_ptr, grid, batch=1, status=None, launch_rows=0):
    cap = coords.shape[0]
    slots = cabi.lib().spconvb_hash_slots(cap)
    table = torch.empty(slots, dtype=torch.int64, device=coords.device)
    cabi.check(cabi.lib().spconvb_hash_build(_ptr(coords), _ptr(n_ptr), cap, launch_rows,
                                             cabi.i3(grid), batch, _ptr(table), slots, 0,
                                             _ptr(status), _stream()), "hash_build")
    return table


def subm_map(coords, n_ptr, grid, table, ksize=(3, 3, 3), dilation=(1, 1, 1), batch=1,
             status=None, launch_rows=0):
    cap = coords.shape[0]
    kvol = int(np.prod(ksize))
    m = torch.empty((kvol, cap), dtype=torch.int32, device=coords.device)
    cabi.check(cabi.lib().spconvb_subm_map(_ptr(coords), _ptr(n_ptr), cap, launch_rows,
                                           cabi.i3(grid), batch, cabi.i3(ksize),
                                           cabi.i3(dilation), _ptr(table), table.numel(), _ptr(m),
                                           _ptr(status), _stream()), "subm_map")
    return m


def out_grid(grid, ksize, stride, pad, dilation=(1, 1, 1)):
    return [int(cabi.lib().spconvb_out_extent(int(g), int(k), int(s), int(p), int(d)))
            for g, k, s, p, d in zip(grid, ksize, stride, pad, dilation)]


def down_map(coords, n_ptr, grid, table, ksize, stride, pad, dilation=(1, 1, 1), cap_out=None,
             batch=1, status=None, want_table=True, launch_rows=0, return_ws=False, in_ws=None):
    """Returns (out_coords, n_out_ptr, map, out_table, out_grid) and, with ``return_ws``,
    the workspace (bitmap + rank prefix of the outputs) as a sixth item.  ``table`` is not
    needed any more and may be None.  ``in_ws``: the workspace of the down_map call that made
    ``coords``; the map is then looked up by rank from the output side
    (spconvb_down_map_ranked), with the same result."""
    dev = coords.device
    cap_in = coords.shape[0]
    og = out_grid(grid, ksize, stride, pad, dilation)
    if cap_out is None:
        cap_out = max(1, min(cap_in * int(np.prod(ksize)), batch * int(np.prod(og))))
    kvol = int(np.prod(ksize))
    ws = torch.empty(cabi.lib().spconvb_down_workspace_bytes(cabi.i3(og), batch),
                     dtype=torch.uint8, device=dev)
    oc = torch.zeros((cap_out, 4), dtype=torch.int32, device=dev)
    n_out = torch.zeros(1, dtype=torch.int32, device=dev)
    m = torch.full((kvol, cap_out), -1, dtype=torch.int32, device=dev)
    slots = cabi.lib().spconvb_hash_slots(cap_out) if want_table else 0
    otab = torch.empty(slots, dtype=torch.int64, device=dev) if want_table else None
    if in_ws is not None:
        cabi.check(cabi.lib().spconvb_down_map_ranked(
            _ptr(coords), _ptr(n_ptr), cap_in, launch_rows, cabi.i3(grid), batch, cabi.i3(ksize),
            cabi.i3(stride), cabi.i3(pad), cabi.i3(dilation), _ptr(in_ws), _ptr(ws),
            _ptr(oc), _ptr(n_out), cap_out, _ptr(m), _ptr(otab), slots, 0, _ptr(status),
            _stream()), "down_map_ranked")
    else:
        cabi.check(cabi.lib().spconvb_down_map(
            _ptr(coords), _ptr(n_ptr), cap_in, launch_rows, cabi.i3(grid), batch, cabi.i3(ksize),
            cabi.i3(stride), cabi.i3(pad), cabi.i3(dilation), _ptr(table),
            table.numel() if table is not None else 0, _ptr(ws),
            _ptr(oc), _ptr(n_out), cap_out, _ptr(m), _ptr(otab), slots, 0, _ptr(status),
            _stream()), "down_map")
    if return_ws:
        return oc, n_out, m, otab, og, ws
    return oc, n_out, m, otab, og


def subm_map_ranked(coords, n_ptr, grid, ws, ksize=(3, 3, 3), dilation=(1, 1, 1), batch=1,
                    status=None, launch_rows=0):
    """SubM map of rows that came out of ``down_map`` (ranked in its workspace ``ws``)."""
    cap = coords.shape[0]
    kvol = int(np.prod(ksize))
    m = torch.empty((kvol, cap), dtype=torch.int32, device=coords.device)
    cabi.check(cabi.lib().spconvb_subm_map_ranked(_ptr(coords), _ptr(n_ptr), cap, launch_rows,
                                                  cabi.i3(grid), batch, cabi.i3(ksize),
                                                  cabi.i3(dilation), _ptr(ws), _ptr(m),
                                                  _ptr(status), _stream()), "subm_map_ranked")
    return m


def inverse_map(coords, n_ptr, grid, ws, cap_coarse, ksize, stride, pad, dilation=(1, 1, 1),
                batch=1, status=None, launch_rows=0):
    """Map of the inverse conv of a strided rulebook: ``coords`` are the rows that went INTO
    ``down_map`` (with ``return_ws=True``), ``ws`` its workspace, ``cap_coarse`` its cap_out."""
    cap = coords.shape[0]
    kvol = int(np.prod(ksize))
    m = torch.empty((kvol, cap), dtype=torch.int32, device=coords.device)
    cabi.check(cabi.lib().spconvb_inverse_map(_ptr(coords), _ptr(n_ptr), cap, launch_rows,
                                              cabi.i3(grid), batch, cabi.i3(ksize), cabi.i3(stride),
                                              cabi.i3(pad), cabi.i3(dilation), _ptr(ws), cap_coarse,
                                              _ptr(m), _ptr(status), _stream()), "inverse_map")
    return m


class ConvWeights:
    """Device copies of one layer's parameters in both kernel formats."""

    def __init__(self, w, compute, scale=None, bias=None, device="cuda"):
        # w: numpy [cout, kvol, cin] int8 (compute I8) or float16 (compute F16)
        w = np.ascontiguousarray(w)
        self.compute = compute
        self.cout, self.kvol, self.cin = w.shape
        assert w.dtype == (np.int8 if compute == I8 else np.float16)
        self.plain = torch.from_numpy(w.copy()).to(device)
        self.packed = None
        lib = cabi.lib()
        if lib.spconvb_conv_supported(compute, self.cin, self.cout):
            nbytes = lib.spconvb_conv_packed_bytes(compute, self.cin, self.cout, self.kvol)
            host = np.zeros(nbytes, np.uint8)
            cabi.check(lib.spconvb_conv_pack_weights(compute, self.cin, self.cout, self.kvol,
                                                     w.ctypes.data_as(C.c_void_p),
                                                     host.ctypes.data_as(C.c_void_p)), "pack")
            self.packed = torch.from_numpy(host).to(device)
        self.scale = None if scale is None else torch.from_numpy(
            np.ascontiguousarray(scale, np.float32)).to(device)
        self.bias = None if bias is None else torch.from_numpy(
            np.ascontiguousarray(bias, np.float32)).to(device)


def conv_forward(x, m, n_out_ptr, wts: ConvWeights, act=ACT_NONE, out_kind=F16,
                 inv_out_scale=1.0, res=None, res_scale=1.0, mid_kind=F16, mid_inv_scale=1.0,
                 mid_scale=1.0, res_relu=False, force_simt=False, status=None, launch_rows=0,
                 out=None, wait_test=0, n_in_ptr=None):
    """``n_in_ptr`` (device row count of ``x``) lets the tensor-core kernel prefetch the input
    rows into L2; results do not depend on it."""
    cap = m.shape[1]
    p = cabi.ConvParams()
    p.compute, p.cin, p.cout, p.kvol = wts.compute, wts.cin, wts.cout, wts.kvol
    p.act, p.out_kind, p.inv_out_scale = act, out_kind, inv_out_scale
    p.res = res.data_ptr() if res is not None else None
    p.res_kind = kind_of(res) if res is not None else F16
    p.res_scale, p.mid_kind = res_scale, mid_kind
    p.mid_inv_scale, p.mid_scale, p.res_relu = mid_inv_scale, mid_scale, int(res_relu)
    p.force_simt = int(force_simt)
    p.wait_test = int(wait_test)
    if n_in_ptr is not None:
        p.n_in_ptr, p.cap_in = n_in_ptr.data_ptr(), x.shape[0]
    if out is None:
        out = torch.empty((cap, wts.cout), dtype=torch.int8 if out_kind == I8 else torch.float16,
                          device=x.device)
    cabi.check(cabi.lib().spconvb_conv_forward(
        C.byref(p), _ptr(x), _ptr(m), cap, _ptr(n_out_ptr), launch_rows, _ptr(wts.plain),
        _ptr(wts.packed), _ptr(wts.scale), _ptr(wts.bias), _ptr(out), _ptr(status), _stream()),
        "conv_forward")
    return out


def add(a, a_scale, b, b_scale, n_ptr, relu, out_kind, inv_out_scale=1.0):
    rows, ch = a.shape
    out = torch.empty((rows, ch), dtype=torch.int8 if out_kind == I8 else torch.float16,
                      device=a.device)
    cabi.check(cabi.lib().spconvb_add(_ptr(a), kind_of(a), a_scale, _ptr(b), kind_of(b), b_scale,
                                      ch, _ptr(n_ptr), rows, int(relu), out_kind, inv_out_scale,
                                      _ptr(out), _stream()), "add")
    return out


def relu(x, n_ptr):
    out = torch.empty_like(x)
    cabi.check(cabi.lib().spconvb_relu(_ptr(x), kind_of(x), x.shape[1], _ptr(n_ptr), x.shape[0],
                                       _ptr(out), _stream()), "relu")
    return out


def convert(x, out_kind, cout_pad, scale_or_inv, n_ptr):
    rows, cin = x.shape
    out = torch.empty((rows, cout_pad), dtype=torch.int8 if out_kind == I8 else torch.float16,
                      device=x.device)
    cabi.check(cabi.lib().spconvb_convert(_ptr(x), kind_of(x), cin, out_kind, cout_pad,
                                          scale_or_inv, _ptr(n_ptr), rows, _ptr(out), _stream()),
               "convert")
    return out


def scatter_dense(feat, coords, n_ptr, grid, batch=1, in_scale=1.0, perm=None):
    ch = feat.shape[1]
    g = [grid[p] for p in perm] if perm is not None else list(grid)
    out = torch.empty((batch, ch, g[0], g[1], g[2]), dtype=torch.float16, device=feat.device)
    cabi.check(cabi.lib().spconvb_scatter_dense(
        _ptr(feat), kind_of(feat), in_scale, _ptr(coords), _ptr(n_ptr), feat.shape[0], ch, batch,
        cabi.i3(grid), cabi.i3(perm) if perm is not None else None, _ptr(out), _stream()),
        "scatter_dense")
    return out


LAYOUTS = {"NCHW": 1, "NCHW32": 2, "NHWzC": 3}


def scatter_dense_layout(feat, coords, n_ptr, grid, layout="NCHW", dynamic_range=0.0, batch=1,
                         in_scale=1.0, perm=None):
    """ScatterDense into ``layout``; int8 with scale ``dynamic_range / 127`` when the range is
    positive, else fp16.  Returns the tensor with the dimensions as they lie in memory."""
    ch = feat.shape[1]
    g = [grid[p] for p in perm] if perm is not None else list(grid)
    lay = LAYOUTS[layout]
    i8 = dynamic_range > 0
    if lay == 2:
        shape = (batch, (ch * g[0] + 31) // 32, g[1], g[2], 32)
    elif lay == 3:
        shape = (batch, g[1], g[2], g[0], ch)
    else:
        shape = (batch, ch, g[0], g[1], g[2])
    out = torch.empty(shape, dtype=torch.int8 if i8 else torch.float16, device=feat.device)
    lib = cabi.lib()
    pp = cabi.i3(perm) if perm is not None else None
    assert lib.spconvb_dense_bytes(ch, batch, cabi.i3(grid), pp, lay, 1 if i8 else 0) == \
        out.numel() * out.element_size()
    inv = float(np.float32(127.0) / np.float32(dynamic_range)) if i8 else 1.0
    cabi.check(lib.spconvb_scatter_dense_layout(
        _ptr(feat), kind_of(feat), in_scale, _ptr(coords), _ptr(n_ptr), feat.shape[0], ch, batch,
        cabi.i3(grid), pp, lay, 1 if i8 else 0, inv, _ptr(out), _stream()), "scatter_dense_layout")
    return out


def voxel_params(prange, vsize, grid_xyz, num_features=5, points_kind=0, max_pts=10,
                 max_voxels=160000, order=0):
    p = cabi.VoxelParams()
    for i in range(3):
        p.range_min[i], p.range_max[i] = prange[i], prange[3 + i]
        p.voxel_size[i], p.grid[i] = vsize[i], grid_xyz[i]
    p.num_features, p.points_kind = num_features, points_kind
    p.max_points_per_voxel, p.max_voxels, p.order = max_pts, max_voxels, order
    return p


def voxelize(points, params, status=None):
    """points: cuda tensor [n, F] float32/float16.  Returns (features, indices, n_ptr)."""
    n = points.shape[0]
    lib = cabi.lib()
    ws = torch.empty(max(256, lib.spconvb_voxelize_workspace_bytes(C.byref(params), max(n, 1))),
                     dtype=torch.uint8, device=points.device)
    feat = torch.zeros((params.max_voxels, params.num_features), dtype=torch.float16,
                       device=points.device)
    idx = torch.zeros((params.max_voxels, 4), dtype=torch.int32, device=points.device)
    n_ptr = torch.zeros(1, dtype=torch.int32, device=points.device)
    cabi.check(lib.spconvb_voxelize(C.byref(params), _ptr(points), n, _ptr(ws), _ptr(feat),
                                    _ptr(idx), _ptr(n_ptr), _ptr(status), _stream()), "voxelize")
    return feat, idx, n_ptr
