"""Python front-end of the engine: the same calls a C++ user makes through
``spconv::load_engine_from_onnx`` / ``Engine::forward``, over the C ABI.

torch owns input memory and streams and gives zero-copy views of the engine's
output buffers; all computation happens inside ``libspconvb.so``.
"""
from __future__ import annotations

import ctypes as C
import os
import tempfile

import numpy as np
import torch

from . import cabi, engine_abi, onnx_writer
from .engine_abi import (BUILD_FORCE_SIMT, BUILD_KEEP_TENSORS, BUILD_NO_FUSION, BUILD_SINGLE_STREAM,  # noqa: F401
                         PRECISION_FP16, PRECISION_INT8)


class _DeviceArray:
    """Exposes a raw device pointer through ``__cuda_array_interface__``."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(int(s) for s in shape), "typestr": typestr,
                                         "data": (int(ptr), False), "version": 2}


def _view(ptr, shape, kind_or_typestr, device):
    typestr = {cabi.F16: "<f2", cabi.I8: "|i1"}.get(kind_or_typestr, kind_or_typestr)
    if int(np.prod(shape)) == 0:
        dt = {"<f2": torch.float16, "|i1": torch.int8, "<i4": torch.int32}[typestr]
        return torch.empty(tuple(shape), dtype=dt, device=device)
    return torch.as_tensor(_DeviceArray(ptr, shape, typestr), device=device)


def _stream_ptr(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


class Engine:
    def __init__(self, handle, device):
        self._h = handle
        self.device = device
        self._lib = cabi.lib()

    # -- construction -------------------------------------------------------
    @classmethod
    def from_onnx(cls, path, precision=PRECISION_FP16, flags=0, fixed_launch_points=0,
                  device=None):
        lib = cabi.lib()
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        err = C.c_int(0)
        with torch.cuda.device(device):
            h = lib.spconvb_engine_load_onnx(os.fsencode(path), precision, flags,
                                             fixed_launch_points, _stream_ptr(), C.byref(err))
        if not h:
            raise RuntimeError("load_engine_from_onnx(%s) failed: %s" % (
                path, lib.spconvb_error_string(err.value).decode()))
        return cls(h, device)

    @classmethod
    def from_model(cls, model: dict, precision=PRECISION_FP16, flags=0, device=None):
        """Serialises the model to an ONNX file and loads it (the file path is
        the interface the reference's users have)."""
        with tempfile.TemporaryDirectory() as d:
            path = os.path.join(d, "model.scn.onnx")
            onnx_writer.save(model, path)
            return cls.from_onnx(path, precision, flags, 0, device)

    def close(self):
        if self._h:
            self._lib.spconvb_engine_destroy(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    # -- execution ----------------------------------------------------------
    def prepare(self, grid, batch=1):
        with torch.cuda.device(self.device):
            cabi.check(self._lib.spconvb_engine_prepare(self._h, cabi.i3(grid), batch), "prepare")

    def forward(self, features, indices, grid, n=None, batch=1, stream=None):
        """features fp16 [rows, C], indices int32 [rows, 4] on the device.  ``n``
        rows are valid (default: all)."""
        assert features.dtype == torch.float16 and indices.dtype == torch.int32
        assert features.is_contiguous() and indices.is_contiguous()
        n = features.shape[0] if n is None else int(n)
        cabi.check(self._lib.spconvb_engine_forward(
            self._h, features.data_ptr(), n, indices.data_ptr(), cabi.i3(grid), batch,
            _stream_ptr(stream)), "forward")

    def forward_dds(self, features, indices, n_dev, grid, batch=1, stream=None):
        """Like forward, with the valid row count in device memory (int32/uint32 [1])."""
        cabi.check(self._lib.spconvb_engine_forward_dds(
            self._h, features.data_ptr(), indices.data_ptr(), features.shape[0], n_dev.data_ptr(),
            cabi.i3(grid), batch, _stream_ptr(stream)), "forward_dds")

    # -- results ------------------------------------------------------------
    def num_outputs(self):
        return self._lib.spconvb_engine_num_outputs(self._h)

    def output(self, i=0):
        """Zero-copy view of output ``i`` (valid after the stream has run)."""
        data = C.c_void_p()
        shape = (C.c_int64 * 8)()
        ndim, kind, dense = C.c_int32(), C.c_int32(), C.c_int32()
        cabi.check(self._lib.spconvb_engine_output(self._h, i, C.byref(data), shape,
                                                   C.byref(ndim), C.byref(kind), C.byref(dense)))
        layout, pshape, pnd, _ = self._output_layout(i)
        if layout > 1:  # NCHW32 / NHWzC: the view has the dimensions as they lie in memory
            return _view(data.value, pshape, kind.value, self.device)
        return _view(data.value, [shape[d] for d in range(ndim.value)], kind.value, self.device)

    def _output_layout(self, i):
        layout, nd, nbytes = C.c_int32(), C.c_int32(), C.c_size_t()
        pshape = (C.c_int64 * 8)()
        cabi.check(self._lib.spconvb_engine_output_layout(self._h, i, C.byref(layout), pshape,
                                                          C.byref(nd), C.byref(nbytes)))
        return layout.value, [pshape[d] for d in range(nd.value)], nd.value, nbytes.value

    def output_layout(self, i=0):
        """Name of the TensorLayout of dense output ``i`` ("NCHW", "NCHW32", "NHWzC"; "None"
        for a sparse output)."""
        return ["None", "NCHW", "NCHW32", "NHWzC"][self._output_layout(i)[0]]

    def output_ptr(self, i=0):
        data = C.c_void_p()
        shape = (C.c_int64 * 8)()
        ndim, kind, dense = C.c_int32(), C.c_int32(), C.c_int32()
        cabi.check(self._lib.spconvb_engine_output(self._h, i, C.byref(data), shape,
                                                   C.byref(ndim), C.byref(kind), C.byref(dense)))
        if dense.value:
            return data.value, self._output_layout(i)[3]
        nbytes = int(np.prod([shape[d] for d in range(ndim.value)])) * (1 if kind.value else 2)
        return data.value, nbytes

    def tensor_names(self):
        return [s for s in self._lib.spconvb_engine_tensor_names(self._h).decode().split("\n") if s]

    def tensor(self, name):
        """dict(features [cap, C] view, coords [cap, 4] view or None, n (host int), scale, kind)."""
        v = engine_abi.TensorView()
        cabi.check(self._lib.spconvb_engine_tensor(self._h, name.encode(), C.byref(v)),
                   "tensor(%s)" % name)
        torch.cuda.current_stream().synchronize()
        n = int(_view(v.n_ptr, [1], "<i4", self.device).item()) if v.n_ptr else 0
        feats = _view(v.features, [v.cap, v.channels], v.kind, self.device) if not v.dense else None
        coords = _view(v.coords, [v.cap, 4], "<i4", self.device) if v.coords else None
        return {"features": feats, "coords": coords, "n": n, "scale": float(v.scale),
                "kind": v.kind, "grid": list(v.grid), "cap": v.cap}

    def rules(self):
        """[(map view [kvol, cap], n_out, n_in)] for every rulebook (after a forward)."""
        out = []
        torch.cuda.current_stream().synchronize()
        for i in range(self._lib.spconvb_engine_num_rules(self._h)):
            m, no, ni = C.c_void_p(), C.c_void_p(), C.c_void_p()
            cap, kvol = C.c_uint32(), C.c_int32()
            cabi.check(self._lib.spconvb_engine_rule(self._h, i, C.byref(m), C.byref(cap),
                                                     C.byref(kvol), C.byref(no), C.byref(ni)))
            out.append((_view(m.value, [kvol.value, cap.value], "<i4", self.device),
                        int(_view(no.value, [1], "<i4", self.device).item()),
                        int(_view(ni.value, [1], "<i4", self.device).item())))
        return out

    def coordset_rows(self, i):
        """Rows of coordinate set ``i`` after the last forward (host int)."""
        p, cap = C.c_void_p(), C.c_uint32()
        cabi.check(self._lib.spconvb_engine_coordset(self._h, i, C.byref(p), C.byref(cap), None))
        torch.cuda.current_stream().synchronize()
        return int(_view(p.value, [1], "<i4", self.device).item())

    def profile(self, features, indices, grid, n=None, batch=1, reps=5, flush=None, stream=None):
        """Per-step device milliseconds of one forward (see spconvb_engine_profile).
        Returns [(describe line, ms)]."""
        n = features.shape[0] if n is None else int(n)
        ns = self._lib.spconvb_engine_num_steps(self._h)
        ms = (C.c_float * ns)()
        cabi.check(self._lib.spconvb_engine_profile(
            self._h, features.data_ptr(), n, indices.data_ptr(), cabi.i3(grid), batch,
            _stream_ptr(stream), ms, ns, reps, flush.data_ptr() if flush is not None else None,
            flush.numel() * flush.element_size() if flush is not None else 0), "profile")
        lines = [ln for ln in self.describe().split("\n") if ln]
        return list(zip(lines, [float(v) for v in ms]))

    def describe(self):
        return self._lib.spconvb_engine_describe(self._h).decode()

    def status(self, stream=None):
        out = (C.c_uint32 * 4)()
        cabi.check(self._lib.spconvb_engine_status(self._h, out, _stream_ptr(stream)), "status")
        return [int(v) for v in out]

    def last_launches(self):
        return int(self._lib.spconvb_engine_last_launches(self._h))

    # -- run-time precision control (the v1.0 interface's setters) -----------------
    def set_node_precision(self, key, compute_precision, output_precision, by_optype=False):
        """Precision of the node called ``key`` (or of every node of operator type ``key``);
        returns how many nodes changed.  Takes effect at the next ``reconfigure``."""
        n = self._lib.spconvb_engine_set_node_precision(self._h, key.encode(), int(by_optype),
                                                        compute_precision, output_precision)
        if n < 0:
            cabi.check(n, "set_node_precision")
        return n

    def set_int8_calibration(self, enable):
        """True (+ ``reconfigure``): run in fp16 and collect every tensor's absmax over the
        forwards that follow.  False: turn the maxima into the graph's dynamic ranges and
        make int8 the main precision (+ ``reconfigure`` to build that engine)."""
        cabi.check(self._lib.spconvb_engine_set_int8_calibration(self._h, int(bool(enable))),
                   "set_int8_calibration")

    def reconfigure(self, stream=None):
        with torch.cuda.device(self.device):
            cabi.check(self._lib.spconvb_engine_reconfigure(self._h, _stream_ptr(stream)),
                       "reconfigure")


def calibrate(model: dict, features, indices, grid) -> dict:
    """Plain absmax calibration on one frame: runs the model in fp16 on the GPU
    with every tensor kept and returns {tensor id: absmax}.  This is what the
    v1.0 interface's set_int8_calibration does in its next forward
    (CUDA-CenterPoint/3rdparty/libspconv/include/spconv/engine.hpp:83-85)."""
    from . import models
    eng = Engine.from_model(model, PRECISION_FP16, BUILD_KEEP_TENSORS | BUILD_NO_FUSION)
    eng.forward(features, indices, grid)
    torch.cuda.synchronize()
    st = eng.status()
    if st[0]:
        raise RuntimeError("calibration frame raised device status %s" % st)
    ranges = {}
    for tid in models.tensor_ids(model):
        if tid == model["inputs"][0][0]:
            ranges[tid] = float(features.float().abs().max().item())
            continue
        t = eng.tensor(tid)
        ranges[tid] = float(t["features"][: t["n"]].float().abs().max().item()) if t["n"] else 1.0
    eng.close()
    return ranges
