"""Python binding with the interface of the reference's `pyscn` module
(libraries/3DSparseConvolution/src/pyscn.cpp:47-146): host arrays in, host arrays out.

    model = SCNModel("centerpoint.scn.PTQ.onnx", "int8")
    features, indices = model.forward(features_fp16, indices_int32, [41, 1440, 1440], stream)

`forward` copies the inputs to the device on `stream` (0 = the current torch stream),
runs the engine, copies output 0 back through pinned buffers and synchronises the stream,
like the reference.  One deviation: the reference wraps the returned indices as float16
(pyscn.cpp:114); here they are int32, what the engine produced.  For a dense output
(ScatterDense) the indices array is empty, shape (0, 4).
"""
from __future__ import annotations

import numpy as np
import torch

from . import cabi, engine as _engine


def set_verbose(enable: bool) -> None:
    """pyscn.cpp:145 `set_verbose`: log level Verb when enabled, Warn otherwise."""
    cabi.lib().spconvb_set_log_level(0 if enable else 1)


class SCNModel:
    def __init__(self, onnx: str, precision: str):
        prec = _engine.PRECISION_FP16 if precision == "fp16" else _engine.PRECISION_INT8
        try:
            self._engine = _engine.Engine.from_onnx(onnx, prec)
        except RuntimeError:
            self._engine = None  # the reference keeps an invalid instance and fails in forward
        self._feat_dev = self._idx_dev = None
        self._feat_pin = self._idx_pin = None
        self._out_pin = None

    def valid(self) -> bool:
        return self._engine is not None

    def _staging(self, rows: int, ch: int):
        dev = self._engine.device
        if self._feat_dev is None or self._feat_dev.shape[0] < rows or self._feat_dev.shape[1] != ch:
            cap = max(rows, 1)
            self._feat_dev = torch.empty((cap, ch), dtype=torch.float16, device=dev)
            self._idx_dev = torch.empty((cap, 4), dtype=torch.int32, device=dev)
            self._feat_pin = torch.empty((cap, ch), dtype=torch.float16).pin_memory()
            self._idx_pin = torch.empty((cap, 4), dtype=torch.int32).pin_memory()

    def forward(self, features, indices, grid_size, stream: int = 0):
        if not self.valid():
            raise BufferError("Invalid engine instance, please makesure your construct")
        features = np.ascontiguousarray(features)
        indices = np.ascontiguousarray(indices)
        if features.dtype != np.float16 or features.ndim != 2:
            raise ValueError("features must be float16 [N, C]")
        if indices.dtype != np.int32 or indices.shape != (features.shape[0], 4):
            raise ValueError("indices must be int32 [N, 4]")
        if len(grid_size) != 3:
            raise ValueError("grid_size must have 3 entries")
        eng = self._engine
        rows, ch = features.shape
        self._staging(rows, ch)
        st = torch.cuda.ExternalStream(stream, device=eng.device) if stream else \
            torch.cuda.current_stream(eng.device)
        with torch.cuda.device(eng.device), torch.cuda.stream(st):
            self._feat_pin[:rows].copy_(torch.from_numpy(features))
            self._idx_pin[:rows].copy_(torch.from_numpy(indices))
            self._feat_dev[:rows].copy_(self._feat_pin[:rows], non_blocking=True)
            self._idx_dev[:rows].copy_(self._idx_pin[:rows], non_blocking=True)
            eng.forward(self._feat_dev, self._idx_dev, list(grid_size), n=rows, stream=st)
            out = eng.output(0)
            if self._out_pin is None or self._out_pin.numel() < out.numel() or \
                    self._out_pin.dtype != out.dtype:
                self._out_pin = torch.empty(out.numel(), dtype=out.dtype).pin_memory()
            host = self._out_pin[:out.numel()].view(out.shape)
            host.copy_(out, non_blocking=True)
            st.synchronize()
        status = eng.status()
        if status[0]:
            raise RuntimeError("engine status %s" % (status,))
        return host.numpy().copy(), np.zeros((0, 4), np.int32)
