"""Engine-level part of the C ABI (graph builder, engine, tensors); see include/spconvb.h."""
from __future__ import annotations

import ctypes as C

_VP = C.c_void_p
_I32P = C.POINTER(C.c_int32)
_I64P = C.POINTER(C.c_int64)
_F32P = C.POINTER(C.c_float)
_U16P = C.POINTER(C.c_uint16)
_CP = C.c_char_p

PRECISION_FP16, PRECISION_INT8 = 1, 2
BUILD_KEEP_TENSORS, BUILD_NO_FUSION, BUILD_FORCE_SIMT, BUILD_SINGLE_STREAM = 1, 2, 4, 8


class TensorView(C.Structure):
    _fields_ = [("features", C.c_void_p), ("kind", C.c_int32), ("channels", C.c_int32),
                ("scale", C.c_float), ("coords", C.c_void_p), ("n_ptr", C.c_void_p),
                ("cap", C.c_uint32), ("grid", C.c_int32 * 3), ("dense", C.c_int32)]


LOG_FN = C.CFUNCTYPE(None, C.c_int32, C.c_char_p)

SYMBOLS = {
    "spconvb_builder_create": (_VP, []),
    "spconvb_builder_destroy": (None, [_VP]),
    "spconvb_builder_input": (C.c_int, [_VP, _CP]),
    "spconvb_builder_sparse_conv": (C.c_int, [
        _VP, _CP, C.c_int, _VP, _I32P, _VP, C.c_int32, _VP, C.c_int32, _CP, _I32P, _I32P, _I32P,
        _I32P, C.c_float, C.c_int32, C.c_uint32, C.c_uint32, _CP, C.c_int32, C.c_int32, _CP,
        C.c_int32]),
    "spconvb_builder_add": (C.c_int, [_VP, _CP, C.c_int, C.c_int, C.c_float, C.c_float, _CP,
                                      C.c_int32, C.c_int32, C.c_uint32]),
    "spconvb_builder_relu": (C.c_int, [_VP, _CP, C.c_int, _CP]),
    "spconvb_builder_dense": (C.c_int, [_VP, _CP, C.c_int, _CP, _CP, _I32P, C.c_int32, _I32P,
                                        C.c_int32, C.c_int32, C.c_float, C.c_uint32]),
    "spconvb_builder_reshape": (C.c_int, [_VP, _CP, C.c_int, _I64P, C.c_int32, _CP]),
    "spconvb_builder_transpose": (C.c_int, [_VP, _CP, C.c_int, _I64P, C.c_int32, _CP]),
    "spconvb_builder_output": (C.c_int, [_VP, C.c_int]),
    "spconvb_builder_build": (_VP, [_VP, C.c_int32, C.c_uint32, _VP, C.POINTER(C.c_int)]),
    "spconvb_engine_load_onnx": (_VP, [_CP, C.c_int32, C.c_uint32, C.c_uint32, _VP,
                                       C.POINTER(C.c_int)]),
    "spconvb_onnx_inspect": (C.c_int, [_CP, _CP, C.c_size_t]),
    "spconvb_engine_destroy": (None, [_VP]),
    "spconvb_engine_forward": (C.c_int, [_VP, _VP, C.c_uint32, _VP, _I32P, C.c_int32, _VP]),
    "spconvb_engine_forward_dds": (C.c_int, [_VP, _VP, _VP, C.c_uint32, _VP, _I32P, C.c_int32,
                                             _VP]),
    "spconvb_engine_prepare": (C.c_int, [_VP, _I32P, C.c_int32]),
    "spconvb_engine_num_outputs": (C.c_int, [_VP]),
    "spconvb_engine_output": (C.c_int, [_VP, C.c_int, C.POINTER(_VP), _I64P, _I32P, _I32P, _I32P]),
    "spconvb_engine_output_layout": (C.c_int, [_VP, C.c_int, _I32P, _I64P, _I32P,
                                               C.POINTER(C.c_size_t)]),
    "spconvb_engine_output_rows": (C.c_int, [_VP, C.c_int, C.POINTER(_VP), C.POINTER(_VP),
                                             C.POINTER(C.c_uint32), _I32P, _I32P]),
    "spconvb_engine_tensor": (C.c_int, [_VP, _CP, C.POINTER(TensorView)]),
    "spconvb_engine_tensor_names": (_CP, [_VP]),
    "spconvb_engine_describe": (_CP, [_VP]),
    "spconvb_engine_num_steps": (C.c_int, [_VP]),
    "spconvb_engine_profile": (C.c_int, [_VP, _VP, C.c_uint32, _VP, _I32P, C.c_int32, _VP, _F32P,
                                         C.c_int32, C.c_int32, _VP, C.c_size_t]),
    "spconvb_engine_coordset": (C.c_int, [_VP, C.c_int, C.POINTER(_VP), C.POINTER(C.c_uint32),
                                          _I32P]),
    "spconvb_engine_num_rules": (C.c_int, [_VP]),
    "spconvb_engine_rule": (C.c_int, [_VP, C.c_int, C.POINTER(_VP), C.POINTER(C.c_uint32), _I32P,
                                      C.POINTER(_VP), C.POINTER(_VP)]),
    "spconvb_read_device": (C.c_int, [_VP, _VP, C.c_size_t, _VP]),
    "spconvb_copy_async": (C.c_int, [_VP, _VP, C.c_size_t, C.c_int32, _VP]),
    "spconvb_engine_status": (C.c_int, [_VP, C.POINTER(C.c_uint32), _VP]),
    "spconvb_engine_last_launches": (C.c_int, [_VP]),
    "spconvb_engine_set_node_precision": (C.c_int, [_VP, C.c_char_p, C.c_int32, C.c_int32,
                                                    C.c_int32]),
    "spconvb_engine_set_int8_calibration": (C.c_int, [_VP, C.c_int32]),
    "spconvb_engine_reconfigure": (C.c_int, [_VP, _VP]),
    "spconvb_set_log_level": (None, [C.c_int32]),
    "spconvb_set_log_callback": (None, [LOG_FN]),
}


def bind(handle):
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(handle, name)
        fn.restype = res
        fn.argtypes = args
