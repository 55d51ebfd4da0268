"""ctypes binding of the C ABI declared in ``include/spconvb.h``.

The library is loaded from ``lidar_ai_solution_b200/lib/libspconvb.so`` (built
in-tree by ``python -m lidar_ai_solution_b200.build``).  There is no fallback:
if the shared object is missing, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# SPCONVB_LIB: path of another build of the same library (to compare two builds)
LIB_PATH = os.environ.get("SPCONVB_LIB") or os.path.join(_PKG, "lib", "libspconvb.so")

OK = 0
F16, I8 = 0, 1
ACT_NONE, ACT_RELU = 0, 1
ST_HASH_FULL, ST_DUPLICATE, ST_OVERFLOW, ST_TIMEOUT, ST_COORD_RANGE = 1, 2, 4, 8, 16
FLAG_PREZEROED = 1
E_SCRATCH_LIMIT = -8
STATIC_SCRATCH_BYTES = 4 << 20


class ConvParams(C.Structure):
    _fields_ = [
        ("compute", C.c_int32), ("cin", C.c_int32), ("cout", C.c_int32), ("kvol", C.c_int32),
        ("act", C.c_int32), ("out_kind", C.c_int32), ("inv_out_scale", C.c_float),
        ("res", C.c_void_p), ("res_kind", C.c_int32), ("res_scale", C.c_float),
        ("mid_kind", C.c_int32), ("mid_inv_scale", C.c_float), ("mid_scale", C.c_float),
        ("res_relu", C.c_int32), ("force_simt", C.c_int32), ("wait_test", C.c_int32),
        ("n_in_ptr", C.c_void_p), ("cap_in", C.c_uint32),
    ]


class VoxelParams(C.Structure):
    _fields_ = [
        ("range_min", C.c_float * 3), ("range_max", C.c_float * 3), ("voxel_size", C.c_float * 3),
        ("grid", C.c_int32 * 3), ("num_features", C.c_int32), ("points_kind", C.c_int32),
        ("max_points_per_voxel", C.c_int32), ("max_voxels", C.c_int32), ("order", C.c_int32),
    ]


# every symbol include/spconvb.h declares: name -> (restype, argtypes)
_I3 = C.POINTER(C.c_int32)
_VP = C.c_void_p
SYMBOLS = {
    "spconvb_version": (C.c_char_p, []),
    "spconvb_error_string": (C.c_char_p, [C.c_int]),
    "spconvb_hash_slots": (C.c_uint32, [C.c_uint32]),
    "spconvb_hash_build": (C.c_int, [_VP, _VP, C.c_uint32, C.c_uint32, _I3, C.c_int32, _VP,
                                     C.c_uint32, C.c_uint32, _VP, _VP]),
    "spconvb_subm_map": (C.c_int, [_VP, _VP, C.c_uint32, C.c_uint32, _I3, C.c_int32, _I3, _I3, _VP,
                                   C.c_uint32, _VP, _VP, _VP]),
    "spconvb_subm_map_ranked": (C.c_int, [_VP, _VP, C.c_uint32, C.c_uint32, _I3, C.c_int32, _I3, _I3,
                                          _VP, _VP, _VP, _VP]),
    "spconvb_inverse_map": (C.c_int, [_VP, _VP, C.c_uint32, C.c_uint32, _I3, C.c_int32, _I3, _I3, _I3,
                                      _I3, _VP, C.c_uint32, _VP, _VP, _VP]),
    "spconvb_out_extent": (C.c_int32, [C.c_int32] * 5),
    "spconvb_down_workspace_bytes": (C.c_size_t, [_I3, C.c_int32]),
    "spconvb_down_map": (C.c_int, [_VP, _VP, C.c_uint32, C.c_uint32, _I3, C.c_int32, _I3, _I3, _I3,
                                   _I3, _VP, C.c_uint32, _VP, _VP, _VP, C.c_uint32, _VP, _VP,
                                   C.c_uint32, C.c_uint32, _VP, _VP]),
    "spconvb_down_map_ranked": (C.c_int, [_VP, _VP, C.c_uint32, C.c_uint32, _I3, C.c_int32, _I3, _I3,
                                          _I3, _I3, _VP, _VP, _VP, _VP, C.c_uint32, _VP, _VP,
                                          C.c_uint32, C.c_uint32, _VP, _VP]),
    "spconvb_down_map_static": (C.c_int, [_VP, _VP, C.c_uint32, C.c_uint32, _I3, C.c_int32, _I3, _I3,
                                          _I3, _I3, _VP, C.c_uint32, _VP, _VP, C.c_uint32, _VP,
                                          _VP, C.c_uint32, C.c_uint32, _VP, _VP]),
    "spconvb_conv_packed_bytes": (C.c_size_t, [C.c_int32] * 4),
    "spconvb_conv_pack_weights": (C.c_int, [C.c_int32] * 4 + [_VP, _VP]),
    "spconvb_conv_supported": (C.c_int, [C.c_int32] * 3),
    "spconvb_conv_forward": (C.c_int, [C.POINTER(ConvParams), _VP, _VP, C.c_uint32, _VP,
                                       C.c_uint32, _VP, _VP, _VP, _VP, _VP, _VP, _VP]),
    "spconvb_add": (C.c_int, [_VP, C.c_int32, C.c_float, _VP, C.c_int32, C.c_float, C.c_int32,
                              _VP, C.c_uint32, C.c_int32, C.c_int32, C.c_float, _VP, _VP]),
    "spconvb_relu": (C.c_int, [_VP, C.c_int32, C.c_int32, _VP, C.c_uint32, _VP, _VP]),
    "spconvb_absmax": (C.c_int, [_VP, C.c_int32, C.c_int32, _VP, C.c_uint32, _VP, _VP]),
    "spconvb_convert": (C.c_int, [_VP, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float,
                                  _VP, C.c_uint32, _VP, _VP]),
    "spconvb_scatter_dense": (C.c_int, [_VP, C.c_int32, C.c_float, _VP, _VP, C.c_uint32,
                                        C.c_int32, C.c_int32, _I3, _I3, _VP, _VP]),
    "spconvb_scatter_dense_layout": (C.c_int, [_VP, C.c_int32, C.c_float, _VP, _VP, C.c_uint32,
                                               C.c_int32, C.c_int32, _I3, _I3, C.c_int32,
                                               C.c_int32, C.c_float, _VP, _VP]),
    "spconvb_dense_bytes": (C.c_size_t, [C.c_int32, C.c_int32, _I3, _I3, C.c_int32, C.c_int32]),
    "spconvb_voxelize_workspace_bytes": (C.c_size_t, [C.POINTER(VoxelParams), C.c_uint32]),
    "spconvb_voxelize": (C.c_int, [C.POINTER(VoxelParams), _VP, C.c_uint32, _VP, _VP, _VP, _VP,
                                   _VP, _VP]),
}

class CpHead(C.Structure):
    """spconvb_cp_head (include/spconvb_centerpoint.h)."""
    _fields_ = [("reg", C.c_void_p), ("height", C.c_void_p), ("dim", C.c_void_p),
                ("rot", C.c_void_p), ("vel", C.c_void_p), ("hm", C.c_void_p),
                ("num_classes", C.c_int32), ("label_offset", C.c_int32)]


class CpParams(C.Structure):
    """spconvb_cp_params (include/spconvb_centerpoint.h)."""
    _fields_ = [("H", C.c_int32), ("W", C.c_int32), ("out_size_factor", C.c_float),
                ("voxel_size", C.c_float * 2), ("pc_range", C.c_float * 2),
                ("score_threshold", C.c_float), ("post_center_range", C.c_float * 6),
                ("nms_iou_threshold", C.c_float), ("max_det", C.c_int32),
                ("nms_post_max", C.c_int32)]


SYMBOLS.update({
    "spconvb_cp_default_params": (None, [C.POINTER(CpParams)]),
    "spconvb_cp_workspace_bytes": (C.c_size_t, [C.POINTER(CpParams), C.c_int32]),
    "spconvb_cp_postprocess": (C.c_int, [C.POINTER(CpHead), C.c_int32, C.POINTER(CpParams), _VP,
                                         C.c_size_t, _VP, _VP, _VP]),
    "spconvb_cp_task_detections": (C.c_int, [C.POINTER(CpParams), C.c_int32, _VP, C.c_int32,
                                             C.POINTER(_VP), C.POINTER(_VP)]),
    "spconvb_cp_rotated_iou": (C.c_int, [_VP, _VP, C.c_int32, _VP, _VP]),
})

_LIB = None


def lib() -> C.CDLL:
    """The loaded library with argtypes set.  Raises if it was not built."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "%s is missing: run `python -m lidar_ai_solution_b200.build` "
                "(there is no CPU fallback)" % LIB_PATH)
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        from . import engine_abi  # engine-level symbols share the handle
        engine_abi.bind(handle)
        _LIB = handle
    return _LIB


def i3(v):
    return (C.c_int32 * 3)(*[int(x) for x in v])


def check(code: int, what: str = "spconvb call"):
    if code != OK:
        raise RuntimeError("%s failed: %s (%d)" % (what, lib().spconvb_error_string(code).decode(),
                                                   code))
