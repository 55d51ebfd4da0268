"""Engine-level part of the C ABI (graph builder, engine, tensors); see include/spconvb.h."""
from __future__ import annotations

SYMBOLS = {}


def bind(handle):
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(handle, name)
        fn.restype = res
        fn.argtypes = args
