"""The reference's tensor file format, as written and read by its tooling and by
`spconv::Tensor::save/load`.

Layout (libraries/3DSparseConvolution/tool/tensor.py:24-69): three int32 words
(magic 0x33ff1101, number of dimensions, dtype code), then the dimensions as int32,
then the raw little-endian data.  dtype codes: 1 int32, 2 float16, 3 float32,
4 int64, 5 uint64, 6 uint32, 7 int8, 8 uint8.
"""
from __future__ import annotations

import numpy as np

MAGIC = 0x33FF1101
_CODE_OF = {"int32": 1, "float16": 2, "float32": 3, "int64": 4, "uint64": 5, "uint32": 6,
            "int8": 7, "uint8": 8}
_DTYPE_OF = {v: np.dtype(k) for k, v in _CODE_OF.items()}


def save(tensor, file) -> None:
    """Writes a numpy array (or anything numpy can convert, torch tensors included)."""
    if not isinstance(tensor, np.ndarray):
        if hasattr(tensor, "detach"):
            tensor = tensor.detach().cpu().numpy()
        else:
            tensor = np.array(tensor)
    name = str(tensor.dtype)
    if name not in _CODE_OF:
        raise RuntimeError("Unsupport dtype %s" % name)
    tensor = np.ascontiguousarray(tensor)
    with open(file, "wb") as f:
        f.write(np.array([MAGIC, tensor.ndim, _CODE_OF[name]], dtype=np.int32).tobytes())
        f.write(np.array(tensor.shape, dtype=np.int32).tobytes())
        f.write(tensor.tobytes())


def load(file, return_torch: bool = False):
    with open(file, "rb") as f:
        head = f.read(12)
        if len(head) != 12:
            raise RuntimeError("%s: not a tensor file (too short)" % file)
        magic, ndim, code = (int(v) for v in np.frombuffer(head, dtype=np.int32))
        if magic != MAGIC:
            raise RuntimeError("%s: not a tensor file (bad magic)" % file)
        if code not in _DTYPE_OF:
            raise RuntimeError("Can not find match dtype for index %d" % code)
        if ndim < 0 or ndim > 16:
            raise RuntimeError("%s: bad number of dimensions %d" % (file, ndim))
        dims = np.frombuffer(f.read(ndim * 4), dtype=np.int32)
        if dims.size != ndim or (dims < 0).any():
            raise RuntimeError("%s: bad dimensions" % file)
        dtype = _DTYPE_OF[code]
        count = int(np.prod(dims, dtype=np.int64)) if ndim else 1
        raw = f.read(count * dtype.itemsize)
        if len(raw) != count * dtype.itemsize:
            raise RuntimeError("%s: truncated data" % file)
        data = np.frombuffer(raw, dtype=dtype).reshape(tuple(int(d) for d in dims))
    if return_torch:
        import torch
        return torch.from_numpy(data.copy())
    return data
