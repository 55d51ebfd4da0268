"""Writes the custom sparse-convolution ONNX files with nothing but ``struct``.

The schema is the one the reference's exporters produce and its loader reads
(libraries/3DSparseConvolution/src/onnx-parser.cpp:130-215): nodes
``SparseConvolution`` (inputs x, weight, bias; fp16 raw initialisers),
``Add``, ``Relu``, ``ScatterDense``, ``Reshape``, ``Transpose`` with the
attributes listed there; the graph input is named "0" and tensors carry
decimal ids (CUDA-CenterPoint/qat/onnx_export/exptool.py:300-372).

Only the protobuf wire format is needed: varints, 32-bit floats and
length-delimited fields.
"""
from __future__ import annotations

import struct

import numpy as np

FLOAT16 = 10
_ATTR_FLOAT, _ATTR_INT, _ATTR_STRING, _ATTR_FLOATS, _ATTR_INTS = 1, 2, 3, 6, 7


def _varint(v: int) -> bytes:
    if v < 0:
        v += 1 << 64
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(field: int, wire: int) -> bytes:
    return _varint((field << 3) | wire)


def _ld(field: int, payload: bytes) -> bytes:
    return _key(field, 2) + _varint(len(payload)) + payload


def _vi(field: int, v: int) -> bytes:
    return _key(field, 0) + _varint(int(v))


def _attribute(name: str, value) -> bytes:
    body = _ld(1, name.encode())
    if isinstance(value, bool):
        value = int(value)
    if isinstance(value, float):
        body += _key(2, 5) + struct.pack("<f", value) + _vi(20, _ATTR_FLOAT)
    elif isinstance(value, (int, np.integer)):
        body += _vi(3, int(value)) + _vi(20, _ATTR_INT)
    elif isinstance(value, str):
        body += _ld(4, value.encode()) + _vi(20, _ATTR_STRING)
    elif len(value) and isinstance(value[0], (float, np.floating)):
        body += _ld(7, b"".join(struct.pack("<f", float(v)) for v in value)) + _vi(20, _ATTR_FLOATS)
    else:
        body += _ld(8, b"".join(_varint(int(v)) for v in value)) + _vi(20, _ATTR_INTS)
    return body


def _node(op: str, inputs, outputs, name: str, attrs: dict) -> bytes:
    body = b"".join(_ld(1, i.encode()) for i in inputs)
    body += b"".join(_ld(2, o.encode()) for o in outputs)
    body += _ld(3, name.encode()) + _ld(4, op.encode())
    for k, v in attrs.items():
        body += _ld(5, _attribute(k, v))
    return body


def _tensor_fp16(name: str, array: np.ndarray) -> bytes:
    a = np.ascontiguousarray(array, np.float16)
    body = _ld(1, b"".join(_varint(int(d)) for d in a.shape))  # packed dims
    body += _vi(2, FLOAT16) + _ld(8, name.encode()) + _ld(9, a.tobytes())
    return body


def _value_info(name: str, shape) -> bytes:
    dims = b"".join(_ld(1, _vi(1, int(d))) for d in shape)
    tensor_type = _vi(1, FLOAT16) + _ld(2, dims)
    return _ld(1, name.encode()) + _ld(2, _ld(1, tensor_type))


def serialize(model: dict) -> bytes:
    """``model``: {"inputs": [(name, shape)], "outputs": [(name, shape)], "nodes": [node dicts]}
    with node dicts as produced by ``models.py``."""
    nodes, inits = [], []
    n_conv = 0
    for nd in model["nodes"]:
        op = nd["op"]
        if op == "conv":
            wname, bname = "spconv%d.weight" % n_conv, "spconv%d.bias" % n_conv
            n_conv += 1
            inits.append(_tensor_fp16(wname, nd["weight"]))
            inits.append(_tensor_fp16(bname, nd["bias"]))
            attrs = {
                "ndim": 3, "in_channels": int(nd["weight"].shape[-1]),
                "out_channels": int(nd["weight"].shape[0]),
                "kernel_size": list(nd["kernel_size"]), "output_bound": int(nd["output_bound"]),
                "stride": list(nd["stride"]), "dilation": list(nd["dilation"]),
                "padding": list(nd["padding"]), "transposed": 0,
                "inverse": int(nd.get("inverse", 0)),
                "subm": int(nd["subm"]), "rulebook": nd.get("rulebook", ""),
                "activation": nd["activation"],
            }
            if "input_dynamic_range" in nd:
                attrs["input_dynamic_range"] = float(nd["input_dynamic_range"])
                attrs["weight_dynamic_ranges"] = [float(v) for v in nd["weight_dynamic_ranges"]]
                attrs["precision"] = nd["precision"]
                attrs["output_precision"] = nd["output_precision"]
            nodes.append(_node("SparseConvolution", [nd["x"], wname, bname], [nd["out"]],
                               nd["name"], attrs))
        elif op == "add":
            attrs = {}
            if "input0_dynamic_range" in nd:
                attrs = {"input0_dynamic_range": float(nd["input0_dynamic_range"]),
                         "input1_dynamic_range": float(nd["input1_dynamic_range"]),
                         "precision": nd["precision"], "output_precision": nd["output_precision"]}
            nodes.append(_node("Add", [nd["a"], nd["b"]], [nd["out"]], nd["name"], attrs))
        elif op == "relu":
            nodes.append(_node("Relu", [nd["x"]], [nd["out"]], nd["name"], {}))
        elif op == "dense":
            attrs = {"input_spatial_shape": list(nd["input_spatial_shape"]),
                     "format": nd["format"], "output_shape": list(nd["output_shape"])}
            if nd.get("output_layout"):
                attrs["output_layout"] = nd["output_layout"]
            if nd.get("input_dynamic_range"):
                attrs["input_dynamic_range"] = float(nd["input_dynamic_range"])
            nodes.append(_node("ScatterDense", [nd["x"]], [nd["out"]], nd["name"], attrs))
        elif op == "reshape":
            nodes.append(_node("Reshape", [nd["x"]], [nd["out"]], nd["name"],
                               {"dims": list(nd["dims"])}))
        elif op == "transpose":
            nodes.append(_node("Transpose", [nd["x"]], [nd["out"]], nd["name"],
                               {"dims": list(nd["dims"])}))
        else:
            raise ValueError("unknown op %r" % op)
    graph = b"".join(_ld(1, n) for n in nodes) + _ld(2, b"scn")
    graph += b"".join(_ld(5, t) for t in inits)
    graph += b"".join(_ld(11, _value_info(n, s)) for n, s in model["inputs"])
    graph += b"".join(_ld(12, _value_info(n, s)) for n, s in model["outputs"])
    opset = _ld(1, b"ai.onnx") + _vi(2, 11)
    return _vi(1, 6) + _ld(2, b"pytorch") + _ld(3, b"1.9") + _ld(7, graph) + _ld(8, opset)


def save(model: dict, path: str) -> None:
    with open(path, "wb") as f:
        f.write(serialize(model))
