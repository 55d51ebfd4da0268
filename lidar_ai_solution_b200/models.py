"""Graph descriptions of the two lidar backbones, with random-init weights.

The layer lists are the ones the benchmark configurations give:

* CenterPoint SCN: SubM 5->16, two residual blocks at 16, then three times
  (stride-2 conv, two residual blocks) with 32, 64, 128 channels (paddings
  (1,1,1), (1,1,1), (0,1,1)), a 128->128 conv with kernel (3,1,1) stride
  (2,1,1), ScatterDense to [1,128,2,180,180] and a Reshape to [1,256,180,180].
* BEVFusion lidar SparseEncoder: the same sequence of layers, dense output
  transposed to put x before y as the exporter does.

Node order, tensor ids, attribute names, the residual block
(conv-ReLU, conv, Add, Relu) and the int8 precision maps follow what the
reference's exporters trace:
CUDA-CenterPoint/qat/onnx_export/exptool.py:69-283 and export-scn.py:57-68,
CUDA-BEVFusion/qat/lean/exptool.py:127-294 and qat/export-scn.py:62-67.
Weights are Kaiming-normal fp16 in the exporter's [Cout, k0, k1, k2, Cin]
layout; BatchNorm is taken as already folded.
"""
from __future__ import annotations

import copy

import numpy as np

GRID_ZYX = (41, 1440, 1440)


class _Ids:
    def __init__(self):
        self.n = 0

    def new(self):
        self.n += 1
        return str(self.n)


def _conv(ids, rng, nodes, x, cin, cout, ksize, stride, pad, subm, rulebook, act, counter,
          output_bound):
    kvol = int(np.prod(ksize))
    w = (rng.standard_normal((cout, *ksize, cin)) * np.sqrt(2.0 / (kvol * cin))).astype(np.float16)
    b = (rng.standard_normal(cout) * 0.02).astype(np.float16)
    out = ids.new()
    nodes.append({"op": "conv", "name": "conv%d" % counter[0], "x": x, "out": out, "weight": w,
                  "bias": b, "activation": act, "kernel_size": list(ksize),
                  "stride": list(stride), "padding": list(pad), "dilation": [1, 1, 1],
                  "subm": int(subm), "rulebook": rulebook, "output_bound": output_bound})
    counter[0] += 1
    return out


def _block(ids, rng, nodes, x, c, key, counter, output_bound):
    """SparseBasicBlock after BN/ReLU fusion: conv(ReLU) -> conv -> Add(identity) -> Relu."""
    first = len(nodes)
    y = _conv(ids, rng, nodes, x, c, c, (3, 3, 3), (1, 1, 1), (1, 1, 1), True, key, "ReLU",
              counter, output_bound)
    y = _conv(ids, rng, nodes, y, c, c, (3, 3, 3), (1, 1, 1), (1, 1, 1), True, key, "None",
              counter, output_bound)
    s = ids.new()
    nodes.append({"op": "add", "name": "add%d" % counter[1], "a": y, "b": x, "out": s})
    r = ids.new()
    nodes.append({"op": "relu", "name": "relu%d" % counter[1], "x": s, "out": r})
    counter[1] += 1
    return r, list(range(first, len(nodes)))


def scn_backbone(kind: str = "centerpoint", seed: int = 0, in_channels: int = 5,
                 grid_zyx=GRID_ZYX, output_bound: int = 200000, channels=(16, 32, 64, 128)):
    """Float model (no quantisation attributes).  Returns the model dict; the
    key "roles" maps role names (conv_input, block0..7, down1..3, extra) to node
    indices for the precision maps."""
    assert kind in ("centerpoint", "bevfusion")
    rng = np.random.default_rng(seed)
    ids, nodes, counter, roles = _Ids(), [], [0, 0], {}
    c0, c1, c2, c3 = channels
    x = "0"
    x = _conv(ids, rng, nodes, x, in_channels, c0, (3, 3, 3), (1, 1, 1), (1, 1, 1), True, "subm0",
              "ReLU", counter, output_bound)
    roles["conv_input"] = [0]
    grid = list(grid_zyx)
    nblock = 0
    for stage, (c, pad) in enumerate(zip((c0, c1, c2, c3), (None, (1, 1, 1), (1, 1, 1), (0, 1, 1)))):
        if stage > 0:
            prev = (c0, c1, c2, c3)[stage - 1]
            roles["down%d" % stage] = [len(nodes)]
            x = _conv(ids, rng, nodes, x, prev, c, (3, 3, 3), (2, 2, 2), pad, False,
                      "down%d" % stage, "ReLU", counter, output_bound)
            grid = [(g + 2 * p - 3) // 2 + 1 for g, p in zip(grid, pad)]
        for _ in range(2):
            x, idx = _block(ids, rng, nodes, x, c, "res%d" % stage, counter, output_bound)
            roles["block%d" % nblock] = idx
            nblock += 1
    roles["extra"] = [len(nodes)]
    x = _conv(ids, rng, nodes, x, c3, c3, (3, 1, 1), (2, 1, 1), (0, 0, 0), False, "extra", "ReLU",
              counter, output_bound)
    grid = [(grid[0] - 3) // 2 + 1, grid[1], grid[2]]
    d = ids.new()
    nodes.append({"op": "dense", "name": "scatter0", "x": x, "out": d,
                  "input_spatial_shape": grid, "format": "zyx",
                  "output_shape": [1, c3, grid[0], grid[1], grid[2]]})
    if kind == "bevfusion":
        t = ids.new()
        nodes.append({"op": "transpose", "name": "transpose0", "x": d, "out": t,
                      "dims": [0, 1, 2, 4, 3]})
        d = t
        out_shape = [1, c3 * grid[0], grid[2], grid[1]]
    else:
        out_shape = [1, c3 * grid[0], grid[1], grid[2]]
    r = ids.new()
    nodes.append({"op": "reshape", "name": "reshape0", "x": d, "out": r, "dims": out_shape})
    return {"kind": kind, "grid": list(grid_zyx), "inputs": [("0", [1, in_channels])],
            "outputs": [(r, out_shape)], "nodes": nodes, "roles": roles,
            "in_channels": in_channels}


def single_layer(cin: int, cout: int, seed: int = 0, subm: bool = True, output_bound=200000):
    """One SparseConvolution node (ReLU fused) whose sparse result is the graph output."""
    rng = np.random.default_rng(seed)
    ids, nodes = _Ids(), []
    if subm:
        y = _conv(ids, rng, nodes, "0", cin, cout, (3, 3, 3), (1, 1, 1), (1, 1, 1), True, "subm0",
                  "ReLU", [0, 0], output_bound)
    else:
        y = _conv(ids, rng, nodes, "0", cin, cout, (3, 3, 3), (2, 2, 2), (1, 1, 1), False, "down",
                  "ReLU", [0, 0], output_bound)
    return {"kind": "layer", "inputs": [("0", [1, cin])], "outputs": [(y, [1, cout])],
            "nodes": nodes, "roles": {"conv_input": [0]}, "in_channels": cin}


def encoder_decoder(channels: int = 16, seed: int = 0, in_channels: int = 16,
                    output_bound=200000):
    """A segmentation-style block: SubM conv, stride-2 conv (rulebook "down0"), SubM conv on
    the coarse rows, SparseInverseConvolution back onto the fine rows through the same
    rulebook, Add with the skip connection, ReLU.  Both the fine sum and the coarse tensor
    are graph outputs (sparse, two outputs)."""
    rng = np.random.default_rng(seed)
    ids, nodes, counter = _Ids(), [], [0, 0]
    c = channels
    x0 = _conv(ids, rng, nodes, "0", in_channels, c, (3, 3, 3), (1, 1, 1), (1, 1, 1), True,
               "subm0", "ReLU", counter, output_bound)
    d = _conv(ids, rng, nodes, x0, c, 2 * c, (3, 3, 3), (2, 2, 2), (1, 1, 1), False, "down0",
              "ReLU", counter, output_bound)
    e = _conv(ids, rng, nodes, d, 2 * c, 2 * c, (3, 3, 3), (1, 1, 1), (1, 1, 1), True, "subm1",
              "ReLU", counter, output_bound)
    u = _conv(ids, rng, nodes, e, 2 * c, c, (3, 3, 3), (2, 2, 2), (1, 1, 1), False, "down0",
              "None", counter, output_bound)
    nodes[-1]["inverse"] = 1
    s = ids.new()
    nodes.append({"op": "add", "name": "add0", "a": u, "b": x0, "out": s})
    r = ids.new()
    nodes.append({"op": "relu", "name": "relu0", "x": s, "out": r})
    return {"kind": "encoder_decoder", "inputs": [("0", [1, in_channels])],
            "outputs": [(r, [1, c]), (e, [1, 2 * c])], "nodes": nodes,
            "roles": {"conv_input": [0]}, "in_channels": in_channels}


def quantize(model: dict, ranges: dict, kind: str | None = None) -> dict:
    """Attach the int8 attributes.  ``ranges`` maps tensor id -> absmax seen in
    calibration (plain absmax on one frame).  Weight ranges are per output
    channel.  The precision map is the exporter's for the model kind."""
    kind = kind or model["kind"]
    m = copy.copy(model)
    m["nodes"] = [dict(n) for n in model["nodes"]]
    nodes, roles = m["nodes"], model["roles"]
    for n in nodes:
        if n["op"] == "conv":
            w = n["weight"].astype(np.float32)
            n["weight_dynamic_ranges"] = np.abs(w).reshape(w.shape[0], -1).max(1).tolist()
            n["input_dynamic_range"] = float(max(ranges[n["x"]], 1e-6))
            n["precision"] = n["output_precision"] = "int8"
        elif n["op"] == "add":
            r = float(max(ranges[n["a"]], ranges[n["b"]], 1e-6))
            n["input0_dynamic_range"] = n["input1_dynamic_range"] = r
            n["precision"] = n["output_precision"] = "int8"
    first = nodes[roles["conv_input"][0]]
    if kind == "centerpoint":
        first["precision"] = first["output_precision"] = "fp16"
        for i in roles.get("block0", []):
            if nodes[i]["op"] == "conv":
                nodes[i]["precision"] = nodes[i]["output_precision"] = "fp16"
            elif nodes[i]["op"] == "add":
                nodes[i]["precision"] = "fp16"
                nodes[i]["output_precision"] = "int8"
    elif kind == "bevfusion":
        first["precision"] = "fp16"
    if "extra" in roles:
        nodes[roles["extra"][0]]["output_precision"] = "fp16"
    else:  # a single layer: its sparse output leaves the engine as fp16
        nodes[-1]["output_precision"] = "fp16"
    return m


def tensor_ids(model: dict):
    """Ids of all sparse tensors in execution order."""
    out = [model["inputs"][0][0]]
    for n in model["nodes"]:
        if n["op"] in ("conv", "add", "relu"):
            out.append(n["out"])
    return out
