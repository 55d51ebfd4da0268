"""Runs a whole model description node by node on the CPU oracle.

TEST INFRASTRUCTURE ONLY (see oracle.py).  The graph semantics restated here
are the ones the reference's exporters imply for its closed engine
(CUDA-CenterPoint/qat/onnx_export/exptool.py:141-231, export-scn.py:57-68):

* a loader precision of fp16 overrides every per-layer attribute
  (CUDA-CenterPoint/3rdparty/libspconv/include/spconv/engine.hpp:97-101);
* an int8 tensor is stored with the dynamic range its consumer declares: the
  first int8 conv consumer's ``input_dynamic_range``, else an Add consumer's
  ``inputN_dynamic_range``, else a ScatterDense ``input_dynamic_range``; a Relu
  passes the range of its own output upstream;
* a conv dequantises with the scale its input was stored with; Add dequantises
  each operand with the operand's stored scale;
* nothing is fused: every node rounds its result to its output precision.

Parity status: unpinned against the closed engine (no golden outputs exist).
"""
from __future__ import annotations

import numpy as np

from . import oracle as orc

F32 = np.float32


def _eff(global_precision, p):
    return "fp16" if global_precision == "fp16" else ("int8" if p == "int8" else "fp16")


def resolve(model, precision):
    """kind ('i8'/'f16') and dynamic range of every tensor id."""
    nodes = model["nodes"]
    consumers = {}
    for i, n in enumerate(nodes):
        for key in ("x", "a", "b"):
            if key in n:
                consumers.setdefault(n[key], []).append(i)
    kind = {model["inputs"][0][0]: "f16"}
    for n in nodes:
        if n["op"] in ("conv", "add"):
            kind[n["out"]] = "i8" if _eff(precision, n.get("output_precision", "fp16")) == "int8" else "f16"
        elif n["op"] == "relu":
            kind[n["out"]] = kind[n["x"]]
        else:
            kind[n["out"]] = "f16"
    dr = {}
    order = [model["inputs"][0][0]] + [n["out"] for n in nodes]
    for t in reversed(order):
        if kind[t] != "i8":
            continue
        v = 0.0
        for c in consumers.get(t, []):
            cn = nodes[c]
            if cn["op"] == "conv" and _eff(precision, cn.get("precision", "fp16")) == "int8":
                v = cn.get("input_dynamic_range", 0.0)
            elif cn["op"] == "add":
                v = cn.get("input0_dynamic_range" if cn["a"] == t else "input1_dynamic_range", 0.0)
            elif cn["op"] == "dense":
                v = cn.get("input_dynamic_range", 0.0)
            elif cn["op"] == "relu":
                v = dr.get(cn["out"], 0.0)
            if v > 0:
                break
        if v > 0:
            dr[t] = float(v)
        else:
            kind[t] = "f16"
    for n in nodes:
        if n["op"] == "relu" and kind[n["x"]] != kind[n["out"]]:
            kind[n["out"]] = kind[n["x"]]
            if n["x"] in dr:
                dr[n["out"]] = dr[n["x"]]
    return kind, dr


def run(model, features, coords, grid, precision="fp16"):
    """Returns (outputs, tensors): outputs = list of numpy arrays for the graph
    outputs, tensors = {id: dict(feat, coords, grid, kind, dr)} for every sparse tensor."""
    kind, dr = resolve(model, precision)
    coords = np.ascontiguousarray(coords, np.int32)
    T = {model["inputs"][0][0]: dict(feat=np.ascontiguousarray(features, np.float16), coords=coords,
                                     grid=list(grid), kind="f16", dr=0.0)}
    dense = {}
    dense_meta = {}
    rule_cache = {}
    named_rules = {}
    for n in model["nodes"]:
        op = n["op"]
        if op == "conv":
            src = T[n["x"]]
            compute = _eff(precision, n.get("precision", "fp16"))
            key = (id(src["coords"]), tuple(n["kernel_size"]), tuple(n["stride"]),
                   tuple(n["padding"]), tuple(n["dilation"]), n["subm"], bool(n.get("inverse")))
            if n.get("inverse"):
                # SparseInverseConvolution (engine.hpp:156 `inverse`): the pairs of the strided
                # rulebook with the same `rulebook` key, input and output swapped; the outputs
                # are that rulebook's input rows
                fwd = named_rules[n["rulebook"]]
                if fwd["coarse"] is not src["coords"]:
                    raise ValueError("inverse conv %s: input is not the output of rulebook %s"
                                     % (n["name"], n["rulebook"]))
                inv = np.full((fwd["map"].shape[0], len(fwd["fine"])), -1, np.int32)
                for k in range(fwd["map"].shape[0]):
                    rows = fwd["map"][k, :fwd["n_coarse"]]
                    o = np.nonzero(rows >= 0)[0]
                    inv[k, rows[o]] = o
                rule_cache[key] = (fwd["fine"], inv, list(fwd["fine_grid"]), len(fwd["fine"]))
            if key not in rule_cache:
                if n["subm"]:
                    m, _ = orc.subm_map(src["coords"], src["grid"], n["kernel_size"], n["dilation"])
                    rule_cache[key] = (src["coords"], m, list(src["grid"]), len(src["coords"]))
                else:
                    oc, m, _, og, n_out = orc.down_map(src["coords"], src["grid"], n["kernel_size"],
                                                       n["stride"], n["padding"], n["dilation"],
                                                       cap=n.get("output_bound"))
                    rule_cache[key] = (oc, m, og, len(oc))
                    if n.get("rulebook"):
                        named_rules[n["rulebook"]] = dict(fine=src["coords"], fine_grid=src["grid"],
                                                          coarse=oc, map=m, n_coarse=n_out)
            oc, m, og, n_out = rule_cache[key]
            w16 = np.ascontiguousarray(n["weight"], np.float16)
            cout, cin = w16.shape[0], w16.shape[-1]
            w16 = w16.reshape(cout, -1, cin)
            bias = n["bias"].astype(np.float32)
            act = orc.ACT_RELU if n["activation"] == "ReLU" else orc.ACT_NONE
            okind = orc.KIND_I8 if kind[n["out"]] == "i8" else orc.KIND_F16
            inv_out = float(F32(127.0) / F32(dr[n["out"]])) if okind == orc.KIND_I8 else 1.0
            if compute == "int8":
                if src["kind"] == "i8":
                    xq, in_scale = src["feat"], F32(src["dr"]) / F32(127.0)
                else:
                    xq = orc.quantize_f16(src["feat"], n["input_dynamic_range"])
                    in_scale = F32(n["input_dynamic_range"]) / F32(127.0)
                amax = np.asarray(n["weight_dynamic_ranges"], np.float32)
                wq = orc.quantize_weights(w16.astype(np.float32), amax)
                scale = (in_scale * (amax / F32(127.0))).astype(np.float32)
                y = orc.conv_i8(xq, m, n_out, wq, scale, bias, act, okind, inv_out)
            else:
                x = src["feat"]
                if src["kind"] == "i8":
                    x = (x.astype(np.float32) * (F32(src["dr"]) / F32(127.0))).astype(np.float16)
                y = orc.conv_f16(x, m, n_out, w16, bias, act, okind, inv_out)
            T[n["out"]] = dict(feat=y, coords=oc, grid=og, kind=kind[n["out"]],
                               dr=dr.get(n["out"], 0.0))
        elif op == "add":
            a, b = T[n["a"]], T[n["b"]]
            okind = orc.KIND_I8 if kind[n["out"]] == "i8" else orc.KIND_F16
            inv_out = float(F32(127.0) / F32(dr[n["out"]])) if okind == orc.KIND_I8 else 1.0
            sa = float(F32(a["dr"]) / F32(127.0)) if a["kind"] == "i8" else 1.0
            sb = float(F32(b["dr"]) / F32(127.0)) if b["kind"] == "i8" else 1.0
            y = orc.add(a["feat"], sa, b["feat"], sb, False, okind, inv_out)
            T[n["out"]] = dict(feat=y, coords=a["coords"], grid=a["grid"], kind=kind[n["out"]],
                               dr=dr.get(n["out"], 0.0))
        elif op == "relu":
            a = T[n["x"]]
            T[n["out"]] = dict(feat=orc.relu(a["feat"]), coords=a["coords"], grid=a["grid"],
                               kind=a["kind"], dr=a["dr"])
        elif op == "dense":
            a = T[n["x"]]
            s = float(F32(a["dr"]) / F32(127.0)) if a["kind"] == "i8" else 1.0
            ddr = float(n.get("input_dynamic_range", 0.0) or 0.0)
            if ddr > 0:  # int8 dense tensor with that range
                if a["kind"] == "i8" and a["dr"] == ddr:
                    q = a["feat"]
                elif a["kind"] == "i8":  # stored with another range: rescale in fp32
                    inv = F32(127.0) / F32(ddr)
                    q = np.clip(np.rint((a["feat"].astype(np.float32) * F32(s)) * inv),
                                -128, 127).astype(np.int8)
                else:
                    q = orc.quantize_f16(a["feat"], ddr)
                dense[n["out"]] = orc.scatter_dense_i8(q, a["coords"], a["grid"], 1)
            else:
                dense[n["out"]] = orc.scatter_dense(a["feat"], a["coords"], a["grid"], 1, s)
            dense_meta[n["out"]] = (n.get("output_layout", "NCHW"), a["feat"].shape[1])
        elif op == "transpose":
            dense[n["out"]] = np.ascontiguousarray(np.transpose(dense[n["x"]], n["dims"]))
            dense_meta[n["out"]] = dense_meta[n["x"]]
        elif op == "reshape":
            dense[n["out"]] = dense[n["x"]].reshape(n["dims"])
            dense_meta[n["out"]] = dense_meta[n["x"]]
        else:
            raise ValueError(op)
    outs = [orc.dense_layout(dense[o], *dense_meta[o]) if o in dense else T[o]["feat"]
            for o, _ in model["outputs"]]
    return outs, T
