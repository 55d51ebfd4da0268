"""CPU-only checks that pin the oracle: golden counts of the reference's input
fixtures, dense cross-correlation, the tensor container, quantisation rules."""
import json
import os
import sys

import numpy as np
import pytest

from lidar_ai_solution_b200 import scenes
from oracle import graph_oracle, oracle as orc

STAGES = [((3, 3, 3), (2, 2, 2), (1, 1, 1)), ((3, 3, 3), (2, 2, 2), (1, 1, 1)),
          ((3, 3, 3), (2, 2, 2), (0, 1, 1)), ((3, 1, 1), (2, 1, 1), (0, 0, 0))]


def _fixture(golden_dir, key):
    zyx = np.load(os.path.join(golden_dir, "fixture_coords.npz"))[key].astype(np.int32)
    return np.concatenate([np.zeros((len(zyx), 1), np.int32), zyx], 1)


@pytest.mark.parametrize("name,key", [("bevfusion", "bevfusion_zyx"),
                                      ("centerpoint", "centerpoint_zyx")])
def test_rulebook_counts_of_reference_frames(golden_dir, name, key):
    """Per-stage voxel and pair counts of the reference's own sample frames."""
    coords = _fixture(golden_dir, key)
    gold = json.load(open(os.path.join(golden_dir, "fixture_counts.json")))[name]
    assert orc.count_duplicates(coords, [41, 1440, 1440]) == 0
    grid = [41, 1440, 1440]
    for (k, s, p), g in zip(STAGES, gold):
        _, pairs = orc.subm_map(coords, grid)
        oc, _, dpairs, og, n_out = orc.down_map(coords, grid, k, s, p)
        assert (len(coords), pairs, n_out, dpairs, og) == (
            g["n"], g["subm_pairs"], g["down_n"], g["down_pairs"], g["down_grid"])
        coords, grid = oc, og
    assert grid == [2, 180, 180]   # 128 channels x 2 = the 256-channel BEV map


def test_known_counts_for_the_centerpoint_frame(golden_dir):
    """The published frame: 79 745 voxels, 591 581 SubM pairs, 69 276 voxels after the first
    stride-2 conv (figures computed independently with a NumPy restatement)."""
    gold = json.load(open(os.path.join(golden_dir, "fixture_counts.json")))["centerpoint"]
    assert [g["n"] for g in gold] == [79745, 69276, 29723, 10335]
    assert [g["subm_pairs"] for g in gold] == [591581, 969672, 483025, 172003]
    assert [g["down_n"] for g in gold] == [69276, 29723, 10335, 7658]
    assert [g["down_pairs"] for g in gold] == [265739, 233074, 98648, 13673]


def _dense_conv(x_sparse, coords, grid, w, stride, pad):
    torch = pytest.importorskip("torch")
    cin = x_sparse.shape[1]
    dense = torch.zeros((1, cin, *grid), dtype=torch.float64)
    dense[0, :, coords[:, 1], coords[:, 2], coords[:, 3]] = torch.from_numpy(
        x_sparse.astype(np.float64)).T
    wt = torch.from_numpy(w.astype(np.float64)).permute(0, 4, 1, 2, 3)  # [O,k0,k1,k2,I] -> OIDHW
    return torch.nn.functional.conv3d(dense, wt, stride=stride, padding=pad)[0].numpy()


@pytest.mark.parametrize("ksize,stride,pad,subm", [
    ((3, 3, 3), (1, 1, 1), (1, 1, 1), True), ((3, 3, 3), (2, 2, 2), (1, 1, 1), False),
    ((3, 3, 3), (2, 2, 2), (0, 1, 1), False), ((3, 1, 1), (2, 1, 1), (0, 0, 0), False)])
def test_conv_equals_dense_cross_correlation_on_active_sites(ksize, stride, pad, subm):
    rng = np.random.default_rng(0)
    grid = (8, 16, 16)
    coords = scenes.make_coords(300, grid, 1)
    x = rng.standard_normal((300, 4)).astype(np.float32)
    w = rng.standard_normal((6, *ksize, 4)).astype(np.float32)
    dense = _dense_conv(x, coords, grid, w, stride, pad)
    if subm:
        m, _ = orc.subm_map(coords, grid, ksize)
        oc, n_out = coords, len(coords)
    else:
        oc, m, _, og, n_out = orc.down_map(coords, grid, ksize, stride, pad)
        assert list(dense.shape[1:]) == og
        # every site the dense conv can reach from an active input is an output, and only those
        reach = np.zeros(dense.shape[1:], bool)
        ones = _dense_conv(np.ones((300, 1), np.float32), coords, grid,
                           np.ones((1, *ksize, 1), np.float32), stride, pad)[0]
        reach[ones > 0] = True
        got = np.zeros_like(reach)
        got[oc[:, 1], oc[:, 2], oc[:, 3]] = True
        assert np.array_equal(got, reach)
        keys = (oc[:, 1] * og[1] + oc[:, 2]) * og[2] + oc[:, 3]
        assert np.all(np.diff(keys) > 0)           # canonical ascending order, no duplicates
    y = orc.conv_f32(x, m, n_out, w.reshape(6, -1, 4))
    ref = dense[:, oc[:, 1], oc[:, 2], oc[:, 3]].T
    assert np.allclose(y, ref, rtol=1e-4, atol=1e-4)


def test_int8_epilogue_rules():
    """q = clamp(rint(x*127/dr)) with ties to even; weights clamp to +-127; y = fma(acc, s, b)."""
    x = np.array([[0.5, 1.5, 2.5, -0.5, -1.5, 200.0, -200.0, 0.49]], np.float16)
    q = orc.quantize_f16(x, 127.0)
    assert q.tolist() == [[0, 2, 2, 0, -2, 127, -128, 0]]
    w = np.array([[1.0, -1.0, 0.5, 3.0]], np.float32)
    assert orc.quantize_weights(w, np.array([1.0], np.float32)).tolist() == [[127, -127, 64, 127]]
    m = np.zeros((1, 1), np.int32)
    xq = np.array([[10, -3]], np.int8)
    wq = np.array([[[7, 5]]], np.int8)
    y = orc.conv_i8(xq, m, 1, wq, np.array([0.25], np.float32), np.array([1.0], np.float32),
                    orc.ACT_NONE, orc.KIND_F32)
    assert y[0, 0] == np.float32(55 * 0.25 + 1.0)
    yq = orc.conv_i8(xq, m, 1, wq, np.array([0.25], np.float32), np.array([1.0], np.float32),
                     orc.ACT_RELU, orc.KIND_I8, 2.0)
    assert yq[0, 0] == 30    # rint(14.75*2) = 30 (29.5 ties to even)


def test_tensor_container_sample(golden_dir):
    """The reference's tensor file format (tool/tensor.py:24-69): int32 magic 0x33ff1101,
    ndim, dtype code, int32 dims, raw data."""
    raw = open(os.path.join(golden_dir, "sample.tensor"), "rb").read()
    magic, ndim, code, d0, d1 = np.frombuffer(raw[:20], np.int32)
    assert (magic, ndim, code, d0, d1) == (0x33FF1101, 2, 2, 40, 5)
    data = np.frombuffer(raw[20:], np.float16).reshape(d0, d1)
    head = np.load(os.path.join(golden_dir, "fixture_coords.npz"))["centerpoint_feat_head"]
    assert np.array_equal(data.view(np.uint16), head.view(np.uint16))
    assert np.all(np.abs(data[:, :2].astype(np.float32)) <= 54.0)   # x, y inside the range


def test_voxelizer_oracle_on_reference_sweep(golden_dir):
    pts = np.load(os.path.join(golden_dir, "sweep_points.npz"))["points"]
    feat, coords, total = orc.voxelize(pts, scenes.CENTERPOINT_RANGE, scenes.CENTERPOINT_VOXEL,
                                       (1440, 1440, 40), 160000, 10, 0)
    assert total == len(coords) and 0 < total < len(pts)
    assert orc.count_duplicates(coords, [41, 1440, 1440]) == 0
    # every voxel's mean lies inside the voxel it was assigned to
    f = feat.astype(np.float32)
    vx = np.floor((f[:, 0] + 54.0) / 0.075)
    assert np.mean(np.abs(vx - coords[:, 3]) <= 1) > 0.999
    # first voxel = first in-range point
    r = scenes.CENTERPOINT_RANGE
    p32 = pts.astype(np.float32)
    inside = ((p32[:, 0] >= r[0]) & (p32[:, 0] < r[3]) & (p32[:, 1] >= r[1]) & (p32[:, 1] < r[4])
              & (p32[:, 2] >= r[2]) & (p32[:, 2] < r[5]))
    first = p32[np.argmax(inside)]
    assert coords[0].tolist() == [0, int(np.floor((first[2] + 5.0) / 0.2)),
                                  int(np.floor((first[1] + 54.0) / 0.075)),
                                  int(np.floor((first[0] + 54.0) / 0.075))]


def test_graph_oracle_int8_matches_float_model_closely():
    """The int8 model tracks the fp16 model (quantisation noise only): a sanity check that
    the scale plumbing (consumer-driven ranges) is coherent."""
    from lidar_ai_solution_b200 import models
    grid = (41, 180, 180)
    coords = scenes.make_coords(3000, grid, 0)
    feats = scenes.make_point_features(coords, 0)
    model = models.scn_backbone("centerpoint", 0, grid_zyx=grid, output_bound=20000)
    outs, T = graph_oracle.run(model, feats, coords, grid, "fp16")
    ranges = {k: float(np.abs(v["feat"].astype(np.float32)).max()) for k, v in T.items()}
    qm = models.quantize(model, ranges)
    kind, dr = graph_oracle.resolve(qm, "int8")
    assert kind["1"] == "f16" and kind[qm["nodes"][-3]["out"]] == "f16"   # conv_input, extra_conv
    assert sum(v == "i8" for v in kind.values()) >= 25
    q_outs, _ = graph_oracle.run(qm, feats, coords, grid, "int8")
    a, b = outs[0].astype(np.float32).ravel(), q_outs[0].astype(np.float32).ravel()
    assert outs[0].shape == (1, 256, 23, 23)
    cos = float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))
    assert cos > 0.98, cos
    # a loader precision of fp16 ignores the int8 attributes
    f_outs, _ = graph_oracle.run(qm, feats, coords, grid, "fp16")
    assert np.array_equal(f_outs[0].view(np.uint16), outs[0].view(np.uint16))


def test_oracle_inverse_conv_equals_dense_transposed_conv():
    """The inverse conv of the graph oracle (pairs of the strided rulebook swapped, same tap
    index) is a dense conv_transpose3d evaluated at the fine active sites."""
    torch = pytest.importorskip("torch")
    from lidar_ai_solution_b200 import models
    grid = (9, 12, 10)
    coords = scenes.make_coords(300, grid, 1)
    m = models.encoder_decoder(8, seed=2, in_channels=8, output_bound=5000)
    feats = np.random.default_rng(0).standard_normal((300, 8)).astype(np.float16)
    _, T = graph_oracle.run(m, feats, coords, grid, "fp16")
    inv = [n for n in m["nodes"] if n.get("inverse")][0]
    e, u = T[inv["x"]], T[inv["out"]]
    assert np.array_equal(u["coords"], coords) and list(u["grid"]) == list(grid)
    og = e["grid"]
    xd = torch.zeros((1, e["feat"].shape[1], *og), dtype=torch.float64)
    for r, (b, z, y, x) in enumerate(e["coords"]):
        xd[0, :, z, y, x] = torch.from_numpy(e["feat"][r].astype(np.float64))
    w = torch.from_numpy(inv["weight"].astype(np.float64)).permute(4, 0, 1, 2, 3).contiguous()
    pad_out = [g - ((o - 1) * 2 - 2 + 3) for g, o in zip(grid, og)]
    yd = torch.nn.functional.conv_transpose3d(xd, w, stride=2, padding=1, output_padding=pad_out)
    ref = np.stack([yd[0, :, z, y, x].numpy() + inv["bias"].astype(np.float64)
                    for (b, z, y, x) in coords])
    got = u["feat"].astype(np.float64)
    assert np.abs(got - ref).max() <= 2e-3 * np.abs(ref).max()


def test_oracle_conv_equals_gather_gemm_scatter_on_config0():
    """Benchmark configuration 0 (20 000 voxels, 16 -> 16, fp32): the oracle's convolution
    equals the per-offset index_select + mm + index_add_ that the PyTorch sparse-conv packages
    run, on the same rulebook."""
    torch = pytest.importorskip("torch")
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                    "oracle"))
    import cpu_baseline_config0 as c0
    coords, x, w = c0.problem(3)
    y, m, pairs = c0.run_oracle(coords, x, w)
    assert pairs == int((m[:, :c0.N] >= 0).sum())
    yt = c0.run_torch(torch, x, w, m)
    assert np.abs(y - yt).max() <= 1e-5 * max(1.0, float(np.abs(yt).max()))


def test_dense_layouts_of_the_oracle():
    """NCHW32 and NHWzC are index permutations of the NCHW tensor: every element of the
    [N, C, D, H, W] scatter must be found at the documented address, padding must be zero,
    and the int8 scatter must agree with the fp16 one on integer-valued rows."""
    rng = np.random.default_rng(5)
    grid, ch, n = (2, 9, 11), 24, 60
    cells = rng.choice(grid[0] * grid[1] * grid[2], n, replace=False)
    coords = np.zeros((n, 4), np.int32)
    coords[:, 1], coords[:, 2], coords[:, 3] = np.unravel_index(cells, grid)
    q = rng.integers(-128, 128, (n, ch)).astype(np.int8)
    d8 = orc.scatter_dense_i8(q, coords, grid, 1)
    dh = orc.scatter_dense(q.astype(np.float16), coords, grid, 1, 1.0)
    assert np.array_equal(d8.astype(np.float16), dh)
    perm = (2, 0, 1)
    d8p = orc.scatter_dense_i8(q, coords, grid, 1, perm)
    assert np.array_equal(d8p.astype(np.float16), orc.scatter_dense(q.astype(np.float16), coords,
                                                                   grid, 1, 1.0, perm))
    c32 = orc.dense_layout(d8, "NCHW32", ch)
    hwzc = orc.dense_layout(d8, "NHWzC", ch)
    assert c32.shape == (1, 2, 9, 11, 32) and hwzc.shape == (1, 9, 11, 2, ch)
    for c in range(ch):
        for z in range(grid[0]):
            m = c * grid[0] + z
            assert np.array_equal(c32[0, m // 32, :, :, m % 32], d8[0, c, z])
            assert np.array_equal(hwzc[0, :, :, z, c], d8[0, c, z])
    assert not c32[0, 1, :, :, 16:].any()  # 48 real channels, 16 of padding
    view4 = d8.reshape(1, ch * grid[0], 9, 11)
    assert np.array_equal(orc.dense_layout(view4, "NCHW32", ch), c32)
    assert np.array_equal(orc.dense_layout(view4, "NHWzC", ch), hwzc)


def test_rotated_iou_known_answers():
    """The bird's-eye overlap of the restated NMS against areas computed by hand."""
    box = lambda x, y, dx, dy, a: [x, y, 0.0, dx, dy, 1.0, a]  # noqa: E731
    a = np.array([box(0, 0, 2, 2, 0.0), box(0, 0, 2, 2, 0.0), box(0, 0, 2, 2, 0.0),
                  box(0, 0, 2, 2, 0.0), box(0, 0, 4, 2, 0.0), box(5, 5, 2, 4, 0.3)], np.float32)
    b = np.array([box(0, 0, 2, 2, 0.0), box(1, 0, 2, 2, 0.0), box(5, 0, 2, 2, 0.0),
                  box(0, 0, 2, 2, np.pi / 4), box(0, 0, 2, 4, np.pi / 2), box(5, 5, 2, 4, 0.3)],
                 np.float32)
    got = orc.rotated_iou(a, b)
    octagon = 8 * (np.sqrt(2) - 1)  # two unit-2 squares, one turned by 45 degrees
    want = [1.0, 2.0 / 6.0, 0.0, octagon / (8 - octagon), 1.0, 1.0]
    assert np.allclose(got, want, atol=2e-5), got


def test_centerpoint_decode_and_nms_on_a_hand_made_head():
    """Three cells above the score threshold: two overlapping boxes of one class and a distant
    one; the decode must rank them by score and the NMS must drop the weaker of the pair."""
    H = W = 16
    head = {"hm": np.full((2, H, W), -9.0), "reg": np.full((2, H, W), 0.5),
            "height": np.full((1, H, W), -1.0), "dim": np.zeros((3, H, W)),
            "rot": np.zeros((2, H, W)), "vel": np.zeros((2, H, W))}
    head["rot"][1] = 1.0                       # sin 0, cos 1 -> yaw 0
    head["dim"][0] = np.log(4.0)               # 4 x 1 x 1 boxes
    head["hm"][1, 5, 5], head["hm"][1, 5, 6], head["hm"][0, 12, 3] = 2.0, 3.0, 0.5
    head["vel"][0, 5, 6] = 1.5
    prm = dict(pc_range=(0.0, 0.0), post_center_range=(-100, -100, -10, 100, 100, 10))
    det, cells = orc.centerpoint_decode(head, prm)
    assert list(cells) == [5 * W + 6, 5 * W + 5, 12 * W + 3]
    assert np.allclose(det[:, 10], 1 / (1 + np.exp(-np.array([3.0, 2.0, 0.5]))), rtol=1e-6)
    assert list(det[:, 9]) == [1.0, 1.0, 0.0]
    assert np.allclose(det[0, :9], [6.5 * 0.6, 5.5 * 0.6, -1.0, np.exp(np.float32(np.float16(np.log(4.0)))), 1.0, 1.0,
                                   1.5, 0.0, 0.0], atol=1e-6)
    boxes, kept, margin = orc.centerpoint_nms(det, label_offset=3, params=prm)
    assert list(kept) == [0, 2] and margin > 1e-3
    assert list(boxes[:, 9]) == [4.0, 3.0] and np.array_equal(boxes[:, :9], det[[0, 2], :9])
    # a score threshold above every cell, and a centre range that excludes everything
    assert len(orc.centerpoint_decode(head, dict(prm, score_threshold=0.99))[0]) == 0
    assert len(orc.centerpoint_decode(head, dict(prm, post_center_range=(50, 50, -10, 60, 60, 10)))[0]) == 0
    # more candidates than max_det: the best max_det by (score, cell) survive
    head["hm"][0] = 1.0
    det, cells = orc.centerpoint_decode(head, dict(prm, max_det=10))
    assert len(det) == 10 and list(cells[:2]) == [5 * W + 6, 5 * W + 5]
    assert list(cells[2:]) == list(range(8))

