"""Kernel-level parity: every CUDA entry point of the C ABI against the CPU oracle
on the same seeded inputs.  Integer and index results must be identical; fp16
tensor-core results are within 1e-2 relative (stated per test)."""
import json
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from lidar_ai_solution_b200 import scenes  # noqa: E402
from oracle import oracle as orc  # noqa: E402
from tests.helpers import int8_problem, kaiming  # noqa: E402

pytestmark = pytest.mark.gpu

STAGES = [((3, 3, 3), (2, 2, 2), (1, 1, 1)), ((3, 3, 3), (2, 2, 2), (1, 1, 1)),
          ((3, 3, 3), (2, 2, 2), (0, 1, 1)), ((3, 1, 1), (2, 1, 1), (0, 0, 0))]


def _ops():
    from lidar_ai_solution_b200 import ops
    return ops


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _status_ok(status):
    s = status.cpu().numpy()
    assert s[0] == 0, "device status %s" % s


# ------------------------------------------------------------------ rulebooks
@pytest.mark.parametrize("n,grid,seed", [(20000, (41, 180, 180), 0), (20000, (41, 180, 180), 3),
                                         (120000, (41, 1440, 1440), 1), (1, (41, 180, 180), 0),
                                         (129, (5, 7, 9), 2)])
def test_subm_map_bit_exact(n, grid, seed):
    ops = _ops()
    coords = scenes.make_coords(n, grid, seed)
    ref, pairs = orc.subm_map(coords, grid)
    dc, n_ptr, st = _dev(coords), ops.device_count(n), ops.new_status()
    table = ops.hash_build(dc, n_ptr, grid, status=st)
    m = ops.subm_map(dc, n_ptr, grid, table, status=st)
    torch.cuda.synchronize()
    _status_ok(st)
    got = m.cpu().numpy()
    assert np.array_equal(got, ref)
    assert int((got >= 0).sum()) == pairs


def test_subm_map_capacity_larger_than_rows():
    """Buffers sized for a bound, row count on the device (the DDS calling pattern)."""
    ops = _ops()
    grid, n, cap = (41, 180, 180), 5000, 8192
    coords = scenes.make_coords(n, grid, 5)
    padded = np.full((cap, 4), 7, np.int32)
    padded[:n] = coords
    ref, _ = orc.subm_map(coords, grid, cap=cap)
    dc, n_ptr, st = _dev(padded), ops.device_count(n), ops.new_status()
    table = ops.hash_build(dc, n_ptr, grid, status=st)
    m = torch.full((27, cap), -1, dtype=torch.int32, device="cuda")
    from lidar_ai_solution_b200 import cabi
    cabi.check(cabi.lib().spconvb_subm_map(dc.data_ptr(), n_ptr.data_ptr(), cap, 2048,
                                           cabi.i3(grid), 1, cabi.i3((3, 3, 3)),
                                           cabi.i3((1, 1, 1)), table.data_ptr(), table.numel(),
                                           m.data_ptr(), st.data_ptr(),
                                           torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    _status_ok(st)
    assert np.array_equal(m.cpu().numpy(), ref)


def test_hash_reports_duplicates_and_range():
    ops = _ops()
    grid = (8, 8, 8)
    coords = np.array([[0, 1, 1, 1], [0, 1, 1, 1], [0, 9, 0, 0]], np.int32)
    st = ops.new_status()
    ops.hash_build(_dev(coords), ops.device_count(3), grid, status=st)
    torch.cuda.synchronize()
    from lidar_ai_solution_b200 import cabi
    bits = int(st.cpu().numpy()[0])
    assert bits & cabi.ST_DUPLICATE and bits & cabi.ST_COORD_RANGE


def _chain(coords, grid):
    """Stage 0 looks neighbours up in the hash table of the caller's rows; later stages rank
    them in the bitmap the strided rulebook left behind (no hash table)."""
    ops = _ops()
    dc, n_ptr, st = _dev(coords), ops.device_count(len(coords)), ops.new_status()
    table = ops.hash_build(dc, n_ptr, grid, status=st)
    ws = None
    out = []
    for k, s, p in STAGES:
        if ws is None:
            m = ops.subm_map(dc, n_ptr, grid, table, status=st)
        else:
            m = ops.subm_map_ranked(dc, n_ptr, grid, ws, status=st)
            by_hash = ops.subm_map(dc, n_ptr, grid, table, status=st)
            assert torch.equal(m[:, : int(n_ptr.item())], by_hash[:, : int(n_ptr.item())])
        in_ws = ws
        oc, n_out, dm, otab, og, ws = ops.down_map(dc, n_ptr, grid, None, k, s, p, status=st,
                                                   return_ws=True)
        if in_ws is not None:
            # rows made by a strided rulebook: the output-side lookup by rank gives the same
            # coordinates, count and map as the input-side scatter
            oc2, n2, dm2, _, _ = ops.down_map(dc, n_ptr, grid, None, k, s, p, status=st,
                                              in_ws=in_ws)
            kk = int(n_out.item())
            assert int(n2.item()) == kk and torch.equal(oc2[:kk], oc[:kk])
            assert torch.equal(dm2[:, :kk], dm[:, :kk])
        torch.cuda.synchronize()
        _status_ok(st)
        out.append((dc, n_ptr, list(grid), m, oc, n_out, dm, og))
        dc, n_ptr, table, grid = oc, n_out, otab, og
    return out


def test_stage_chain_matches_oracle_and_fixture_counts(golden_dir):
    """The reference's 79 745-voxel CenterPoint frame through the backbone's four
    resolutions: maps and output coordinates identical to the oracle, counts equal
    to the committed golden counts."""
    z = np.load(os.path.join(golden_dir, "fixture_coords.npz"))
    counts = json.load(open(os.path.join(golden_dir, "fixture_counts.json")))
    for name, key in (("centerpoint", "centerpoint_zyx"), ("bevfusion", "bevfusion_zyx")):
        zyx = z[key].astype(np.int32)
        coords = np.concatenate([np.zeros((len(zyx), 1), np.int32), zyx], 1)
        grid = [41, 1440, 1440]
        c_ref = coords
        for stage, (dc, n_ptr, g, m, oc, n_out, dm, og) in enumerate(_chain(coords, grid)):
            n = int(n_ptr.item())
            ref_m, pairs = orc.subm_map(c_ref, g)
            assert np.array_equal(m.cpu().numpy()[:, :n], ref_m)
            k, s, p = STAGES[stage]
            roc, rdm, dpairs, rog, rn = orc.down_map(c_ref, g, k, s, p, cap=oc.shape[0])
            assert int(n_out.item()) == rn and og == rog
            assert np.array_equal(oc.cpu().numpy()[:rn], roc)
            assert np.array_equal(dm.cpu().numpy()[:, :rn], rdm[:, :rn])
            gold = counts[name][stage]
            assert (n, pairs, rn, dpairs) == (gold["n"], gold["subm_pairs"], gold["down_n"],
                                              gold["down_pairs"])
            c_ref = roc


@pytest.mark.parametrize("k,s,p,d", [
    ((3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1)),   # every strided layer of the backbones
    ((3, 3, 3), (3, 3, 3), (0, 0, 0), (1, 1, 1)),   # stride that is not a power of two
    ((5, 3, 1), (2, 1, 3), (2, 0, 1), (1, 1, 1)),   # mixed extents, stride 1 on an axis
    ((2, 2, 2), (2, 2, 2), (0, 0, 0), (1, 1, 1)),   # even kernel
    ((1, 1, 1), (2, 2, 2), (0, 0, 0), (1, 1, 1)),   # pure subsampling
    ((3, 3, 7), (1, 2, 1), (1, 1, 3), (1, 1, 1)),   # runs of up to 7 adjacent output cells
    ((3, 3, 3), (2, 2, 2), (2, 1, 2), (2, 1, 2)),   # dilated: the tap-pruning path
])
def test_down_map_geometries_match_the_oracle(k, s, p, d):
    """Output coordinates, their order, the count and the whole map of a strided rulebook for
    kernel / stride / padding / dilation combinations beyond the backbones', from the caller's
    rows (input-side scatter) and again from rulebook-made rows (output-side lookup)."""
    ops = _ops()
    grid = (9, 70, 83)
    coords = scenes.make_coords(6000, grid, 5)
    st = ops.new_status()
    dc = _dev(coords)
    oc, n_out, dm, _, og, ws = ops.down_map(dc, ops.device_count(len(coords)), grid, None, k, s, p,
                                            dilation=d, status=st, want_table=False,
                                            return_ws=True)
    roc, rdm, pairs, rog, rn = orc.down_map(coords, grid, k, s, p, d, cap=oc.shape[0])
    _status_ok(st)
    assert int(n_out.item()) == rn and list(og) == list(rog) and pairs > 0
    assert np.array_equal(oc.cpu().numpy()[:rn], roc)
    assert np.array_equal(dm.cpu().numpy()[:, :rn], rdm[:, :rn])
    # second level: the rows just made are the input, looked up by rank from the output side
    k2, s2, p2 = (3, 3, 3), (2, 2, 2), (1, 1, 1)
    oc2, n2, dm2, _, og2 = ops.down_map(oc, n_out, og, None, k2, s2, p2, status=st,
                                        want_table=False, in_ws=ws)
    roc2, rdm2, _, rog2, rn2 = orc.down_map(roc, rog, k2, s2, p2, cap=oc2.shape[0])
    _status_ok(st)
    assert int(n2.item()) == rn2 and list(og2) == list(rog2)
    assert np.array_equal(oc2.cpu().numpy()[:rn2], roc2)
    assert np.array_equal(dm2.cpu().numpy()[:, :rn2], rdm2[:, :rn2])
    # and the geometry under test on rulebook-made rows (the outputs' bitmap then comes from
    # the inputs' bitmap): first a 3x3x3 stride-1 rulebook over the caller's rows, whose
    # outputs are ranked, then the geometry on those
    fo, fn, _, _, fg, fws = ops.down_map(dc, ops.device_count(len(coords)), grid, None, (3, 3, 3),
                                         (1, 1, 1), (1, 1, 1), status=st, want_table=False,
                                         return_ws=True)
    rfo, _, _, rfg, rfn = orc.down_map(coords, grid, (3, 3, 3), (1, 1, 1), (1, 1, 1),
                                       cap=fo.shape[0])
    assert int(fn.item()) == rfn
    oc3, n3, dm3, _, og3 = ops.down_map(fo, fn, fg, None, k, s, p, dilation=d, status=st,
                                        want_table=False, in_ws=fws)
    roc3, rdm3, _, rog3, rn3 = orc.down_map(rfo, rfg, k, s, p, d, cap=oc3.shape[0])
    _status_ok(st)
    assert int(n3.item()) == rn3 and list(og3) == list(rog3)
    assert np.array_equal(oc3.cpu().numpy()[:rn3], roc3)
    assert np.array_equal(dm3.cpu().numpy()[:, :rn3], rdm3[:, :rn3])


def test_down_map_overflow_sets_status():
    ops = _ops()
    from lidar_ai_solution_b200 import cabi
    grid = (9, 33, 33)
    coords = scenes.make_coords(600, grid, 4)
    dc, n_ptr, st = _dev(coords), ops.device_count(600), ops.new_status()
    table = ops.hash_build(dc, n_ptr, grid, status=st)
    oc, n_out, dm, _, _ = ops.down_map(dc, n_ptr, grid, table, (3, 3, 3), (2, 2, 2), (1, 1, 1),
                                       cap_out=64, status=st)
    torch.cuda.synchronize()
    assert int(n_out.item()) == 64
    assert int(st.cpu().numpy()[0]) & cabi.ST_OVERFLOW
    roc, rdm, _, _, rn = orc.down_map(coords, grid, (3, 3, 3), (2, 2, 2), (1, 1, 1), cap=64)
    assert rn > 64 and np.array_equal(oc.cpu().numpy(), roc)
    assert np.array_equal(dm.cpu().numpy(), rdm)


# --------------------------------------------------------------- convolutions
def _int8_layer(n, c_in, c_out, seed, simt, out_kind, grid=(41, 180, 180), hint=False):
    ops = _ops()
    pb = int8_problem(n, c_in, c_out, grid, seed)
    m_ref, _ = orc.subm_map(pb["coords"], grid)
    y32 = orc.conv_i8(pb["xq"], m_ref, n, pb["wq"], pb["scale"], pb["bias"], orc.ACT_RELU,
                      orc.KIND_F32)
    inv_out = np.float32(127.0) / np.float32(max(float(np.abs(y32).max()), 1e-6))
    ref = orc.conv_i8(pb["xq"], m_ref, n, pb["wq"], pb["scale"], pb["bias"], orc.ACT_RELU,
                      out_kind, float(inv_out))
    n_ptr, st = ops.device_count(n), ops.new_status()
    wts = ops.ConvWeights(pb["wq"], ops.I8, pb["scale"], pb["bias"])
    out = ops.conv_forward(_dev(pb["xq"]), _dev(m_ref), n_ptr, wts, act=ops.ACT_RELU,
                           out_kind=out_kind, inv_out_scale=float(inv_out), force_simt=simt,
                           status=st, n_in_ptr=n_ptr if hint else None)
    torch.cuda.synchronize()
    _status_ok(st)
    return out.cpu().numpy(), ref


@pytest.mark.parametrize("c", [16, 32, 64, 128])
@pytest.mark.parametrize("simt", [False, True])
def test_conv_int8_bit_exact(c, simt):
    """int8 x int8 -> int32 is exact, the epilogue is defined operation by operation,
    so the requantised int8 output must be identical (tolerance 0 LSB)."""
    got, ref = _int8_layer(3000 if simt else 10000, c, c, seed=c, simt=simt, out_kind=orc.KIND_I8)
    assert got.dtype == np.int8 and np.array_equal(got, ref)


@pytest.mark.parametrize("c", [16, 32, 64, 128])
@pytest.mark.parametrize("n", [120000, 200000])
def test_conv_int8_bit_exact_at_benchmark_sizes(c, n):
    """The layer sweep of the benchmark configurations: SubM 3x3x3, Cin = Cout = c, on the
    41x1440x1440 grid with 120 k and 200 k voxels (many tiles per CTA, balanced tile heights,
    the L2 prefetch running ahead of the gather): identical to the oracle."""
    got, ref = _int8_layer(n, c, c, seed=c + n, simt=False, out_kind=orc.KIND_I8,
                           grid=(41, 1440, 1440), hint=True)
    assert got.dtype == np.int8 and np.array_equal(got, ref)


@pytest.mark.parametrize("cin,cout", [(16, 32), (32, 64), (64, 128), (128, 16)])
def test_conv_int8_mixed_channels_fp16_out(cin, cout):
    got, ref = _int8_layer(4097, cin, cout, seed=cin + cout, simt=False, out_kind=orc.KIND_F16)
    assert np.array_equal(got.view(np.uint16), ref.view(np.uint16))


@pytest.mark.parametrize("n", [0, 1, 127, 128, 129, 257])
def test_conv_int8_ragged_row_counts(n):
    if n == 0:
        ops = _ops()
        wts = ops.ConvWeights(np.zeros((16, 27, 16), np.int8), ops.I8, np.ones(16, np.float32),
                              np.zeros(16, np.float32))
        st = ops.new_status()
        out = ops.conv_forward(torch.zeros((1, 16), dtype=torch.int8, device="cuda"),
                               torch.full((27, 1), -1, dtype=torch.int32, device="cuda"),
                               ops.device_count(0), wts, out_kind=ops.I8, status=st)
        torch.cuda.synchronize()
        _status_ok(st)
        assert out.shape == (1, 16)
        return
    got, ref = _int8_layer(n, 32, 32, seed=n, simt=False, out_kind=orc.KIND_I8, grid=(5, 9, 11))
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("n", [1, 3, 255, 256, 257, 511, 513])
@pytest.mark.parametrize("out_kind", ["i8", "f16"])
def test_conv_int8_ragged_row_counts_wide_outputs(n, out_kind):
    """Tiles are 256 rows and the epilogue stores groups of 4 rows per lane quad: partial
    tiles, partial groups, single-row inputs, with 2 weight replicas on the lanes."""
    kind = orc.KIND_I8 if out_kind == "i8" else orc.KIND_F16
    got, ref = _int8_layer(n, 32, 64, seed=100 + n, simt=False, out_kind=kind, grid=(7, 11, 13))
    assert np.array_equal(got.view(np.uint8), ref.view(np.uint8))


def _f16_problem(n, cin, cout, seed, grid=(41, 180, 180), kvol=27):
    rng = np.random.default_rng(seed)
    coords = scenes.make_coords(n, grid, seed)
    x = rng.standard_normal((n, cin)).astype(np.float16)
    w = kaiming(rng, cout, kvol, cin).astype(np.float16)
    bias = (rng.standard_normal(cout) * 0.1).astype(np.float32)
    return coords, x, w, bias


@pytest.mark.parametrize("c", [16, 32, 64, 128])
def test_conv_fp16_tensor_core(c):
    """fp16 operands, fp32 accumulation in a different order than the oracle:
    tolerance 1e-2 relative to the layer's output magnitude."""
    ops = _ops()
    grid, n = (41, 180, 180), 8000
    coords, x, w, bias = _f16_problem(n, c, c, seed=c + 1)
    m_ref, _ = orc.subm_map(coords, grid)
    ref = orc.conv_f16(x, m_ref, n, w, bias, orc.ACT_RELU, orc.KIND_F16).astype(np.float32)
    wts = ops.ConvWeights(w, ops.F16, None, bias)
    st = ops.new_status()
    out = ops.conv_forward(_dev(x), _dev(m_ref), ops.device_count(n), wts, act=ops.ACT_RELU,
                           out_kind=ops.F16, status=st)
    torch.cuda.synchronize()
    _status_ok(st)
    got = out.cpu().numpy().astype(np.float32)
    tol = 1e-2 * max(float(np.abs(ref).max()), 1e-6)
    assert float(np.abs(got - ref).max()) <= tol


def test_conv_fp16_cuda_core_bit_exact_and_first_layer_padding():
    """Cin = 5 padded to 8 (the backbone's first layer) on the tensor-core kernel vs the
    CUDA-core kernel on the unpadded data; the CUDA-core kernel equals the oracle bit for bit."""
    ops = _ops()
    grid, n = (41, 180, 180), 6000
    coords, x, w, bias = _f16_problem(n, 5, 16, seed=11)
    m_ref, _ = orc.subm_map(coords, grid)
    ref = orc.conv_f16(x, m_ref, n, w, bias, orc.ACT_RELU, orc.KIND_F16)
    n_ptr, md = ops.device_count(n), _dev(m_ref)
    simt = ops.conv_forward(_dev(x), md, n_ptr, ops.ConvWeights(w, ops.F16, None, bias),
                            act=ops.ACT_RELU, out_kind=ops.F16, force_simt=True)
    assert np.array_equal(simt.cpu().numpy().view(np.uint16), ref.view(np.uint16))
    wp = np.zeros((16, 27, 8), np.float16)
    wp[:, :, :5] = w
    xp = ops.convert(_dev(x), ops.F16, 8, 1.0, n_ptr)
    st = ops.new_status()
    tc = ops.conv_forward(xp, md, n_ptr, ops.ConvWeights(wp, ops.F16, None, bias),
                          act=ops.ACT_RELU, out_kind=ops.F16, status=st)
    torch.cuda.synchronize()
    _status_ok(st)
    r32 = ref.astype(np.float32)
    assert float(np.abs(tc.cpu().numpy().astype(np.float32) - r32).max()) <= 1e-2 * np.abs(r32).max()


@pytest.mark.parametrize("c,n", [(16, 5000), (32, 5001), (64, 5000), (64, 4999), (128, 2050)])
@pytest.mark.parametrize("res_kind", ["i8", "f16"])
def test_conv_int8_fused_residual_all_widths(c, n, res_kind):
    """Fused conv + Add&ReLU == oracle conv (stored int8) followed by oracle add, for every
    output width (8, 4, 2 or 1 copies of the weights on the accumulator lanes), int8 and
    fp16 residual operands, row counts that leave partial tiles."""
    ops = _ops()
    grid = (41, 180, 180)
    pb = int8_problem(n, c, c, grid, seed=40 + c)
    m_ref, _ = orc.subm_map(pb["coords"], grid)
    rng = np.random.default_rng(6)
    if res_kind == "i8":
        res, res_scale = rng.integers(-128, 128, (n, c)).astype(np.int8), 0.031
    else:
        res, res_scale = (rng.standard_normal((n, c)) * 2).astype(np.float16), 1.0
    mid_dr, out_dr = 3.0, 4.5
    mid = orc.conv_i8(pb["xq"], m_ref, n, pb["wq"], pb["scale"], pb["bias"], orc.ACT_NONE,
                      orc.KIND_I8, float(np.float32(127.0) / np.float32(mid_dr)))
    ref = orc.add(mid, float(np.float32(mid_dr) / np.float32(127.0)), res, res_scale, True,
                  orc.KIND_I8, float(np.float32(127.0) / np.float32(out_dr)))
    wts = ops.ConvWeights(pb["wq"], ops.I8, pb["scale"], pb["bias"])
    st = ops.new_status()
    out = ops.conv_forward(_dev(pb["xq"]), _dev(m_ref), ops.device_count(n), wts,
                           act=ops.ACT_NONE, out_kind=ops.I8,
                           inv_out_scale=float(np.float32(127.0) / np.float32(out_dr)),
                           res=_dev(res), res_scale=res_scale, mid_kind=ops.I8,
                           mid_inv_scale=float(np.float32(127.0) / np.float32(mid_dr)),
                           mid_scale=float(np.float32(mid_dr) / np.float32(127.0)),
                           res_relu=True, status=st)
    torch.cuda.synchronize()
    _status_ok(st)
    assert np.array_equal(out.cpu().numpy(), ref)


@pytest.mark.parametrize("simt", [False, True])
def test_conv_int8_fused_residual_equals_conv_then_add(simt):
    """Fused conv + Add&ReLU epilogue == oracle conv (stored int8) followed by oracle add."""
    ops = _ops()
    grid, n, c = (41, 180, 180), 5000, 64
    pb = int8_problem(n, c, c, grid, seed=21)
    m_ref, _ = orc.subm_map(pb["coords"], grid)
    rng = np.random.default_rng(5)
    res = rng.integers(-128, 128, (n, c)).astype(np.int8)
    res_scale, mid_dr, out_dr = 0.031, 3.0, 4.5
    mid = orc.conv_i8(pb["xq"], m_ref, n, pb["wq"], pb["scale"], pb["bias"], orc.ACT_NONE,
                      orc.KIND_I8, float(np.float32(127.0) / np.float32(mid_dr)))
    ref = orc.add(mid, float(np.float32(mid_dr) / np.float32(127.0)), res, res_scale, True,
                  orc.KIND_I8, float(np.float32(127.0) / np.float32(out_dr)))
    wts = ops.ConvWeights(pb["wq"], ops.I8, pb["scale"], pb["bias"])
    st = ops.new_status()
    out = ops.conv_forward(_dev(pb["xq"]), _dev(m_ref), ops.device_count(n), wts,
                           act=ops.ACT_NONE, out_kind=ops.I8,
                           inv_out_scale=float(np.float32(127.0) / np.float32(out_dr)),
                           res=_dev(res), res_scale=res_scale, mid_kind=ops.I8,
                           mid_inv_scale=float(np.float32(127.0) / np.float32(mid_dr)),
                           mid_scale=float(np.float32(mid_dr) / np.float32(127.0)),
                           res_relu=True, force_simt=simt, status=st)
    torch.cuda.synchronize()
    _status_ok(st)
    assert np.array_equal(out.cpu().numpy(), ref)


def test_strided_conv_int8_through_down_map():
    ops = _ops()
    grid, n = (41, 180, 180), 20000
    pb = int8_problem(n, 16, 32, grid, seed=8)
    roc, rdm, _, og, rn = orc.down_map(pb["coords"], grid, (3, 3, 3), (2, 2, 2), (1, 1, 1))
    ref = orc.conv_i8(pb["xq"], rdm, rn, pb["wq"], pb["scale"], pb["bias"], orc.ACT_RELU,
                      orc.KIND_I8, 20.0)
    dc, n_ptr, st = _dev(pb["coords"]), ops.device_count(n), ops.new_status()
    table = ops.hash_build(dc, n_ptr, grid, status=st)
    oc, n_out, dm, _, _ = ops.down_map(dc, n_ptr, grid, table, (3, 3, 3), (2, 2, 2), (1, 1, 1),
                                       status=st)
    wts = ops.ConvWeights(pb["wq"], ops.I8, pb["scale"], pb["bias"])
    out = ops.conv_forward(_dev(pb["xq"]), dm, n_out, wts, act=ops.ACT_RELU, out_kind=ops.I8,
                           inv_out_scale=20.0, status=st)
    torch.cuda.synchronize()
    _status_ok(st)
    assert int(n_out.item()) == rn
    assert np.array_equal(out.cpu().numpy()[:rn], ref)


# ---------------------------------------------------------------- elementwise
@pytest.mark.parametrize("ak,bk,ok", [(1, 1, 1), (0, 0, 1), (0, 0, 0), (1, 0, 0)])
@pytest.mark.parametrize("ch", [16, 24])
def test_add_relu(ak, bk, ok, ch):
    ops = _ops()
    rng = np.random.default_rng(ak * 4 + bk * 2 + ok)
    n = 3001

    def mk(kind):
        return (rng.integers(-128, 128, (n, ch)).astype(np.int8) if kind
                else rng.standard_normal((n, ch)).astype(np.float16))
    a, b = mk(ak), mk(bk)
    ref = orc.add(a, 0.05, b, 0.021, True, ok, 9.3)
    out = ops.add(_dev(a), 0.05, _dev(b), 0.021, ops.device_count(n), True, ok, 9.3)
    assert np.array_equal(out.cpu().numpy().view(np.uint8), ref.view(np.uint8))


def test_relu_and_convert():
    ops = _ops()
    rng = np.random.default_rng(0)
    n = 1000
    x8 = rng.integers(-128, 128, (n, 16)).astype(np.int8)
    xh = rng.standard_normal((n, 16)).astype(np.float16)
    n_ptr = ops.device_count(n)
    assert np.array_equal(ops.relu(_dev(x8), n_ptr).cpu().numpy(), orc.relu(x8))
    assert np.array_equal(ops.relu(_dev(xh), n_ptr).cpu().numpy().view(np.uint16),
                          orc.relu(xh).view(np.uint16))
    q = ops.convert(_dev(xh), ops.I8, 16, float(np.float32(127.0) / np.float32(3.0)), n_ptr)
    assert np.array_equal(q.cpu().numpy(), orc.quantize_f16(xh, 3.0))


@pytest.mark.parametrize("perm", [None, (0, 2, 1)])
@pytest.mark.parametrize("kind", [0, 1])
def test_scatter_dense(perm, kind):
    ops = _ops()
    grid, n, ch = (2, 180, 180), 7000, 128
    coords = scenes.make_coords(n, grid, 2)
    rng = np.random.default_rng(1)
    feat = (rng.integers(-128, 128, (n, ch)).astype(np.int8) if kind
            else rng.standard_normal((n, ch)).astype(np.float16))
    ref = orc.scatter_dense(feat, coords, grid, 1, 0.02, perm)
    out = ops.scatter_dense(_dev(feat), _dev(coords), ops.device_count(n), grid, 1, 0.02, perm)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), ref.view(np.uint16))


@pytest.mark.parametrize("perm", [None, (2, 0, 1)])
@pytest.mark.parametrize("in_kind,dynamic_range", [(0, 0.0), (0, 2.5), (1, 0.0), (1, 2.54), (1, 3.0)])
@pytest.mark.parametrize("layout,ch", [("NCHW", 128), ("NCHW32", 128), ("NCHW32", 24), ("NHWzC", 128),
                                       ("NHWzC", 24)])
def test_scatter_dense_layouts(layout, ch, in_kind, dynamic_range, perm):
    """Dense outputs in the engine's three layouts, fp16 or int8 (input_dynamic_range > 0):
    bit-exact against the restatement, padding channels and empty cells zero.  The int8 rows
    carry the scale 0.02 = 2.54 / 127, so the range 2.54 is the byte-copy case and 3.0 the
    rescaling one."""
    ops = _ops()
    grid, n = (2, 90, 100), 5000
    coords = scenes.make_coords(n, grid, 2)
    rng = np.random.default_rng(1)
    feat = (rng.integers(-128, 128, (n, ch)).astype(np.int8) if in_kind
            else rng.standard_normal((n, ch)).astype(np.float16))
    in_scale = float(np.float32(2.54) / np.float32(127.0)) if in_kind else 1.0
    if dynamic_range > 0:
        if in_kind and dynamic_range == 2.54:
            q = feat
        elif in_kind:
            inv = np.float32(127.0) / np.float32(dynamic_range)
            q = np.clip(np.rint((feat.astype(np.float32) * np.float32(in_scale)) * inv),
                        -128, 127).astype(np.int8)
        else:
            q = orc.quantize_f16(feat, dynamic_range)
        ref = orc.scatter_dense_i8(q, coords, grid, 1, perm)
    else:
        ref = orc.scatter_dense(feat, coords, grid, 1, in_scale, perm)
    ref = orc.dense_layout(ref, layout, ch)
    out = ops.scatter_dense_layout(_dev(feat), _dev(coords), ops.device_count(n), grid, layout,
                                   dynamic_range, 1, in_scale, perm).cpu().numpy()
    assert out.shape == ref.shape and out.dtype == ref.dtype
    assert np.array_equal(out.view(np.uint8), ref.view(np.uint8))


# ------------------------------------------------------------------ voxelizer
@pytest.mark.parametrize("kind", ["f32", "f16"])
def test_voxelizer_matches_sequential_reference(kind, golden_dir):
    ops = _ops()
    if kind == "f32":
        pts = scenes.make_points(120000, seed=3)
    else:
        pts = np.load(os.path.join(golden_dir, "sweep_points.npz"))["points"]
    prange, vs = scenes.CENTERPOINT_RANGE, scenes.CENTERPOINT_VOXEL
    gxyz = (1440, 1440, 40)
    rf, rc, rn = orc.voxelize(pts, prange, vs, gxyz, 160000, 10, 0)
    params = ops.voxel_params(prange, vs, gxyz, 5, 0 if kind == "f32" else 1, 10, 160000, 0)
    st = ops.new_status()
    feat, idx, n_ptr = ops.voxelize(_dev(pts), params, status=st)
    torch.cuda.synchronize()
    _status_ok(st)
    n = int(n_ptr.item())
    assert n == rn
    assert np.array_equal(idx.cpu().numpy()[:n], rc)
    assert np.array_equal(feat.cpu().numpy()[:n].view(np.uint16), rf.view(np.uint16))


def test_voxelizer_max_voxels_clips():
    ops = _ops()
    from lidar_ai_solution_b200 import cabi
    pts = scenes.make_points(20000, seed=9)
    prange, vs, gxyz = scenes.CENTERPOINT_RANGE, scenes.CENTERPOINT_VOXEL, (1440, 1440, 40)
    rf, rc, rn = orc.voxelize(pts, prange, vs, gxyz, 1000, 10, 1)
    params = ops.voxel_params(prange, vs, gxyz, 5, 0, 10, 1000, 1)
    st = ops.new_status()
    feat, idx, n_ptr = ops.voxelize(_dev(pts), params, status=st)
    torch.cuda.synchronize()
    assert rn > 1000 and int(n_ptr.item()) == 1000
    assert int(st.cpu().numpy()[0]) & cabi.ST_OVERFLOW
    assert np.array_equal(idx.cpu().numpy(), rc)
    assert np.array_equal(feat.cpu().numpy().view(np.uint16), rf.view(np.uint16))


def test_inverse_map_is_the_strided_map_with_rows_swapped():
    """spconvb_inverse_map: map[k][i] = o exactly for the pairs (k, i, o) of the strided
    rulebook (oracle down_map), -1 elsewhere."""
    ops = _ops()
    grid, n = (21, 180, 180), 15000
    coords = scenes.make_coords(n, grid, 31)
    ks, st_, pd = (3, 3, 3), (2, 2, 2), (1, 1, 1)
    roc, rdm, _, og, rn = orc.down_map(coords, grid, ks, st_, pd)
    ref = np.full((27, n), -1, np.int32)
    for k in range(27):
        o = np.nonzero(rdm[k, :rn] >= 0)[0]
        ref[k, rdm[k, o]] = o
    dc, n_ptr, st = _dev(coords), ops.device_count(n), ops.new_status()
    oc, n_out, dm, _, _, ws = ops.down_map(dc, n_ptr, grid, None, ks, st_, pd, status=st,
                                           want_table=False, return_ws=True)
    inv = ops.inverse_map(dc, n_ptr, grid, ws, oc.shape[0], ks, st_, pd, status=st)
    torch.cuda.synchronize()
    _status_ok(st)
    assert int(n_out.item()) == rn
    assert np.array_equal(inv.cpu().numpy(), ref)
    # asymmetric geometry: kernel (3,1,1), stride (2,1,1), no padding
    ks, st_, pd = (3, 1, 1), (2, 1, 1), (0, 0, 0)
    roc, rdm, _, og, rn = orc.down_map(coords, grid, ks, st_, pd)
    ref = np.full((3, n), -1, np.int32)
    for k in range(3):
        o = np.nonzero(rdm[k, :rn] >= 0)[0]
        ref[k, rdm[k, o]] = o
    oc, n_out, dm, _, _, ws = ops.down_map(dc, n_ptr, grid, None, ks, st_, pd, status=st,
                                           want_table=False, return_ws=True)
    inv = ops.inverse_map(dc, n_ptr, grid, ws, oc.shape[0], ks, st_, pd, status=st)
    torch.cuda.synchronize()
    assert np.array_equal(inv.cpu().numpy(), ref)


def test_conv_bounded_wait_runs_out_and_the_context_survives():
    """Failure detection without a GPU fault: with `wait_test` the producers of the
    tensor-core kernel never signal a stage, so the MMA role's wait on it must run out
    (250 ms), raise the CTA-wide abort flag, let every role leave its loop, free TMEM and
    return with SPCONVB_ST_TIMEOUT in the status block.  The next launch on the same
    context is then bit-exact again."""
    ops = _ops()
    from lidar_ai_solution_b200 import cabi
    grid, n, c = (41, 180, 180), 2000, 32
    pb = int8_problem(n, c, c, grid, seed=77)
    m_ref, _ = orc.subm_map(pb["coords"], grid)
    ref = orc.conv_i8(pb["xq"], m_ref, n, pb["wq"], pb["scale"], pb["bias"], orc.ACT_RELU,
                      orc.KIND_I8, 9.0)
    wts = ops.ConvWeights(pb["wq"], ops.I8, pb["scale"], pb["bias"])
    x, m, n_ptr = _dev(pb["xq"]), _dev(m_ref), ops.device_count(n)
    st = ops.new_status()
    ops.conv_forward(x, m, n_ptr, wts, act=ops.ACT_RELU, out_kind=ops.I8, inv_out_scale=9.0,
                     status=st, wait_test=1)
    torch.cuda.synchronize()
    assert int(st.cpu().numpy()[0]) & cabi.ST_TIMEOUT
    st.zero_()
    out = ops.conv_forward(x, m, n_ptr, wts, act=ops.ACT_RELU, out_kind=ops.I8,
                           inv_out_scale=9.0, status=st)
    torch.cuda.synchronize()
    _status_ok(st)
    assert np.array_equal(out.cpu().numpy(), ref)


def _shape_sweep_cases():
    rng = np.random.default_rng(2024)
    chans = [16, 32, 64, 128]
    cases = []
    for i in range(28):
        cin, cout = int(rng.choice(chans)), int(rng.choice(chans))
        n = int(rng.choice([1, 31, 33, 255, 257, 1000, 4736, 4737, 9473, 20000, 37889]))
        kind = ["subm", "down", "k311"][i % 3]
        cases.append((cin, cout, n, kind, i % 2 == 0, 100 + i))
    return cases


@pytest.mark.parametrize("cin,cout,n,kind,i8_out,seed", _shape_sweep_cases())
def test_conv_int8_shape_sweep_bit_exact(cin, cout, n, kind, i8_out, seed):
    """Channel pairs select how many copies of the weights sit on the accumulator lanes and
    whether they stay resident; row counts select the tile height (32..256) and leave
    partial tiles; the three rulebook kinds give 27 or 3 taps.  Everything int8, so the
    tensor-core kernel must match the oracle bit for bit."""
    ops = _ops()
    grid = (41, 180, 180)
    kvol = 3 if kind == "k311" else 27
    pb = int8_problem(n, cin, cout, grid, seed=seed, kvol=kvol)
    if kind == "subm":
        m_ref, _ = orc.subm_map(pb["coords"], grid)
        n_out = n
    elif kind == "down":
        _, m_ref, _, _, n_out = orc.down_map(pb["coords"], grid, (3, 3, 3), (2, 2, 2), (1, 1, 1))
    else:
        _, m_ref, _, _, n_out = orc.down_map(pb["coords"], grid, (3, 1, 1), (2, 1, 1), (0, 0, 0))
    okind = orc.KIND_I8 if i8_out else orc.KIND_F16
    inv = 11.0 if i8_out else 1.0
    ref = orc.conv_i8(pb["xq"], m_ref, n_out, pb["wq"], pb["scale"], pb["bias"], orc.ACT_RELU,
                      okind, inv)
    wts = ops.ConvWeights(pb["wq"], ops.I8, pb["scale"], pb["bias"])
    assert wts.packed is not None
    st = ops.new_status()
    md = _dev(np.ascontiguousarray(m_ref))
    out = ops.conv_forward(_dev(pb["xq"]), md, ops.device_count(n_out), wts, act=ops.ACT_RELU,
                           out_kind=ops.I8 if i8_out else ops.F16, inv_out_scale=inv, status=st)
    torch.cuda.synchronize()
    _status_ok(st)
    assert np.array_equal(out.cpu().numpy()[:n_out].view(np.uint8), ref[:n_out].view(np.uint8))
