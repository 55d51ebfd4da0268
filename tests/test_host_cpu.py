"""CPU-only checks of the host side: the C-ABI library loads and exports every
symbol its header declares, the ONNX writer and the protobuf-free reader agree,
loader errors, scene generator, frame sharding over two gloo ranks."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from lidar_ai_solution_b200 import models, onnx_writer, scenes, sharding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    from lidar_ai_solution_b200 import cabi
    return cabi, cabi.lib()


def test_library_exports_every_declared_symbol():
    cabi, lib = _lib()
    header = open(os.path.join(ROOT, "include", "spconvb.h")).read() + \
        open(os.path.join(ROOT, "include", "spconvb_centerpoint.h")).read()
    declared = set(re.findall(r"SPCONVB_API[^;(]*?\b(spconvb_\w+)\s*\(", header))
    assert len(declared) >= 52
    from lidar_ai_solution_b200 import engine_abi
    bound = set(cabi.SYMBOLS) | set(engine_abi.SYMBOLS)
    for name in sorted(declared):
        assert hasattr(lib, name), "libspconvb.so does not export %s" % name
    assert declared <= bound, "symbols without a ctypes signature: %s" % sorted(declared - bound)
    assert b"sm_100a" in lib.spconvb_version()
    assert lib.spconvb_error_string(0) == b"ok"


def test_host_side_size_helpers_need_no_gpu():
    cabi, lib = _lib()
    from lidar_ai_solution_b200 import centerpoint_post
    cp = centerpoint_post.default_params()
    assert (cp.H, cp.W, cp.max_det, cp.nms_post_max) == (180, 180, 1000, 83)
    assert abs(cp.nms_iou_threshold - 0.2) < 1e-7 and abs(cp.post_center_range[3] - 61.2) < 1e-6
    need = lib.spconvb_cp_workspace_bytes(cabi.C.byref(cp), 6)
    assert 6 * (180 * 180 * 8 + 1000 * (44 + 32 + 128)) <= need < 4 << 20
    assert lib.spconvb_cp_workspace_bytes(cabi.C.byref(cp), 9) == 0
    cp.max_det = 2000
    assert lib.spconvb_cp_workspace_bytes(cabi.C.byref(cp), 6) == 0
    assert lib.spconvb_hash_slots(120000) == 262144
    assert lib.spconvb_out_extent(41, 3, 2, 1, 1) == 21
    assert lib.spconvb_out_extent(11, 3, 2, 0, 1) == 5
    assert lib.spconvb_out_extent(5, 3, 2, 0, 1) == 2
    assert lib.spconvb_down_workspace_bytes(cabi.i3((21, 720, 720)), 1) <= cabi.STATIC_SCRATCH_BYTES
    assert lib.spconvb_conv_supported(cabi.I8, 64, 64) == 1
    assert lib.spconvb_conv_supported(cabi.I8, 5, 16) == 0
    assert lib.spconvb_conv_supported(cabi.F16, 8, 16) == 1
    assert lib.spconvb_conv_packed_bytes(cabi.I8, 16, 16, 27) == 4 * 16 * 128


def test_argument_checks_come_before_any_device_work():
    """Calls that are refused for their arguments return before the first CUDA call, so they
    can be checked without a GPU: the allocation-free strided rulebook refuses null buffers, an
    output table that is not a power of two or too small, and grids beyond its scratch area;
    the elementwise entry points refuse a zero capacity."""
    cabi, lib = _lib()
    g, k, s, p, d = (cabi.i3(v) for v in ((21, 64, 64), (3, 3, 3), (2, 2, 2), (1, 1, 1), (1, 1, 1)))
    fake = 0x1000  # never dereferenced: every call below is refused first

    def static(coords=fake, out_coords=fake, table=None, slots=0, grid=g, cap_out=1000, s=s):
        return lib.spconvb_down_map_static(coords, fake, 1000, 0, grid, 1, k, s, p, d, None, 0,
                                           out_coords, fake, cap_out, fake, table, slots, 0, None,
                                           None)
    assert static(coords=None) == -1 and static(out_coords=None) == -1       # SPCONVB_E_ARG
    assert static(table=fake, slots=3000) == -1      # not a power of two
    assert static(table=fake, slots=1024) == -1      # fewer than 2 * cap_out slots
    # stride 1 keeps 85 M output cells: far beyond the scratch area
    assert static(grid=cabi.i3((41, 1440, 1440)), s=cabi.i3((1, 1, 1))) == cabi.E_SCRATCH_LIMIT
    assert lib.spconvb_relu(fake, cabi.I8, 16, fake, 0, fake, None) == -1
    assert lib.spconvb_convert(fake, cabi.F16, 5, cabi.F16, 4, 1.0, fake, 100, fake, None) == -1


def test_weight_packing_layout():
    """Chunk j, row n, 16-byte segment c is stored at segment c ^ (n % 8) of row n."""
    cabi, lib = _lib()
    cout, kvol, cin = 16, 27, 16
    w = np.arange(cout * kvol * cin, dtype=np.int64).reshape(cout, kvol, cin)
    w = ((w * 7 + 3) % 251 - 125).astype(np.int8)
    nbytes = lib.spconvb_conv_packed_bytes(cabi.I8, cin, cout, kvol)
    dst = np.zeros(nbytes, np.uint8)
    assert lib.spconvb_conv_pack_weights(cabi.I8, cin, cout, kvol, w.ctypes.data_as(C.c_void_p),
                                         dst.ctypes.data_as(C.c_void_p)) == 0
    flat = np.zeros((cout, 4 * 128), np.int8)
    flat[:, : kvol * cin] = w.reshape(cout, -1)
    img = dst.view(np.int8).reshape(4, cout // 8, 8, 8, 16)      # chunk, group, row, seg, byte
    for j in range(4):
        for n in range(cout):
            for c in range(8):
                want = flat[n, j * 128 + c * 16: j * 128 + c * 16 + 16]
                assert np.array_equal(img[j, n // 8, n % 8, c ^ (n % 8)], want)


def _inspect(lib, path):
    buf = C.create_string_buffer(1 << 20)
    rc = lib.spconvb_onnx_inspect(os.fsencode(path), buf, len(buf))
    return rc, buf.value.decode()


def test_onnx_writer_and_reader_round_trip(tmp_path):
    cabi, lib = _lib()
    model = models.scn_backbone("bevfusion", seed=3)
    ranges = {t: 1.0 + i for i, t in enumerate(models.tensor_ids(model))}
    qm = models.quantize(model, ranges)
    path = str(tmp_path / "bev.scn.onnx")
    onnx_writer.save(qm, path)
    rc, text = _inspect(lib, path)
    assert rc == 0
    lines = text.strip().split("\n")
    assert lines[0].startswith("Input 0 ")
    convs = [ln for ln in lines if ln.startswith("SparseConvolution")]
    assert len(convs) == 21 and len([ln for ln in lines if ln.startswith("Add")]) == 8
    assert "cin=5 cout=16 k=3,3,3 s=1,1,1 p=1,1,1 d=1,1,1 subm=1 relu=1 bound=200000 rulebook=subm0 prec=1 out_prec=2" in convs[0]
    assert "k=3,3,3 s=2,2,2 p=0,1,1" in convs[15] and "cin=64 cout=128" in convs[15]
    assert "k=3,1,1 s=2,1,1 p=0,0,0" in convs[20] and "out_prec=1" in convs[20]
    assert "n_wdr=128 bias=128" in convs[20]
    node = qm["nodes"][1]
    assert ("in_dr=%.9g" % np.float32(node["input_dynamic_range"])) in convs[1]
    assert any(ln.startswith("Transpose") and "dims=0,1,2,4,3," in ln for ln in lines)
    assert lines[-1] == "Output %s" % qm["outputs"][0][0]
    assert "Reshape" in lines[-2] and "dims=1,256,180,180," in lines[-2]
    dense = [ln for ln in lines if ln.startswith("ScatterDense")]
    assert len(dense) == 1 and dense[0].endswith(" layout=1 in_dr=0")
    # output_layout and input_dynamic_range of ScatterDense survive the file
    for layout, code in (("NCHW32", 2), ("NHWzC", 3)):
        m2 = dict(qm, nodes=[dict(n) for n in qm["nodes"]])
        d = [n for n in m2["nodes"] if n["op"] == "dense"][0]
        d["output_layout"], d["input_dynamic_range"] = layout, 4.25
        onnx_writer.save(m2, path)
        rc, text = _inspect(lib, path)
        assert rc == 0
        assert (" layout=%d in_dr=4.25" % code) in text


def test_loader_error_codes(tmp_path):
    cabi, lib = _lib()
    blob = onnx_writer.serialize(models.single_layer(16, 32))
    cases = {"trunc.onnx": blob[: len(blob) // 3], "empty.onnx": b"",
             "badop.onnx": blob.replace(b"SparseConvolution", b"SparseConvolutioX"),
             "garbage.onnx": bytes(range(256)) * 8}
    for name, data in cases.items():
        p = tmp_path / name
        p.write_bytes(data)
        rc, _ = _inspect(lib, str(p))
        assert rc in (-4, -5), (name, rc)
    assert _inspect(lib, str(tmp_path / "missing.onnx"))[0] == -4
    rc, _ = _inspect(lib, str(tmp_path / "badop.onnx"))
    assert rc == -5                              # unsupported operator, like the reference loader


def test_scene_generator_is_seeded_and_unique():
    a = scenes.make_coords(20000, (41, 180, 180), 0)
    b = scenes.make_coords(20000, (41, 180, 180), 0)
    c = scenes.make_coords(20000, (41, 180, 180), 1)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    keys = (a[:, 1] * 180 + a[:, 2]) * 180 + a[:, 3]
    assert len(np.unique(keys)) == 20000 and a[:, 0].max() == 0
    assert a[:, 1].max() < 41 and a[:, 2].max() < 180 and a[:, 3].max() < 180
    ground = np.mean((a[:, 1] >= 2) & (a[:, 1] <= 6))
    assert ground > 0.7            # the ground band plus the boxes that fall inside it
    f = scenes.make_point_features(a, 0)
    assert f.dtype == np.float16 and f.shape == (20000, 5)
    assert scenes.make_coords(0).shape == (0, 4)


def test_frame_assignment():
    seeds0, seeds1 = sharding.frame_seeds(0, 16), sharding.frame_seeds(1, 16)
    assert len(set(seeds0) | set(seeds1)) == 32
    counts = [200, 60, 150, 90, 120, 180, 70, 110]
    parts = sharding.assign_frames(counts, 2)
    assert sorted(parts[0] + parts[1]) == list(range(8))
    loads = [sum(counts[i] for i in p) for p in parts]
    assert abs(loads[0] - loads[1]) <= 60
    assert sharding.aggregate(3.5, 16) == (3.5, 16)


_RANK_SCRIPT = r"""
import os, sys
sys.path.insert(0, %(root)r)
import torch.distributed as dist
from lidar_ai_solution_b200 import sharding
rank = int(os.environ["RANK"])
dist.init_process_group("gloo")
seeds = sharding.frame_seeds(rank, 4)
ms, frames = sharding.aggregate(10.0 + 5.0 * rank, len(seeds), dist)
gathered = [None, None]
dist.all_gather_object(gathered, seeds)
assert not (set(gathered[0]) & set(gathered[1]))
assert (ms, frames) == (15.0, 8), (ms, frames)
dist.barrier()
dist.destroy_process_group()
print("rank %%d ok" %% rank)
"""


def test_two_rank_aggregation_over_gloo(tmp_path):
    """world_size 2 on CPU: the timed region's only communication (max of the elapsed time,
    sum of frames) and the disjoint seeds."""
    pytest.importorskip("torch")
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT % {"root": ROOT})
    port = 29500 + (os.getpid() % 2000)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    for rank, p in enumerate(procs):
        out, _ = p.communicate(timeout=180)
        assert p.returncode == 0, out
        assert "rank %d ok" % rank in out


# ------------------------------------------------------------------ tensor files, CLI
def test_tensor_file_round_trip_matches_reference_bytes(tmp_path):
    """tool/tensor.py:24-69: header of three int32, int32 dims, raw data; a file written
    here must be byte-identical to the fixture written in that format."""
    from lidar_ai_solution_b200 import tensor_file
    golden = os.path.join(os.path.dirname(__file__), "golden", "sample.tensor")
    a = tensor_file.load(golden)
    assert a.shape == (40, 5) and a.dtype == np.float16
    out = tmp_path / "x.tensor"
    tensor_file.save(a, out)
    assert open(out, "rb").read() == open(golden, "rb").read()
    for dt in (np.int32, np.float32, np.int8, np.uint8, np.int64):
        x = (np.arange(24).reshape(2, 3, 4) % 100).astype(dt)
        tensor_file.save(x, out)
        y = tensor_file.load(out)
        assert y.dtype == dt and np.array_equal(x, y)


def test_tensor_file_rejects_bad_files(tmp_path):
    from lidar_ai_solution_b200 import tensor_file
    bad = tmp_path / "bad.tensor"
    bad.write_bytes(b"\x00" * 32)
    with pytest.raises(RuntimeError):
        tensor_file.load(bad)
    bad.write_bytes(np.array([0x33FF1101, 2, 2, 4, 4], np.int32).tobytes() + b"\x00" * 8)
    with pytest.raises(RuntimeError):
        tensor_file.load(bad)  # truncated data
    with pytest.raises(RuntimeError):
        tensor_file.save(np.zeros(3, np.complex64), bad)


def test_infer_cli_options_follow_the_reference():
    """Option names and defaults of src/infer.cpp:475-491."""
    from lidar_ai_solution_b200 import infer
    a = infer.parse_args(["--onnx", "m.onnx", "--feature", "f", "--indice", "i",
                          "--grid_size", "41,1440,1440"])
    assert a.fp16 and not a.int8 and not a.cudagraph and not a.dds and not a.profiling
    assert a.fixed_points == 10000 and not a.search_best_perf and not a.stress
    a = infer.parse_args(["--synthetic", "centerpoint", "--int8", "--cudagraph=true", "--dds",
                          "--blackwell", "--sortmask=false", "--fixed_points", "4096"])
    assert a.int8 and a.cudagraph and a.dds and a.blackwell and not a.sortmask
    assert a.fixed_points == 4096
