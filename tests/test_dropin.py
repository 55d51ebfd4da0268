"""The drop-in boundary: C++ programs written against the reference's two header
generations build against include/spconv (v1.3) and include/spconv_v10 (v1.0), link with
libspconv.so / libspconv_v10.so, and (on a GPU) give the same output as the C ABI."""
import os
import shutil
import subprocess

import numpy as np
import pytest

from lidar_ai_solution_b200 import models, onnx_writer, scenes

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "lidar_ai_solution_b200", "lib")
# the reference checkout: $SPCONV_REFERENCE_ROOT, else a "reference" directory beside this repo
REF = os.environ.get("SPCONV_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))
NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"

pytestmark = pytest.mark.skipif(not os.path.exists(NVCC), reason="nvcc not available")


def _build_libs():
    from lidar_ai_solution_b200 import build
    build.build()


def _nvcc(args, cwd=None):
    r = subprocess.run([NVCC, "-std=c++17", "-O1", *args], capture_output=True, text=True, cwd=cwd)
    assert r.returncode == 0, r.stdout + r.stderr


def _link_flags(v10=False):
    libs = ["-lspconv_v10", "-lspconvb"] if v10 else ["-lspconv", "-lspconvb"]
    return ["-L", LIB, *libs, "-Xlinker", "-rpath," + LIB]


def _compile_driver(tmp_path, v10):
    _build_libs()
    src = os.path.join(ROOT, "tests", "cpp", "dropin_v10.cpp" if v10 else "dropin_v13.cpp")
    inc = os.path.join(ROOT, "include", "spconv_v10") if v10 else os.path.join(ROOT, "include")
    exe = str(tmp_path / ("dropin_v10" if v10 else "dropin_v13"))
    _nvcc(["-I", inc, src, "-o", exe, *_link_flags(v10)])
    return exe


def test_own_drivers_compile_and_link(tmp_path):
    assert os.path.exists(_compile_driver(tmp_path, v10=False))
    assert os.path.exists(_compile_driver(tmp_path, v10=True))


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference checkout not mounted")
def test_reference_sources_compile_and_link_unchanged(tmp_path):
    """The reference's own demo (`pro`: src/main.cpp + src/voxelization.cu) and its BEVFusion
    lidar wrapper (lidar-scn.cpp + lidar-voxelization.cu) are compiled where they lie, against
    this repository's headers, and linked against its libraries.  Their protobuf-based
    onnx-parser.cpp is left out: libspconv.so exports a loader with the same signature."""
    _build_libs()
    inc = os.path.join(ROOT, "include")
    sc = os.path.join(REF, "libraries", "3DSparseConvolution", "src")
    objs = []
    for name in ("main.cpp", "voxelization.cu"):
        obj = str(tmp_path / (name + ".o"))
        # their .cu files lean on <stdint.h> arriving through older CUDA headers
        _nvcc(["--pre-include", "stdint.h", "-I", inc, "-I", sc, "-c", os.path.join(sc, name),
               "-o", obj])
        objs.append(obj)
    _nvcc([*objs, "-o", str(tmp_path / "pro"), *_link_flags()])

    bev = os.path.join(REF, "CUDA-BEVFusion", "src")
    objs = []
    for name in ("bevfusion/lidar-scn.cpp", "bevfusion/lidar-voxelization.cu"):
        obj = str(tmp_path / (os.path.basename(name) + ".o"))
        _nvcc(["--pre-include", "stdint.h", "-I", inc, "-I", bev, "-Xcompiler", "-fPIC", "-c",
               os.path.join(bev, name), "-o", obj])
        objs.append(obj)
    # shared object with no unresolved spconv symbols left
    out = str(tmp_path / "liblidar_scn.so")
    _nvcc(["-shared", *objs, "-o", out, *_link_flags(), "-Xlinker", "--no-undefined",
           "-Xlinker", "--unresolved-symbols=report-all", "-Xlinker", "--allow-shlib-undefined"])
    assert os.path.exists(out)


def _write_tensor(path, array):
    codes = {"float16": 2, "int32": 1}
    with open(path, "wb") as f:
        f.write(np.array([0x33FF1101, array.ndim, codes[str(array.dtype)]], np.int32).tobytes())
        f.write(np.array(array.shape, np.int32).tobytes())
        f.write(np.ascontiguousarray(array).tobytes())


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["v13", "v13-dds", "v10"])
def test_cpp_interfaces_match_the_c_abi(tmp_path, mode):
    import torch
    from lidar_ai_solution_b200 import engine
    grid = (41, 360, 360)
    coords = scenes.make_coords(9000, grid, 7)
    feats = scenes.make_point_features(coords, 7)
    model = models.scn_backbone("centerpoint", seed=7, grid_zyx=grid, output_bound=30000)
    df, dc = torch.from_numpy(feats).cuda(), torch.from_numpy(coords).cuda()
    qm = models.quantize(model, engine.calibrate(model, df, dc, grid))
    onnx = str(tmp_path / "centerpoint.scn.PTQ.onnx")
    onnx_writer.save(qm, onnx)
    e = engine.Engine.from_onnx(onnx, engine.PRECISION_INT8)
    e.forward(df, dc, grid)
    torch.cuda.synchronize()
    want = e.output(0).cpu().numpy()

    if mode == "v10":
        exe = _compile_driver(tmp_path, v10=True)
        feats.tofile(str(tmp_path / "f.bin"))
        coords.tofile(str(tmp_path / "i.bin"))
        out = str(tmp_path / "out.bin")
        r = subprocess.run([exe, onnx, "int8", str(tmp_path / "f.bin"), str(tmp_path / "i.bin"),
                            str(len(feats)), "5", *map(str, grid), out], capture_output=True,
                           text=True)
        assert r.returncode == 0, r.stdout + r.stderr
        got = np.fromfile(out, np.float16).reshape(want.shape)
    else:
        exe = _compile_driver(tmp_path, v10=False)
        _write_tensor(str(tmp_path / "f.tensor"), feats)
        _write_tensor(str(tmp_path / "i.tensor"), coords)
        out = str(tmp_path / "out.tensor")
        args = [exe, onnx, "int8", str(tmp_path / "f.tensor"), str(tmp_path / "i.tensor"),
                *map(str, grid), out] + (["dds"] if mode.endswith("dds") else [])
        r = subprocess.run(args, capture_output=True, text=True)
        assert r.returncode == 0, r.stdout + r.stderr
        assert "1.3.2" in r.stdout and "1 x 256 x 45 x 45" in r.stdout
        raw = open(out, "rb").read()
        head = np.frombuffer(raw[:12], np.int32)
        assert head[0] == 0x33FF1101 and head[1] == 4 and head[2] == 2
        got = np.frombuffer(raw[12 + 16:], np.float16).reshape(want.shape)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@pytest.mark.gpu
@pytest.mark.parametrize("dds", [False, True])
def test_sparse_output_through_the_cpp_interface(tmp_path, dds):
    """A graph whose output is a sparse tensor (EngineBuilder::push_output on a convolution,
    engine.hpp:158): output(0) carries features, indices, grid and the device-side row count,
    and reports the input's row count when the host knows it."""
    import torch
    from lidar_ai_solution_b200 import engine
    grid = (41, 360, 360)
    n = 5000
    coords = scenes.make_coords(n, grid, 9)
    feats = scenes.make_point_features(coords, 9)
    model = models.single_layer(5, 16, seed=9, output_bound=8000)
    onnx = str(tmp_path / "layer.onnx")
    onnx_writer.save(model, onnx)
    e = engine.Engine.from_onnx(onnx, engine.PRECISION_FP16)
    e.forward(torch.from_numpy(feats).cuda(), torch.from_numpy(coords).cuda(), grid)
    torch.cuda.synchronize()
    want = e.output(0)[:n].cpu().numpy()
    exe = _compile_driver(tmp_path, v10=False)
    _write_tensor(str(tmp_path / "f.tensor"), feats)
    _write_tensor(str(tmp_path / "i.tensor"), coords)
    out = str(tmp_path / "out.tensor")
    args = [exe, onnx, "fp16", str(tmp_path / "f.tensor"), str(tmp_path / "i.tensor"),
            *map(str, grid), out] + (["dds"] if dds else [])
    r = subprocess.run(args, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    rows = 8000 if dds else n   # the capacity when only the device knows the count
    assert "sparse output: indices %d x 4, rows on device %d, grid 41 360 360" % (rows, n) in r.stdout, \
        r.stdout
    raw = open(out, "rb").read()
    head = np.frombuffer(raw[:12 + 8], np.int32)
    assert head[0] == 0x33FF1101 and head[1] == 2 and tuple(head[3:5]) == (rows, 16)
    got = np.frombuffer(raw[12 + 8:], np.float16).reshape(rows, 16)
    assert np.array_equal(got[:n].view(np.uint16), want.view(np.uint16))
