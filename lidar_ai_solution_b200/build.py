"""Builds the native libraries in-tree with nvcc for sm_100a.

    python -m lidar_ai_solution_b200.build [--force] [--verbose]

Outputs (next to the sources, git-ignored):
    lidar_ai_solution_b200/lib/libspconvb.so   kernels + engine behind the C ABI
    lidar_ai_solution_b200/lib/libspconv.so    C++ facade with the reference's
                                               v1.3 `spconv::` interface
    lidar_ai_solution_b200/lib/libspconv_v10.so  the v1.0 interface CUDA-CenterPoint uses
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(PKG, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


# Sources whose float arithmetic must round operation by operation (no multiply-add contraction)
PER_FILE_FLAGS = {"centerpoint_post.cu": ("-fmad=false",)}


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA extension cannot be built")


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src: str, obj: str, verbose: bool, extra=()):
    cmd = [_nvcc(), *extra, *NVCC_FLAGS, "-c", src, "-o", obj]  # extra include dirs come first
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    if verbose:
        print(r.stderr)
    return obj


def _link(objs, out, libs=(), verbose=False):
    cmd = [_nvcc(), "-shared", "-o", out, *objs, "-Xlinker", "-rpath,$ORIGIN", *libs]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed for %s:\n%s\n%s" % (out, r.stdout, r.stderr))


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.hpp")) + \
        glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(ROOT, "include", "**", "*.h*"), recursive=True)

    core_srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))
    jobs = []
    for s in core_srcs:
        o = os.path.join(OBJDIR, os.path.basename(s) + ".o")
        if force or _newer(o, [s] + headers):
            jobs.append((s, o))
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        list(ex.map(lambda so: _compile(so[0], so[1], verbose,
                                        PER_FILE_FLAGS.get(os.path.basename(so[0]), ())), jobs))
    objs = [os.path.join(OBJDIR, os.path.basename(s) + ".o") for s in core_srcs]
    core = os.path.join(LIBDIR, "libspconvb.so")
    if force or jobs or not os.path.exists(core):
        _link(objs, core, verbose=verbose)

    # C++ facades with the reference's class interfaces, one library per header generation
    for sub, name, inc in (("facade_v13", "libspconv.so", os.path.join(ROOT, "include")),
                           ("facade_v10", "libspconv_v10.so",
                            os.path.join(ROOT, "include", "spconv_v10"))):
        srcs = sorted(glob.glob(os.path.join(CSRC, sub, "*.cpp")))
        if not srcs:
            continue
        fobjs, changed = [], False
        for s in srcs:
            o = os.path.join(OBJDIR, sub + "_" + os.path.basename(s) + ".o")
            if force or _newer(o, [s] + headers):
                _compile(s, o, verbose, extra=("-I", inc))
                changed = True
            fobjs.append(o)
        out = os.path.join(LIBDIR, name)
        if force or changed or not os.path.exists(out) or _newer(out, [core]):
            _link(fobjs, out, libs=("-L", LIBDIR, "-lspconvb"), verbose=verbose)
    return core


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
