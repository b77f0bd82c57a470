"""In-tree build of the two native artefacts (no JIT cache, no install step):

  chunk_attn/lib/libchunk_attn_b200.so     CUDA kernels + host planner behind the C ABI of
                                           include/chunk_attn_b200.h, sm_100a only
  chunk_attn/lib/chunk_attn_c<ext>.so      C++ host (prefix tree, chunk pool, Attention) with the
                                           reference's pybind11 surface, linked against libtorch

Usage: python build.py [--force] [--abi-only]
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "chunk_attn", "lib")
OBJ = os.path.join(HERE, "build")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

ABI_LIB = os.path.join(LIB, "libchunk_attn_b200.so")
EXT_LIB = os.path.join(LIB, "chunk_attn_c" + sysconfig.get_config_var("EXT_SUFFIX"))

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", INCLUDE]
CU_SOURCES = ["ca_attn_fast.cu", "ca_attn_wide.cu", "ca_attn_generic.cu", "ca_pool_ops.cu", "ca_abi.cu", "ca_noalloc.cu", "ca_ops.cu"]
CPP_SOURCES = ["ca_plan.cpp"]
HOST_SOURCES = ["host/chunk.cpp", "host/prefix_tree.cpp", "host/attention.cpp", "host/ops.cpp", "host/bindings.cpp"]


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout[-4000:] + r.stderr[-8000:] + "\n")
        raise RuntimeError("build step failed: " + " ".join(cmd[:1] + cmd[-1:]))
    return r.stdout + r.stderr


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _all_headers():
    hs = [os.path.join(INCLUDE, "chunk_attn_b200.h")]
    for root, _, files in os.walk(CSRC):
        hs += [os.path.join(root, f) for f in files if f.endswith((".h", ".cuh"))]
    return hs


def build_abi(force=False, verbose=False):
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    headers = _all_headers()
    jobs, objs = [], []
    for s in CU_SOURCES:
        src, obj = os.path.join(CSRC, s), os.path.join(OBJ, s + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            extra = ["-Xptxas", "-v"] if verbose else []
            jobs.append(["nvcc"] + NVCC_FLAGS + extra + ["-c", src, "-o", obj])
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    for s in CPP_SOURCES:
        src, obj = os.path.join(CSRC, s), os.path.join(OBJ, s + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-I", INCLUDE,
                         "-I", os.path.join(cuda_home, "include"), "-c", src, "-o", obj])
    out = ""
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            out = "".join(ex.map(_run, jobs))
    if jobs or not os.path.exists(ABI_LIB):
        # static cudart: the library loads (and its host-only entry points run) without a driver
        _run(["nvcc", "-shared", "-cudart", "static", "-o", ABI_LIB] + objs)
    return out


def build_ext(force=False):
    import torch
    tdir = os.path.dirname(torch.__file__)
    headers = _all_headers()
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = [INCLUDE, os.path.join(tdir, "include"),
           os.path.join(tdir, "include", "torch", "csrc", "api", "include"),
           os.path.join(cuda_home, "include"), sysconfig.get_paths()["include"]]
    flags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-w",
             "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
             "-DTORCH_EXTENSION_NAME=chunk_attn_c"] + [x for i in inc for x in ("-I", i)]
    jobs, objs = [], []
    for s in HOST_SOURCES:
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ, s.replace("/", "_") + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            jobs.append(["g++"] + flags + ["-c", src, "-o", obj])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            list(ex.map(_run, jobs))
    if jobs or not os.path.exists(EXT_LIB) or _stale(EXT_LIB, [ABI_LIB]):
        tlib = os.path.join(tdir, "lib")
        _run(["g++", "-shared"] + objs +
             ["-L", LIB, "-lchunk_attn_b200", "-L", tlib, "-ltorch", "-ltorch_cpu", "-ltorch_cuda",
              "-lc10", "-lc10_cuda", "-ltorch_python",
              "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib, "-o", EXT_LIB])


def build_all(force=False, verbose=False):
    out = build_abi(force, verbose)
    build_ext(force)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--abi-only", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas resource usage")
    a = ap.parse_args()
    text = build_abi(a.force, a.verbose)
    if a.verbose:
        print(text)
    if not a.abi_only:
        build_ext(a.force)
    print("built", ABI_LIB, "" if a.abi_only else EXT_LIB)
