"""Build the UNMODIFIED reference into oracle/_ref/ (test infrastructure, never shipped).

Two artefacts, both compiled from the reference's sources where they lie (nothing is copied):

  oracle/_ref/cpu/chunk_attn_c<ext>.so    reference host + its MKL CPU kernels
                                          (cpp/chunk_attn/{chunk,chunk_allocator,attention,
                                          kernel_cpu_mkl,logging,str_utils,task_executor,
                                          python_exports}.cpp, -DUSE_MKL=1)
  oracle/_ref/cuda/chunk_attn_c<ext>.so   reference host + its CUDA kernels recompiled for
                                          sm_100a (kernel_cuda.cu, -DUSE_CUDA=1); optional,
                                          only with --cuda

Deviations from the reference's CMake build, none touching its sources: oneMKL's two headers
are replaced by the shims in oracle/shim (sgemm_/vsExp exported by libtorch_cpu), the C++
standard is 17, the libstdc++ ABI is the one torch was built with, spdlog headers come from
the copy bundled in the flashinfer wheel, and the CUDA build force-includes a fmt formatter
for caffe2::TypeMeta (the reference logs tensor.dtype() through fmt, which fmt >= 10 rejects).

Usage: python oracle/build_ref.py [--cuda] [--ref /path/to/reference] [--force]
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

HOST_SOURCES = ["chunk.cpp", "chunk_allocator.cpp", "attention.cpp", "logging.cpp",
                "str_utils.cpp", "task_executor.cpp", "python_exports.cpp"]


def _paths():
    import torch
    tdir = os.path.dirname(torch.__file__)
    site = os.path.dirname(tdir)
    inc = [os.path.join(HERE, "shim"),
           os.path.join(tdir, "include"),
           os.path.join(tdir, "include", "torch", "csrc", "api", "include"),
           os.path.join(site, "flashinfer", "data", "spdlog", "include"),
           sysconfig.get_paths()["include"]]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    return tdir, inc, abi


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout[-4000:] + r.stderr[-8000:] + "\n")
        raise RuntimeError("reference build step failed: " + cmd[-1])


def ref_so(kind):
    return os.path.join(OUT, kind, "chunk_attn_c" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_cpu(ref, force=False):
    target = ref_so("cpu")
    if os.path.exists(target) and not force:
        return target
    src = os.path.join(ref, "cpp", "chunk_attn")
    tdir, inc, abi = _paths()
    odir = os.path.join(OUT, "cpu", "obj")
    os.makedirs(odir, exist_ok=True)
    flags = ["-O2", "-std=c++17", "-fPIC", "-fopenmp", "-w", "-DUSE_MKL=1", "-DNVTX_DISABLE",
             "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi, "-I", src] + [x for i in inc for x in ("-I", i)]
    srcs = HOST_SOURCES + ["kernel_cpu_mkl.cpp"]
    objs = [os.path.join(odir, s.replace(".cpp", ".o")) for s in srcs]
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        list(ex.map(lambda so: _run(["g++"] + flags + ["-c", os.path.join(src, so[0]), "-o", so[1]]),
                    zip(srcs, objs)))
    tlib = os.path.join(tdir, "lib")
    _run(["g++", "-shared", "-fopenmp"] + objs +
         ["-L", tlib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python",
          "-Wl,-rpath," + tlib, "-o", target])
    return target


def build_cuda(ref, force=False):
    target = ref_so("cuda")
    if os.path.exists(target) and not force:
        return target
    src = os.path.join(ref, "cpp", "chunk_attn")
    tdir, inc, abi = _paths()
    odir = os.path.join(OUT, "cuda", "obj")
    os.makedirs(odir, exist_ok=True)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    fmt_shim = os.path.join(HERE, "shim", "fmt_typemeta.h")
    # a distinct pybind11 internals id keeps this module's "Attention"/"Chunk" type registry
    # apart from the CPU reference module's, so both load in one interpreter
    common = ["-DUSE_CUDA=1", "-DNVTX_DISABLE", "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi,
              '-DPYBIND11_INTERNALS_KIND="_ca_refcuda"', '-DPYBIND11_BUILD_ABI="_ca_refcuda"',
              "-I", src, "-I", os.path.join(cuda_home, "include")] + \
             [x for i in inc for x in ("-I", i)]
    gxx = ["-O2", "-std=c++17", "-fPIC", "-w", "-include", fmt_shim] + common
    objs = []
    jobs = []
    for s in HOST_SOURCES:
        o = os.path.join(odir, s.replace(".cpp", ".o"))
        objs.append(o)
        jobs.append(["g++"] + gxx + ["-c", os.path.join(src, s), "-o", o])
    ko = os.path.join(odir, "kernel_cuda.o")
    objs.append(ko)
    jobs.append(["nvcc", "-std=c++17", "-O3", "--expt-relaxed-constexpr", "-w",
                 "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
                 "-include", fmt_shim] + common + ["-c", os.path.join(src, "kernel_cuda.cu"), "-o", ko])
    # the vLLM-derived `ops` submodule is referenced by python_exports.cpp when USE_CUDA is set
    for s in ["python_exports_ops.cpp"]:
        o = os.path.join(odir, s.replace(".cpp", ".o"))
        objs.append(o)
        jobs.append(["g++"] + gxx + ["-c", os.path.join(src, s), "-o", o])
    for s in ["layernorm_kernels.cu", "pos_encoding_kernels.cu"]:
        o = os.path.join(odir, s.replace(".cu", ".o"))
        objs.append(o)
        jobs.append(["nvcc", "-std=c++17", "-O3", "--expt-relaxed-constexpr", "-w",
                     "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"] +
                    common + ["-c", os.path.join(src, s), "-o", o])
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        list(ex.map(_run, jobs))
    tlib = os.path.join(tdir, "lib")
    _run(["g++", "-shared"] + objs +
         ["-L", tlib, "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
          "-ltorch_python", "-L", os.path.join(cuda_home, "lib64"), "-lcudart",
          "-Wl,-rpath," + tlib, "-o", target])
    return target


def install_models(ref):
    """Install (copy, unchanged) the reference's pure-Python model layer -- src/chunk_attn/models: llama_hf and
    ModelHost -- into oracle/_ref/py/models, the git-ignored output folder, so that the drop-in test can run
    those very files on top of this repository's `chunk_attn` package on a machine that has no reference tree."""
    import shutil
    src = os.path.join(ref, "src", "chunk_attn", "models")
    dst = os.path.join(OUT, "py", "models")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__"))
    return dst


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("CHUNK_ATTN_REFERENCE_TREE"), required="CHUNK_ATTN_REFERENCE_TREE" not in os.environ,
                    help="source tree of the unmodified reference (or set CHUNK_ATTN_REFERENCE_TREE)")
    ap.add_argument("--cuda", action="store_true")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    if not os.path.isdir(a.ref):
        print("reference tree not found at %s: keeping whatever is already in %s" % (a.ref, OUT))
        return
    print(build_cpu(a.ref, a.force))
    print(install_models(a.ref))
    if a.cuda:
        print(build_cuda(a.ref, a.force))


if __name__ == "__main__":
    main()
