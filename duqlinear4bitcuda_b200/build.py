"""Build the package's native code in-tree:

  libduq4.so   the C-ABI CUDA library (include/duq4.h), nvcc for sm_100a
  _CUDA.*.so   the pybind11 operator module (csrc/bindings.cpp) with the names of the reference's
               compiled extension qlinear4bit._CUDA; host C++ only, linked against libduq4.so and torch

    python -m duqlinear4bitcuda_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. The outputs land next to this file so that they travel
with the source tree; they are never installed into site-packages.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libduq4.so")
SOURCES = ["quantize.cu", "dequant.cu", "gemv_decode.cu", "gemm_tc.cu", "gemm_tc2.cu", "abi.cu", "host_pipeline.cu", "peer.cu", "row_parallel.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Wno-deprecated-gpu-targets",
         "-Xcompiler", "-fPIC"]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f != "bindings.cpp"] + [os.path.join(HERE, "..", "include", "duq4.h")]
    return any(os.path.getmtime(d) > t for d in deps)


EXT = os.path.join(HERE, "_CUDA" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build_binding(force=False, verbose=False):
    """The pybind11 module `_CUDA` (g++; torch and pybind11 headers of the running interpreter)."""
    src = os.path.join(CSRC, "bindings.cpp")
    deps = [src, os.path.join(HERE, "..", "include", "duq4.h"), LIB]
    if not force and os.path.exists(EXT) and all(os.path.getmtime(EXT) >= os.path.getmtime(d) for d in deps):
        return EXT
    import torch
    from torch.utils import cpp_extension as ce
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    # the system g++ (the host compiler nvcc uses): its libstdc++ is the shared one torch itself is linked to
    cmd = [os.environ.get("DUQ4_CXX", "/usr/bin/g++"), "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden",
           "-DTORCH_EXTENSION_NAME=_CUDA", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI), src, "-o", EXT,
           "-I", sysconfig.get_paths()["include"], "-I", "/usr/local/cuda/include"]
    for inc in ce.include_paths():
        cmd += ["-isystem", inc]
    cmd += ["-L", HERE, "-l:libduq4.so", "-L", tlib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or p.returncode:
        sys.stderr.write(f"--- bindings.cpp\n{p.stdout}\n")
    if p.returncode:
        raise RuntimeError("building the _CUDA binding failed")
    return EXT


def build(force=False, verbose=False):
    build_library(force, verbose)
    build_binding(force, verbose)
    return LIB


def build_library(force=False, verbose=False):
    if not force and not _stale():
        return LIB
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    for src in SOURCES:
        obj = os.path.join(HERE, "build", src.replace(".cu", ".o"))
        cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(f"--- {src}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.check_call([NVCC, "-shared", "-o", LIB] + objs + ["-Xcompiler", "-fPIC", "-Xlinker", "-soname=libduq4.so"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
