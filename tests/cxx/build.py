"""Builds tests/cxx/libtorch_pipeline (needs the torch headers/libraries of the running interpreter)."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
EXE = os.path.join(HERE, "_build", "libtorch_pipeline")


def build(force=False):
    src = os.path.join(HERE, "libtorch_pipeline.cpp")
    deps = [src] + [os.path.join(ROOT, "include", f) for f in ("linear.h", "quant_tensor.h", "gemm.h", "quant.h", "duq4.h")]
    if not force and os.path.exists(EXE) and all(os.path.getmtime(EXE) >= os.path.getmtime(d) for d in deps):
        return EXE
    import torch
    from torch.utils import cpp_extension as ce
    sys.path.insert(0, ROOT)
    import duqlinear4bitcuda_b200.lib as L
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    os.makedirs(os.path.dirname(EXE), exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O1", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI), src, "-o", EXE,
           "-I", os.path.join(ROOT, "include"), "-I", "/usr/local/cuda/include"]
    for inc in ce.include_paths():
        cmd += ["-isystem", inc]
    cmd += [L.LIB_PATH, "-L", tlib, "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
            "-L", "/usr/local/cuda/lib64", "-lcudart", "-ldl",
            "-Wl,-rpath," + tlib, "-Wl,-rpath," + os.path.dirname(L.LIB_PATH), "-Wl,--no-as-needed"]
    subprocess.check_call(cmd)
    return EXE


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
