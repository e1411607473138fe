"""include/linear.h and include/quant_tensor.h (the reference's libtorch C++ API): the parity
program tests/cxx/libtorch_pipeline.cpp compiles against the torch headers (CPU test) and, on a
GPU, reports that Quantizer4bit -> Linear4bit / Linear4bitDUQ and the tensor-level functions equal
the reference's own CUDA launchers (oracle/_ref/libduq_ref.so, compiled from the reference's
sources) bit for bit."""
import os
import subprocess

from tests import _util as U

import pytest

from tests.cxx import build as cxx_build


def test_libtorch_headers_compile_and_link():
    exe = cxx_build.build()
    assert exe.endswith("libtorch_pipeline")


@pytest.mark.gpu
def test_libtorch_pipeline_matches_reference_composition():
    exe = cxx_build.build()
    ref = os.path.join(U.ROOT, "oracle", "_ref", "libduq_ref.so")
    if not os.path.exists(ref):
        pytest.skip("reference kernels not built (make -C oracle ref)")
    r = subprocess.run([exe, ref], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "libtorch pipeline ok" in r.stdout
