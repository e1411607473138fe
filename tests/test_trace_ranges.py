"""CPU-only: the library's entry points open an NVTX range named after themselves (domain "duq4").
A test-only NVTX injection library (tests/c/nvtx_listener.c) records what the library pushes; the calls
used here are rejected for their arguments before any CUDA call, so no GPU is needed."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import ctypes
import duqlinear4bitcuda_b200.lib as L
c = L.cdll
P = ctypes.c_void_p(0x1000)
e = L.Epilogue(); e.mode = L.MODE_SYM; e.scale_row = 0x1000; e.scale_col_1 = 0x1000
assert c.duq4_linear_w4a4(None, P, 4, 8, 64, ctypes.byref(e), P, None, None) == -1
assert c.duq4_sym_quant(None, P, 4, 64, 32, P, None) == -1
assert c.duq4_linear_w4a4_from_fp16(P, P, 4, 8, 100, L.MODE_SYM, 1.0, ctypes.byref(e), P, P, 1 << 20, None) == -2
"""


def test_entry_points_push_named_ranges(tmp_path):
    so = tmp_path / "libnvtx_listener.so"
    subprocess.run(["gcc", "-O1", "-shared", "-fPIC", "-I", os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/include",
                    os.path.join(ROOT, "tests", "c", "nvtx_listener.c"), "-o", str(so)], check=True)
    log = tmp_path / "ranges.log"
    env = dict(os.environ, NVTX_INJECTION64_PATH=str(so), DUQ4_NVTX_LOG=str(log), PYTHONPATH=ROOT)
    subprocess.run([sys.executable, "-c", CHILD], check=True, env=env, cwd=ROOT, timeout=300)
    lines = log.read_text().split("\n")
    assert "domain duq4" in lines
    for name in ("duq4_linear_w4a4", "duq4_sym_quant", "duq4_linear_w4a4_from_fp16"):
        assert f"push {name}" in lines, lines
    assert sum(l.startswith("push ") for l in lines) == sum(l.startswith("pop") for l in lines) == 3
