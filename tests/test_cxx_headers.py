"""CPU-only: the reference-named C++ headers (include/gemm.h, include/quant.h) compile with a
plain host compiler, link against libduq4.so, and report a rejected argument by throwing."""
import os
import subprocess
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SRC = r'''
#include "gemm.h"
#include "quant.h"
#include <cstdio>
int main() {
    static_assert(QUANT_COL_K == 10 && qmax_sym == 6 && kElementsPerVector == 2, "reference constants");
    static_assert(QUANT_COL_ST == ((((__uint128_t)1 << 5) - 1) | ((((__uint128_t)1 << 5) - 1) << 10)), "bits 0-4 and 10-14");
    static_assert(((QUANT_COL_ST << 0) & 1) == 1 && ((QUANT_COL_ST << 1) & 1) == 0, "the reference's selector holds for column 0 only");
    int caught = 0;
    try { matmul_host_4bit(nullptr, nullptr, 4, 4, 64, nullptr); } catch (const std::runtime_error &) { ++caught; }
    try { sym_quant_host(nullptr, nullptr, 4, 64, 32, nullptr); } catch (const std::runtime_error &) { ++caught; }
    try { asym_dual_dequant_host(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 1, 1, nullptr); }
    catch (const std::runtime_error &) { ++caught; }
    const Int4Storage *a[1] = {nullptr}; int32_t *c[1] = {nullptr};
    try { batch_matmul_host_4bit(a, a, 4, 4, 64, c, 1); } catch (const std::runtime_error &) { ++caught; }
    return caught == 4 ? 0 : 1;
}
'''


def test_headers_compile_link_and_throw():
    import duqlinear4bitcuda_b200.lib as L
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "t.cpp"); exe = os.path.join(d, "t")
        open(src, "w").write(SRC)
        subprocess.check_call(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-I", "/usr/local/cuda/include", src,
                               "-o", exe, L.LIB_PATH, "-Wl,-rpath," + os.path.dirname(L.LIB_PATH)])
        assert subprocess.call([exe]) == 0
