"""numpy/ctypes front-end of the CPU oracle (oracle/duq_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's
CPU-baseline leg; never by the product package. All arrays are numpy; fp16 tensors are
passed as np.float16 (bit patterns are what matters). The reference lines each function
follows are cited in duq_oracle.c.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libduq_oracle.so")
_lib = None

QUANT_COL_K = 10  # include/quant.h:5 of the reference
QMAX_SYM = 6      # include/common.h:54 of the reference: (7 - 1e-8) truncates to 6


def build(force=False):
    """Compile duq_oracle.c with gcc (seconds)."""
    src = os.path.join(_HERE, "duq_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a)
    assert a.dtype == dt, (a.dtype, dt)
    return a


u32 = ctypes.c_uint32


def sym_quant(x, scale, nudge=0, cols_dst=None):
    x = _c(x, np.float16); scale = _c(scale.reshape(-1), np.float16)
    rows, cols = x.shape
    cd = (cols + 1) // 2 if cols_dst is None else cols_dst
    q = np.zeros((rows, cd), np.uint8)
    lib().duqo_sym_quant(_p(x), _p(scale), u32(rows), u32(cols), u32(cd), _p(q), ctypes.c_int(nudge))
    return q


def sym_dual_quant(x, s1, s2, nudge=0):
    x = _c(x, np.float16); s1 = _c(s1.reshape(-1), np.float16); s2 = _c(s2.reshape(-1), np.float16)
    rows, cols = x.shape
    cd = (cols + 1) // 2
    q = np.zeros((rows, cd), np.uint8)
    lib().duqo_sym_dual_quant(_p(x), _p(s1), _p(s2), u32(rows), u32(cols), u32(cd), _p(q), ctypes.c_int(nudge))
    return q


def asym_quant(x, scale, zeros, nudge=0):
    x = _c(x, np.float16); scale = _c(scale.reshape(-1), np.float16); zeros = _c(zeros.reshape(-1), np.float16)
    rows, cols = x.shape
    cd = (cols + 1) // 2
    q = np.zeros((rows, cd), np.uint8)
    lib().duqo_asym_quant(_p(x), _p(scale), _p(zeros), u32(rows), u32(cols), u32(cd), _p(q), ctypes.c_int(nudge))
    return q


def asym_dual_quant(x, s1, z1, s2, z2, nudge=0):
    x = _c(x, np.float16)
    s1, z1, s2, z2 = (_c(v.reshape(-1), np.float16) for v in (s1, z1, s2, z2))
    rows, cols = x.shape
    cd = (cols + 1) // 2
    q = np.zeros((rows, cd), np.uint8)
    lib().duqo_asym_dual_quant(_p(x), _p(s1), _p(z1), _p(s2), _p(z2), u32(rows), u32(cols), u32(cd), _p(q),
                               ctypes.c_int(nudge))
    return q


def asym_quant_8bit(x, scale, zeros):
    x = _c(x, np.float32); scale = _c(scale.reshape(-1), np.float32); zeros = _c(zeros.reshape(-1), np.float32)
    rows, cols = x.shape
    q = np.zeros((rows, cols), np.int8)
    lib().duqo_asym_quant_8bit(_p(x), _p(scale), _p(zeros), u32(rows), u32(cols), _p(q))
    return q


def sym_scales(x, clip=1.0, c0=0, c1=None):
    x = _c(x, np.float16)
    rows, cols = x.shape
    c1 = cols if c1 is None else c1
    s = np.zeros(rows, np.float16)
    lib().duqo_sym_scales(_p(x), u32(rows), u32(cols), u32(c0), u32(c1), ctypes.c_float(clip), _p(s))
    return s


def asym_scales_zeros(x, c0=0, c1=None):
    x = _c(x, np.float16)
    rows, cols = x.shape
    c1 = cols if c1 is None else c1
    s = np.zeros(rows, np.float16); z = np.zeros(rows, np.float16)
    lib().duqo_asym_scales_zeros(_p(x), u32(rows), u32(cols), u32(c0), u32(c1), _p(s), _p(z))
    return s, z


def matmul_4bit(A, B):
    A = _c(A, np.uint8); B = _c(B, np.uint8)
    M, kb = A.shape; N = B.shape[0]
    assert B.shape[1] == kb
    C = np.zeros((M, N), np.int32)
    lib().duqo_matmul_4bit(_p(A), _p(B), u32(M), u32(N), u32(kb * 2), _p(C))
    return C


def matmul_8bit(A, B):
    A = _c(A, np.int8); B = _c(B, np.int8)
    M, K = A.shape; N = B.shape[0]
    C = np.zeros((M, N), np.int32)
    lib().duqo_matmul_8bit(_p(A), _p(B), u32(M), u32(N), u32(K), _p(C))
    return C


def batch_matmul_4bit(A, B):
    A = _c(A, np.uint8); B = _c(B, np.uint8)
    b, M, kb = A.shape; N = B.shape[1]
    C = np.zeros((b, M, N), np.int32)
    lib().duqo_batch_matmul_4bit(_p(A), _p(B), u32(M), u32(N), u32(kb * 2), _p(C), u32(b))
    return C


def sym_dequant(q, sr, sc):
    q = _c(q, np.int32); sr = _c(sr.reshape(-1), np.float16); sc = _c(sc.reshape(-1), np.float16)
    rows, cols = q.shape
    x = np.zeros((rows, cols), np.float16)
    lib().duqo_sym_dequant(_p(q), _p(sr), _p(sc), u32(rows), u32(cols), _p(x))
    return x


def sym_dual_dequant(q, sr, sc1, sc2, col0=0):
    q = _c(q, np.int32)
    sr, sc1, sc2 = (_c(v.reshape(-1), np.float16) for v in (sr, sc1, sc2))
    rows, cols = q.shape
    x = np.zeros((rows, cols), np.float16)
    lib().duqo_sym_dual_dequant(_p(q), _p(sr), _p(sc1), _p(sc2), u32(rows), u32(cols), u32(col0), _p(x))
    return x


def asym_dequant(q, sr, zr, sc, zc):
    q = _c(q, np.int32)
    sr, zr, sc, zc = (_c(v.reshape(-1), np.float16) for v in (sr, zr, sc, zc))
    rows, cols = q.shape
    x = np.zeros((rows, cols), np.float16)
    lib().duqo_asym_dequant(_p(q), _p(sr), _p(zr), _p(sc), _p(zc), u32(rows), u32(cols), _p(x))
    return x


def asym_dual_dequant(q, sr, zr, sc1, zc1, sc2, zc2, col0=0):
    q = _c(q, np.int32)
    sr, zr, sc1, zc1, sc2, zc2 = (_c(v.reshape(-1), np.float16) for v in (sr, zr, sc1, zc1, sc2, zc2))
    rows, cols = q.shape
    x = np.zeros((rows, cols), np.float16)
    lib().duqo_asym_dual_dequant(_p(q), _p(sr), _p(zr), _p(sc1), _p(zc1), _p(sc2), _p(zc2), u32(rows), u32(cols),
                                 u32(col0), _p(x))
    return x


def asym_batch_dequant(q, sr, zr, sc, zc):
    q = _c(q, np.int32)
    sr, zr, sc, zc = (_c(v.reshape(-1), np.float16) for v in (sr, zr, sc, zc))
    b, rows, cols = q.shape
    x = np.zeros((b, rows, cols), np.float16)
    lib().duqo_asym_batch_dequant(_p(q), _p(sr), _p(zr), _p(sc), _p(zc), u32(b), u32(rows), u32(cols), _p(x))
    return x


def asym_dequant_hprec(q, sr, zr, sc, zc):
    q = _c(q, np.int32)
    sr, zr, sc, zc = (_c(v.reshape(-1), np.float32) for v in (sr, zr, sc, zc))
    rows, cols = q.shape
    x = np.zeros((rows, cols), np.float32)
    lib().duqo_asym_dequant_hprec(_p(q), _p(sr), _p(zr), _p(sc), _p(zc), u32(rows), u32(cols), _p(x))
    return x


def add_bias(x, bias):
    x = _c(x, np.float16).copy(); bias = _c(bias.reshape(-1), np.float16)
    rows, cols = x.shape
    lib().duqo_add_bias(_p(x), _p(bias), u32(rows), u32(cols))
    return x


def weight_sym_quant_pack(w):
    w = _c(w, np.float16)
    N, K = w.shape
    s = np.zeros(N, np.float16); q = np.zeros((N, K // 2), np.uint8)
    lib().duqo_weight_sym_quant_pack(_p(w), u32(N), u32(K), _p(s), _p(q))
    return q, s


def unpack_s4(q):
    """uint8 [.., K/2] -> int8 [.., K] signed nibbles, low nibble first."""
    lo = (q & 0xF).astype(np.int8); hi = (q >> 4).astype(np.int8)
    lo = np.where(lo >= 8, lo - 16, lo).astype(np.int8); hi = np.where(hi >= 8, hi - 16, hi).astype(np.int8)
    out = np.empty(q.shape[:-1] + (q.shape[-1] * 2,), np.int8)
    out[..., 0::2] = lo; out[..., 1::2] = hi
    return out


def pack_s4(v):
    """int [.., K] in [-8,15] -> uint8 [.., K/2]."""
    v = (np.asarray(v).astype(np.int16) & 0xF).astype(np.uint8)
    return (v[..., 0::2] | (v[..., 1::2] << 4)).astype(np.uint8)


# ---- whole-layer compositions (what the reference modules compute) ---------------------

def linear_w4a4(mode, qa, qw, sr, zr, sc1, zc1, sc2, zc2, bias=None, col0=0):
    """matmul + the mode's dequant (+ bias): qlinear4bit/nn/linear.py forward methods."""
    acc = matmul_4bit(qa, qw)
    if mode == "sym":
        out = sym_dequant(acc, sr, sc1)
    elif mode == "sym_dual":
        out = sym_dual_dequant(acc, sr, sc1, sc2, col0)
    elif mode == "asym":
        out = asym_dequant(acc, sr, zr, sc1, zc1)
    elif mode == "asym_dual":
        out = asym_dual_dequant(acc, sr, zr, sc1, zc1, sc2, zc2, col0)
    else:
        raise ValueError(mode)
    if bias is not None:
        out = add_bias(out, bias)
    return acc, out
