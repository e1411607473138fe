"""Seeded synthetic inputs shaped like the benchmark configurations, and comparison helpers."""
import ctypes
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def acts(M, K, seed, mean=0.0, outlier_frac=0.01, outlier_mul=20.0):
    """fp16 activations ~N(mean,1) with a fraction of K-channels scaled up (outliers)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K), dtype=np.float32) + np.float32(mean)
    n_out = int(outlier_frac * K)
    if n_out:
        ch = rng.permutation(K)[:n_out]
        x[:, ch] *= np.float32(outlier_mul)
    return x.astype(np.float16)


def rand_codes(rows, K, seed):
    """Random packed int4 rows (every nibble value occurs)."""
    rng = np.random.default_rng(seed)
    return rng.integers(0, 256, (rows, K // 2), dtype=np.uint8)


def rand_scales(n, seed, lo=0.002, hi=0.05):
    rng = np.random.default_rng(seed)
    return (lo + (hi - lo) * rng.random(n)).astype(np.float16)


def rand_zeros(n, seed):
    rng = np.random.default_rng(seed)
    return rng.integers(0, 16, n).astype(np.float16)


def bits_equal(a, b):
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b)
    if a.dtype == np.float16:
        a = a.view(np.uint16); b = b.view(np.uint16)
    elif a.dtype == np.float32:
        a = a.view(np.uint32); b = b.view(np.uint32)
    return a.shape == b.shape and np.array_equal(a, b)


def f16_equal_nan(a, b):
    """Bit equality, except that any NaN matches any NaN (payloads are not specified)."""
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b)
    if a.shape != b.shape:
        return False
    both_nan = np.isnan(a) & np.isnan(b)
    return bool(np.all(both_nan | (a.view(np.uint16) == b.view(np.uint16))))


def codes_within_bracket(got, exact, lo, hi):
    """GPU codes must equal the exact-division codes except where the approximate-reciprocal
    divide is within 2 fp32 ulps of a rounding boundary (there either neighbour is allowed).
    Returns (ok, number of such near-tie elements)."""
    from oracle import oracle as o
    g, e, l, h = (o.unpack_s4(v).astype(np.int16) for v in (got, exact, lo, hi))
    mn = np.minimum(l, h); mx = np.maximum(l, h)
    ok = ((g == e) | ((g >= mn) & (g <= mx)))
    return bool(ok.all()), int((g != e).sum())


def load_ref_lib():
    """The reference's own CUDA kernels (built by oracle/Makefile target `ref`), or None."""
    p = os.path.join(ROOT, "oracle", "_ref", "libduq_ref.so")
    if not os.path.exists(p):
        return None
    try:
        return ctypes.CDLL(p)
    except OSError:
        return None
