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


# ---- the library's own quantizer output as the oracle's input ---------------------------------
_FUSED = {"sym": "duq4_quantize_sym_fused", "sym_dual": "duq4_quantize_sym_dual_fused",
          "asym": "duq4_quantize_asym_fused", "asym_dual": "duq4_quantize_asym_dual_fused"}


def i8_codes_to_packed(a8):
    """Tensor-core-ready activations (int8 = 16 * code, K permuted inside 128-blocks, as
    duq4_quantize_fused_i8 writes them) -> packed int4 codes [M, K/2] in the reference's format."""
    from oracle import oracle as o
    a8 = np.ascontiguousarray(a8)
    K = a8.shape[1]
    assert np.all((a8.astype(np.int16) & 15) == 0), "int8 activations are not multiples of 16"
    pos = np.arange(K); blk, r = pos // 128, pos % 128
    src = blk * 128 + 32 * (r // 32) + 2 * (r % 16) + ((r % 32) // 16)   # position pos holds column src
    codes = np.empty(a8.shape, dtype=np.int8)
    codes[:, src] = (a8.astype(np.int16) // 16).astype(np.int8)
    return o.pack_s4(codes)


def check_gpu_codes(torch, L, mode, x, qa, s1, z1=None, s2=None, z2=None, clip=1.0):
    """`qa` (packed codes) and the per-token vectors are what the library's fused quantizer made of
    the fp16 tokens `x` (numpy). Requires: scales / zero-points bit-identical to the oracle's, codes
    equal to the oracle's except at proven near-ties of the GPU divide (bracket of +-2 fp32 ulps),
    and -- when the reference's own kernels were built -- codes bit-identical to the reference's
    quantize kernel run on the GPU with those scales."""
    from oracle import oracle as o
    asym, dual = mode.startswith("asym"), mode.endswith("dual")
    if mode == "sym":
        exp = [o.sym_scales(x, clip)]; ora = lambda n: o.sym_quant(x, exp[0], n); got = [s1]
    elif mode == "sym_dual":
        exp = [o.sym_scales(x, clip, 0, 10), o.sym_scales(x, clip, 10)]; got = [s1, s2]
        ora = lambda n: o.sym_dual_quant(x, exp[0], exp[1], n)
    elif mode == "asym":
        exp = list(o.asym_scales_zeros(x)); got = [s1, z1]
        ora = lambda n: o.asym_quant(x, exp[0], exp[1], n)
    else:
        exp = list(o.asym_scales_zeros(x, 0, 10)) + list(o.asym_scales_zeros(x, 10)); got = [s1, z1, s2, z2]
        ora = lambda n: o.asym_dual_quant(x, exp[0], exp[1], exp[2], exp[3], n)
    for g, e in zip(got, exp):
        assert f16_equal_nan(np.asarray(g).reshape(-1), e), f"{mode}: per-token scale / zero-point differs from the oracle"
    ok, _ = codes_within_bracket(qa, ora(0), ora(-2), ora(2))
    assert ok, f"{mode}: a code differs from the oracle where the divide is not on a rounding near-tie"
    ref = load_ref_lib()
    if ref is not None:
        rows, cols = x.shape
        dx = torch.from_numpy(np.ascontiguousarray(x)).cuda()
        dv = [torch.from_numpy(np.ascontiguousarray(np.asarray(g).reshape(-1))).cuda() for g in got]
        q2 = torch.zeros((rows, cols // 2), dtype=torch.uint8, device="cuda")
        fn = getattr(ref, f"ref_{mode}_quant")
        fn.argtypes = [ctypes.c_void_p] * (1 + len(dv)) + [ctypes.c_uint32] * 3 + [ctypes.c_void_p]
        fn.restype = ctypes.c_int
        assert fn(L.ptr(dx), *[L.ptr(a) for a in dv], rows, cols, cols // 2, L.ptr(q2)) == 0
        assert np.array_equal(q2.cpu().numpy(), qa), f"{mode}: codes differ from the reference's own quantize kernel"


def gpu_quantize(torch, L, mode, x, clip=1.0, check=True):
    """Runs the library's fused quantizer on the fp16 tokens `x` (numpy [M, K], K even) and returns
    (packed codes, s1, z1, s2, z2) as numpy arrays (vectors a mode does not produce are None), after
    check_gpu_codes. Layer tests feed these to the oracle's GEMM + dequant, so that every output row
    is compared exactly."""
    M, K = x.shape
    dx = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    q = torch.zeros((M, K // 2), dtype=torch.uint8, device="cuda")
    vec = lambda: torch.zeros(M, dtype=torch.float16, device="cuda")
    s1, z1, s2, z2 = vec(), vec(), vec(), vec()
    st = L.current_stream()
    if mode == "sym":
        L.call(_FUSED[mode], L.ptr(dx), M, K, clip, L.ptr(q), L.ptr(s1), st)
    elif mode == "sym_dual":
        L.call(_FUSED[mode], L.ptr(dx), M, K, clip, L.ptr(q), L.ptr(s1), L.ptr(s2), st)
    elif mode == "asym":
        L.call(_FUSED[mode], L.ptr(dx), M, K, L.ptr(q), L.ptr(s1), L.ptr(z1), st)
    else:
        L.call(_FUSED[mode], L.ptr(dx), M, K, L.ptr(q), L.ptr(s1), L.ptr(z1), L.ptr(s2), L.ptr(z2), st)
    torch.cuda.synchronize()
    asym, dual = mode.startswith("asym"), mode.endswith("dual")
    out = (q.cpu().numpy(), s1.cpu().numpy(), z1.cpu().numpy() if asym else None, s2.cpu().numpy() if dual else None,
           z2.cpu().numpy() if mode == "asym_dual" else None)
    if check:
        check_gpu_codes(torch, L, mode, x, *out, clip=clip)
    return out


def from_fp16_scratch(ws, M, K):
    """Decodes the scratch duq4_linear_w4a4_from_fp16 leaves behind (numpy uint8 copy of it): packed
    codes [M, K/2] and the four per-token fp16 vectors (scale_1, zeros_1, scale_2, zeros_2). Layout:
    codes (packed for M <= 16, else tensor-core-ready int8 with the row count padded to 32 for
    17..31 tokens), then the four vectors, every region 256-byte aligned."""
    al = lambda v: (v + 255) // 256 * 256
    small = M <= 16
    rows = 32 if (16 < M < 32) else M
    cbytes = M * (K // 2) if small else rows * K
    if small:
        qa = ws[: M * (K // 2)].reshape(M, K // 2).copy()
    else:
        qa = i8_codes_to_packed(ws[: M * K].view(np.int8).reshape(M, K))
    off, vec = al(cbytes), al(2 * M)
    vs = [ws[off + i * vec: off + i * vec + 2 * M].view(np.float16).copy() for i in range(4)]
    return (qa, *vs)
