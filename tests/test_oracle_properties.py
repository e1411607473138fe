"""CPU-only property tests of the oracle (the checker itself has to be right): identities that hold
for every input size, checked on random shapes with hypothesis against plain numpy."""
import numpy as np
from hypothesis import given, settings, strategies as st

from tests import _util as U


def _o():
    from oracle import oracle as o
    return o


@settings(max_examples=25, deadline=None)
@given(st.integers(1, 9), st.integers(1, 40), st.integers(0, 2**31 - 1))
def test_pack_unpack_round_trip(rows, half_cols, seed):
    o = _o()
    v = np.random.default_rng(seed).integers(-8, 8, (rows, 2 * half_cols)).astype(np.int8)
    q = o.pack_s4(v)
    assert q.shape == (rows, half_cols) and q.dtype == np.uint8
    assert np.array_equal(o.unpack_s4(q), v)
    # low nibble = even element, high nibble = odd element, two's complement
    assert np.array_equal(q & 0xF, v[:, 0::2].astype(np.uint8) & 0xF)
    assert np.array_equal(q >> 4, v[:, 1::2].astype(np.uint8) & 0xF)


@settings(max_examples=20, deadline=None)
@given(st.integers(1, 7), st.integers(1, 9), st.integers(1, 4), st.integers(0, 2**31 - 1))
def test_matmul_equals_numpy_on_unpacked_nibbles(M, N, kblocks, seed):
    """The int4 GEMM is the exact integer contraction of the signed nibbles (numpy int64 as the yardstick),
    additive over K blocks (split-K) and over output rows/columns (sharding)."""
    o = _o()
    K = 64 * kblocks
    A = U.rand_codes(M, K, seed); B = U.rand_codes(N, K, seed + 1)
    C = o.matmul_4bit(A, B)
    want = o.unpack_s4(A).astype(np.int64) @ o.unpack_s4(B).astype(np.int64).T
    assert C.dtype == np.int32 and np.array_equal(C.astype(np.int64), want)
    if kblocks > 1:   # K-split: partial accumulators add up
        h = 32 * (kblocks // 2)   # packed bytes of the first part (a multiple of 32 = 64 elements)
        part = o.matmul_4bit(np.ascontiguousarray(A[:, :h]), np.ascontiguousarray(B[:, :h])) + \
            o.matmul_4bit(np.ascontiguousarray(A[:, h:]), np.ascontiguousarray(B[:, h:]))
        assert np.array_equal(part, C)
    if N > 1:         # column shards concatenate
        n0 = N // 2
        cat = np.concatenate([o.matmul_4bit(A, np.ascontiguousarray(B[:n0])), o.matmul_4bit(A, np.ascontiguousarray(B[n0:]))], axis=1)
        assert np.array_equal(cat, C)


@settings(max_examples=20, deadline=None)
@given(st.integers(1, 6), st.integers(1, 6), st.integers(0, 2**31 - 1))
def test_symmetric_quantizer_properties(rows, col_blocks, seed):
    """Codes stay in the reference's clamp window [-8, 6]; the scale is half(half(absmax)/7); quantizing the
    dequantized codes with the same scale returns the same codes (idempotence); an all-zero row gives
    scale 0 and codes 0."""
    o = _o()
    cols = 16 * col_blocks
    x = U.acts(rows, cols, seed % 100000)
    x[0, :] = 0
    s = o.sym_scales(x, 1.0)
    amax = np.abs(x.astype(np.float32)).max(axis=1).astype(np.float16)
    assert U.bits_equal(s, (amax.astype(np.float32) / np.float32(7)).astype(np.float16))
    q = o.sym_quant(x, s)
    v = o.unpack_s4(q)
    assert v.min() >= -8 and v.max() <= 6
    assert s[0] == 0 and not v[0].any()
    back = (v.astype(np.float32) * s.astype(np.float32)[:, None]).astype(np.float16)   # exact: |v| <= 8
    assert np.array_equal(o.unpack_s4(o.sym_quant(back, s)), v)


@settings(max_examples=20, deadline=None)
@given(st.integers(1, 5), st.integers(1, 12), st.integers(0, 2**31 - 1))
def test_dequant_matches_fp16_numpy_steps(M, N, seed):
    """sym: (s_row * s_col) * half(acc); asym: (s_row * s_col) * ((half(acc) - z_row) - z_col); every step
    rounded to fp16, accumulators beyond 65504 become inf -- restated with numpy float16 arithmetic."""
    o = _o()
    rng = np.random.default_rng(seed)
    acc = rng.integers(-70000, 70000, (M, N)).astype(np.int32)
    sr = U.rand_scales(M, seed % 1000); sc = U.rand_scales(N, seed % 1000 + 1)
    zr = U.rand_zeros(M, seed % 1000 + 2); zc = U.rand_zeros(N, seed % 1000 + 3)
    h = lambda a: np.asarray(a, dtype=np.float32).astype(np.float16)
    with np.errstate(over="ignore", invalid="ignore"):
        e = h(acc.astype(np.float32))
        ss = h(sr.astype(np.float32)[:, None] * sc.astype(np.float32)[None, :])
        want_sym = h(ss.astype(np.float32) * e.astype(np.float32))
        t = h(h(e.astype(np.float32) - zr.astype(np.float32)[:, None]).astype(np.float32) - zc.astype(np.float32)[None, :])
        want_asym = h(ss.astype(np.float32) * t.astype(np.float32))
    assert U.f16_equal_nan(o.sym_dequant(acc, sr, sc), want_sym)
    assert U.f16_equal_nan(o.asym_dequant(acc, sr, zr, sc, zc), want_asym)
