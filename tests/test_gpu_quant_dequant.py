"""GPU parity of the quantize / dequantize entry points, called through the C ABI, against
the CPU oracle (bit-exact) and, when it was built, the reference's own CUDA kernels."""
import ctypes

import numpy as np
import pytest

from tests import _util as U

pytestmark = pytest.mark.gpu

SHAPES = [(1, 64), (16, 4096), (33, 200), (5, 7), (3, 10), (2, 12), (257, 11008), (4, 28672), (2, 40000)]


@pytest.fixture(scope="module")
def env():
    import torch
    import duqlinear4bitcuda_b200.lib as L
    from oracle import oracle as o
    return torch, L, o


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _x(rows, cols, seed, asym):
    x = U.acts(rows, cols, seed, mean=0.1 if asym else 0.0, outlier_frac=0.01, outlier_mul=20.0)
    if rows > 2:
        x[1, :] = 0          # all-zero token: scale 0
        x[2, :] = x[2, 0]    # constant token: asymmetric range 0
    return x


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("mode", ["sym", "sym_dual", "asym", "asym_dual"])
def test_quant_given_scales(env, rows, cols, mode):
    torch, L, o = env
    x = _x(rows, cols, rows * 1000 + cols, "asym" in mode)
    cd = (cols + 1) // 2
    if mode == "sym":
        s1 = o.sym_scales(x); args = (s1,)
        ora = lambda n: o.sym_quant(x, s1, n)
    elif mode == "sym_dual":
        s1 = o.sym_scales(x, c0=0, c1=10); s2 = o.sym_scales(x, c0=10); args = (s1, s2)
        ora = lambda n: o.sym_dual_quant(x, s1, s2, n)
    elif mode == "asym":
        s1, z1 = o.asym_scales_zeros(x); args = (s1, z1)
        ora = lambda n: o.asym_quant(x, s1, z1, n)
    else:
        s1, z1 = o.asym_scales_zeros(x, 0, 10); s2, z2 = o.asym_scales_zeros(x, 10); args = (s1, z1, s2, z2)
        ora = lambda n: o.asym_dual_quant(x, s1, z1, s2, z2, n)
    dx = dev(torch, x); dargs = [dev(torch, a) for a in args]
    q = torch.zeros((rows, cd), dtype=torch.uint8, device="cuda")
    L.call(f"duq4_{mode}_quant", L.ptr(dx), *[L.ptr(a) for a in dargs], rows, cols, cd, L.ptr(q), L.current_stream())
    torch.cuda.synchronize()
    ok, near = U.codes_within_bracket(q.cpu().numpy(), ora(0), ora(-2), ora(2))
    assert ok
    assert near <= max(2, rows * cols // 100000)  # near-ties of the approximate divide are rare

    ref = U.load_ref_lib()
    if ref is not None:  # the reference's kernel, same inputs: bit-exact, no bracket
        q2 = torch.zeros_like(q)
        fn = getattr(ref, f"ref_{mode}_quant")
        fn.argtypes = [ctypes.c_void_p] * (1 + len(dargs)) + [ctypes.c_uint32] * 3 + [ctypes.c_void_p]
        assert fn(L.ptr(dx), *[L.ptr(a) for a in dargs], rows, cols, cd, L.ptr(q2)) == 0
        assert torch.equal(q, q2)


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("mode", ["sym", "sym_dual", "asym", "asym_dual"])
def test_quant_fused(env, rows, cols, mode):
    torch, L, o = env
    x = _x(rows, cols, rows * 77 + cols, "asym" in mode)
    clip = 0.9 if rows % 2 else 1.0
    cd = (cols + 1) // 2
    dx = dev(torch, x)
    q = torch.zeros((rows, cd), dtype=torch.uint8, device="cuda")
    vec = lambda: torch.zeros(rows, dtype=torch.float16, device="cuda")
    st = L.current_stream()
    if mode == "sym":
        s1 = vec(); outs = [s1]
        L.call("duq4_quantize_sym_fused", L.ptr(dx), rows, cols, clip, L.ptr(q), L.ptr(s1), st)
        exp = [o.sym_scales(x, clip)]
        ora = lambda n: o.sym_quant(x, exp[0], n)
    elif mode == "sym_dual":
        s1, s2 = vec(), vec(); outs = [s1, s2]
        L.call("duq4_quantize_sym_dual_fused", L.ptr(dx), rows, cols, clip, L.ptr(q), L.ptr(s1), L.ptr(s2), st)
        exp = [o.sym_scales(x, clip, 0, 10), o.sym_scales(x, clip, 10)]
        ora = lambda n: o.sym_dual_quant(x, exp[0], exp[1], n)
    elif mode == "asym":
        s1, z1 = vec(), vec(); outs = [s1, z1]
        L.call("duq4_quantize_asym_fused", L.ptr(dx), rows, cols, L.ptr(q), L.ptr(s1), L.ptr(z1), st)
        exp = list(o.asym_scales_zeros(x))
        ora = lambda n: o.asym_quant(x, exp[0], exp[1], n)
    else:
        s1, z1, s2, z2 = vec(), vec(), vec(), vec(); outs = [s1, z1, s2, z2]
        L.call("duq4_quantize_asym_dual_fused", L.ptr(dx), rows, cols, L.ptr(q), L.ptr(s1), L.ptr(z1), L.ptr(s2),
               L.ptr(z2), st)
        exp = list(o.asym_scales_zeros(x, 0, 10)) + list(o.asym_scales_zeros(x, 10))
        ora = lambda n: o.asym_dual_quant(x, exp[0], exp[1], exp[2], exp[3], n)
    torch.cuda.synchronize()
    for got, e in zip(outs, exp):
        assert U.f16_equal_nan(got.cpu().numpy(), e), mode
    ok, near = U.codes_within_bracket(q.cpu().numpy(), ora(0), ora(-2), ora(2))
    assert ok
    assert near <= max(2, rows * cols // 100000)


def test_quant_golden_fixture(env, golden):
    """Scales, zero-points and codes of the fused kernels against the fixture made by the
    reference's own quantizer modules."""
    torch, L, o = env
    for name in ("symq_a", "symq_b"):
        x = golden[name + "_x"]; x2 = np.ascontiguousarray(x.reshape(-1, x.shape[-1]))
        rows, cols = x2.shape
        dx = dev(torch, x2)
        q = torch.zeros((rows, cols // 2), dtype=torch.uint8, device="cuda"); s = torch.zeros(rows, dtype=torch.float16, device="cuda")
        L.call("duq4_quantize_sym_fused", L.ptr(dx), rows, cols, float(golden[name + "_clip"]), L.ptr(q), L.ptr(s),
               L.current_stream())
        torch.cuda.synchronize()
        assert U.bits_equal(s.cpu().numpy(), golden[name + "_scales"].reshape(-1))
        want = o.pack_s4(np.minimum(o.unpack_s4(golden[name + "_q7"].reshape(rows, -1)), 6))  # CUDA clamp bound
        assert np.array_equal(q.cpu().numpy(), want)
    x = golden["asymq_x"]; x2 = np.ascontiguousarray(x.reshape(-1, x.shape[-1]))
    rows, cols = x2.shape
    dx = dev(torch, x2)
    q = torch.zeros((rows, cols // 2), dtype=torch.uint8, device="cuda")
    s = torch.zeros(rows, dtype=torch.float16, device="cuda"); z = torch.zeros_like(s)
    L.call("duq4_quantize_asym_fused", L.ptr(dx), rows, cols, L.ptr(q), L.ptr(s), L.ptr(z), L.current_stream())
    torch.cuda.synchronize()
    assert U.bits_equal(s.cpu().numpy(), golden["asymq_scales"].reshape(-1))
    assert U.bits_equal(z.cpu().numpy(), golden["asymq_zeros"].reshape(-1))
    assert np.array_equal(q.cpu().numpy(), golden["asymq_q"].reshape(rows, -1))


def test_quant_8bit(env):
    torch, L, o = env
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((37, 130)) * 3).astype(np.float32)
    mn = x.min(1); mx = x.max(1)
    scale = ((mx - mn) / 127).astype(np.float32); zeros = np.rint(-mn / scale).astype(np.float32)
    dx, ds, dz = dev(torch, x), dev(torch, scale), dev(torch, zeros)
    q = torch.zeros((37, 130), dtype=torch.int8, device="cuda")
    L.call("duq4_asym_quant_8bit", L.ptr(dx), L.ptr(ds), L.ptr(dz), 37, 130, L.ptr(q), L.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(q.cpu().numpy(), o.asym_quant_8bit(x, scale, zeros))


DQ_SHAPES = [(1, 8), (16, 4096), (5, 33), (130, 1000), (64, 28672)]


@pytest.mark.parametrize("rows,cols", DQ_SHAPES)
def test_dequant_all_variants(env, rows, cols):
    torch, L, o = env
    rng = np.random.default_rng(rows * 31 + cols)
    q = rng.integers(-300000, 300000, (rows, cols), dtype=np.int32)
    q[0, : min(cols, 8)] = [0, 1, -1, 65504, 65520, -65520, 2047, 2049][: min(cols, 8)]
    sr = U.rand_scales(rows, 1, 0.01, 0.5); sc1 = U.rand_scales(cols, 2); sc2 = U.rand_scales(cols, 3)
    zr = U.rand_zeros(rows, 4); zc1 = U.rand_zeros(cols, 5); zc2 = U.rand_zeros(cols, 6)
    d = {k: dev(torch, v) for k, v in dict(q=q, sr=sr, sc1=sc1, sc2=sc2, zr=zr, zc1=zc1, zc2=zc2).items()}
    P = lambda k: L.ptr(d[k])
    st = L.current_stream()
    out = lambda: torch.zeros((rows, cols), dtype=torch.float16, device="cuda")
    ref = U.load_ref_lib()
    cases = {
        "sym": (("q", "sr", "sc1"), o.sym_dequant(q, sr, sc1)),
        "sym_dual": (("q", "sr", "sc1", "sc2"), o.sym_dual_dequant(q, sr, sc1, sc2)),
        "asym": (("q", "sr", "zr", "sc1", "zc1"), o.asym_dequant(q, sr, zr, sc1, zc1)),
        "asym_dual": (("q", "sr", "zr", "sc1", "zc1", "sc2", "zc2"), o.asym_dual_dequant(q, sr, zr, sc1, zc1, sc2, zc2)),
    }
    for name, (keys, want) in cases.items():
        x = out()
        L.call(f"duq4_{name}_dequant", *[P(k) for k in keys], rows, cols, L.ptr(x), st)
        torch.cuda.synchronize()
        assert U.f16_equal_nan(x.cpu().numpy(), want), name
        if ref is not None:
            x2 = out()
            fn = getattr(ref, f"ref_{name}_dequant")
            fn.argtypes = [ctypes.c_void_p] * len(keys) + [ctypes.c_uint32] * 2 + [ctypes.c_void_p]
            assert fn(*[P(k) for k in keys], rows, cols, L.ptr(x2)) == 0
            assert U.f16_equal_nan(x.cpu().numpy(), x2.cpu().numpy()), name + " vs reference kernel"


def test_dequant_batched_and_hprec(env):
    torch, L, o = env
    rng = np.random.default_rng(11)
    B, rows, cols = 3, 20, 48
    q = rng.integers(-5000, 5000, (B, rows, cols), dtype=np.int32)
    sr = U.rand_scales(B * rows, 1).reshape(B, rows); zr = U.rand_zeros(B * rows, 2).reshape(B, rows)
    sc = U.rand_scales(B * cols, 3).reshape(B, cols); zc = U.rand_zeros(B * cols, 4).reshape(B, cols)
    dq, dsr, dzr, dsc, dzc = (dev(torch, v) for v in (q, sr, zr, sc, zc))
    x = torch.zeros((B, rows, cols), dtype=torch.float16, device="cuda")
    L.call("duq4_asym_batch_dequant", L.ptr(dq), L.ptr(dsr), L.ptr(dzr), L.ptr(dsc), L.ptr(dzc), B, rows, cols, L.ptr(x),
           L.current_stream())
    torch.cuda.synchronize()
    assert U.f16_equal_nan(x.cpu().numpy(), o.asym_batch_dequant(q, sr, zr, sc, zc))
    # fp32 "hprec" dequant of the 8-bit side path
    q2 = q[0]
    fsr = rng.random(rows, dtype=np.float32); fzr = rng.integers(0, 127, rows).astype(np.float32)
    fsc = rng.random(cols, dtype=np.float32); fzc = rng.integers(0, 127, cols).astype(np.float32)
    d = [dev(torch, v) for v in (q2, fsr, fzr, fsc, fzc)]
    y = torch.zeros((rows, cols), dtype=torch.float32, device="cuda")
    L.call("duq4_asym_dequant_hprec", *[L.ptr(v) for v in d], rows, cols, L.ptr(y), L.current_stream())
    torch.cuda.synchronize()
    assert U.bits_equal(y.cpu().numpy(), o.asym_dequant_hprec(q2, fsr, fzr, fsc, fzc))


def test_empty_and_rejected_arguments(env):
    torch, L, o = env
    x = torch.zeros((4, 64), dtype=torch.float16, device="cuda"); s = torch.ones(4, dtype=torch.float16, device="cuda")
    q = torch.zeros((4, 32), dtype=torch.uint8, device="cuda")
    st = L.current_stream()
    assert L.cdll.duq4_sym_quant(L.ptr(x), L.ptr(s), 0, 64, 32, L.ptr(q), st) == 0          # empty: ok, no launch
    assert L.cdll.duq4_sym_quant(None, L.ptr(s), 4, 64, 32, L.ptr(q), st) == -1             # NULL rejected
    assert L.cdll.duq4_quantize_sym_fused(L.ptr(x), 4, 0, 1.0, L.ptr(q), L.ptr(s), st) == -2  # zero columns
    assert L.cdll.duq4_matmul_4bit(L.ptr(q), L.ptr(q), 4, 4, 48, L.ptr(q), st) == -2         # K % 64 != 0
    with pytest.raises(L.Duq4Error):
        L.call("duq4_sym_dequant", None, L.ptr(s), L.ptr(s), 4, 4, L.ptr(x), st)
    torch.cuda.synchronize()
