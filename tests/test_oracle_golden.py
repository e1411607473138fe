"""The CPU oracle against fixtures produced by the reference's own Python code
(tests/golden/make_golden.py). CPU only."""
import numpy as np

from oracle import oracle as o


def test_pack_unpack(golden):
    assert np.array_equal(o.pack_s4(golden["pack_in_s"]), golden["pack_out_s"])
    assert np.array_equal(o.pack_s4(golden["pack_in_u"]), golden["pack_out_u"])
    assert np.array_equal(o.unpack_s4(golden["unpack_in"]).astype(np.int32), golden["unpack_out"])


def _clamp6(q7):
    """Apply the CUDA kernel's upper bound 6 to codes clamped at 7 by the torch path."""
    v = o.unpack_s4(q7)
    return o.pack_s4(np.minimum(v, o.QMAX_SYM))


def test_sym_quantizer_scales_and_codes(golden):
    for name in ("symq_a", "symq_b"):
        x = golden[name + "_x"]
        x2 = x.reshape(-1, x.shape[-1])
        s = o.sym_scales(x2, clip=float(golden[name + "_clip"]))
        # reference returns scales with shape [B,1,S] (unsqueeze(1)); flattened order is row order
        assert np.array_equal(s.view(np.uint16), golden[name + "_scales"].reshape(-1).view(np.uint16))
        q = o.sym_quant(x2, s)
        assert np.array_equal(q, _clamp6(golden[name + "_q7"].reshape(q.shape)))
    # the all-zero token quantizes to code 0 with scale 0
    assert golden["symq_a_scales"].reshape(-1)[0] == 0
    assert not o.sym_quant(golden["symq_a_x"].reshape(-1, 192)[:1], np.zeros(1, np.float16)).any()


def test_asym_quantizer(golden):
    x = golden["asymq_x"]
    x2 = x.reshape(-1, x.shape[-1])
    s, z = o.asym_scales_zeros(x2)
    assert np.array_equal(s.view(np.uint16), golden["asymq_scales"].reshape(-1).view(np.uint16))
    assert np.array_equal(z.view(np.uint16), golden["asymq_zeros"].reshape(-1).view(np.uint16))
    q = o.asym_quant(x2, s, z)
    assert np.array_equal(q, golden["asymq_q"].reshape(q.shape))


def test_matmul_accumulators(golden):
    assert np.array_equal(o.matmul_4bit(golden["mm_A"], golden["mm_B"]), golden["mm_C"])
    # batched = per-batch
    A = np.stack([golden["mm_A"], golden["mm_A"][::-1]]); B = np.stack([golden["mm_B"], golden["mm_B"][::-1]])
    C = o.batch_matmul_4bit(A, B)
    assert np.array_equal(C[0], golden["mm_C"])
    assert np.array_equal(C[1], golden["mm_C"][::-1, ::-1])


def test_all_nibble_pairs():
    """Every signed nibble pair through the GEMM restatement."""
    v = np.arange(-8, 8, dtype=np.int8)
    A = np.zeros((16, 64), np.int8); B = np.zeros((16, 64), np.int8)
    A[:, 0] = v; B[:, 0] = v
    C = o.matmul_4bit(o.pack_s4(A), o.pack_s4(B))
    assert np.array_equal(C, np.outer(v.astype(np.int32), v.astype(np.int32)))


def test_dequant_formulas_by_hand():
    """Dequant restatement against numpy float16 arithmetic written out per operation."""
    rng = np.random.default_rng(7)
    q = rng.integers(-70000, 70000, (5, 24), dtype=np.int32)
    sr = (rng.random(5) * 0.1).astype(np.float16); sc = (rng.random(24) * 0.01).astype(np.float16)
    zr = rng.integers(0, 16, 5).astype(np.float16); zc = rng.integers(0, 16, 24).astype(np.float16)
    sc2 = (rng.random(24) * 0.01).astype(np.float16); zc2 = rng.integers(0, 16, 24).astype(np.float16)
    with np.errstate(over="ignore", invalid="ignore"):
        e = q.astype(np.float32).astype(np.float16)          # +-inf beyond the half range
        ss = (sr[:, None] * sc[None, :]).astype(np.float16)  # numpy rounds each half op once
        sym = (ss * e).astype(np.float16)
        asym = (ss * ((e - zr[:, None]).astype(np.float16) - zc[None, :]).astype(np.float16)).astype(np.float16)
        scd = np.where(np.arange(24) < 10, sc, sc2)
        symd = ((sr[:, None] * scd[None, :]).astype(np.float16) * e).astype(np.float16)
        sca = np.where(np.arange(24) == 0, sc, sc2); zca = np.where(np.arange(24) == 0, zc, zc2)
        asymd = ((sr[:, None] * sca[None, :]).astype(np.float16)
                 * ((e - zr[:, None]).astype(np.float16) - zca[None, :]).astype(np.float16)).astype(np.float16)
    eq = lambda a, b: np.array_equal(a.view(np.uint16), b.view(np.uint16))
    assert np.isinf(e).any()
    assert eq(o.sym_dequant(q, sr, sc), sym)
    assert eq(o.asym_dequant(q, sr, zr, sc, zc), asym)
    assert eq(o.sym_dual_dequant(q, sr, sc, sc2), symd)
    assert eq(o.asym_dual_dequant(q, sr, zr, sc, zc, sc2, zc2), asymd)
    qb = np.stack([q, q[::-1]])
    srb = np.stack([sr, sr[::-1]]); zrb = np.stack([zr, zr[::-1]])
    got = o.asym_batch_dequant(qb, srb, zrb, np.stack([sc, sc]), np.stack([zc, zc]))
    assert eq(got[0], asym) and eq(got[1], asym[::-1])


def test_dual_quant_selector():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 40)).astype(np.float16)
    s1 = o.sym_scales(x, c0=0, c1=10); s2 = o.sym_scales(x, c0=10)
    q = o.sym_dual_quant(x, s1, s2)
    left = o.sym_quant(np.ascontiguousarray(x[:, :10]), s1); right = o.sym_quant(np.ascontiguousarray(x[:, 10:]), s2)
    assert np.array_equal(q[:, :5], left) and np.array_equal(q[:, 5:], right)
    # asym dual: add before rounding
    sa1, za1 = o.asym_scales_zeros(x, 0, 10); sa2, za2 = o.asym_scales_zeros(x, 10)
    qd = o.unpack_s4(o.asym_dual_quant(x, sa1, za1, sa2, za2)).astype(np.int32) & 0xF
    with np.errstate(all="ignore"):
        d = np.concatenate([(x[:, :10] / sa1[:, None]).astype(np.float16) + za1[:, None],
                            (x[:, 10:] / sa2[:, None]).astype(np.float16) + za2[:, None]], 1).astype(np.float16)
    assert np.array_equal(qd, np.clip(np.rint(d.astype(np.float32)), 0, 15).astype(np.int32))


def test_odd_columns_leave_high_nibble_zero():
    x = np.ones((2, 7), np.float16); s = np.full(2, 0.25, np.float16)
    q = o.sym_quant(x, s)
    assert q.shape == (2, 4) and (q[:, 3] >> 4 == 0).all() and (q[:, 3] & 0xF == 4).all()


def test_asym_weight_prep_matches_reference(golden):
    """Linear4bitASQ.from_linear of the reference vs the package's host-side weight prep."""
    import torch
    from duqlinear4bitcuda_b200.tools import quantization as qz
    w = torch.from_numpy(golden["asq_w"])
    wq, sc, zr = qz.asym_weight_quant(w)
    assert np.array_equal(wq.numpy(), golden["asq_weight"])
    assert np.array_equal(sc.numpy().view(np.uint16), golden["asq_scales"].view(np.uint16))
    assert np.array_equal(zr.numpy().view(np.uint16), golden["asq_zeros"].view(np.uint16))
