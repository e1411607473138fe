"""GPU parity of the integer GEMMs and the fused W4A4 linear layer, through the C ABI.

int32 accumulators are compared bit-exactly with the CPU oracle; fp16 outputs too (the
epilogue performs the reference's fp16 operations one by one), which is stricter than the
1e-3 relative tolerance the task allows. Full-size shapes are checked through a
size-independent property (row sums of C against A * (sum of B rows)) plus oracle-checked
row samples."""
import ctypes

import numpy as np
import pytest

from tests import _util as U

pytestmark = pytest.mark.gpu

REL_TOL = 1e-3  # max |got - want| / max|want| allowed for fp16 outputs (bit equality is expected)


@pytest.fixture(scope="module")
def env():
    import torch
    import duqlinear4bitcuda_b200.lib as L
    from oracle import oracle as o
    return torch, L, o


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def tc_status(L):
    v = ctypes.c_int32(-1)
    L.call("duq4_last_device_status", L.current_stream(), ctypes.byref(v))
    return v.value


def run_linear(torch, L, o, mode, M, N, K, seed, bias=True, col0=0, want_acc=True):
    qa = U.rand_codes(M, K, seed); qw = U.rand_codes(N, K, seed + 1)
    sr = U.rand_scales(M, seed + 2, 0.01, 0.3); zr = U.rand_zeros(M, seed + 3)
    sc1 = U.rand_scales(N, seed + 4); zc1 = U.rand_zeros(N, seed + 5)
    sc2 = U.rand_scales(N, seed + 6); zc2 = U.rand_zeros(N, seed + 7)
    b = (np.random.default_rng(seed + 8).standard_normal(N)).astype(np.float16) if bias else None
    acc_w, out_w = o.linear_w4a4(mode, qa, qw, sr, zr, sc1, zc1, sc2, zc2, b, col0)
    t = {k: (None if v is None else dev(torch, v)) for k, v in
         dict(qa=qa, qw=qw, sr=sr, zr=zr, sc1=sc1, zc1=zc1, sc2=sc2, zc2=zc2, b=b).items()}
    asym = mode.startswith("asym"); dual = mode.endswith("dual")
    epi = L.make_epilogue(mode, t["sr"], t["zr"] if asym else None, t["sc1"], t["zc1"] if asym else None,
                          t["sc2"] if dual else None, t["zc2"] if mode == "asym_dual" else None, t["b"], col0)
    out = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    acc = torch.full((M, N), -7, dtype=torch.int32, device="cuda") if want_acc else None
    L.call("duq4_linear_w4a4", L.ptr(t["qa"]), L.ptr(t["qw"]), M, N, K, ctypes.byref(epi), L.ptr(out), L.ptr(acc),
           L.current_stream())
    torch.cuda.synchronize()
    if M > 16:
        assert tc_status(L) == 0
    if want_acc:
        assert np.array_equal(acc.cpu().numpy(), acc_w), f"int32 accumulators differ ({mode} M={M} N={N} K={K})"
    got = out.cpu().numpy()
    fin = np.isfinite(out_w)
    denom = max(float(np.abs(out_w[fin]).max()), 1e-6)
    assert float(np.abs(got[fin].astype(np.float32) - out_w[fin].astype(np.float32)).max()) / denom <= REL_TOL
    assert U.f16_equal_nan(got, out_w), f"fp16 outputs not bit-identical ({mode} M={M} N={N} K={K})"


# ---- small-M (decode) kernel ---------------------------------------------------------------
@pytest.mark.parametrize("M", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("N,K", [(16, 64), (40, 192), (4096, 4096), (1000, 1088), (12288, 4096), (4096, 11008)])
def test_decode_linear_sym(env, M, N, K):
    torch, L, o = env
    run_linear(torch, L, o, "sym", M, N, K, seed=M * 7 + N + K)


@pytest.mark.parametrize("mode", ["sym_dual", "asym", "asym_dual"])
@pytest.mark.parametrize("M", [1, 5, 16])
def test_decode_linear_modes(env, mode, M):
    torch, L, o = env
    run_linear(torch, L, o, mode, M, 264, 512, seed=M + 100, bias=(M != 5))
    run_linear(torch, L, o, mode, M, 264, 512, seed=M + 200, col0=8)  # sharded: global column offset


@pytest.mark.parametrize("mode", ["sym_dual", "asym", "asym_dual"])
@pytest.mark.parametrize("M,N,K", [(1, 264, 4096), (7, 1000, 4160), (16, 4744, 8192), (12, 40, 5120)])
def test_decode_streaming_kernel_modes(env, mode, M, N, K):
    """Ragged N, K not a multiple of the 2048-element stage, every epilogue mode, sharded column
    offset, on both small-M kernels (the dispatcher picks by shape; the debug variable
    DUQ4_GEMV_VARIANT pins one)."""
    torch, L, o = env
    run_linear(torch, L, o, mode, M, N, K, seed=M + N, bias=(M != 7), col0=(6 if M == 16 else 0))


@pytest.mark.parametrize("variant", ["0", "1", "3"])
def test_decode_both_kernels_pinned(variant):
    """Each small-M kernel forced for every shape, in a fresh process (the choice is read once)."""
    import os, subprocess, sys
    env2 = dict(os.environ, DUQ4_GEMV_VARIANT=variant)
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", os.path.abspath(__file__), "-k",
                        "decode_streaming_kernel_modes or decode_linear_sym or decode_few_tokens or decode_streaming_kernel_batched"],
                       env=env2, capture_output=True, text=True, cwd=U.ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("N,K", [(1, 64), (8, 64), (333, 1088), (4096, 4096), (5000, 11008), (130, 28672)])
def test_decode_few_tokens_shapes(env, M, N, K):
    """1..4 tokens: single rows, ragged N, K that is not a multiple of a k-step, long rows."""
    torch, L, o = env
    mode = ["sym", "asym", "sym_dual", "asym_dual"][M - 1]
    run_linear(torch, L, o, mode, M, N, K, seed=M * 3 + N, bias=(N % 2 == 0), col0=(3 if M == 4 else 0))


def test_decode_streaming_kernel_batched(env):
    torch, L, o = env
    B, M, N, K = 3, 5, 200, 4096
    qa = U.rand_codes(B * M, K, 1).reshape(B, M, K // 2); qw = U.rand_codes(B * N, K, 2).reshape(B, N, K // 2)
    da, dw = dev(torch, qa), dev(torch, qw)
    C = torch.zeros((B, M, N), dtype=torch.int32, device="cuda")
    L.call("duq4_batch_matmul_4bit", L.ptr(da), L.ptr(dw), M, N, K, L.ptr(C), B, L.current_stream())
    torch.cuda.synchronize()
    assert tc_status(L) == 0
    assert np.array_equal(C.cpu().numpy(), o.batch_matmul_4bit(qa, qw))


def test_decode_matmul_int32_all_nibble_pairs(env):
    torch, L, o = env
    v = np.arange(-8, 8, dtype=np.int8)
    A = np.zeros((16, 64), np.int8); B = np.zeros((16, 64), np.int8)
    for k in range(64):
        A[:, k] = np.roll(v, k); B[:, k] = np.roll(v, 3 * k)
    qa, qb = o.pack_s4(A), o.pack_s4(B)
    da, db = dev(torch, qa), dev(torch, qb)
    C = torch.zeros((16, 16), dtype=torch.int32, device="cuda")
    L.call("duq4_matmul_4bit", L.ptr(da), L.ptr(db), 16, 16, 64, L.ptr(C), L.current_stream())
    torch.cuda.synchronize()
    assert np.array_equal(C.cpu().numpy(), A.astype(np.int32) @ B.astype(np.int32).T)
    assert np.array_equal(C.cpu().numpy(), o.matmul_4bit(qa, qb))


# ---- tensor-core kernel -------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(17, 128, 64), (128, 256, 128), (300, 520, 192), (128, 128, 1024), (257, 1000, 4096),
                                   (1024, 4096, 4096)])
def test_tc_matmul_int32(env, M, N, K):
    torch, L, o = env
    qa = U.rand_codes(M, K, M + N); qb = U.rand_codes(N, K, K + 1)
    da, db = dev(torch, qa), dev(torch, qb)
    C = torch.full((M, N), -3, dtype=torch.int32, device="cuda")
    L.call("duq4_matmul_4bit", L.ptr(da), L.ptr(db), M, N, K, L.ptr(C), L.current_stream())
    torch.cuda.synchronize()
    assert tc_status(L) == 0
    assert np.array_equal(C.cpu().numpy(), o.matmul_4bit(qa, qb))
    ref = U.load_ref_lib()
    if ref is not None and N % 4 == 0:   # the reference's CUTLASS int4 GEMM on the same inputs
        C2 = torch.zeros_like(C)
        ref.ref_matmul_4bit.argtypes = [ctypes.c_void_p] * 2 + [ctypes.c_uint32] * 3 + [ctypes.c_void_p]
        if ref.ref_matmul_4bit(L.ptr(da), L.ptr(db), M, N, K, L.ptr(C2)) == 0:
            assert torch.equal(C, C2)


@pytest.mark.parametrize("mode", ["sym", "sym_dual", "asym", "asym_dual"])
def test_tc_linear_modes(env, mode):
    torch, L, o = env
    run_linear(torch, L, o, mode, 200, 392, 256, seed=41)
    run_linear(torch, L, o, mode, 130, 264, 128, seed=42, bias=False, col0=4)
    run_linear(torch, L, o, mode, 512, 2048, 1024, seed=43, want_acc=False)


def test_tc_output_row_stride(env):
    """Writing into a column slice of a wider [M, N_total] buffer (N-sharded layers)."""
    torch, L, o = env
    M, N, K, NT = 150, 256, 128, 768
    qa = U.rand_codes(M, K, 1); qw = U.rand_codes(N, K, 2)
    sr = U.rand_scales(M, 3); sc = U.rand_scales(N, 4)
    _, want = o.linear_w4a4("sym", qa, qw, sr, None, sc, None, None, None)
    t = [dev(torch, v) for v in (qa, qw, sr, sc)]
    big = torch.zeros((M, NT), dtype=torch.float16, device="cuda")
    epi = L.make_epilogue("sym", t[2], None, t[3], ldo=NT)
    L.call("duq4_linear_w4a4", L.ptr(t[0]), L.ptr(t[1]), M, N, K, ctypes.byref(epi),
           ctypes.c_void_p(big.data_ptr() + 256 * 2), None, L.current_stream())
    torch.cuda.synchronize()
    got = big.cpu().numpy()
    assert U.f16_equal_nan(got[:, 256:512], want) and not got[:, :256].any() and not got[:, 512:].any()


@pytest.mark.parametrize("M,N,K", [(64, 128, 64), (200, 300, 208), (128, 256, 4096)])
def test_tc_matmul_8bit(env, M, N, K):
    torch, L, o = env
    rng = np.random.default_rng(M)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8); B = rng.integers(-128, 128, (N, K), dtype=np.int8)
    da, db = dev(torch, A), dev(torch, B)
    C = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    L.call("duq4_matmul_8bit", L.ptr(da), L.ptr(db), M, N, K, L.ptr(C), L.current_stream())
    torch.cuda.synchronize()
    assert tc_status(L) == 0
    assert np.array_equal(C.cpu().numpy(), o.matmul_8bit(A, B))


@pytest.mark.parametrize("B,M,N,K", [(3, 8, 48, 128), (4, 100, 160, 192), (8, 256, 4096, 4096)])
def test_batched(env, B, M, N, K):
    torch, L, o = env
    qa = U.rand_codes(B * M, K, 9).reshape(B, M, K // 2); qw = U.rand_codes(B * N, K, 10).reshape(B, N, K // 2)
    da, dw = dev(torch, qa), dev(torch, qw)
    C = torch.zeros((B, M, N), dtype=torch.int32, device="cuda")
    L.call("duq4_batch_matmul_4bit", L.ptr(da), L.ptr(dw), M, N, K, L.ptr(C), B, L.current_stream())
    torch.cuda.synchronize()
    want = o.batch_matmul_4bit(qa, qw)
    assert np.array_equal(C.cpu().numpy(), want)
    # fused batched asymmetric epilogue = asym_batch_dequant of the accumulators
    sr = U.rand_scales(B * M, 1).reshape(B, M); zr = U.rand_zeros(B * M, 2).reshape(B, M)
    sc = U.rand_scales(B * N, 3).reshape(B, N); zc = U.rand_zeros(B * N, 4).reshape(B, N)
    t = [dev(torch, v) for v in (sr, zr, sc, zc)]
    epi = L.make_epilogue("asym", t[0], t[1], t[2], t[3])
    out = torch.zeros((B, M, N), dtype=torch.float16, device="cuda")
    L.call("duq4_linear_w4a4_batched", L.ptr(da), L.ptr(dw), M, N, K, B, ctypes.byref(epi), L.ptr(out), None,
           L.current_stream())
    torch.cuda.synchronize()
    assert U.f16_equal_nan(out.cpu().numpy(), o.asym_batch_dequant(want, sr, zr, sc, zc))


@pytest.mark.parametrize("M", [1, 4, 20, 31, 300])   # 1: single launch; 20, 31: the int8 code buffer is padded to 32 rows
@pytest.mark.parametrize("mode", ["sym", "sym_dual", "asym", "asym_dual"])
def test_linear_from_fp16(env, M, mode):
    """quantize -> GEMM -> dequant in one call, scratch supplied by the caller. The codes and per-token
    vectors the call leaves in its scratch are checked against the oracle (and the reference's quantize
    kernel) by U.check_gpu_codes; the oracle's GEMM + dequant on exactly those codes must then give every
    output row bit for bit."""
    torch, L, o = env
    N, K = 520, 1024
    asym, dual = mode.startswith("asym"), mode.endswith("dual")
    x = U.acts(M, K, 5, mean=0.1 if asym else 0.0)
    w = (np.random.default_rng(6).standard_normal((N, K)) * 0.02).astype(np.float16)
    qw, sw = o.weight_sym_quant_pack(w)
    zc = U.rand_zeros(N, 7); sw2 = U.rand_scales(N, 8); zc2 = U.rand_zeros(N, 9)
    dx, dw, dsw, dzc, dsw2, dzc2 = (dev(torch, v) for v in (x, qw, sw, zc, sw2, zc2))
    nbytes = L.cdll.duq4_linear_from_fp16_workspace_bytes(M, K)
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    epi = L.make_epilogue(mode, None, None, dsw, dzc if asym else None, dsw2 if dual else None, dzc2 if mode == "asym_dual" else None)
    out = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    for _ in range(2):  # the scratch is reused between calls
        L.call("duq4_linear_w4a4_from_fp16", L.ptr(dx), L.ptr(dw), M, N, K, L.MODES[mode], 1.0, ctypes.byref(epi), L.ptr(out),
               L.ptr(ws), nbytes, L.current_stream())
    torch.cuda.synchronize()
    if M > 16:
        assert tc_status(L) == 0
    if M > 1:    # two launches: the codes and per-token vectors the call's quantizer wrote are in its scratch
        qa, s1, z1, s2, z2 = U.from_fp16_scratch(ws.cpu().numpy(), M, K)
        U.check_gpu_codes(torch, L, mode, x, qa, s1, z1 if asym else None, s2 if dual else None, z2 if mode == "asym_dual" else None)
    else:        # one launch, codes never leave the CTAs' shared memory (their parity: test_small_m_fused_quantizer_codes);
        # the oracle runs on the stand-alone fused quantizer's codes, which U.gpu_quantize checks
        assert not ws.any(), "the single-launch route must leave the workspace untouched"
        qa, s1, z1, s2, z2 = U.gpu_quantize(torch, L, mode, x)
    # the epilogue uses set 1 of the per-token vectors (the reference modules carry one row-scale vector)
    _, want = o.linear_w4a4(mode, qa, qw, s1, z1 if asym else None, sw, zc if asym else None, sw2 if dual else None,
                            zc2 if mode == "asym_dual" else None)
    assert U.f16_equal_nan(out.cpu().numpy(), want), f"{mode} M={M}: fp16 outputs differ from the oracle on the call's own codes"
    assert L.cdll.duq4_linear_w4a4_from_fp16(L.ptr(dx), L.ptr(dw), M, N, K, L.MODES[mode], 1.0, ctypes.byref(epi), L.ptr(out),
                                             L.ptr(ws), nbytes - 1, L.current_stream()) == -4


@pytest.mark.parametrize("variant", [None, "0", "1", "3"])
@pytest.mark.parametrize("mode", ["sym", "sym_dual", "asym", "asym_dual"])
def test_small_m_fused_quantizer_codes(env, mode, variant):
    """The single-launch route of duq4_linear_w4a4_from_fp16: the CTAs of the small-M kernel quantize the tokens in
    shared memory. It is taken for one token by default; DUQ4_FUSEQ_MAX_M=16 (set here, in a fresh process) lets
    every token count up to 16 take it, so the in-kernel quantizer is checked for all of them.
    The codes are made visible through the public entry point with a weight matrix that copies them out: weight
    row n holds code 1 at input channel n and 0 elsewhere, all per-channel scales 1 (zero-points 0), so the fp16
    output element [m, n] is (s_m * 1) * (code[m, n] (- z_m)) -- a different value for each of the 16 codes.
    Scales, zero-points and codes must equal those of the stand-alone fused quantizer (which U.gpu_quantize
    checks against the oracle and the reference's kernel), for every token count 1..16, on each of the three
    small-M kernels (variant pins one in a fresh process), including an all-zero token, a constant token and
    tokens holding inf / NaN."""
    import os
    if variant is not None or os.environ.get("DUQ4_FUSEQ_MAX_M") != "16":
        import subprocess, sys
        env2 = dict(os.environ, DUQ4_FUSEQ_MAX_M="16")
        if variant is not None:
            env2["DUQ4_GEMV_VARIANT"] = variant
        r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu",
                            f"{os.path.abspath(__file__)}::test_small_m_fused_quantizer_codes[{mode}-None]"],
                           env=env2, capture_output=True, text=True, cwd=U.ROOT)
        assert r.returncode == 0 and " passed" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
        return
    torch, L, o = env
    asym, dual = mode.startswith("asym"), mode.endswith("dual")
    for K in (64, 704, 4096):
        eye = np.zeros((K, K), dtype=np.int8); np.fill_diagonal(eye, 1)
        dw = dev(torch, o.pack_s4(eye))
        one = torch.ones(K, dtype=torch.float16, device="cuda"); zero = torch.zeros(K, dtype=torch.float16, device="cuda")
        epi = L.make_epilogue(mode, None, None, one, zero if asym else None, one if dual else None, zero if mode == "asym_dual" else None)
        for M in (1, 2, 3, 5, 8, 9, 13, 16):
            if M * (K // 2 * 5 + 64) + 1024 > 96 * 1024:
                continue   # staging copy + code rows exceed the shared-memory budget: the call takes two launches
            x = U.acts(M, K, 100 + M + K, mean=0.1 if asym else 0.0)
            if M >= 5:
                x[1] = 0; x[2] = x[2, 0]; x[3, 5] = np.inf; x[4, 7] = np.nan
            dx = dev(torch, x)
            nbytes = L.cdll.duq4_linear_from_fp16_workspace_bytes(M, K)
            ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
            out = torch.full((M, K), float("nan"), dtype=torch.float16, device="cuda")
            L.call("duq4_linear_w4a4_from_fp16", L.ptr(dx), L.ptr(dw), M, K, K, L.MODES[mode], 0.9, ctypes.byref(epi), L.ptr(out),
                   L.ptr(ws), nbytes, L.current_stream())
            torch.cuda.synchronize()
            qa, s1, z1, s2, z2 = U.gpu_quantize(torch, L, mode, x, clip=0.9, check=(M < 5))   # inf/NaN tokens: no oracle bracket
            codes = o.unpack_s4(qa).astype(np.int32)   # asymmetric codes 8..15 read back as -8..-1, as the GEMM reads them
            want = o.asym_dequant(codes, s1, z1, np.ones(K, np.float16), np.zeros(K, np.float16)) if asym else \
                o.sym_dequant(codes, s1, np.ones(K, np.float16))
            assert U.f16_equal_nan(out.cpu().numpy(), want), f"{mode} K={K} M={M}"


@pytest.mark.parametrize("M,chunk_rows,pinned,pitch", [(4, 0, True, 0), (300, 0, True, 0), (1300, 256, True, 0),
                                                      (1300, 512, False, 0), (777, 256, True, 24), (2048, 0, True, 0)])
def test_linear_from_fp16_host_entry_equals_device_entry(env, M, chunk_rows, pinned, pitch):
    """Host-buffer entry (chunked, three streams) == device-buffer entry bit for bit: every stage is
    per token, so cutting the tokens into row chunks changes nothing. Covers ragged last chunks (20 rows
    of 1300: tensor-core kernel; 9 rows of 777: small-M kernel), an output row pitch, pageable host
    memory, and two calls in a row on the same staging area."""
    torch, L, o = env
    N, K = 776, 1024
    x = U.acts(M, K, 15, mean=0.05)
    w = (np.random.default_rng(16).standard_normal((N, K)) * 0.02).astype(np.float16)
    qw, sw = o.weight_sym_quant_pack(w)
    zc = U.rand_zeros(N, 17)
    b = np.random.default_rng(18).standard_normal(N).astype(np.float16)
    dx, dw, dsw, dzc, db = (dev(torch, v) for v in (x, qw, sw, zc, b))
    ldo = N + pitch
    for mode in ("sym", "asym"):
        epi = L.make_epilogue(mode, None, None, dsw, dzc if mode == "asym" else None, None, None, db)
        nbytes = L.cdll.duq4_linear_from_fp16_workspace_bytes(M, K)
        ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        want = torch.zeros((M, N), dtype=torch.float16, device="cuda")
        L.call("duq4_linear_w4a4_from_fp16", L.ptr(dx), L.ptr(dw), M, N, K, L.MODES[mode], 1.0, ctypes.byref(epi),
               L.ptr(want), L.ptr(ws), nbytes, L.current_stream())
        xh = torch.from_numpy(x.copy())
        oh = torch.full((M, ldo), -3.0, dtype=torch.float16)
        if pinned:
            xh, oh = xh.pin_memory(), oh.pin_memory()
        sbytes = L.cdll.duq4_linear_host_staging_bytes(M, N, K, chunk_rows)
        staging = torch.zeros(sbytes, dtype=torch.uint8, device="cuda")
        epi_h = L.make_epilogue(mode, None, None, dsw, dzc if mode == "asym" else None, None, None, db, ldo=ldo)
        for _ in range(2):
            L.call("duq4_linear_w4a4_from_fp16_host", xh.data_ptr(), L.ptr(dw), M, N, K, L.MODES[mode], 1.0,
                   ctypes.byref(epi_h), oh.data_ptr(), chunk_rows, L.ptr(staging), sbytes, L.current_stream())
        torch.cuda.synchronize()   # the helper streams joined the caller's stream before the call returned
        assert tc_status(L) == 0
        got = oh.numpy()
        assert U.f16_equal_nan(got[:, :N], want.cpu().numpy()), f"{mode}: host entry differs from device entry"
        if pitch:
            assert np.all(got[:, N:] == np.float16(-3.0)), "padding columns of the host result were written"
        assert L.cdll.duq4_linear_w4a4_from_fp16_host(xh.data_ptr(), L.ptr(dw), M, N, K, L.MODES[mode], 1.0, ctypes.byref(epi_h),
                                                      oh.data_ptr(), chunk_rows, L.ptr(staging), sbytes - 1,
                                                      L.current_stream()) == -4


def test_full_size_property_prefill(env):
    """Benchmark-size prefill layer (M=4096, K=8192, N=28672): row sums of the int32 result must
    equal A * (sum of weight rows), and sampled rows must match the oracle exactly."""
    torch, L, o = env
    M, N, K = 4096, 28672, 8192
    g = torch.Generator(device="cuda").manual_seed(0)
    qa = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device="cuda", generator=g)
    qw = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device="cuda", generator=g)
    C = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    L.call("duq4_matmul_4bit", L.ptr(qa), L.ptr(qw), M, N, K, L.ptr(C), L.current_stream())
    torch.cuda.synchronize()
    assert tc_status(L) == 0

    def unpack(q):  # torch-side signed unpack, used only for the property
        lo = (q & 0xF).to(torch.int16); hi = (q >> 4).to(torch.int16)
        lo = torch.where(lo >= 8, lo - 16, lo); hi = torch.where(hi >= 8, hi - 16, hi)
        return torch.stack([lo, hi], -1).reshape(q.shape[0], -1)

    wsum = torch.zeros(K, dtype=torch.float64, device="cuda")
    for i in range(0, N, 4096):
        wsum += unpack(qw[i:i + 4096]).to(torch.float64).sum(0)
    rows = C.to(torch.float64).sum(1)
    want = torch.zeros(M, dtype=torch.float64, device="cuda")
    for i in range(0, M, 1024):
        want[i:i + 1024] = unpack(qa[i:i + 1024]).to(torch.float64) @ wsum
    assert torch.equal(rows, want)
    idx = [0, 1, 127, 128, 2047, 4095]
    sub = o.matmul_4bit(qa[idx].cpu().numpy(), qw.cpu().numpy())
    assert np.array_equal(C[idx].cpu().numpy(), sub)


@pytest.mark.parametrize("M,N,K", [(8192, 512, 256), (4500, 520, 384), (2304, 256, 16512), (8192, 256, 128)])
def test_banded_tile_order_covers_every_tile_once(env, M, N, K):
    """Problems with more row blocks than one band of the CTA-pair kernel's tile order (16 row blocks; 8 when
    K > 16384), ragged last bands included: the int32 accumulators of the packed route and of the pre-laid-out route
    (with the K-split) must equal an fp32 matrix product of the unpacked codes (exact: every partial sum is an integer
    below 2^24) in every element -- a tile computed twice or left out would show."""
    torch, L, o = env
    g = torch.Generator(device="cuda").manual_seed(M + K)
    qa = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device="cuda", generator=g)
    qw = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device="cuda", generator=g)
    st = L.current_stream()

    def unpack(q):
        lo = (q & 0xF).to(torch.int16); hi = (q >> 4).to(torch.int16)
        lo = torch.where(lo >= 8, lo - 16, lo); hi = torch.where(hi >= 8, hi - 16, hi)
        return torch.stack([lo, hi], -1).reshape(q.shape[0], -1)

    ai, wi = unpack(qa), unpack(qw)
    want = (ai.float() @ wi.float().T).to(torch.int32)
    C = torch.full((M, N), -7, dtype=torch.int32, device="cuda")
    L.call("duq4_matmul_4bit", L.ptr(qa), L.ptr(qw), M, N, K, L.ptr(C), st)
    torch.cuda.synchronize()
    assert torch.equal(C, want)
    # the pre-laid-out route: the same codes as tensor-core-ready int8 (16 * code, K permuted inside 128-blocks by the
    # library's own re-layout of the packed tensor, which works on any packed [rows, K/2] tensor)
    a8 = torch.empty((M, K), dtype=torch.int8, device="cuda"); w8 = torch.empty((N, K), dtype=torch.int8, device="cuda")
    L.call("duq4_weight_prelayout_i8", L.ptr(qa), M, K, L.ptr(a8), st)
    L.call("duq4_weight_prelayout_i8", L.ptr(qw), N, K, L.ptr(w8), st)
    sk = torch.empty(L.cdll.duq4_gemm_split_scratch_bytes(), dtype=torch.uint8, device="cuda")
    C2 = torch.full((M, N), -7, dtype=torch.int32, device="cuda")
    L.call("duq4_linear_w4a4_prelaid", L.ptr(a8), L.ptr(w8), M, N, K, ctypes.byref(L.make_epilogue("none")), None, L.ptr(C2), L.ptr(sk), sk.numel(), st)
    torch.cuda.synchronize()
    assert tc_status(L) == 0
    assert torch.equal(C2, want)


@pytest.mark.parametrize("M", [4096, 512])
def test_full_size_headline_route_equals_packed_route(env, M):
    """The route bench.py times at the benchmark size (K=8192, N=28672; 4096 tokens, and 512 where the last round of
    tiles is split along K over eight CTA pairs): fused quantizer to tensor-core-ready int8 codes, weights pre-laid-out
    to int8, CTA-pair GEMM with the K-split. Its int32 accumulators must equal those of duq4_matmul_4bit on the packed
    codes of the same tokens in every one of the M x N elements, and their row sums must equal codes * (sum of the
    weight rows) computed in fp64 from the packed tensors."""
    torch, L, o = env
    N, K = 28672, 8192
    g = torch.Generator(device="cuda").manual_seed(M)
    x = (torch.randn((M, K), device="cuda", generator=g) * (1 + 19 * (torch.rand(K, device="cuda", generator=g) < 0.01))).half()
    qw = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device="cuda", generator=g)
    st = L.current_stream()
    qa = torch.empty((M, K // 2), dtype=torch.uint8, device="cuda"); s_p = torch.empty(M, dtype=torch.float16, device="cuda")
    a8 = torch.empty((M, K), dtype=torch.int8, device="cuda"); s_8 = torch.empty(M, dtype=torch.float16, device="cuda")
    L.call("duq4_quantize_sym_fused", L.ptr(x), M, K, 1.0, L.ptr(qa), L.ptr(s_p), st)
    L.call("duq4_quantize_fused_i8", L.MODE_SYM, L.ptr(x), M, K, 1.0, L.ptr(a8), L.ptr(s_8), None, None, None, st)
    w8 = torch.empty((N, K), dtype=torch.int8, device="cuda")
    L.call("duq4_weight_prelayout_i8", L.ptr(qw), N, K, L.ptr(w8), st)
    sk = torch.empty(L.cdll.duq4_gemm_split_scratch_bytes(), dtype=torch.uint8, device="cuda")
    C = torch.full((M, N), -7, dtype=torch.int32, device="cuda"); C_ref = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    L.call("duq4_linear_w4a4_prelaid", L.ptr(a8), L.ptr(w8), M, N, K, ctypes.byref(L.make_epilogue("none")), None, L.ptr(C), L.ptr(sk), sk.numel(), st)
    L.call("duq4_matmul_4bit", L.ptr(qa), L.ptr(qw), M, N, K, L.ptr(C_ref), st)
    torch.cuda.synchronize()
    assert tc_status(L) == 0
    assert torch.equal(s_p.view(torch.int16), s_8.view(torch.int16))
    assert torch.equal(C, C_ref)

    def unpack(q):
        lo = (q & 0xF).to(torch.int16); hi = (q >> 4).to(torch.int16)
        lo = torch.where(lo >= 8, lo - 16, lo); hi = torch.where(hi >= 8, hi - 16, hi)
        return torch.stack([lo, hi], -1).reshape(q.shape[0], -1)

    wsum = torch.zeros(K, dtype=torch.float64, device="cuda")
    for i in range(0, N, 4096):
        wsum += unpack(qw[i:i + 4096]).to(torch.float64).sum(0)
    want = torch.zeros(M, dtype=torch.float64, device="cuda")
    for i in range(0, M, 1024):
        want[i:i + 1024] = unpack(qa[i:i + 1024]).to(torch.float64) @ wsum
    assert torch.equal(C.to(torch.float64).sum(1), want)


@pytest.mark.parametrize("mode", ["sym", "sym_dual", "asym", "asym_dual"])
@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (130, 264, 192), (512, 1024, 2048),
                                   # up to 128 tokens: narrow-tile launches (tile width picked by N: 160 / 128 / 96 / 64)
                                   (17, 22016, 256), (64, 1000, 1088), (100, 20000, 192), (128, 4104, 448), (33, 12288, 320)])
def test_preunpacked_activations_match_packed_path(env, mode, M, N, K):
    """duq4_quantize_fused_i8 + duq4_linear_w4a4_preunpacked give the scales and outputs of
    duq4_quantize_*_fused + duq4_linear_w4a4, and the int32 accumulators of the oracle."""
    torch, L, o = env
    x = U.acts(M, K, M + K, mean=0.1 if "asym" in mode else 0.0)
    dx = dev(torch, x)
    qw = U.rand_codes(N, K, 3); dqw = dev(torch, qw)
    sc1 = dev(torch, U.rand_scales(N, 4)); zc1 = dev(torch, U.rand_zeros(N, 5))
    sc2 = dev(torch, U.rand_scales(N, 6)); zc2 = dev(torch, U.rand_zeros(N, 7))
    vec = lambda: torch.zeros(M, dtype=torch.float16, device="cuda")
    st = L.current_stream()
    s1, z1, s2, z2 = vec(), vec(), vec(), vec()
    t1, y1, t2, y2 = vec(), vec(), vec(), vec()
    q = torch.zeros((M, K // 2), dtype=torch.uint8, device="cuda")
    a8 = torch.zeros((M, K), dtype=torch.int8, device="cuda")
    if mode == "sym":
        L.call("duq4_quantize_sym_fused", L.ptr(dx), M, K, 1.0, L.ptr(q), L.ptr(s1), st)
    elif mode == "sym_dual":
        L.call("duq4_quantize_sym_dual_fused", L.ptr(dx), M, K, 1.0, L.ptr(q), L.ptr(s1), L.ptr(s2), st)
    elif mode == "asym":
        L.call("duq4_quantize_asym_fused", L.ptr(dx), M, K, L.ptr(q), L.ptr(s1), L.ptr(z1), st)
    else:
        L.call("duq4_quantize_asym_dual_fused", L.ptr(dx), M, K, L.ptr(q), L.ptr(s1), L.ptr(z1), L.ptr(s2), L.ptr(z2), st)
    L.call("duq4_quantize_fused_i8", L.MODES[mode], L.ptr(dx), M, K, 1.0, L.ptr(a8), L.ptr(t1), L.ptr(y1), L.ptr(t2), L.ptr(y2), st)
    torch.cuda.synchronize()
    assert torch.equal(s1.view(torch.int16), t1.view(torch.int16))
    if "asym" in mode:
        assert torch.equal(z1.view(torch.int16), y1.view(torch.int16))
    # the int8 buffer is 16 * code, K-permuted inside 128-blocks: undo the permutation and compare
    codes = o.unpack_s4(q.cpu().numpy()).astype(np.int16)
    a = a8.cpu().numpy().astype(np.int16)
    pos = np.arange(K); blk, r = pos // 128, pos % 128
    src = blk * 128 + 32 * (r // 32) + 2 * (r % 16) + ((r % 32) // 16)
    assert np.array_equal(a, 16 * codes[:, src])
    asym = mode.startswith("asym"); dual = mode.endswith("dual")
    epi = L.make_epilogue(mode, s1, z1 if asym else None, sc1, zc1 if asym else None, sc2 if dual else None,
                          zc2 if mode == "asym_dual" else None)
    out_a = torch.zeros((M, N), dtype=torch.float16, device="cuda"); out_b = torch.zeros_like(out_a)
    acc_b = torch.zeros((M, N), dtype=torch.int32, device="cuda")
    L.call("duq4_linear_w4a4", L.ptr(q), L.ptr(dqw), M, N, K, ctypes.byref(epi), L.ptr(out_a), None, st)
    L.call("duq4_linear_w4a4_preunpacked", L.ptr(a8), L.ptr(dqw), M, N, K, ctypes.byref(epi), L.ptr(out_b), L.ptr(acc_b), st)
    torch.cuda.synchronize()
    assert tc_status(L) == 0
    assert np.array_equal(acc_b.cpu().numpy(), o.matmul_4bit(q.cpu().numpy(), qw))
    assert U.f16_equal_nan(out_a.cpu().numpy(), out_b.cpu().numpy())


@pytest.mark.parametrize("mode", ["sym", "asym_dual"])
@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (17, 1000, 128), (300, 520, 256), (2000, 2100, 384), (512, 4096, 4096), (300, 520, 2048)])
def test_prelaid_int8_weights_match_packed_weights(env, mode, M, N, K):
    """duq4_weight_prelayout_i8 + duq4_linear_w4a4_prelaid (both operands int8 in the tensor-core-ready layout, no
    in-kernel unpack) give the int32 accumulators of the oracle and the fp16 outputs of the packed-weight path."""
    torch, L, o = env
    asym, dual = mode.startswith("asym"), mode.endswith("dual")
    x = U.acts(M, K, M + K, mean=0.1 if asym else 0.0); dx = dev(torch, x)
    qw = U.rand_codes(N, K, 3); dqw = dev(torch, qw)
    sc1 = dev(torch, U.rand_scales(N, 4)); zc1 = dev(torch, U.rand_zeros(N, 5))
    sc2 = dev(torch, U.rand_scales(N, 6)); zc2 = dev(torch, U.rand_zeros(N, 7))
    vec = lambda: torch.zeros(M, dtype=torch.float16, device="cuda")
    s1, z1, s2, z2 = vec(), vec(), vec(), vec()
    a8 = torch.zeros((M, K), dtype=torch.int8, device="cuda")
    w8 = torch.zeros((N, K), dtype=torch.int8, device="cuda")
    st = L.current_stream()
    L.call("duq4_quantize_fused_i8", L.MODES[mode], L.ptr(dx), M, K, 1.0, L.ptr(a8), L.ptr(s1), L.ptr(z1), L.ptr(s2), L.ptr(z2), st)
    L.call("duq4_weight_prelayout_i8", L.ptr(dqw), N, K, L.ptr(w8), st)
    torch.cuda.synchronize()
    assert np.array_equal(U.i8_codes_to_packed(w8.cpu().numpy()), qw)   # the same layout the activation quantizer writes
    epi = L.make_epilogue(mode, s1, z1 if asym else None, sc1, zc1 if asym else None, sc2 if dual else None, zc2 if dual and asym else None)
    out_a = torch.zeros((M, N), dtype=torch.float16, device="cuda"); out_b = torch.full_like(out_a, float("nan"))
    acc_b = torch.full((M, N), -5, dtype=torch.int32, device="cuda")
    L.call("duq4_linear_w4a4_preunpacked", L.ptr(a8), L.ptr(dqw), M, N, K, ctypes.byref(epi), L.ptr(out_a), None, st)
    L.call("duq4_linear_w4a4_prelaid", L.ptr(a8), L.ptr(w8), M, N, K, ctypes.byref(epi), L.ptr(out_b), L.ptr(acc_b), None, 0, st)
    # ... and with scratch for the K-split of the last round of tiles (same bits: the partial sums are exact)
    split = torch.full((L.cdll.duq4_gemm_split_scratch_bytes(),), 0x5A, dtype=torch.uint8, device="cuda")
    out_c = torch.full_like(out_a, float("nan")); acc_c = torch.full_like(acc_b, -5)
    L.call("duq4_linear_w4a4_prelaid", L.ptr(a8), L.ptr(w8), M, N, K, ctypes.byref(epi), L.ptr(out_c), L.ptr(acc_c), L.ptr(split), split.numel(), st)
    torch.cuda.synchronize()
    assert torch.equal(acc_c, acc_b) and torch.equal(out_c.view(torch.int16), out_b.view(torch.int16))
    torch.cuda.synchronize()
    assert tc_status(L) == 0
    assert np.array_equal(acc_b.cpu().numpy(), o.matmul_4bit(U.i8_codes_to_packed(a8.cpu().numpy()), qw))
    assert U.f16_equal_nan(out_a.cpu().numpy(), out_b.cpu().numpy())
    assert L.cdll.duq4_weight_prelayout_i8(L.ptr(dqw), N, 192, L.ptr(w8), st) == -2   # K must be a multiple of 128


@pytest.mark.parametrize("mode", ["sym", "sym_dual", "asym", "asym_dual"])
@pytest.mark.parametrize("M,N,K", [(5, 264, 128), (300, 520, 1024), (2100, 2000, 256),
                                   # launches whose last round of tiles is split along K: 6 tiles by 8 pairs each (32 k-steps),
                                   # 150 tiles = 2 full rounds + 2 tiles by 2 pairs each (8 k-steps), 76 tiles = 1 round + 2 tiles by 8
                                   (300, 520, 4096), (512, 19200, 1024), (256, 19456, 4224)])
def test_linear_from_fp16_prelaid_equals_packed_weight_entry(env, mode, M, N, K):
    """The one-call layer on pre-laid-out int8 weights == the one-call layer on the packed weights, bit for bit
    (the packed-weight entry is checked against the oracle elsewhere), including launches that split the tiles of
    their last round along K and add int32 partial tiles before the dequant."""
    torch, L, o = env
    asym, dual = mode.startswith("asym"), mode.endswith("dual")
    dx = dev(torch, U.acts(M, K, 3, mean=0.1 if asym else 0.0)); dqw = dev(torch, U.rand_codes(N, K, 4))
    sc1, zc1, sc2, zc2 = (dev(torch, v) for v in (U.rand_scales(N, 5), U.rand_zeros(N, 6), U.rand_scales(N, 7), U.rand_zeros(N, 8)))
    bias = dev(torch, np.random.default_rng(9).standard_normal(N).astype(np.float16))
    epi = L.make_epilogue(mode, None, None, sc1, zc1 if asym else None, sc2 if dual else None, zc2 if mode == "asym_dual" else None, bias)
    w8 = torch.zeros((N, K), dtype=torch.int8, device="cuda")
    L.call("duq4_weight_prelayout_i8", L.ptr(dqw), N, K, L.ptr(w8), L.current_stream())
    nbytes = L.cdll.duq4_linear_from_fp16_prelaid_workspace_bytes(M, K)
    assert nbytes >= L.cdll.duq4_linear_from_fp16_workspace_bytes(M, K)
    ws = torch.full((nbytes,), 0xAB, dtype=torch.uint8, device="cuda")   # the call must not rely on a cleared workspace
    want = torch.zeros((M, N), dtype=torch.float16, device="cuda"); got = torch.full_like(want, float("nan"))
    L.call("duq4_linear_w4a4_from_fp16", L.ptr(dx), L.ptr(dqw), M, N, K, L.MODES[mode], 0.9, ctypes.byref(epi), L.ptr(want), L.ptr(ws), nbytes,
           L.current_stream())
    for _ in range(2):   # twice: the arrival counters of the K-split are cleared by every call
        L.call("duq4_linear_w4a4_from_fp16_prelaid", L.ptr(dx), L.ptr(w8), M, N, K, L.MODES[mode], 0.9, ctypes.byref(epi), L.ptr(got), L.ptr(ws), nbytes,
               L.current_stream())
    torch.cuda.synchronize()
    assert tc_status(L) == 0
    assert U.f16_equal_nan(got.cpu().numpy(), want.cpu().numpy())
    assert L.cdll.duq4_linear_w4a4_from_fp16_prelaid(L.ptr(dx), L.ptr(w8), M, N, K, L.MODES[mode], 0.9, ctypes.byref(epi), L.ptr(got), L.ptr(ws),
                                                     M * K, L.current_stream()) == -4


@pytest.mark.parametrize("mode", ["sym", "asym"])
@pytest.mark.parametrize("M,N,K,G", [(8, 264, 256, 2), (300, 520, 1024, 2), (1000, 1032, 768, 3), (2100, 2000, 512, 4)])
def test_row_parallel_pieces_on_one_gpu_equal_unsharded_layer(env, mode, M, N, K, G):
    """The K-sharded layer's pieces, with the G ranks emulated one after the other on one GPU (every 'rank' has its own
    slab buffer; no kernel waits for another): per-slice statistics -> max / min over the ranks -> codes from the given
    statistics -> GEMM partial accumulators stored into the owners' slabs -> owner's reduce + dequant + bias. The result
    must equal the unsharded layer bit for bit (scales / zero-points and codes equal the fused quantizer's)."""
    torch, L, o = env
    asym = mode == "asym"
    x = U.acts(M, K, 7 + M, mean=0.1 if asym else 0.0)
    if M > 4:
        x[1] = 0; x[2] = x[2, 0]
    qw = U.rand_codes(N, K, 8); sc = U.rand_scales(N, 9); zc = U.rand_zeros(N, 10)
    bias = np.random.default_rng(11).standard_normal(N).astype(np.float16)
    dx, dqw, dsc, dzc, db = (dev(torch, v) for v in (x, qw, sc, zc, bias))
    st = L.current_stream()
    per = -(-(K // 64) // G) * 64
    bounds = [(min(K, r * per), min(K, (r + 1) * per)) for r in range(G)]
    # 1. statistics per slice, reduced
    sa = [torch.zeros(M, dtype=torch.float16, device="cuda") for _ in range(G)]
    sb = [torch.zeros(M, dtype=torch.float16, device="cuda") for _ in range(G)]
    xs = [dx[:, b:e].contiguous() for b, e in bounds]
    for r, (b, e) in enumerate(bounds):
        if e > b:
            L.call("duq4_row_stats", L.MODES[mode], L.ptr(xs[r]), M, e - b, L.ptr(sa[r]), L.ptr(sb[r]), st)
        else:
            sa[r].fill_(float("inf") if asym else 0.0); sb[r].fill_(float("-inf"))
    ga = torch.stack(sa).amin(0) if asym else torch.stack(sa).amax(0)
    gb = torch.stack(sb).amax(0)
    # 2. + 3. codes with the global statistics, partial accumulators to the owners' slabs
    rpo = -(-M // G)
    slabs = [torch.full((G, rpo, N), 12345, dtype=torch.int32, device="cuda") for _ in range(G)]   # owner o's buffer
    scale = torch.zeros(M, dtype=torch.float16, device="cuda"); zeros = torch.zeros(M, dtype=torch.float16, device="cuda")
    n_slabs = 0
    for r, (b, e) in enumerate(bounds):
        if e == b:
            continue
        n_slabs += 1
        a8 = torch.zeros((M, e - b), dtype=torch.int8, device="cuda")
        L.call("duq4_quantize_i8_from_stats", L.MODES[mode], L.ptr(xs[r]), M, e - b, L.ptr(ga), L.ptr(gb), 1.0, L.ptr(a8), L.ptr(scale), L.ptr(zeros), st)
        wk = dqw[:, b // 2: e // 2].contiguous()
        epi = L.make_epilogue("none", acc_owners=[t.data_ptr() for t in slabs], acc_rows_per_owner=rpo, acc_slot=r)
        L.call("duq4_linear_w4a4_preunpacked", L.ptr(a8), L.ptr(wk), M, N, e - b, ctypes.byref(epi), None, None, st)
    # 4. every owner: reduce + dequant + bias into the one result
    out = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    for o_ in range(G):
        row0 = min(M, o_ * rpo); rows = min(M, row0 + rpo) - row0
        epi2 = L.make_epilogue(mode, scale, zeros if asym else None, dsc, dzc if asym else None, None, None, db, ldo=N)
        L.call("duq4_reduce_dequant_gather", L.ptr(slabs[o_]), n_slabs, rpo, row0, rows, N, ctypes.byref(epi2), L.ptr(out), st)
    torch.cuda.synchronize()
    assert tc_status(L) == 0
    # the unsharded layer: the fused quantizer's terms and codes (checked against the oracle), the oracle's GEMM + dequant
    qa, s1, z1, _, _ = U.gpu_quantize(torch, L, mode, x)
    assert U.f16_equal_nan(scale.cpu().numpy(), s1) and (not asym or U.f16_equal_nan(zeros.cpu().numpy(), z1))
    _, want = o.linear_w4a4(mode, qa, qw, s1, z1 if asym else None, sc, zc if asym else None, None, None, bias)
    assert U.f16_equal_nan(out.cpu().numpy(), want)
    assert L.cdll.duq4_row_stats(L.MODE_SYM_DUAL, L.ptr(xs[0]), M, 64, L.ptr(sa[0]), None, st) == -3   # dual schemes do not commute with a K split


@pytest.mark.parametrize("mode,M,N,K,G,R", [("sym", 700, 520, 512, 3, 256), ("asym_dual", 1000, 1032, 256, 4, 250), ("sym", 100, 392, 256, 2, 64),
                                            ("asym", 12, 264, 512, 3, 4), ("sym_dual", 16, 136, 128, 8, 2), ("sym", 2048, 2048, 1024, 8, 256)])
def test_fused_gather_row_routing_delivers_each_row_to_its_owner_only(env, mode, M, N, K, G, R):
    """duq4_epilogue.out_rows_per_owner: row m of a launch is stored only into out_peers[m // R]. With G buffers on
    one GPU (NaN-filled) each buffer must end up holding exactly its block of rows of the ordinary result and NaN
    elsewhere -- through every kernel family: the CTA-pair kernel on pre-laid-out and on packed weights, the narrow-tile
    kernel (M <= 128) and the small-M kernels (M <= 16)."""
    torch, L, o = env
    asym, dual = mode.startswith("asym"), mode.endswith("dual")
    x = U.acts(M, K, 21 + M, mean=0.1 if asym else 0.0)
    qw = U.rand_codes(N, K, 22); sc1 = U.rand_scales(N, 23); zc1 = U.rand_zeros(N, 24); sc2 = U.rand_scales(N, 25); zc2 = U.rand_zeros(N, 26)
    bias = np.random.default_rng(27).standard_normal(N).astype(np.float16)
    dx, dqw, dsc1, dzc1, dsc2, dzc2, db = (dev(torch, v) for v in (x, qw, sc1, zc1, sc2, zc2, bias))
    st = L.current_stream()
    vecs = (dsc1, dzc1 if asym else None, dsc2 if dual else None, dzc2 if mode == "asym_dual" else None, db)
    ws = torch.empty(max(L.cdll.duq4_linear_from_fp16_workspace_bytes(M, K), L.cdll.duq4_linear_from_fp16_prelaid_workspace_bytes(M, K)),
                     dtype=torch.uint8, device="cuda")
    want = torch.empty((M, N), dtype=torch.float16, device="cuda")
    L.call("duq4_linear_w4a4_from_fp16", L.ptr(dx), L.ptr(dqw), M, N, K, L.MODES[mode], 1.0,
           ctypes.byref(L.make_epilogue(mode, None, None, *vecs)), L.ptr(want), L.ptr(ws), ws.numel(), st)
    routes = ["packed"] + (["prelaid"] if K % 128 == 0 and M > 16 else [])
    for route in routes:
        bufs = [torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda") for _ in range(G)]
        epi = L.make_epilogue(mode, None, None, *vecs, ldo=N, out_peers=[b.data_ptr() for b in bufs], out_rows_per_owner=R)
        if route == "packed":
            L.call("duq4_linear_w4a4_from_fp16", L.ptr(dx), L.ptr(dqw), M, N, K, L.MODES[mode], 1.0, ctypes.byref(epi), None, L.ptr(ws), ws.numel(), st)
        else:
            w8 = torch.empty((N, K), dtype=torch.int8, device="cuda")
            L.call("duq4_weight_prelayout_i8", L.ptr(dqw), N, K, L.ptr(w8), st)
            L.call("duq4_linear_w4a4_from_fp16_prelaid", L.ptr(dx), L.ptr(w8), M, N, K, L.MODES[mode], 1.0, ctypes.byref(epi), None, L.ptr(ws), ws.numel(), st)
        torch.cuda.synchronize()
        assert tc_status(L) == 0
        for g, b in enumerate(bufs):
            lo, hi = min(M, g * R), min(M, (g + 1) * R)
            assert torch.equal(b[lo:hi].view(torch.int16), want[lo:hi].view(torch.int16)), (route, g)
            rest = torch.cat([b[:lo], b[hi:]])
            assert bool(torch.isnan(rest).all()), (route, g)
    # too few owners for the rows, multicast together with routing, an entry point without routing
    bad = L.make_epilogue(mode, None, None, *vecs, ldo=N, out_peers=[want.data_ptr()], out_rows_per_owner=max(1, M - 1))
    if M > 1:
        assert L.cdll.duq4_linear_w4a4_from_fp16(L.ptr(dx), L.ptr(dqw), M, N, K, L.MODES[mode], 1.0, ctypes.byref(bad), None, L.ptr(ws), ws.numel(), st) == -2
    bad2 = L.make_epilogue(mode, None, None, *vecs, ldo=N, out_rows_per_owner=R)
    assert L.cdll.duq4_linear_w4a4_from_fp16(L.ptr(dx), L.ptr(dqw), M, N, K, L.MODES[mode], 1.0, ctypes.byref(bad2), L.ptr(want), L.ptr(ws), ws.numel(), st) == -3


@pytest.mark.parametrize("mode,M,N,K,chunk", [("sym", 700, 520, 512, 256), ("asym", 40, 264, 256, 0), ("sym_dual", 2048, 1024, 1024, 512)])
def test_host_rows_pipeline_with_one_rank_equals_device_entry(env, mode, M, N, K, chunk):
    """duq4_linear_w4a4_from_fp16_to_host_rows with a single rank (its exchange is then a plain store into the rank's own
    buffer and its barrier has nobody to wait for): chunked arithmetic, barrier epochs and the download of the owned rows
    give the same bits as the device entry point; a second call reuses buffers and continues the epochs."""
    torch, L, o = env
    asym, dual = mode.startswith("asym"), mode.endswith("dual")
    x = U.acts(M, K, 31 + M, mean=0.1 if asym else 0.0)
    qw = U.rand_codes(N, K, 32); sc1 = U.rand_scales(N, 33); zc1 = U.rand_zeros(N, 34); sc2 = U.rand_scales(N, 35); zc2 = U.rand_zeros(N, 36)
    dx, dqw, dsc1, dzc1, dsc2, dzc2 = (dev(torch, v) for v in (x, qw, sc1, zc1, sc2, zc2))
    st = L.current_stream()
    vecs = (dsc1, dzc1 if asym else None, dsc2 if dual else None, dzc2 if mode == "asym_dual" else None, None)
    ws = torch.empty(L.cdll.duq4_linear_from_fp16_workspace_bytes(M, K), dtype=torch.uint8, device="cuda")
    want = torch.empty((M, N), dtype=torch.float16, device="cuda")
    L.call("duq4_linear_w4a4_from_fp16", L.ptr(dx), L.ptr(dqw), M, N, K, L.MODES[mode], 1.0,
           ctypes.byref(L.make_epilogue(mode, None, None, *vecs)), L.ptr(want), L.ptr(ws), ws.numel(), st)
    ldo, col_begin = N + 64, 32   # the block sits inside a wider result
    buf = torch.zeros((M, ldo), dtype=torch.float16, device="cuda")
    flags = torch.zeros(1, dtype=torch.int64, device="cuda")
    flag_ptrs = (ctypes.c_void_p * 1)(flags.data_ptr())
    out_host = torch.full((M, ldo), -3.0, dtype=torch.float16).pin_memory()
    staging = torch.empty(max(256, L.cdll.duq4_linear_pipeline_staging_bytes(0, 0, M, N, K, chunk)), dtype=torch.uint8, device="cuda")
    epi = L.make_epilogue(mode, None, None, *vecs, ldo=ldo, out_peers=[buf.data_ptr()])
    epoch = ctypes.c_uint64(0)
    for call in range(2):
        L.call("duq4_linear_w4a4_from_fp16_to_host_rows", L.ptr(dx), L.ptr(dqw), 0, M, N, K, L.MODES[mode], 1.0, ctypes.byref(epi), col_begin, 0,
               flag_ptrs, ctypes.byref(epoch), 0, out_host.data_ptr(), chunk, L.ptr(staging), staging.numel(), st)
        torch.cuda.synchronize()
        assert tc_status(L) == 0
        assert torch.equal(out_host[:, col_begin:col_begin + N].contiguous().view(torch.int16), want.cpu().view(torch.int16))
        assert bool((out_host[:, :col_begin] == 0).all()) and bool((out_host[:, col_begin + N:] == 0).all())   # the rest of the owned rows as the buffer had it
        out_host.fill_(-3.0)
    rows = chunk if chunk else max(256, -(-((M + 15) // 16) // 256) * 256)
    assert epoch.value == 2 * (1 + -(-M // min(M, rows)))


@pytest.mark.parametrize("K", [512, 4096])
def test_decode_static_weights_overlap_keeps_stream_order(env, K):
    """With duq4_set_static_weights(1) the small-M kernels start streaming weights before the
    previous kernel of the stream has finished. Activations written by that previous kernel
    (here: a device copy queued right before each call) must still be seen, and a chain of calls
    that reuse one output buffer must leave the last result."""
    torch, L, o = env
    M, N = 4, 1032
    qw = U.rand_codes(N, K, 1); sw = U.rand_scales(N, 2)
    dw, dsw = dev(torch, qw), dev(torch, sw)
    srcs = [dev(torch, U.rand_codes(M, K, 10 + i)) for i in range(6)]
    sa = dev(torch, U.rand_scales(M, 3))
    qa = torch.zeros((M, K // 2), dtype=torch.uint8, device="cuda")
    outs = [torch.zeros((M, N), dtype=torch.float16, device="cuda") for _ in range(6)]
    epi = L.make_epilogue("sym", sa, None, dsw)
    prev = L.cdll.duq4_set_static_weights(1)
    try:
        for i in range(6):
            tmp = torch.bitwise_xor(srcs[i], 0)   # a kernel that produces the activations ...
            qa = tmp                               # ... consumed by the very next launch
            L.call("duq4_linear_w4a4", L.ptr(qa), L.ptr(dw), M, N, K, ctypes.byref(epi), L.ptr(outs[i]), None, L.current_stream())
        torch.cuda.synchronize()
    finally:
        L.cdll.duq4_set_static_weights(prev)
    for i in range(6):
        _, want = o.linear_w4a4("sym", srcs[i].cpu().numpy(), qw, sa.cpu().numpy(), None, sw, None, None, None)
        assert U.f16_equal_nan(outs[i].cpu().numpy(), want), i


@pytest.mark.parametrize("mode", ["sym", "sym_dual", "asym", "asym_dual"])
def test_pair_kernel_shapes(env, mode):
    """Problems with at least 60 tiles of 256x256 run on CTA pairs (cta_group::2): ragged M and N,
    K with a partial last stage, every epilogue mode, int32 accumulators, packed activations."""
    torch, L, o = env
    run_linear(torch, L, o, mode, 2000, 2100, 448, seed=71, col0=5)


@pytest.mark.parametrize("width", ["160", "192", "224", "32"])
def test_pair_kernel_tile_widths_pinned(width):
    """The CTA-pair kernel picks its tile width per launch (narrower tiles when they fill the last
    round of tiles better); each width forced for the pair-kernel cases, in a fresh process (the
    choice is read once). Covers packed and pre-unpacked activations, ragged N against every width,
    int32 accumulators and all epilogue modes."""
    import os, subprocess, sys
    env2 = dict(os.environ, DUQ4_TC_BN=width)
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", os.path.abspath(__file__), "-k",
                        "pair_kernel_shapes or pair_kernel_batched or preunpacked_activations_match_packed_path or full_size_property"],
                       env=env2, capture_output=True, text=True, cwd=U.ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def test_pair_kernel_batched(env):
    torch, L, o = env
    B, M, N, K = 8, 512, 1024, 256   # 8 x 2 x 4 = 64 pair tiles
    qa = U.rand_codes(B * M, K, 9).reshape(B, M, K // 2); qw = U.rand_codes(B * N, K, 10).reshape(B, N, K // 2)
    da, dw = dev(torch, qa), dev(torch, qw)
    C = torch.zeros((B, M, N), dtype=torch.int32, device="cuda")
    L.call("duq4_batch_matmul_4bit", L.ptr(da), L.ptr(dw), M, N, K, L.ptr(C), B, L.current_stream())
    torch.cuda.synchronize()
    assert tc_status(L) == 0
    assert np.array_equal(C.cpu().numpy(), o.batch_matmul_4bit(qa, qw))


@pytest.mark.parametrize("M,N,K", [(1, 12288, 4096), (16, 12288, 4096), (4, 4096, 11008)])
def test_next_weights_hint_changes_nothing_but_timing(env, M, N, K):
    """The L2 prefetch hint for the following layer (duq4_epilogue.next_weights) is never dereferenced by
    the arithmetic: outputs with a hint (aligned, misaligned, shorter than the skipped head, huge) equal
    the outputs without one, on every small-M kernel."""
    torch, L, o = env
    qa = dev(torch, U.rand_codes(M, K, 1)); qw = dev(torch, U.rand_codes(N, K, 2))
    sr = dev(torch, U.rand_scales(M, 3)); sc = dev(torch, U.rand_scales(N, 4))
    nxt = torch.randint(0, 256, (40 << 20,), dtype=torch.uint8, device="cuda")
    outs = []
    for hint in (None, nxt, nxt[1:], nxt[: 1 << 20], nxt[16: (13 << 20) + 48]):
        epi = L.make_epilogue("sym", sr, None, sc, next_weights=hint)
        out = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        L.call("duq4_linear_w4a4", L.ptr(qa), L.ptr(qw), M, N, K, ctypes.byref(epi), L.ptr(out), None, L.current_stream())
        torch.cuda.synchronize()
        outs.append(out)
    for x in outs[1:]:
        assert torch.equal(x.view(torch.int16), outs[0].view(torch.int16))
    assert torch.equal(nxt[:64].cpu(), nxt[:64].cpu())   # the hinted buffer is untouched (still readable)
