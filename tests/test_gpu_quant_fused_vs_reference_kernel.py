"""The fused per-token quantizers -- the ones on every hot path -- against the reference's OWN quantize
kernels, bit for bit, with no tolerance of any kind.

The fused kernels code a token with a short path (one approximate reciprocal per token, fp16x2
magic-number rounding) instead of the reference's per-element __hdiv + __half2int_rn + clamp
(src/kernels/quant.cu:12-61, :100-147; src/kernels/quant2.cu:10-60, :102-156). The claim is that the
codes are identical. Here each fused entry point (packed output, and the tensor-core-ready int8 output
un-permuted) quantizes tokens drawn from the benchmark distributions at the benchmark widths; then the
reference's kernel, compiled from its sources into oracle/_ref/libduq_ref.so, codes the same tokens
with the scales / zero-points the fused kernel wrote, and the packed codes must be equal everywhere.
"""
import ctypes

import numpy as np
import pytest

from tests import _util as U

pytestmark = pytest.mark.gpu

# (tokens, K): the headline prefill layer, the decode configuration, and the long rows of the
# 11008 -> 4096 and 28672 -> 8192 layers
SHAPES = [(4096, 8192), (16, 4096), (300, 11008), (130, 28672)]
MODES = ["sym", "sym_dual", "asym", "asym_dual"]


def _tokens(torch, M, K, mode, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    asym = mode.startswith("asym")
    x = torch.randn((M, K), generator=g, dtype=torch.float32, device="cuda") + (0.1 if asym else 0.0)
    frac, mul = (200, 30.0) if asym else (100, 20.0)     # 0.5 % x30 / 1 % x20 outlier channels
    ch = torch.randperm(K, generator=g, device="cuda")[: K // frac]
    x[:, ch] *= mul
    x = x.to(torch.float16)
    if M > 4:
        x[1] = 0                      # all-zero token (scale 0)
        x[2] = x[2, 0]                # constant token (asymmetric range 0)
        x[3, 5] = float("inf")        # tokens holding inf / NaN take the element-by-element path
        x[4, 7] = float("nan")
    return x.contiguous()


@pytest.mark.parametrize("M,K", SHAPES)
@pytest.mark.parametrize("mode", MODES)
def test_fused_quantizer_codes_equal_reference_kernel(mode, M, K):
    import torch
    import duqlinear4bitcuda_b200.lib as L
    ref = U.load_ref_lib()
    if ref is None:
        pytest.skip("reference kernels not built (make -C oracle ref)")
    asym, dual = mode.startswith("asym"), mode.endswith("dual")
    x = _tokens(torch, M, K, mode, seed=M + K)
    st = L.current_stream()
    vec = lambda: torch.zeros(M, dtype=torch.float16, device="cuda")
    s1, z1, s2, z2 = vec(), vec(), vec(), vec()
    t1, y1, t2, y2 = vec(), vec(), vec(), vec()
    q = torch.zeros((M, K // 2), dtype=torch.uint8, device="cuda")
    a8 = torch.zeros((M, K), dtype=torch.int8, device="cuda")
    clip = 0.9 if (M == 16 and not asym) else 1.0
    if mode == "sym":
        L.call("duq4_quantize_sym_fused", L.ptr(x), M, K, clip, L.ptr(q), L.ptr(s1), st)
    elif mode == "sym_dual":
        L.call("duq4_quantize_sym_dual_fused", L.ptr(x), M, K, clip, L.ptr(q), L.ptr(s1), L.ptr(s2), st)
    elif mode == "asym":
        L.call("duq4_quantize_asym_fused", L.ptr(x), M, K, L.ptr(q), L.ptr(s1), L.ptr(z1), st)
    else:
        L.call("duq4_quantize_asym_dual_fused", L.ptr(x), M, K, L.ptr(q), L.ptr(s1), L.ptr(z1), L.ptr(s2), L.ptr(z2), st)
    L.call("duq4_quantize_fused_i8", L.MODES[mode], L.ptr(x), M, K, clip, L.ptr(a8), L.ptr(t1), L.ptr(y1), L.ptr(t2), L.ptr(y2), st)
    torch.cuda.synchronize()

    vecs = {"sym": [s1], "sym_dual": [s1, s2], "asym": [s1, z1], "asym_dual": [s1, z1, s2, z2]}[mode]
    vecs8 = {"sym": [t1], "sym_dual": [t1, t2], "asym": [t1, y1], "asym_dual": [t1, y1, t2, y2]}[mode]
    for a, b in zip(vecs, vecs8):   # both outputs of the fused kernel carry the same per-token vectors
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))

    q_ref = torch.full_like(q, 0xAB)
    fn = getattr(ref, f"ref_{mode}_quant")
    fn.argtypes = [ctypes.c_void_p] * (1 + len(vecs)) + [ctypes.c_uint32] * 3 + [ctypes.c_void_p]
    fn.restype = ctypes.c_int
    assert fn(L.ptr(x), *[L.ptr(v) for v in vecs], M, K, K // 2, L.ptr(q_ref)) == 0
    torch.cuda.synchronize()
    bad = int((q != q_ref).sum())
    assert bad == 0, f"{mode} M={M} K={K}: {bad} packed bytes differ from the reference's quantize kernel"
    packed8 = torch.from_numpy(U.i8_codes_to_packed(a8.cpu().numpy())).cuda()
    assert torch.equal(packed8, q_ref), f"{mode} M={M} K={K}: int8 output (un-permuted) differs from the reference's kernel"
