"""The reference's own CUDA path against this library, on the same GPU and the same inputs.

The reference layer is four pieces (qlinear4bit/nn/quantizer.py:10-16 SymQuantizer,
qlinear4bit/nn/linear.py:60-78 Linear4bitSQ.forward): torch ops for the per-token scale, then
sym_quant_host (src/kernels/quant.cu:48-61), matmul_host_4bit (src/kernels/gemm.cu:8-43, CUTLASS
Sm80 int4 tensor-op GEMM) and sym_dequant_host (src/kernels/quant.cu:83-97). Those launchers are
compiled from the reference's sources into oracle/_ref/libduq_ref.so; this test runs them for the
layer shapes of the headline benchmark, checks that duq4_linear_w4a4_from_fp16 returns the same
bits, and requires it to be faster. Timings are printed (run with -s to see them).
"""
import ctypes

import pytest

from tests import _util as U

pytestmark = pytest.mark.gpu

SHAPES = [  # (name, M, K, N)
    ("decode_M1_4096x22016", 1, 4096, 22016),
    ("decode_M16_4096x4096", 16, 4096, 4096),
    ("prefill_M4096_8192x28672", 4096, 8192, 28672),
]


def _time_ms(torch, fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


@pytest.mark.parametrize("name,M,K,N", SHAPES)
def test_layer_beats_reference_cuda_kernels(name, M, K, N):
    import torch
    import duqlinear4bitcuda_b200.lib as L
    ref = U.load_ref_lib()
    if ref is None:
        pytest.skip("reference kernels not built (make -C oracle ref)")
    g = torch.Generator().manual_seed(7)
    x = torch.randn((M, K), generator=g, dtype=torch.float32)
    x[:, torch.randperm(K, generator=g)[: K // 100]] *= 20.0
    x = x.to(torch.float16).cuda()
    qw = torch.from_numpy(U.rand_codes(N, K, 8)).cuda()
    sw = torch.from_numpy(U.rand_scales(N, 9)).cuda()

    # ---- the reference's four pieces, on the legacy default stream as the reference launches them
    q = torch.empty((M, K // 2), dtype=torch.uint8, device="cuda")
    acc = torch.empty((M, N), dtype=torch.int32, device="cuda")
    out_ref = torch.empty((M, N), dtype=torch.float16, device="cuda")

    def reference_layer():
        s = (torch.max(torch.abs(x), dim=-1, keepdim=True)[0] / 7).to(torch.float16) * 1.0
        assert ref.ref_sym_quant(L.ptr(x), L.ptr(s), M, K, K // 2, L.ptr(q)) == 0
        assert ref.ref_matmul_4bit(L.ptr(q), L.ptr(qw), M, N, K, L.ptr(acc)) == 0
        assert ref.ref_sym_dequant(L.ptr(acc), L.ptr(s), L.ptr(sw), M, N, L.ptr(out_ref)) == 0

    for f in (ref.ref_sym_quant, ref.ref_matmul_4bit, ref.ref_sym_dequant):
        f.restype = ctypes.c_int
    ref.ref_sym_quant.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p]
    ref.ref_matmul_4bit.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p]
    ref.ref_sym_dequant.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p]

    # ---- this library: one call
    nbytes = L.cdll.duq4_linear_from_fp16_workspace_bytes(M, K)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    out = torch.empty((M, N), dtype=torch.float16, device="cuda")
    epi = L.make_epilogue("sym", None, None, sw)

    def our_layer():
        L.call("duq4_linear_w4a4_from_fp16", L.ptr(x), L.ptr(qw), M, N, K, L.MODE_SYM, 1.0, ctypes.byref(epi), L.ptr(out),
               L.ptr(ws), nbytes, L.current_stream())

    with torch.cuda.stream(torch.cuda.default_stream()):
        reference_layer()
        our_layer()
        torch.cuda.synchronize()
        # same divide instruction, same roundings, exact integer GEMM: every output bit must agree
        bad_rows = int((out.view(torch.int16) != out_ref.view(torch.int16)).any(dim=1).sum())
        assert bad_rows == 0, f"{bad_rows} of {M} rows differ from the reference's CUDA path"
        iters = 20 if M > 16 else 200
        t_ref = _time_ms(torch, reference_layer, iters)
        t_our = _time_ms(torch, our_layer, iters)
    ops = 2.0 * M * N * K
    print(f"\n[{name}] reference CUDA path {t_ref * 1e3:9.1f} us ({ops / t_ref / 1e9:8.1f} TOPS)   "
          f"this library {t_our * 1e3:9.1f} us ({ops / t_our / 1e9:8.1f} TOPS)   speed-up {t_ref / t_our:6.1f}x   rows differing {bad_rows}")
    assert t_our < t_ref, f"{name}: {t_our:.4f} ms is not faster than the reference's {t_ref:.4f} ms"
