"""duq4_linear_w4a4_from_fp16_static -- the entry point for callers that cannot allocate or lend
device memory (a plugin inside a server whose allocator owns the whole GPU, code on a latency
path that must not trigger an allocation's device synchronisation). Its scratch is a fixed
2 MiB array inside the library, so this test checks, through the C ABI:

  * two calls in a row give exactly the output of the workspace-taking entry point
    (bit-identical fp16, the tolerance the other GPU tests use), although the second call finds
    the first call's leftovers in the shared array -- on every kernel the call can route to
    (small-M register and TMA-streamed kernels, the single-CTA tensor-core kernel including the
    17..31-token case whose code buffer is padded to 32 rows, and the CTA-pair kernel) -- and the
    workspace-taking entry point is itself checked against the CPU oracle on the same inputs;
  * the calls leave the library's TMA descriptor cache (host heap) untouched;
  * a problem whose scratch need exceeds the array is refused with DUQ4_ERR_TOO_LARGE (-8)
    before anything is launched.

The file is named so that pytest collects it last."""
import ctypes

import numpy as np
import pytest

from tests import _util as U

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,mode", [(1, 4096, 4096, "asym"),        # one token: single-launch route, no scratch used at all
                                        (4, 520, 1024, "sym"), (16, 384, 4096, "asym"), (100, 264, 2048, "sym"),
                                        (20, 520, 1024, "asym"),        # 17..31 tokens: 32-row padded code buffer
                                        (9, 9600, 4096, "sym"),         # small-M TMA-streamed kernel
                                        (200, 22016, 4096, "sym")])     # CTA-pair tensor-core kernel
def test_static_scratch_entry_matches_workspace_entry_twice(M, N, K, mode):
    import torch
    import duqlinear4bitcuda_b200.lib as L
    from oracle import oracle as o

    st = L.current_stream()
    dw = torch.from_numpy(U.rand_codes(N, K, 11)).cuda()
    dsw = torch.from_numpy(U.rand_scales(N, 12)).cuda()
    dzc = torch.from_numpy(U.rand_zeros(N, 13)).cuda()
    bias = torch.from_numpy(np.random.default_rng(14).standard_normal(N).astype(np.float16)).cuda()
    epi = L.make_epilogue(mode, None, None, dsw, dzc if mode == "asym" else None, bias=bias)
    nbytes = L.cdll.duq4_linear_from_fp16_workspace_bytes(M, K)
    assert nbytes <= 2 << 20
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    for call in range(2):  # different activations per call: the second sees the first's leftovers
        x = torch.from_numpy(U.acts(M, K, 20 + call, mean=0.1 if mode == "asym" else 0.0)).cuda()
        want = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        got = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        L.call("duq4_linear_w4a4_from_fp16", L.ptr(x), L.ptr(dw), M, N, K, L.MODES[mode], 1.0, ctypes.byref(epi), L.ptr(want),
               L.ptr(ws), nbytes, st)
        torch.cuda.synchronize()
        cached = L.cdll.duq4_tensor_map_cache_entries()
        L.call("duq4_linear_w4a4_from_fp16_static", L.ptr(x), L.ptr(dw), M, N, K, L.MODES[mode], 1.0, ctypes.byref(epi),
               L.ptr(got), st)
        torch.cuda.synchronize()
        assert L.cdll.duq4_tensor_map_cache_entries() == cached, "the static entry point touched the descriptor cache"
        assert U.f16_equal_nan(got.cpu().numpy(), want.cpu().numpy()), f"call {call}"
        assert not torch.isnan(got).all()
        if call == 0:   # the workspace entry point against the oracle, on the codes it left in its scratch
            xn = x.cpu().numpy()
            if M > 1:
                qa, s1, z1, _, _ = U.from_fp16_scratch(ws.cpu().numpy(), M, K)
                U.check_gpu_codes(torch, L, mode, xn, qa, s1, z1 if mode == "asym" else None)
            else:   # one token: a single launch, the codes stay in shared memory
                qa, s1, z1, _, _ = U.gpu_quantize(torch, L, mode, xn)
            _, ora = o.linear_w4a4(mode, qa, dw.cpu().numpy(), s1, z1 if mode == "asym" else None, dsw.cpu().numpy(),
                                   dzc.cpu().numpy() if mode == "asym" else None, None, None, bias.cpu().numpy())
            assert U.f16_equal_nan(want.cpu().numpy(), ora), "workspace entry point differs from the oracle"
    status = ctypes.c_int32(-1)
    L.call("duq4_last_device_status", st, ctypes.byref(status))
    assert status.value == 0


def test_static_scratch_entry_rejects_oversized_problem():
    import torch
    import duqlinear4bitcuda_b200.lib as L

    M, N, K = 512, 128, 8192  # needs 4 MiB of scratch
    assert L.cdll.duq4_linear_from_fp16_workspace_bytes(M, K) > 2 << 20
    x = torch.zeros((M, K), dtype=torch.float16, device="cuda")
    w = torch.zeros((N, K // 2), dtype=torch.uint8, device="cuda")
    s = torch.ones(N, dtype=torch.float16, device="cuda")
    out = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    epi = L.make_epilogue("sym", None, None, s)
    rc = L.cdll.duq4_linear_w4a4_from_fp16_static(L.ptr(x), L.ptr(w), M, N, K, L.MODE_SYM, 1.0, ctypes.byref(epi), L.ptr(out),
                                                  L.current_stream())
    assert rc == -8
    assert b"scratch" in L.cdll.duq4_error_string(rc)
    torch.cuda.synchronize()
