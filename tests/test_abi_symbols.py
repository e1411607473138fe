"""CPU-only: the C-ABI library loads and exports every function include/duq4.h declares."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    src = open(os.path.join(ROOT, "include", "duq4.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(duq4_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    import duqlinear4bitcuda_b200.lib as L
    names = declared_functions()
    assert len(names) >= 25
    for n in names:
        assert hasattr(L.cdll, n), f"libduq4.so does not export {n}"
        assert n in L.SIGNATURES, f"lib.py has no signature for {n}"
    assert sorted(L.SIGNATURES) == names


def test_metadata_calls_without_gpu():
    import duqlinear4bitcuda_b200.lib as L
    assert L.cdll.duq4_dual_quant_col_k() == 10
    assert b"sm_100a" in L.cdll.duq4_version()
    assert L.cdll.duq4_error_string(-4).startswith(b"workspace")
    assert L.cdll.duq4_linear_from_fp16_workspace_bytes(16, 4096) == 16 * 2048 + 4 * 256


def test_arguments_are_rejected_before_any_launch():
    """Status codes for bad arguments come back without a GPU: every entry point validates pointers,
    modes, shapes and workspaces before it touches the CUDA runtime. Pointers below are fake non-NULL
    addresses; a call that got as far as a launch would fail differently (positive cudaError_t)."""
    import ctypes
    import duqlinear4bitcuda_b200.lib as L
    c = L.cdll
    P = ctypes.c_void_p(0x1000)          # "some device pointer"
    NULL = None
    e = L.Epilogue()
    e.mode = L.MODE_SYM
    e.scale_row = 0x1000
    e.scale_col_1 = 0x1000
    ep = ctypes.byref(e)
    # NULL operands
    assert c.duq4_sym_quant(NULL, P, 4, 64, 32, P, NULL) == -1
    assert c.duq4_matmul_4bit(P, NULL, 4, 8, 64, P, NULL) == -1
    assert c.duq4_linear_w4a4(NULL, P, 4, 8, 64, ep, P, NULL, NULL) == -1
    # K must be a multiple of 64
    assert c.duq4_matmul_4bit(P, P, 4, 8, 100, P, NULL) == -2
    assert c.duq4_linear_w4a4_from_fp16(P, P, 4, 8, 100, L.MODE_SYM, 1.0, ep, P, P, 1 << 20, NULL) == -2
    # unknown modes; the dual schemes are refused by the gate/up entry point
    bad = L.Epilogue(); bad.mode = 99
    assert c.duq4_linear_w4a4(P, P, 4, 8, 64, ctypes.byref(bad), P, NULL, NULL) == -3
    assert c.duq4_linear_w4a4_from_fp16(P, P, 4, 8, 64, 9, 1.0, ep, P, P, 1 << 20, NULL) == -3
    dual = L.Epilogue(); dual.mode = L.MODE_SYM_DUAL; dual.scale_row = 0x1000; dual.scale_col_1 = 0x1000; dual.scale_col_2 = 0x1000
    assert c.duq4_linear_w4a4_gate_up_silu(P, 1, P, 4, 8, 64, ctypes.byref(dual), P, NULL) == -3
    # an asymmetric epilogue needs zero-points
    asym = L.Epilogue(); asym.mode = L.MODE_ASYM; asym.scale_row = 0x1000; asym.scale_col_1 = 0x1000
    assert c.duq4_linear_w4a4(P, P, 4, 8, 64, ctypes.byref(asym), P, NULL, NULL) == -1
    # workspaces: missing, too small, misaligned
    need = c.duq4_linear_from_fp16_workspace_bytes(4, 64)
    assert c.duq4_linear_w4a4_from_fp16(P, P, 4, 8, 64, L.MODE_SYM, 1.0, ep, P, NULL, need, NULL) == -4
    assert c.duq4_linear_w4a4_from_fp16(P, P, 4, 8, 64, L.MODE_SYM, 1.0, ep, P, P, need - 1, NULL) == -4
    assert c.duq4_linear_w4a4_from_fp16(P, P, 4, 8, 64, L.MODE_SYM, 1.0, ep, P, ctypes.c_void_p(0x1010), need, NULL) == -4
    # built-in scratch: problems that do not fit are refused
    assert c.duq4_linear_w4a4_from_fp16_static(P, P, 4096, 8, 8192, L.MODE_SYM, 1.0, ep, P, NULL) == -8
    # host-buffer entry point: peers are not allowed, staging is checked
    peers = L.Epilogue(); peers.mode = L.MODE_SYM; peers.scale_col_1 = 0x1000; peers.n_out_peers = 1; peers.out_peers[0] = 0x1000
    assert c.duq4_linear_w4a4_from_fp16_host(P, P, 300, 8, 64, L.MODE_SYM, 1.0, ctypes.byref(peers), P, 0, P, 1 << 30, NULL) == -3
    assert c.duq4_linear_w4a4_from_fp16_host(P, P, 300, 8, 64, L.MODE_SYM, 1.0, ep, P, 0, NULL, 1 << 30, NULL) == -4
    # row routing of the fused gather: needs peers, no multicast, enough owners for the rows, an entry point that routes
    routed = L.Epilogue(); routed.mode = L.MODE_SYM; routed.scale_row = 0x1000; routed.scale_col_1 = 0x1000; routed.out_rows_per_owner = 2
    assert c.duq4_linear_w4a4(P, P, 4, 8, 64, ctypes.byref(routed), P, NULL, NULL) == -3            # no peers
    routed.n_out_peers = 1; routed.out_peers[0] = 0x1000
    assert c.duq4_linear_w4a4(P, P, 4, 8, 64, ctypes.byref(routed), NULL, NULL, NULL) == -2         # 1 owner x 2 rows < 4 rows
    routed.out_multicast = 0x2000
    assert c.duq4_linear_w4a4(P, P, 2, 8, 64, ctypes.byref(routed), NULL, NULL, NULL) == -3         # multicast and routing exclude each other
    routed.out_multicast = None
    assert c.duq4_linear_w4a4_batched(P, P, 2, 8, 64, 1, ctypes.byref(routed), NULL, NULL, NULL) == -3   # the batched entry point does not route
    # host result by rows: flags, rank index, full width, routing chosen by the call itself
    flags = (ctypes.c_void_p * 2)(0x3000, 0x4000)
    epoch = ctypes.c_uint64(0)
    two = L.Epilogue(); two.mode = L.MODE_SYM; two.scale_col_1 = 0x1000; two.ldo = 64; two.n_out_peers = 2; two.out_peers[0] = 0x1000; two.out_peers[1] = 0x2000
    rows = lambda e_, col, self_, fl, ep_: c.duq4_linear_w4a4_from_fp16_to_host_rows(P, P, 0, 4, 8, 64, L.MODE_SYM, 1.0, ctypes.byref(e_), col, self_, fl,
                                                                                   ep_, 0, P, 0, P, 1 << 20, NULL)
    assert rows(two, 0, 0, None, ctypes.byref(epoch)) == -1          # no barrier flags
    assert rows(two, 0, 2, flags, ctypes.byref(epoch)) == -2         # rank index outside the peer list
    assert rows(two, 60, 0, flags, ctypes.byref(epoch)) == -2        # the block does not fit the result's width
    two.out_rows_per_owner = 2
    assert rows(two, 0, 0, flags, ctypes.byref(epoch)) == -3         # the routing is the call's own choice
    assert epoch.value == 0
    # empty problems are fine and do nothing
    assert c.duq4_linear_w4a4_from_fp16(P, P, 0, 8, 64, L.MODE_SYM, 1.0, ep, P, P, 1 << 20, NULL) == 0
    # sizes of the host-buffer staging area: device copies of x and of the result + one chunk's quantizer scratch
    M, N, K = 4096, 28672, 8192
    chunk = 256   # a sixteenth of M, already a multiple of 256
    assert c.duq4_linear_host_staging_bytes(M, N, K, 0) == M * K * 2 + M * N * 2 + c.duq4_linear_from_fp16_workspace_bytes(chunk, K)
    for code in range(-8, 0):
        assert len(c.duq4_error_string(code)) > 3
