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
