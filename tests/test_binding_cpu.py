"""CPU-only: the compiled operator module (the drop-in for the reference's qlinear4bit._CUDA,
src/export/bindings.cpp:772-921) imports without a GPU, exports the reference's names, and its
argument checks raise before anything touches a device."""
import pytest

REFERENCE_NAMES = ["matmul", "matmul_8bit", "batched_matmul", "sym_quant", "sym_dual_quant", "sym_dequant", "sym_dual_dequant",
                   "asym_quant", "asym_quant_8bit", "asym_batch_dequant", "asym_dequant", "asym_dequant_hprec", "asym_dual_quant",
                   "asym_dual_dequant", "get_dual_quant_col_k"]


def test_operator_module_exports_the_reference_names():
    import qlinear4bit._CUDA as ops
    for n in REFERENCE_NAMES:
        assert callable(getattr(ops, n)), n
    assert ops.get_dual_quant_col_k() == 10


def test_wrong_element_types_are_reported_before_the_device_check():
    """fp32 scale buffers (torch's default for a module filled by load_state_dict), a bf16 bias or
    fp32 activations must raise, not be read as fp16. The type check comes first, so it fires here
    on CPU tensors; right types on CPU tensors then fail the CUDA check. Nothing is launched."""
    import torch
    import qlinear4bit._CUDA as ops
    M, N, K = 4, 8, 64
    A = torch.zeros((M, K // 2), dtype=torch.uint8); W = torch.zeros((N, K // 2), dtype=torch.uint8)
    h = lambda n: torch.ones(n, dtype=torch.float16)
    x = torch.zeros((M, K), dtype=torch.float16)
    with pytest.raises(RuntimeError, match="scale_col_1 to have dtype"):
        ops.linear_w4a4("sym", A, W, h(M), None, torch.ones(N))
    with pytest.raises(RuntimeError, match="scale_row to have dtype"):
        ops.linear_w4a4("sym", A, W, torch.ones(M), None, h(N))
    with pytest.raises(RuntimeError, match="bias to have dtype"):
        ops.linear_w4a4("sym", A, W, h(M), None, h(N), bias=torch.ones(N, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="A to have dtype"):
        ops.linear_w4a4("sym", A.to(torch.int8), W, h(M), None, h(N))
    with pytest.raises(RuntimeError, match="x to have dtype"):
        ops.linear_w4a4_from_fp16("sym", x.float(), W, h(N))
    with pytest.raises(RuntimeError, match="scale_col_1 to have dtype"):
        ops.linear_w4a4_from_fp16("sym", x, W, torch.ones(N))
    with pytest.raises(RuntimeError, match="W_prelaid to have dtype"):
        ops.linear_w4a4_from_fp16("sym", x, W, h(N), W_prelaid=torch.zeros((N, K), dtype=torch.uint8))
    with pytest.raises(RuntimeError, match="scale_col to have dtype"):
        ops.linear_w4a4_gate_up_silu("sym", A, W, h(M), None, torch.ones(N))
    with pytest.raises(RuntimeError, match="zeros_row to have dtype"):
        ops.linear_w4a4_batched("asym", A[None], W[None], h(M), torch.zeros(M), h(N), h(N))
    for f in (ops.quantize_sym_fused, ops.quantize_asym_fused, ops.quantize_sym_dual_fused, ops.quantize_asym_dual_fused):
        with pytest.raises(RuntimeError, match="x to have dtype"):
            f(x.float())
    with pytest.raises(RuntimeError, match="gate_up to have dtype"):
        ops.silu_mul_quantize_fused(x.float())
    # right types, host tensors: refused by the device check
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops.linear_w4a4("sym", A, W, h(M), None, h(N))
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops.quantize_sym_fused(x)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops.sym_quant(x, h(M))
