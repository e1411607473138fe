"""Tensor-level operator module with the names, keyword names and return conventions of the
reference's compiled extension `qlinear4bit._CUDA` (ref: src/export/bindings.cpp:768-932),
implemented over the C ABI of libduq4.so.

Every function validates its tensors the way the reference binding does (contiguous, CUDA,
same GPU, leading-dimension sizes), allocates its result with torch on the input's device and
launches on torch's CURRENT stream (the reference always used the legacy default stream).
Functions the reference does not have are marked "(new)".
"""
import ctypes

import torch

from . import lib as _L

__all__ = [
    "matmul", "matmul_8bit", "batched_matmul", "sym_quant", "sym_dual_quant", "sym_dequant", "sym_dual_dequant",
    "asym_quant", "asym_quant_8bit", "asym_batch_dequant", "asym_dequant", "asym_dequant_hprec", "asym_dual_quant",
    "asym_dual_dequant", "get_dual_quant_col_k", "quantize_sym_fused", "quantize_asym_fused",
    "quantize_sym_dual_fused", "quantize_asym_dual_fused", "silu_mul_quantize_fused", "linear_w4a4", "linear_w4a4_from_fp16", "linear_w4a4_batched",
]


def _check(fn, **tensors):
    first = None
    for name, t in tensors.items():
        if t is None:
            continue
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{fn}: {name} must be a torch.Tensor")
        if not t.is_cuda:
            raise RuntimeError(f"{fn}: expected {name} to be a CUDA tensor")
        if not t.is_contiguous():
            raise RuntimeError(f"{fn}: expected {name} to be contiguous")
        if first is None:
            first = t
        elif t.device != first.device:
            raise RuntimeError(f"{fn}: expected {name} to be on the same GPU as the first argument")
    return first


def _size0(fn, name, t, n, dim=0):
    if t.size(dim) != n:
        raise RuntimeError(f"{fn}: expected {name}.size({dim}) == {n}, got {t.size(dim)}")


def _bits(bits):
    if bits != 32:
        raise RuntimeError("Unsupported data type")


def _run(name, dev_tensor, *args):
    with torch.cuda.device(dev_tensor.device):
        _L.call(name, *args, _L.current_stream())


_p = _L.ptr


def get_dual_quant_col_k():
    """ref: bindings.cpp:471-473."""
    return _L.cdll.duq4_dual_quant_col_k()


# ---- GEMMs -------------------------------------------------------------------------------
def matmul(A, B):
    """int4 x int4 -> int32, C[M,N] = A[M,K/2] . B[N,K/2]^T (ref: bindings.cpp:10-26)."""
    _check("matmul", A=A, B=B)
    M, N, K = A.size(0), B.size(0), A.size(1) * 2
    C = torch.empty((M, N), dtype=torch.int32, device=A.device)
    _run("duq4_matmul_4bit", A, _p(A), _p(B), M, N, K, _p(C))
    return C


def matmul_8bit(A, B):
    """int8 x int8 -> int32 (ref: bindings.cpp:28-44)."""
    _check("matmul_8bit", A=A, B=B)
    M, N, K = A.size(0), B.size(0), A.size(1)
    C = torch.empty((M, N), dtype=torch.int32, device=A.device)
    _run("duq4_matmul_8bit", A, _p(A), _p(B), M, N, K, _p(C))
    return C


def batched_matmul(A, B):
    """A [b,M,K/2], B [b,N,K/2] -> int32 [b,M,N] (ref: bindings.cpp:46-84, which does not work
    there: it hands host pointer arrays to the device)."""
    _check("batched_matmul", A=A, B=B)
    b, M, N, K = A.size(0), A.size(1), B.size(1), A.size(2) * 2
    _size0("batched_matmul", "B", B, b)
    C = torch.empty((b, M, N), dtype=torch.int32, device=A.device)
    _run("duq4_batch_matmul_4bit", A, _p(A), _p(B), M, N, K, _p(C), b)
    return C


# ---- quantize, scales given --------------------------------------------------------------
def _quant_out(x):
    rows, cols = x.size(0), x.size(1)
    cd = (cols + 1) // 2
    return rows, cols, cd, torch.empty((rows, cd), dtype=torch.uint8, device=x.device)


def sym_quant(x, scale):
    """ref: bindings.cpp:88-105."""
    _check("sym_quant", x=x, scale=scale)
    _size0("sym_quant", "scale", scale, x.size(0))
    rows, cols, cd, q = _quant_out(x)
    _run("duq4_sym_quant", x, _p(x), _p(scale), rows, cols, cd, _p(q))
    return q


def sym_dual_quant(x, scale_1, scale_2):
    """ref: bindings.cpp:107-127."""
    _check("sym_dual_quant", x=x, scale_1=scale_1, scale_2=scale_2)
    _size0("sym_dual_quant", "scale_1", scale_1, x.size(0)); _size0("sym_dual_quant", "scale_2", scale_2, x.size(0))
    rows, cols, cd, q = _quant_out(x)
    _run("duq4_sym_dual_quant", x, _p(x), _p(scale_1), _p(scale_2), rows, cols, cd, _p(q))
    return q


def asym_quant(x, scale, zeros):
    """ref: bindings.cpp:221-243."""
    _check("asym_quant", x=x, scale=scale, zeros=zeros)
    _size0("asym_quant", "scale", scale, x.size(0)); _size0("asym_quant", "zeros", zeros, x.size(0))
    rows, cols, cd, q = _quant_out(x)
    _run("duq4_asym_quant", x, _p(x), _p(scale), _p(zeros), rows, cols, cd, _p(q))
    return q


def asym_dual_quant(x, scale_1, zeros_1, scale_2, zeros_2):
    """ref: bindings.cpp:393-421 (whose wrapper forgets to return its tensor; this one returns it)."""
    _check("asym_dual_quant", x=x, scale_1=scale_1, zeros_1=zeros_1, scale_2=scale_2, zeros_2=zeros_2)
    for n, t in (("scale_1", scale_1), ("zeros_1", zeros_1), ("scale_2", scale_2), ("zeros_2", zeros_2)):
        _size0("asym_dual_quant", n, t, x.size(0))
    rows, cols, cd, q = _quant_out(x)
    _run("duq4_asym_dual_quant", x, _p(x), _p(scale_1), _p(zeros_1), _p(scale_2), _p(zeros_2), rows, cols, cd, _p(q))
    return q


def asym_quant_8bit(x, scale, zeros):
    """fp32 in, int8 codes in [0,126] out (ref: bindings.cpp:245-266)."""
    _check("asym_quant_8bit", x=x, scale=scale, zeros=zeros)
    _size0("asym_quant_8bit", "scale", scale, x.size(0)); _size0("asym_quant_8bit", "zeros", zeros, x.size(0))
    q = torch.empty((x.size(0), x.size(1)), dtype=torch.int8, device=x.device)
    _run("duq4_asym_quant_8bit", x, _p(x), _p(scale), _p(zeros), x.size(0), x.size(1), _p(q))
    return q


# ---- fused quantizers (new) ---------------------------------------------------------------
def quantize_sym_fused(x, clip_ratio=1.0):
    """(new) x fp16 [rows, K] -> (codes uint8 [rows, K/2], scales fp16 [rows]); one kernel doing
    what SymQuantizer's abs/max/div/mul torch ops plus sym_quant do."""
    _check("quantize_sym_fused", x=x)
    rows, cols, cd, q = _quant_out(x)
    s = torch.empty((rows,), dtype=torch.float16, device=x.device)
    _run("duq4_quantize_sym_fused", x, _p(x), rows, cols, float(clip_ratio), _p(q), _p(s))
    return q, s


def quantize_asym_fused(x):
    """(new) -> (codes, scales fp16 [rows], zeros fp16 [rows])."""
    _check("quantize_asym_fused", x=x)
    rows, cols, cd, q = _quant_out(x)
    s = torch.empty((rows,), dtype=torch.float16, device=x.device); z = torch.empty_like(s)
    _run("duq4_quantize_asym_fused", x, _p(x), rows, cols, _p(q), _p(s), _p(z))
    return q, s, z


def quantize_sym_dual_fused(x, clip_ratio=1.0):
    """(new) dual-uniform: one scale for columns < get_dual_quant_col_k(), one for the rest."""
    _check("quantize_sym_dual_fused", x=x)
    rows, cols, cd, q = _quant_out(x)
    s1 = torch.empty((rows,), dtype=torch.float16, device=x.device); s2 = torch.empty_like(s1)
    _run("duq4_quantize_sym_dual_fused", x, _p(x), rows, cols, float(clip_ratio), _p(q), _p(s1), _p(s2))
    return q, s1, s2


def quantize_asym_dual_fused(x):
    """(new) -> (codes, scale_1, zeros_1, scale_2, zeros_2)."""
    _check("quantize_asym_dual_fused", x=x)
    rows, cols, cd, q = _quant_out(x)
    s1 = torch.empty((rows,), dtype=torch.float16, device=x.device)
    z1, s2, z2 = torch.empty_like(s1), torch.empty_like(s1), torch.empty_like(s1)
    _run("duq4_quantize_asym_dual_fused", x, _p(x), rows, cols, _p(q), _p(s1), _p(z1), _p(s2), _p(z2))
    return q, s1, z1, s2, z2


def silu_mul_quantize_fused(gate_up, mode="sym", clip_ratio=1.0, tensor_core_ready=False):
    """(new) SiLU-gated MLP glue in one kernel: gate_up fp16 [rows, 2*I] holds the gate projection in
    columns [0, I) and the up projection in [I, 2I); returns the per-token quantization of
    h = F.silu(gate) * up (the fp16 tensor those torch ops would produce) without storing h:
    (codes, scales) for mode "sym", (codes, scales, zeros) for "asym". Codes are packed uint8
    [rows, I/2], or int8 [rows, I] in the GEMM's tensor-core-ready layout when requested."""
    _check("silu_mul_quantize_fused", gate_up=gate_up)
    rows, ld = gate_up.size(0), gate_up.size(1)
    inter = ld // 2
    if ld % 2 or gate_up.dtype != torch.float16:
        raise RuntimeError("silu_mul_quantize_fused: expected fp16 [rows, 2*I]")
    q = torch.empty((rows, inter) if tensor_core_ready else (rows, inter // 2),
                    dtype=torch.int8 if tensor_core_ready else torch.uint8, device=gate_up.device)
    s = torch.empty((rows,), dtype=torch.float16, device=gate_up.device)
    z = torch.empty_like(s) if mode == "asym" else None
    _run("duq4_silu_mul_quantize_fused", gate_up, _L.MODES[mode], _p(gate_up), rows, inter, ld, inter, float(clip_ratio), _p(q),
         1 if tensor_core_ready else 0, _p(s), _p(z))
    return (q, s) if z is None else (q, s, z)


# ---- dequantize ---------------------------------------------------------------------------
def sym_dequant(q, scale_row, scale_col, bits):
    """ref: bindings.cpp:130-170."""
    _check("sym_dequant", q=q, scale_row=scale_row, scale_col=scale_col)
    rows, cols = q.size(0), q.size(1)
    _size0("sym_dequant", "scale_row", scale_row, rows); _size0("sym_dequant", "scale_col", scale_col, cols)
    _bits(bits)
    x = torch.empty((rows, cols), dtype=torch.float16, device=q.device)
    _run("duq4_sym_dequant", q, _p(q), _p(scale_row), _p(scale_col), rows, cols, _p(x))
    return x


def sym_dual_dequant(q, scale_row, scale_col_1, scale_col_2, bits):
    """ref: bindings.cpp:172-217."""
    _check("sym_dual_dequant", q=q, scale_row=scale_row, scale_col_1=scale_col_1, scale_col_2=scale_col_2)
    rows, cols = q.size(0), q.size(1)
    _size0("sym_dual_dequant", "scale_row", scale_row, rows)
    _size0("sym_dual_dequant", "scale_col_1", scale_col_1, cols); _size0("sym_dual_dequant", "scale_col_2", scale_col_2, cols)
    _bits(bits)
    x = torch.empty((rows, cols), dtype=torch.float16, device=q.device)
    _run("duq4_sym_dual_dequant", q, _p(q), _p(scale_row), _p(scale_col_1), _p(scale_col_2), rows, cols, _p(x))
    return x


def asym_dequant(q, scale_row, zeros_row, scale_col, zeros_col, bits):
    """ref: bindings.cpp:268-307."""
    _check("asym_dequant", q=q, scale_row=scale_row, zeros_row=zeros_row, scale_col=scale_col, zeros_col=zeros_col)
    rows, cols = q.size(0), q.size(1)
    _size0("asym_dequant", "scale_row", scale_row, rows); _size0("asym_dequant", "zeros_row", zeros_row, rows)
    _size0("asym_dequant", "scale_col", scale_col, cols); _size0("asym_dequant", "zeros_col", zeros_col, cols)
    _bits(bits)
    x = torch.empty((rows, cols), dtype=torch.float16, device=q.device)
    _run("duq4_asym_dequant", q, _p(q), _p(scale_row), _p(zeros_row), _p(scale_col), _p(zeros_col), rows, cols, _p(x))
    return x


def asym_dual_dequant(q, scale_row, zeros_row, scale_col_1, zeros_col_1, scale_col_2, zeros_col_2, bits):
    """ref: bindings.cpp:423-467."""
    _check("asym_dual_dequant", q=q, scale_row=scale_row, zeros_row=zeros_row, scale_col_1=scale_col_1,
           zeros_col_1=zeros_col_1, scale_col_2=scale_col_2, zeros_col_2=zeros_col_2)
    rows, cols = q.size(0), q.size(1)
    _size0("asym_dual_dequant", "scale_row", scale_row, rows); _size0("asym_dual_dequant", "zeros_row", zeros_row, rows)
    for n, t in (("scale_col_1", scale_col_1), ("zeros_col_1", zeros_col_1), ("scale_col_2", scale_col_2),
                 ("zeros_col_2", zeros_col_2)):
        _size0("asym_dual_dequant", n, t, cols)
    _bits(bits)
    x = torch.empty((rows, cols), dtype=torch.float16, device=q.device)
    _run("duq4_asym_dual_dequant", q, _p(q), _p(scale_row), _p(zeros_row), _p(scale_col_1), _p(zeros_col_1),
         _p(scale_col_2), _p(zeros_col_2), rows, cols, _p(x))
    return x


def asym_batch_dequant(q, scale_row, zeros_row, scale_col, zeros_col, bits):
    """q [b,rows,cols]; row vectors with size(1) == rows, column vectors with size(1) == cols
    (ref: bindings.cpp:351-391)."""
    _check("asym_batch_dequant", q=q, scale_row=scale_row, zeros_row=zeros_row, scale_col=scale_col, zeros_col=zeros_col)
    b, rows, cols = q.size(0), q.size(1), q.size(2)
    _size0("asym_batch_dequant", "scale_row", scale_row, rows, 1); _size0("asym_batch_dequant", "zeros_row", zeros_row, rows, 1)
    _size0("asym_batch_dequant", "scale_col", scale_col, cols, 1); _size0("asym_batch_dequant", "zeros_col", zeros_col, cols, 1)
    _bits(bits)
    x = torch.empty((b, rows, cols), dtype=torch.float16, device=q.device)
    _run("duq4_asym_batch_dequant", q, _p(q), _p(scale_row), _p(zeros_row), _p(scale_col), _p(zeros_col), b, rows, cols, _p(x))
    return x


def asym_dequant_hprec(q, scale_row, zeros_row, scale_col, zeros_col, bits):
    """fp32 dequant of the 8-bit path (ref: bindings.cpp:309-348)."""
    _check("asym_dequant_hprec", q=q, scale_row=scale_row, zeros_row=zeros_row, scale_col=scale_col, zeros_col=zeros_col)
    rows, cols = q.size(0), q.size(1)
    _size0("asym_dequant_hprec", "scale_row", scale_row, rows); _size0("asym_dequant_hprec", "scale_col", scale_col, cols)
    _bits(bits)
    x = torch.empty((rows, cols), dtype=torch.float32, device=q.device)
    _run("duq4_asym_dequant_hprec", q, _p(q), _p(scale_row), _p(zeros_row), _p(scale_col), _p(zeros_col), rows, cols, _p(x))
    return x


# ---- fused linear (new) -------------------------------------------------------------------
def linear_w4a4(mode, A, W, scale_row, zeros_row=None, scale_col_1=None, zeros_col_1=None, scale_col_2=None,
                zeros_col_2=None, bias=None, col_offset=0, out=None, return_acc=False, next_weights=None):
    """(new) fp16 [M,N] = dequant_mode(A [M,K/2] . W [N,K/2]^T) (+ bias): GEMM, dequant and bias in
    one kernel; results identical to matmul -> *_dequant -> `+ bias`. `mode` is one of
    "sym", "sym_dual", "asym", "asym_dual". `out` may be a column slice view of a wider
    row-major buffer (its row stride is honoured). `next_weights`: the packed weights of the layer
    that follows on this stream -- a hint that lets the small-M kernels warm L2 with them."""
    _check("linear_w4a4", A=A, W=W, scale_row=scale_row, zeros_row=zeros_row, scale_col_1=scale_col_1,
           zeros_col_1=zeros_col_1, scale_col_2=scale_col_2, zeros_col_2=zeros_col_2, bias=bias)
    M, N, K = A.size(0), W.size(0), A.size(1) * 2
    if W.size(1) != A.size(1):
        raise RuntimeError("linear_w4a4: A and W disagree on K")
    _size0("linear_w4a4", "scale_row", scale_row, M)
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=A.device)
    elif out.dtype != torch.float16 or out.size(0) != M or out.size(1) != N or out.stride(1) != 1:
        raise RuntimeError("linear_w4a4: out must be fp16 [M,N] with unit column stride")
    acc = torch.empty((M, N), dtype=torch.int32, device=A.device) if return_acc else None
    epi = _L.make_epilogue(mode, scale_row, zeros_row, scale_col_1, zeros_col_1, scale_col_2, zeros_col_2, bias,
                           col_offset, out.stride(0) if M > 1 else max(out.stride(0), N), next_weights=next_weights)
    _run("duq4_linear_w4a4", A, _p(A), _p(W), M, N, K, ctypes.byref(epi), _p(out), _p(acc))
    return (out, acc) if return_acc else out


_WS = {}   # per-device scratch for linear_w4a4_from_fp16, grown on demand


def linear_w4a4_from_fp16(mode, x, W, scale_col_1, zeros_col_1=None, scale_col_2=None, zeros_col_2=None, bias=None,
                          clip_ratio=1.0, act_mode=None):
    """(new) fp16 activations [M,K] -> per-token quantize -> GEMM -> dequant (+bias) in one library call
    (two launches, the quantized activations stay in an internal scratch tensor in the GEMM's
    tensor-core-ready layout). Same result as quantizer module + linear_w4a4. `act_mode` defaults to
    the single-scale quantizer of the epilogue's family ("sym" for sym/sym_dual, "asym" otherwise),
    which is what the reference modules pair with each linear variant."""
    _check("linear_w4a4_from_fp16", x=x, W=W, scale_col_1=scale_col_1, zeros_col_1=zeros_col_1, scale_col_2=scale_col_2,
           zeros_col_2=zeros_col_2, bias=bias)
    if x.dtype != torch.float16 or x.dim() != 2:
        raise RuntimeError("linear_w4a4_from_fp16: x must be fp16 [M, K]")
    M, K, N = x.size(0), x.size(1), W.size(0)
    if W.size(1) * 2 != K:
        raise RuntimeError("linear_w4a4_from_fp16: x and W disagree on K")
    if act_mode is None:
        act_mode = "sym" if mode in ("sym", "sym_dual") else "asym"
    need = _L.cdll.duq4_linear_from_fp16_workspace_bytes(M, K)
    ws = _WS.get(x.device)
    if ws is None or ws.numel() < need:
        ws = _WS[x.device] = torch.empty(need, dtype=torch.uint8, device=x.device)
    out = torch.empty((M, N), dtype=torch.float16, device=x.device)
    epi = _L.make_epilogue(mode, None, None, scale_col_1, zeros_col_1, scale_col_2, zeros_col_2, bias)
    _run("duq4_linear_w4a4_from_fp16", x, _p(x), _p(W), M, N, K, _L.MODES[act_mode], float(clip_ratio), ctypes.byref(epi),
         _p(out), _p(ws), ws.numel())
    return out


def linear_w4a4_gate_up_silu(mode, A, W, scale_row, zeros_row=None, scale_col=None, zeros_col=None, bias=None):
    """(new) SiLU-gated gate/up projection in one launch: W packed [2*I, K/2] = gate rows then up rows,
    `scale_col` / `zeros_col` / `bias` with 2*I entries; returns h fp16 [M, I] equal to
    `F.silu(y[:, :I]) * y[:, I:]` for y = linear_w4a4(mode, A, W, ...), without writing y. A is either
    packed int4 activations uint8 [M, K/2] or the tensor-core-ready int8 [M, K] of
    silu_mul_quantize_fused / duq4_quantize_fused_i8. mode: "sym" or "asym"."""
    _check("linear_w4a4_gate_up_silu", A=A, W=W, scale_row=scale_row, zeros_row=zeros_row, scale_col=scale_col,
           zeros_col=zeros_col, bias=bias)
    if mode not in ("sym", "asym"):
        raise RuntimeError("linear_w4a4_gate_up_silu: mode must be 'sym' or 'asym'")
    a_is_int8 = A.dtype == torch.int8
    M, K = A.size(0), (A.size(1) if a_is_int8 else A.size(1) * 2)
    if W.size(0) % 2 != 0 or W.size(1) * 2 != K:
        raise RuntimeError("linear_w4a4_gate_up_silu: W must be [2*I, K/2]")
    inter = W.size(0) // 2
    _size0("linear_w4a4_gate_up_silu", "scale_row", scale_row, M)
    _size0("linear_w4a4_gate_up_silu", "scale_col", scale_col, 2 * inter)
    h = torch.empty((M, inter), dtype=torch.float16, device=A.device)
    epi = _L.make_epilogue(mode, scale_row, zeros_row, scale_col, zeros_col, None, None, bias)
    _run("duq4_linear_w4a4_gate_up_silu", A, _p(A), 1 if a_is_int8 else 0, _p(W), M, inter, K, ctypes.byref(epi), _p(h))
    return h


def linear_w4a4_batched(mode, A, W, scale_row, zeros_row=None, scale_col_1=None, zeros_col_1=None, scale_col_2=None,
                        zeros_col_2=None):
    """(new) batched form: A [b,M,K/2], W [b,N,K/2], row vectors [b,M], column vectors [b,N]."""
    _check("linear_w4a4_batched", A=A, W=W, scale_row=scale_row, zeros_row=zeros_row, scale_col_1=scale_col_1,
           zeros_col_1=zeros_col_1, scale_col_2=scale_col_2, zeros_col_2=zeros_col_2)
    b, M, N, K = A.size(0), A.size(1), W.size(1), A.size(2) * 2
    out = torch.empty((b, M, N), dtype=torch.float16, device=A.device)
    epi = _L.make_epilogue(mode, scale_row, zeros_row, scale_col_1, zeros_col_1, scale_col_2, zeros_col_2)
    _run("duq4_linear_w4a4_batched", A, _p(A), _p(W), M, N, K, b, ctypes.byref(epi), _p(out), None)
    return out
