"""Functional wrappers: flatten leading dimensions, call the operator module, restore the
shape. Names and argument order follow `qlinear4bit/tools/tensor_utils.py` of the reference
(cited per function); `linear` is new and runs the fused kernel."""
import torch

from .. import _CUDA as ops


class PackedQuantizedTensor:
    """Quantized activations travelling between a quantizer and a linear module
    (ref: tensor_utils.py:20-39): packed codes, per-token scales, optional zero-points."""

    def __init__(self, quantized_x: torch.Tensor, scales_x: torch.Tensor, zeros_x: torch.Tensor = None):
        self.quantized_x = quantized_x
        self.scales_x = scales_x
        self.zeros_x = zeros_x

    def size(self):
        return self.quantized_x.size()

    @property
    def device(self):
        return self.quantized_x.device

    @property
    def dtype(self):
        return self.quantized_x.dtype


def _rows(t):
    """[..., C] -> ([rows, C], leading shape)."""
    return t.view(-1, t.shape[-1]), tuple(t.shape[:-1])


def _need(cond, msg):
    if not cond:
        raise AssertionError(msg)


def _k_ok(A):
    _need(A.shape[-1] % 32 == 0, "A.shape[-1]: {} must be multiplication of 32".format(A.shape[-1]))


def matmul(A, B):
    """ref: tensor_utils.py:51-55."""
    _k_ok(A)
    a, lead_a = _rows(A)
    b, lead_b = _rows(B)
    return ops.matmul(a, b).view(*lead_a, *lead_b)


def matmul_8bit(A, B):
    """ref: tensor_utils.py:57-61."""
    _k_ok(A)
    a, lead_a = _rows(A)
    b, lead_b = _rows(B)
    return ops.matmul_8bit(a, b).view(*lead_a, *lead_b)


def batched_matmul(A, B):
    """A [b,M,K/2], B [b,N,K/2] -> int32 [b,M,N] (ref: tensor_utils.py:63-68, which stops in an
    interactive shell before calling a kernel that does not work)."""
    _k_ok(A)
    return ops.batched_matmul(A, B)


def _f16(*ts):
    _need(all(t.dtype == torch.float16 for t in ts), "expected torch.float16 tensors")


def sym_quant(x, scale):
    """ref: tensor_utils.py:70-73."""
    _f16(x, scale)
    x2, lead = _rows(x)
    return ops.sym_quant(x2, scale.view(-1)).view(*lead, -1)


def sym_dual_quant(x, scale_1, scale_2):
    """ref: tensor_utils.py:75-78."""
    _f16(x, scale_1, scale_2)
    x2, lead = _rows(x)
    return ops.sym_dual_quant(x2, scale_1.view(-1), scale_2.view(-1)).view(*lead, -1)


def sym_dequant(q, scale_row, scale_col, bits=32):
    """ref: tensor_utils.py:80-84."""
    _need(q.dtype == torch.int32, "q must be int32")
    _f16(scale_row, scale_col)
    q2, lead = _rows(q)
    return ops.sym_dequant(q2, scale_row.view(-1), scale_col, bits).view(*lead, -1)


def sym_dual_dequant(q, scale_row, scale_col_1, scale_col_2, bits=32):
    """ref: tensor_utils.py:86-90."""
    _need(q.dtype == torch.int32, "q must be int32")
    _f16(scale_row, scale_col_1, scale_col_2)
    q2, lead = _rows(q)
    return ops.sym_dual_dequant(q2, scale_row.view(-1), scale_col_1, scale_col_2, bits).view(*lead, -1)


def asym_quant(q, scale, zero):
    """ref: tensor_utils.py:92-96."""
    _f16(q, scale, zero)
    x2, lead = _rows(q)
    return ops.asym_quant(x2, scale.view(-1), zero.view(-1)).view(*lead, -1)


def asym_quant_8bit(q, scale, zero):
    """ref: tensor_utils.py:98-102."""
    _need(q.dtype == scale.dtype == zero.dtype == torch.float32, "expected torch.float32 tensors")
    x2, lead = _rows(q)
    return ops.asym_quant_8bit(x2, scale.view(-1), zero.view(-1)).view(*lead, -1)


def asym_dequant(q, scale_row, zeros_row, scale_col, zeros_col, bits=32):
    """ref: tensor_utils.py:104-108."""
    _need(q.dtype == torch.int32, "q must be int32")
    _f16(scale_row, zeros_row, scale_col, zeros_col)
    q2, lead = _rows(q)
    return ops.asym_dequant(q2, scale_row.view(-1), zeros_row.view(-1), scale_col.view(-1), zeros_col.view(-1),
                            bits).view(*lead, -1)


def asym_dequant_hprec(q, scale_row, zeros_row, scale_col, zeros_col, bits=32):
    """ref: tensor_utils.py:110-114."""
    _need(q.dtype == torch.int32, "q must be int32")
    _need(all(t.dtype == torch.float32 for t in (scale_row, zeros_row, scale_col, zeros_col)), "expected torch.float32")
    q2, lead = _rows(q)
    return ops.asym_dequant_hprec(q2, scale_row.view(-1), zeros_row.view(-1), scale_col.view(-1), zeros_col.view(-1),
                                  bits).view(*lead, -1)


def asym_batch_dequant(q, scale_row, zeros_row, scale_col, zeros_col, bits=32):
    """ref: tensor_utils.py:116-124."""
    _need(q.dtype == torch.int32, "q must be int32")
    _f16(scale_row, zeros_row, scale_col, zeros_col)
    lead, (r, c) = tuple(q.shape[:-2]), q.shape[-2:]
    q3 = q.view(-1, r, c)
    return ops.asym_batch_dequant(q3, scale_row, zeros_row, scale_col, zeros_col, bits).view(*lead, r, c)


def asym_dual_quant(q, scale_1, zeros1, scale_2, zeros2):
    """ref: tensor_utils.py:126-134 (which asserts an int32 input by mistake; the kernel takes
    fp16 activations, as here)."""
    _f16(q, scale_1, zeros1, scale_2, zeros2)
    x2, lead = _rows(q)
    return ops.asym_dual_quant(x2, scale_1.view(-1), zeros1.view(-1), scale_2.view(-1), zeros2.view(-1)).view(*lead, -1)


def asym_dual_dequant(q, scale_row, zeros_row, scale_col_1, zeros_col_1, scale_col_2, zeros_col_2, bits=32):
    """ref: tensor_utils.py:136-143."""
    _need(q.dtype == torch.int32, "q must be int32")
    _f16(scale_row, zeros_row, scale_col_1, zeros_col_1, scale_col_2, zeros_col_2)
    q2, lead = _rows(q)
    return ops.asym_dual_dequant(q2, scale_row.view(-1), zeros_row.view(-1), scale_col_1.view(-1), zeros_col_1.view(-1),
                                 scale_col_2.view(-1), zeros_col_2.view(-1), bits).view(*lead, -1)


def get_dual_quant_col():
    """ref: tensor_utils.py:144-145."""
    return ops.get_dual_quant_col_k()


def linear(mode, packed: PackedQuantizedTensor, weight, scale_col_1, zeros_col_1=None, scale_col_2=None,
           zeros_col_2=None, bias=None):
    """(new) the whole forward of a 4-bit linear module on quantized input: one fused kernel."""
    _k_ok(packed.quantized_x)
    a, lead = _rows(packed.quantized_x)
    zr = None if packed.zeros_x is None else packed.zeros_x.reshape(-1)
    flat = lambda t: None if t is None else t.reshape(-1)
    out = ops.linear_w4a4(mode, a, weight, packed.scales_x.reshape(-1), zr, flat(scale_col_1), flat(zeros_col_1),
                          flat(scale_col_2), flat(zeros_col_2), bias)
    return out.view(*lead, -1)
