"""Activation x activation quantized matmul modules (ref: qlinear4bit/nn/matmul.py). Both
operands are quantized per row at run time; the batched product is ONE launch of the batched
fused kernel instead of the reference's Python loop over the batch plus a separate dequant."""
import math

import torch
import torch.nn as nn

from .. import _CUDA as ops
from ..tools import tensor_utils
from .quantizer import AsymQuantizer, SymQuantizer


class AsymQuantMatMul(nn.Module):
    """A [..,HA,W] x B [..,HB,W]^T -> fp16 [..,HA,HB] with asymmetric 4-bit operands
    (ref: nn/matmul.py:20-68). W must be a multiple of 64."""

    def __init__(self, transpose_B=False):
        super().__init__()
        self.quantizer_A = AsymQuantizer()
        self.quantizer_B = AsymQuantizer()
        self.transpose_B = transpose_B

    def forward(self, A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
        if self.transpose_B:
            B = B.transpose(-1, -2)
        lead_a, lead_b = tuple(A.shape[:-2]), tuple(B.shape[:-2])
        if any(x != y for x, y in zip(lead_a, lead_b)):
            raise AssertionError("Batch dimensions must match")
        nb = math.prod(lead_a)
        HA, HB = A.shape[-2], B.shape[-2]
        qa = self.quantizer_A(A.reshape(nb, HA, A.shape[-1]))
        qb = self.quantizer_B(B.reshape(nb, HB, B.shape[-1]))
        out = ops.linear_w4a4_batched("asym", qa.quantized_x, qb.quantized_x,
                                      qa.scales_x.reshape(nb, HA), qa.zeros_x.reshape(nb, HA),
                                      qb.scales_x.reshape(nb, HB), qb.zeros_x.reshape(nb, HB))
        return out.view(*lead_a, HA, HB)


class SymQuantMatMul(nn.Module):
    """2-D symmetric variant (ref: nn/matmul.py:72-84)."""

    def __init__(self):
        super().__init__()
        self.quantizer_A = SymQuantizer()
        self.quantizer_B = SymQuantizer()

    def forward(self, A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
        qa = self.quantizer_A(A)
        qb = self.quantizer_B(B)
        return tensor_utils.linear("sym", qa, qb.quantized_x, qb.scales_x)
