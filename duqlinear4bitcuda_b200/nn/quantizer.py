"""Per-token activation quantizer modules (same class names, constructor arguments and return
type as `qlinear4bit/nn/quantizer.py` of the reference). Each forward is ONE fused kernel
launch instead of the reference's chain of torch reductions followed by a quantize launch;
scales, zero-points and codes are bit-identical to that chain."""
import torch

from .. import _CUDA as ops
from ..tools import tensor_utils
from ..tools.tensor_utils import PackedQuantizedTensor


def _as_rows(x):
    if not x.is_contiguous():
        x = x.contiguous()
    return x.view(-1, x.shape[-1]), tuple(x.shape[:-1])


def _scale_shape(lead):
    """The reference computes `max(|x|, -1)[0].unsqueeze(1)`: for x [B,S,K] its scales have
    shape [B,1,S]; for x [R,K] they are [R,1]. Consumers flatten them, so only the element
    order matters, which is the row order."""
    if len(lead) <= 1:
        return (*lead, 1)
    return (lead[0], 1, *lead[1:])


class SymQuantizer(torch.nn.Module):
    """ref: nn/quantizer.py:5-16. scale = half(half(max|x|)/7) * input_clip_ratio per token,
    codes clamp(rn(x/scale), -8, 6)."""

    def __init__(self, input_clip_ratio=1.0):
        super().__init__()
        self.input_clip_ratio = input_clip_ratio

    def forward(self, x) -> PackedQuantizedTensor:
        x2, lead = _as_rows(x)
        q, s = ops.quantize_sym_fused(x2, self.input_clip_ratio)
        return PackedQuantizedTensor(q.view(*lead, -1), s.view(_scale_shape(lead)))


class AsymQuantizer(torch.nn.Module):
    """ref: nn/quantizer.py:18-35. scale = (max-min)/15, zero = round(-min/scale); like the
    reference, `input_clip_ratio` is stored and not used."""

    def __init__(self, input_clip_ratio: float = 1.0):
        super().__init__()
        self.n_levels = 2 ** 4
        self.input_clip_ratio = input_clip_ratio

    def forward(self, x) -> PackedQuantizedTensor:
        x2, lead = _as_rows(x)
        q, s, z = ops.quantize_asym_fused(x2)
        return PackedQuantizedTensor(q.view(*lead, -1), s.view(*lead, 1), z.view(*lead, 1))


class AsymQuantizer8bit(torch.nn.Module):
    """ref: nn/quantizer.py:38-55. 8-bit side path on fp32 activations: the statistics stay in
    torch (it is not part of the 4-bit hot path), the coding runs in the library."""

    def __init__(self, input_clip_ratio: float = 1.0):
        super().__init__()
        self.n_levels = 2 ** 7
        self.input_clip_ratio = input_clip_ratio

    def forward(self, x) -> PackedQuantizedTensor:
        if not x.is_contiguous():
            x = x.contiguous()
        lo = x.amin(dim=-1, keepdim=True)
        hi = x.amax(dim=-1, keepdim=True)
        scale = (hi - lo) / (self.n_levels - 1)
        zeros = (-lo / scale).round().to(torch.float32)
        q = tensor_utils.asym_quant_8bit(x, scale, zeros)
        return PackedQuantizedTensor(q, scale, zeros)
