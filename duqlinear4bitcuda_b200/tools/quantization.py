"""Host-side (pure torch) helpers: nibble packing and fake-quantization.

Same names and results as `qlinear4bit/tools/quantization.py` of the reference (cited per
function); they run on any device and are used for one-off weight preparation, not on the
hot path. The int4 storage format is: element 2j in the low nibble of byte j, element 2j+1
in the high nibble, two's complement.
"""
import torch


def two_compl(x, bits: int):
    """Two's-complement image of signed integers in `bits` bits (ref: quantization.py:4-5)."""
    return torch.where(x < 0, x + (1 << bits), x)


def get_minq_maxq(bits: int, sym: bool):
    """Integer range of a `bits`-bit code (ref: quantization.py:7-15)."""
    if sym:
        hi = (1 << (bits - 1)) - 1
        return torch.tensor(-hi - 1), torch.tensor(hi)
    return torch.tensor(0), torch.tensor((1 << bits) - 1)


def sym_quant(x, scale, maxq):
    """round(x/scale) clamped to [-(maxq+1), maxq] (ref: quantization.py:29-32)."""
    scale = scale.to(x.device)
    return torch.clamp(torch.round(x / scale), -(maxq + 1), maxq), scale


def sym_dequant(q, scale):
    return scale * q


def sym_quant_dequant(x, scale, maxq):
    q, s = sym_quant(x, scale, maxq)
    return sym_dequant(q, s)


def asym_quant(x, scale, zero, maxq):
    """round(x/scale) + zero clamped to [0, maxq] (ref: quantization.py:17-21)."""
    scale, zero = scale.to(x.device), zero.to(x.device)
    return torch.clamp(torch.round(x / scale) + zero, 0, maxq), scale, zero


def asym_dequant(q, scale, zero):
    return scale * (q - zero)


def asym_quant_dequant(x, scale, zero, maxq):
    q, s, z = asym_quant(x, scale, zero, maxq)
    return asym_dequant(q, s, z)


def pack_i4(q, sym=True):
    """Signed integer tensor [..., K] with values in the 4-bit range -> uint8 [..., K/2]
    (ref: quantization.py:40-47)."""
    if not torch.is_signed(q):
        raise AssertionError("The tensor to be packed should be signed int")
    lo, hi = get_minq_maxq(4, sym)
    if not bool(torch.all((q >= lo) & (q <= hi))):
        raise AssertionError("values outside the int4 range")
    nib = two_compl(q.to(torch.int8), 4).to(torch.uint8)
    return nib[..., 0::2] | (nib[..., 1::2] << 4)


def unpack_i4(x: torch.Tensor):
    """uint8 [..., K/2] -> int32 [..., K], every nibble read as a signed value
    (ref: quantization.py:50-72)."""
    if x.dtype != torch.uint8:
        raise AssertionError("The tensor to be unpacked should be stored in uint8")
    pair = torch.stack((x & 0x0F, x >> 4), dim=-1).to(torch.int32)
    pair = torch.where(pair >= 8, pair - 16, pair)
    return pair.reshape(*x.shape[:-1], x.shape[-1] * 2)


# ---- weight preparation used by the nn modules' from_float / from_linear -----------------

def asym_weight_quant(w, levels=16):
    """Per-output-row asymmetric weight quantization exactly as the reference's
    `Linear4bitASQ.from_linear` does it (ref: qlinear4bit/nn/linear.py:126-137): the range is
    [min|w|, max|w|] of the ABSOLUTE values, so negative weights clamp to code 0.
    Returns (packed uint8 [N, K/2] on CPU, scales fp16 [N,1], zeros fp16 [N,1])."""
    mag = w.abs()
    hi = mag.max(dim=-1, keepdim=True)[0]
    lo = mag.min(dim=-1, keepdim=True)[0]
    scale = (hi - lo) / (levels - 1)
    zeros = (-lo / scale).round().to(torch.float16)
    codes = torch.clamp(torch.round(w / scale) + zeros, 0, levels - 1)
    return pack_i4(codes.to(torch.int8), sym=False).cpu(), scale.to(torch.float16), zeros


def sym_weight_quant(w, scales):
    """round(w / scales) packed as signed int4 (ref: qlinear4bit/nn/linear.py:72-73). Values
    outside [-8, 7] are an error there (pack_i4 asserts) and here."""
    return pack_i4((w / scales).round().to(torch.int8)).cpu()
