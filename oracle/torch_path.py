"""CPU restatement, in plain torch ops, of the reference's PyTorch fake-quant / integer-matmul path for
one symmetric W4A4 linear layer. TEST AND BENCHMARK INFRASTRUCTURE ONLY (the timed CPU baseline of
bench.py and its checker in tests/); nothing in the product imports it.

It follows, step by step:
  * qlinear4bit/nn/quantizer.py:10-16      per-token scale  (max|x| / 7).half() * clip
  * qlinear4bit/tools/quantization.py:28-31 sym_quant        clamp(round(x / scale), -(maxq+1), maxq), maxq = 7
  * qlinear4bit/tools/quantization.py:40-47 pack_i4          two's-complement nibbles, even column in the low nibble
  * qlinear4bit/tools/quantization.py:50-72 unpack_i4        back to int32 (both operands)
  * the integer contraction C = A_int @ B_int^T as a float matmul of the unpacked codes (exact: |C| < 2^24)
  * qlinear4bit/nn/linear.py:42-56 with src/kernels/quant.cu:79-80   x = (s_row * s_col) * half(C), fp16 ops
The clamp bound here is the Python path's 7 (the CUDA kernels of the reference clamp to 6, which is what the
C oracle and the GPU library reproduce); `qmax` selects either so that the two checkers can be compared.
"""
import torch


def per_token_sym_scales(x: torch.Tensor, clip: float = 1.0) -> torch.Tensor:
    return (torch.max(torch.abs(x), dim=-1)[0].unsqueeze(1) / 7).to(torch.float16) * clip


def sym_quant(x: torch.Tensor, scale: torch.Tensor, qmax: int = 7) -> torch.Tensor:
    return torch.clamp(torch.round(x / scale), -8, qmax)


def pack_i4(q: torch.Tensor) -> torch.Tensor:
    b = q.to(torch.int8)
    b = torch.where(b < 0, b + 16, b).to(torch.uint8)
    return b[:, 0::2] | (b[:, 1::2] << 4)


def unpack_i4(p: torch.Tensor) -> torch.Tensor:
    lo = (p & 0x0F).to(torch.int8)
    hi = ((p & 0xF0) >> 4).to(torch.int8)
    lo = torch.where(lo >= 8, lo - 16, lo)
    hi = torch.where(hi >= 8, hi - 16, hi)
    out = torch.empty((p.shape[0], p.shape[1] * 2), dtype=torch.int32)
    out[:, 0::2] = lo
    out[:, 1::2] = hi
    return out


def linear_w4a4_sym(x: torch.Tensor, w_codes_f32: torch.Tensor, w_scales: torch.Tensor, clip: float = 1.0, qmax: int = 7):
    """x fp16 [M, K]; w_codes_f32 = unpack_i4(packed weights).float() [N, K] (prepared once, like the packed weight
    buffer of a module); w_scales fp16 [N]. Returns (packed activation codes, per-token scales, int32 accumulators,
    fp16 output)."""
    s = per_token_sym_scales(x, clip)
    q = sym_quant(x.float(), s.float(), qmax)          # fp16 CPU division is emulated through fp32 by torch as well
    packed = pack_i4(q)
    a = unpack_i4(packed).float()
    acc = (a @ w_codes_f32.t()).to(torch.int32)
    out = (s * w_scales.view(1, -1)) * acc.to(torch.float16)
    return packed, s.view(-1), acc, out
