"""4-bit linear modules with the class names, constructor arguments, buffer names/shapes/dtypes
and conversion helpers of `qlinear4bit/nn/linear.py` of the reference, so that a reference
`state_dict` loads unchanged. The forward of every 4-bit variant is one fused kernel (GEMM +
dequant + bias) whose results equal the reference's matmul -> *_dequant -> `+ bias` sequence.
"""
import torch

from ..tools import quantization as qz
from ..tools import tensor_utils
from ..tools.tensor_utils import PackedQuantizedTensor
from .quantizer import AsymQuantizer, AsymQuantizer8bit


class _PackedLinearBase(torch.nn.Module):
    """Shared plumbing: the packed weight buffer (uint8 [out, in/2], initialised like the
    reference with randint(1,7)), optional bias, and the per-channel vectors a variant names."""
    _mode = None
    _vectors = ()          # buffer names, each [out_features, 1]
    _vector_dtype = None   # None: torch default (the symmetric variants of the reference)

    def _setup(self, in_features, out_features, bias, bias_dtype):
        self.in_features = in_features
        self.out_features = out_features
        for name in self._vectors:
            kw = {} if self._vector_dtype is None else {"dtype": self._vector_dtype}
            self.register_buffer(name, torch.zeros((out_features, 1), requires_grad=False, **kw))
        self.register_buffer("weight", torch.randint(1, 7, (out_features, in_features // 2), dtype=torch.uint8,
                                                     requires_grad=False))
        if bias:
            self.register_buffer("bias", torch.zeros((out_features,), dtype=bias_dtype))
        else:
            self.bias = None

    def _vec(self, name):
        """Per-channel vector `name` as the kernels read it: fp16. The symmetric variants register their
        scales with torch's default dtype (fp32), as the reference does, so a module that was built
        directly and filled by load_state_dict holds fp32 scales; those are converted once and the
        fp16 copy is kept until the buffer changes."""
        t = getattr(self, name, None) if name in self._vectors else None
        if t is None or t.dtype == torch.float16:
            return t
        cache = self.__dict__.setdefault("_f16_vectors", {})
        key = (t.data_ptr(), t._version, t.device)
        hit = cache.get(name)
        if hit is None or hit[0] != key:
            hit = cache[name] = (key, t.to(torch.float16))
        return hit[1]

    def _bias_f16(self):
        b = self.bias
        if b is None or b.dtype == torch.float16:
            return b
        raise TypeError(f"{type(self).__name__}: bias must be float16 for the fused kernel, got {b.dtype}")

    # Weight pre-layout cache: forwards that see at least this many tokens run on an int8 copy of the packed
    # weights in the tensor-core kernel's operand layout (no in-kernel unpack: 3.7 vs 3.1 POPS on the 8192 -> 28672
    # layer at 4096 tokens). The copy is derived lazily from `weight` on first use (0.1 ms for that layer), costs
    # K bytes per output channel beside the K/2 of the packed tensor, is rebuilt when `weight` changes and is NOT part
    # of the state_dict (the packed tensor stays the format of record). Set `weight_prelayout = False` on a module
    # (or the class) to keep only the packed weights.
    weight_prelayout = True
    prelayout_min_tokens = 256

    def _prelaid_weight(self, tokens):
        from .. import _CUDA as ops
        w = self.weight
        if not self.weight_prelayout or tokens < self.prelayout_min_tokens or not w.is_cuda or self.in_features % 128 != 0:
            return None
        key = (w.data_ptr(), w._version, w.device)
        hit = self.__dict__.get("_prelaid")
        if hit is None or hit[0] != key:
            hit = self.__dict__["_prelaid"] = (key, ops.weight_prelayout_i8(w))
        return hit[1]

    def _fused_fp16(self, x):
        """fp16 input of a module that owns its quantizer: quantize + GEMM + dequant in one library
        call; the activations never exist as packed codes in HBM."""
        from .. import _CUDA as ops
        if not x.is_contiguous():
            x = x.contiguous()
        flat = lambda t: None if t is None else t.reshape(-1)
        first = lambda a, b: self._vec(a) if a in self._vectors else self._vec(b)
        y = ops.linear_w4a4_from_fp16(self._mode, x.view(-1, x.shape[-1]), self.weight,
                                      flat(first("weight_scales", "weight_scales_1")), flat(first("weight_zeros", "weight_zeros_1")),
                                      flat(self._vec("weight_scales_2")), flat(self._vec("weight_zeros_2")), self._bias_f16(),
                                      W_prelaid=self._prelaid_weight(x.numel() // x.shape[-1]))
        return y.view(*x.shape[:-1], -1)

    def _fused(self, packed):
        if type(packed) is not PackedQuantizedTensor:
            raise AssertionError("Input should be quantized tensor, or require_quantizer should be passed as initial argument")
        return tensor_utils.linear(self._mode, packed, self.weight,
                                   self._vec("weight_scales") if "weight_scales" in self._vectors else self._vec("weight_scales_1"),
                                   self._vec("weight_zeros") if "weight_zeros" in self._vectors else self._vec("weight_zeros_1"),
                                   self._vec("weight_scales_2"), self._vec("weight_zeros_2"), self._bias_f16())


class Linear4bitSQ(_PackedLinearBase):
    """Symmetric W4A4 linear (ref: nn/linear.py:24-78). forward takes a PackedQuantizedTensor."""
    _mode = "sym"
    _vectors = ("weight_scales",)

    def __init__(self, in_features, out_features, bias=False, dtype=torch.float16):
        super().__init__()
        self._setup(in_features, out_features, bias, dtype)

    def forward(self, x):
        return self._fused(x)

    @staticmethod
    def from_float(module: torch.nn.Linear, weight_scales=None):
        """ref: nn/linear.py:58-78. `weight_scales` [out,1]; round(W/scales) must already lie in
        [-8,7] (no clamp, as in the reference: packing asserts the range)."""
        w = module.weight.data
        new = Linear4bitSQ(module.in_features, module.out_features, bias=module.bias is not None, dtype=w.dtype).to(w.dtype)
        if weight_scales is not None:
            if tuple(weight_scales.shape) != (module.out_features, 1):
                raise AssertionError("weight_scales should have shape (out_features, 1)")
            w = w.cuda()
            new.weight_scales.copy_(weight_scales.to(w.dtype))
            new.weight.copy_(qz.sym_weight_quant(w, weight_scales.cuda()))
            if module.bias is not None:
                new.bias.copy_(module.bias.detach())
        return new


class Linear4bitDUSQ(_PackedLinearBase):
    """Symmetric dual-uniform W4A4 linear (ref: nn/linear.py:147-206): input columns below
    get_dual_quant_col() were quantized with weight_scales_1, the rest with weight_scales_2.
    The dequant picks the set by OUTPUT column, as the reference kernel does."""
    _mode = "sym_dual"
    _vectors = ("weight_scales_1", "weight_scales_2")

    def __init__(self, in_features, out_features, bias=False, dtype=torch.float16):
        super().__init__()
        self._setup(in_features, out_features, bias, dtype)

    def forward(self, x):
        return self._fused(x)

    @staticmethod
    def from_float(module: torch.nn.Linear, weight_scales_1=None, weight_scales_2=None):
        """ref: nn/linear.py:178-206."""
        w = module.weight.data
        new = Linear4bitDUSQ(module.in_features, module.out_features, bias=module.bias is not None, dtype=w.dtype).to(w.dtype)
        if weight_scales_1 is not None and weight_scales_2 is not None:
            for name, s in (("weight_scales_1", weight_scales_1), ("weight_scales_2", weight_scales_2)):
                if tuple(s.shape) != (module.out_features, 1):
                    raise AssertionError(f"{name} should have shape (out_features, 1)")
            w = w.cuda()
            new.weight_scales_1.copy_(weight_scales_1.to(w.dtype))
            new.weight_scales_2.copy_(weight_scales_2.to(w.dtype))
            split = tensor_utils.get_dual_quant_col()
            codes = torch.cat([(w[:, :split] / weight_scales_1.cuda()).round(),
                               (w[:, split:] / weight_scales_2.cuda()).round()], dim=-1)
            new.weight.copy_(qz.pack_i4(codes.to(torch.int8)).cpu())
            if module.bias is not None:
                new.bias.copy_(module.bias.detach())
        return new


class Linear4bitASQ(_PackedLinearBase):
    """Asymmetric W4A4 linear (ref: nn/linear.py:80-145). With require_quantizer=True the module
    quantizes fp16 input itself (AsymQuantizer)."""
    _mode = "asym"
    _vectors = ("weight_scales", "weight_zeros")
    _vector_dtype = torch.float16

    def __init__(self, in_features, out_features, bias=False, require_quantizer=True):
        super().__init__()
        self.require_quantizer = require_quantizer
        self._setup(in_features, out_features, bias, torch.float16)
        if require_quantizer:
            self.quantizer = AsymQuantizer()

    def forward(self, x):
        if self.require_quantizer:
            if isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.float16 and x.shape[-1] % 64 == 0:
                return self._fused_fp16(x)   # same result as self.quantizer(x) followed by the fused linear
            x = self.quantizer(x)
        return self._fused(x)

    @classmethod
    def from_linear(cls, module: torch.nn.Linear, require_quantizer: bool = True):
        """ref: nn/linear.py:117-145 (range taken over |w|, so negative weights clamp to code 0)."""
        new = cls(module.in_features, module.out_features, bias=module.bias is not None, require_quantizer=require_quantizer)
        packed, scale, zeros = qz.asym_weight_quant(module.weight.data)
        new.weight.copy_(packed)
        new.weight_scales.copy_(scale)
        new.weight_zeros.copy_(zeros)
        if module.bias is not None:
            new.bias.copy_(module.bias.detach())
        return new


class LinearQuant4bitDUASQ(_PackedLinearBase):
    """Asymmetric dual-uniform W4A4 linear (ref: nn/linear.py:209-297)."""
    _mode = "asym_dual"
    _vectors = ("weight_scales_1", "weight_zeros_1", "weight_scales_2", "weight_zeros_2")
    _vector_dtype = torch.float16

    def __init__(self, in_features, out_features, bias=False, require_quantizer=True):
        super().__init__()
        self.require_quantizer = require_quantizer
        self._setup(in_features, out_features, bias, torch.float16)
        if require_quantizer:
            self.quantizer = AsymQuantizer()

    def forward(self, x):
        if self.require_quantizer:
            if isinstance(x, torch.Tensor) and x.is_cuda and x.dtype == torch.float16 and x.shape[-1] % 64 == 0:
                return self._fused_fp16(x)   # same result as self.quantizer(x) followed by the fused linear
            x = self.quantizer(x)
        return self._fused(x)

    @classmethod
    def from_linear(cls, module: torch.nn.Linear, require_quantizer=True):
        """ref: nn/linear.py:252-297: the two column ranges are quantized independently."""
        new = cls(module.in_features, module.out_features, bias=module.bias is not None, require_quantizer=require_quantizer)
        w = module.weight.data
        split = tensor_utils.get_dual_quant_col()
        halves = []
        for idx, part in ((1, w[:, :split]), (2, w[:, split:])):
            mag = part.abs()
            hi = mag.max(dim=-1, keepdim=True)[0]
            lo = mag.min(dim=-1, keepdim=True)[0]
            scale = (hi - lo) / 15
            zeros = (-lo / scale).round().to(torch.float16)
            halves.append(torch.clamp(torch.round(part / scale) + zeros, 0, 15))
            getattr(new, f"weight_scales_{idx}").copy_(scale.to(torch.float16))
            getattr(new, f"weight_zeros_{idx}").copy_(zeros)
        new.weight.copy_(qz.pack_i4(torch.cat(halves, dim=-1).to(torch.int8), sym=False).cpu())
        if module.bias is not None:
            new.bias.copy_(module.bias.detach())
        return new


class LinearQuant8bitASQ(torch.nn.Module):
    """8-bit asymmetric linear of the reference's side path (ref: nn/linear.py:300-368): int8
    weights [out,in], fp32 scales/zeros, int8 tensor-core GEMM + fp32 dequant."""

    def __init__(self, in_features, out_features, bias=False, require_quantizer=True):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.require_quantizer = require_quantizer
        self.register_buffer("weight_scales", torch.zeros((out_features, 1), requires_grad=False, dtype=torch.float32))
        self.register_buffer("weight_zeros", torch.zeros((out_features, 1), requires_grad=False, dtype=torch.float32))
        self.register_buffer("weight", torch.randint(1, 7, (out_features, in_features), dtype=torch.int8, requires_grad=False))
        if bias:
            self.register_buffer("bias", torch.zeros((out_features,), dtype=torch.float32))
        else:
            self.bias = None
        if require_quantizer:
            self.quantizer = AsymQuantizer8bit()

    def forward(self, x):
        if self.require_quantizer:
            x = self.quantizer(x)
        if type(x) is not PackedQuantizedTensor:
            raise AssertionError("Input should be quantized tensor, or require_quantizer should be passed as initial argument")
        acc = tensor_utils.matmul_8bit(x.quantized_x, self.weight)
        y = tensor_utils.asym_dequant_hprec(acc, x.scales_x, x.zeros_x, self.weight_scales, self.weight_zeros)
        return y if self.bias is None else y + self.bias

    @classmethod
    def from_linear(cls, module: torch.nn.Linear, require_quantizer=True):
        new = cls(module.in_features, module.out_features, bias=module.bias is not None, require_quantizer=require_quantizer)
        w = module.weight.data
        mag = w.abs()
        hi = mag.max(dim=-1, keepdim=True)[0]
        lo = mag.min(dim=-1, keepdim=True)[0]
        scale = (hi - lo) / 127
        zeros = (-lo / scale).round().to(torch.float32)
        codes = torch.clamp(torch.round(w / scale) + zeros, 0, 127)
        new.weight.copy_(codes.to(torch.int8).cpu())
        new.weight_scales.copy_(scale.to(torch.float32))
        new.weight_zeros.copy_(zeros)
        if module.bias is not None:
            new.bias.copy_(module.bias.detach())
        return new
