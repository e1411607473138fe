"""Generate the golden fixtures in this directory from the reference's own Python code.

Run once, in a container that has a checkout of the reference project:

    python tests/golden/make_golden.py --ref /path/to/DUQLinear4bitCUDA

The reference's quantizer modules (qlinear4bit/nn/quantizer.py) and its pure-torch tools
(qlinear4bit/tools/quantization.py) run on CPU; its compiled extension `qlinear4bit._CUDA`
cannot, so a stand-in module is injected whose quantize calls are the reference's own
fake-quant functions (tools/quantization.py: sym_quant, asym_quant, pack_i4). The scales
and zero-points are therefore exactly what the reference's modules compute; the codes are
what its torch path computes (symmetric clamp [-8, 7]; its CUDA kernel clamps to [-8, 6],
which the tests apply on top, see `qmax_sym` in the reference's include/common.h:54).
Integer accumulators come from `unpack_i4(A) @ unpack_i4(B).T`.

Outputs: golden_ref.npz (a few hundred KB). The tests read only that file.
"""
import argparse
import os
import sys
import types

import numpy as np
import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default="/root/reference")
    args = ap.parse_args()
    sys.path.insert(0, args.ref)

    import qlinear4bit.tools.quantization as rq  # reference, pure torch

    captured = {}
    stub = types.ModuleType("qlinear4bit._CUDA")

    def _sym_quant(x, scale):
        q, _ = rq.sym_quant(x, scale.view(-1, 1), torch.tensor(7))
        return rq.pack_i4(q.to(torch.int8))

    def _asym_quant(x, scale, zeros):
        q, _, _ = rq.asym_quant(x, scale.view(-1, 1), zeros.view(-1, 1), torch.tensor(15))
        return rq.pack_i4(q.to(torch.int8), sym=False)

    stub.sym_quant = _sym_quant
    stub.asym_quant = _asym_quant
    stub.get_dual_quant_col_k = lambda: 10
    sys.modules["qlinear4bit._CUDA"] = stub
    import qlinear4bit.nn.quantizer as rquant  # reference modules, now importable on CPU
    import qlinear4bit.nn.linear as rlin

    g = torch.Generator().manual_seed(1234)
    out = {}

    # 1. nibble packing
    v_s = torch.randint(-8, 8, (6, 64), generator=g, dtype=torch.int8)
    v_u = torch.randint(0, 16, (6, 64), generator=g, dtype=torch.int8)
    raw = torch.randint(0, 256, (5, 48), generator=g, dtype=torch.uint8)
    out["pack_in_s"] = v_s.numpy(); out["pack_out_s"] = rq.pack_i4(v_s).numpy()
    out["pack_in_u"] = v_u.numpy(); out["pack_out_u"] = rq.pack_i4(v_u, sym=False).numpy()
    out["unpack_in"] = raw.numpy(); out["unpack_out"] = rq.unpack_i4(raw).numpy()

    # 2. activations with outlier channels (shape of the benchmark inputs, small)
    def acts(shape, mean, outlier_frac, outlier_mul):
        x = torch.randn(shape, generator=g) + mean
        K = shape[-1]
        n_out = max(1, int(outlier_frac * K))
        ch = torch.randperm(K, generator=g)[:n_out]
        x[..., ch] *= outlier_mul
        return x.to(torch.float16)

    for name, clip in (("symq_a", 1.0), ("symq_b", 0.9)):
        x = acts((3, 5, 192), 0.0, 0.01, 20.0)
        if name == "symq_a":
            x[0, 0, :] = 0  # an all-zero token: scale 0, 0/0 -> NaN -> code 0
        p = rquant.SymQuantizer(clip)(x)
        out[name + "_x"] = x.numpy(); out[name + "_clip"] = np.float32(clip)
        out[name + "_scales"] = p.scales_x.numpy(); out[name + "_q7"] = p.quantized_x.numpy()

    x = acts((2, 7, 256), 0.1, 0.005, 30.0)
    p = rquant.AsymQuantizer()(x)
    out["asymq_x"] = x.numpy(); out["asymq_scales"] = p.scales_x.numpy()
    out["asymq_zeros"] = p.zeros_x.numpy(); out["asymq_q"] = p.quantized_x.numpy()

    # 3. integer accumulators
    A = torch.randint(0, 256, (16, 96), generator=g, dtype=torch.uint8)
    B = torch.randint(0, 256, (40, 96), generator=g, dtype=torch.uint8)
    out["mm_A"] = A.numpy(); out["mm_B"] = B.numpy()
    out["mm_C"] = (rq.unpack_i4(A).to(torch.int32) @ rq.unpack_i4(B).to(torch.int32).T).numpy()

    # 4. asymmetric weight preparation (runs on CPU as shipped): Linear4bitASQ.from_linear and
    #    LinearQuant4bitDUASQ.from_linear
    lin = torch.nn.Linear(128, 24, bias=True)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(24, 128, generator=g) * 0.02)
        lin.bias.copy_(torch.randn(24, generator=g))
    lin = lin.half()
    m = rlin.Linear4bitASQ.from_linear(lin, require_quantizer=True)
    out["asq_w"] = lin.weight.data.numpy(); out["asq_b"] = lin.bias.data.numpy()
    out["asq_weight"] = m.weight.numpy(); out["asq_scales"] = m.weight_scales.numpy()
    out["asq_zeros"] = m.weight_zeros.numpy(); out["asq_bias"] = m.bias.detach().numpy()
    m2 = rlin.LinearQuant4bitDUASQ.from_linear(lin, require_quantizer=True)
    out["duasq_weight"] = m2.weight.numpy()
    for k in ("weight_scales_1", "weight_zeros_1", "weight_scales_2", "weight_zeros_2"):
        out["duasq_" + k] = getattr(m2, k).numpy()

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_ref.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main()
