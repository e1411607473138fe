// libtorch (C++) module API of the 4-bit linear layers: class names, public members,
// constructor and method signatures of DUQLinear4bitCUDA's include/linear.h (lines 31-60
// there; src/module/linear.cu:87-281), header-only over the C ABI. forward() is ONE fused
// kernel (GEMM + dequant + bias) whose output equals the reference's
// matmul_host_4bit -> sym(_dual)_dequant -> `+ bias` sequence bit for bit.
// The plain fp `Linear` / `LinearPlain<T>` helpers of the reference header are not part of
// the W4A4 path and are not provided.
#pragma once
#include "quant_tensor.h"

namespace duq4_torch {
inline torch::Tensor fused_forward(int mode, const PackedQuantizedTensor &in, const torch::Tensor &weight,
                                   const torch::Tensor &s1, const torch::Tensor *s2, const torch::Tensor &bias) {
    const torch::Tensor &x = in.quantized_x;
    TORCH_CHECK(x.size(-1) % 32 == 0, "packed K must be a multiple of 32");
    need_cuda_contig("Linear4bit::forward", {&x, &weight});
    c10::cuda::CUDAGuard guard(x.device());
    auto A = x.view({-1, x.size(-1)});
    const uint32_t M = A.size(0), N = weight.size(0), K = A.size(1) * 2;
    auto srow = in.scale.contiguous().view(-1);
    TORCH_CHECK(srow.size(0) == M && srow.scalar_type() == torch::kFloat16, "per-token scales: fp16 [M]");
    auto out = torch::empty({M, N}, torch::dtype(torch::kFloat16).device(x.device()));
    duq4_epilogue e = {};
    e.mode = mode;
    e.scale_row = srow.data_ptr();
    e.scale_col_1 = s1.data_ptr();
    if (s2) e.scale_col_2 = s2->data_ptr();
    if (bias.defined()) e.bias = bias.data_ptr();
    ok("Linear4bit::forward", duq4_linear_w4a4(A.data_ptr<uint8_t>(), weight.data_ptr<uint8_t>(), M, N, K, &e, out.data_ptr(),
                                              nullptr, stream()));
    std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end());
    shape.back() = N;
    return out.view(shape);
}
inline void init_buffers(torch::Tensor &weight, uint32_t input_dim, uint32_t output_dim) {
    weight = torch::randint(1, 7, {output_dim, input_dim / 2}, torch::kUInt8).to(torch::kCUDA);
    weight.set_requires_grad(false);
}
}  // namespace duq4_torch

// include/linear.h:31-45 of the reference
class Linear4bit : public torch::nn::Module {
public:
    torch::Tensor weight;        // uint8 [out, in/2]
    torch::Tensor weight_scale;  // fp16 [out, 1]
    torch::Tensor bias;          // [out], undefined when the layer has none

    Linear4bit(uint32_t input_dim, uint32_t output_dim, bool bias, torch::Dtype dtype = torch::kFloat16) {
        duq4_torch::init_buffers(weight, input_dim, output_dim);
        weight_scale = torch::zeros({output_dim, 1}, torch::dtype(torch::kFloat16).device(torch::kCUDA));
        if (bias) this->bias = torch::zeros({output_dim}, torch::dtype(dtype).device(torch::kCUDA));
    }
    torch::Tensor forward(PackedQuantizedTensor input) {
        return duq4_torch::fused_forward(DUQ4_MODE_SYM, input, weight, weight_scale, nullptr, bias);
    }
    // src/module/linear.cu:161-176: round(W / scales) packed as int4 (no clamp: out-of-range values are an error)
    static Linear4bit from_float(torch::nn::Linear &linear, torch::Tensor weight_scales) {
        auto w = linear->weight.data().to(torch::kCUDA);
        Linear4bit m(w.size(-1), w.size(0), linear->bias.defined(), torch::kFloat16);
        m.weight_scale.copy_(weight_scales.to(torch::kCUDA, w.scalar_type()));
        m.weight.copy_(pack_i4(torch::round(w / m.weight_scale).to(torch::kInt8)));
        if (linear->bias.defined()) m.bias.copy_(linear->bias.data());
        return m;
    }
};

// include/linear.h:47-60: dual-uniform symmetric weights (columns < QUANT_COL_K use set 1)
class Linear4bitDUQ : public torch::nn::Module {
public:
    torch::Tensor weight;
    torch::Tensor weight_scale_1;
    torch::Tensor weight_scale_2;
    torch::Tensor bias;

    Linear4bitDUQ(uint32_t input_dim, uint32_t output_dim, bool bias, torch::Dtype dtype = torch::kFloat16) {
        duq4_torch::init_buffers(weight, input_dim, output_dim);
        weight_scale_1 = torch::zeros({output_dim, 1}, torch::dtype(torch::kFloat16).device(torch::kCUDA));
        weight_scale_2 = torch::zeros({output_dim, 1}, torch::dtype(torch::kFloat16).device(torch::kCUDA));
        if (bias) this->bias = torch::zeros({output_dim}, torch::dtype(dtype).device(torch::kCUDA));
    }
    torch::Tensor forward(PackedQuantizedTensor input) {
        return duq4_torch::fused_forward(DUQ4_MODE_SYM_DUAL, input, weight, weight_scale_1, &weight_scale_2, bias);
    }
    // src/module/linear.cu:254-281
    static Linear4bitDUQ from_float(torch::nn::Linear &linear, torch::Tensor weight_scales_1, torch::Tensor weight_scales_2) {
        using namespace torch::indexing;
        auto w = linear->weight.data().to(torch::kCUDA);
        Linear4bitDUQ m(w.size(-1), w.size(0), linear->bias.defined(), torch::kFloat16);
        m.weight_scale_1.copy_(weight_scales_1.to(torch::kCUDA, w.scalar_type()));
        m.weight_scale_2.copy_(weight_scales_2.to(torch::kCUDA, w.scalar_type()));
        const int64_t split = duq4_dual_quant_col_k();
        auto left = torch::round(w.index({Slice(), Slice(None, split)}) / m.weight_scale_1);
        auto right = torch::round(w.index({Slice(), Slice(split, None)}) / m.weight_scale_2);
        m.weight.copy_(pack_i4(torch::cat({left, right}, -1).to(torch::kInt8)));
        if (linear->bias.defined()) m.bias.copy_(linear->bias.data());
        return m;
    }
};
