// libtorch (C++) tensor-level API of the 4-bit path: the class and function names, members and
// signatures of DUQLinear4bitCUDA's include/quant_tensor.h (lines 11-90 there), implemented
// header-only over the C ABI in duq4.h. Launches go to torch's CURRENT CUDA stream.
//
// Quantizer4bit::forward is one fused kernel (row abs-max, scale, codes) whose scales and codes
// equal the reference's abs/max/div/mul chain followed by sym_quant
// (src/module/quant_tensor.cu:151-161 there).
#pragma once
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/torch.h>

#include "common.h"
#include "duq4.h"

namespace duq4_torch {
inline void ok(const char *fn, int status) { TORCH_CHECK(status == 0, fn, ": ", duq4_error_string(status)); }
inline void *stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline void need_cuda_contig(const char *fn, std::initializer_list<const torch::Tensor *> ts) {
    const torch::Tensor *first = nullptr;
    for (const torch::Tensor *t : ts) {
        TORCH_CHECK(t->is_cuda(), fn, ": expected a CUDA tensor");
        TORCH_CHECK(t->is_contiguous(), fn, ": expected a contiguous tensor");
        if (!first) first = t;
        TORCH_CHECK(t->device() == first->device(), fn, ": tensors must be on the same GPU");
    }
}
}  // namespace duq4_torch

// include/quant_tensor.h:11-25 of the reference
class PackedQuantizedTensor {
public:
    torch::Tensor quantized_x;
    torch::Tensor scale;
    PackedQuantizedTensor(torch::Tensor quantized_x, torch::Tensor scale) : quantized_x(quantized_x), scale(scale) {}
    torch::IntArrayRef sizes() const { return quantized_x.sizes(); }
    torch::Device device() const { return quantized_x.device(); }
};

// :28-44
class PackedDoubleQuantizedTensor {
public:
    torch::Tensor quantized_x;
    torch::Tensor scale_1;
    torch::Tensor scale_2;
    PackedDoubleQuantizedTensor(torch::Tensor quantized_x, torch::Tensor scale_1, torch::Tensor scale_2)
        : quantized_x(quantized_x), scale_1(scale_1), scale_2(scale_2) {}
    torch::IntArrayRef sizes() const { return quantized_x.sizes(); }
    torch::Device device() const { return quantized_x.device(); }
};

// :46 (src/module/quant_tensor.cu:11-29): x fp16 [rows, cols], scale fp16 [rows] -> uint8 [rows, ceil(cols/2)]
inline torch::Tensor sym_quant(const torch::Tensor &x, const torch::Tensor &scale) {
    duq4_torch::need_cuda_contig("sym_quant", {&x, &scale});
    TORCH_CHECK(scale.size(0) == x.size(0), "sym_quant: scale.size(0) must equal x.size(0)");
    c10::cuda::CUDAGuard guard(x.device());
    const uint32_t rows = x.size(0), cols = x.size(1), cd = (cols + 1) / 2;
    auto q = torch::empty({rows, cd}, torch::dtype(torch::kUInt8).device(x.device()));
    duq4_torch::ok("sym_quant", duq4_sym_quant(x.data_ptr(), scale.data_ptr(), rows, cols, cd, q.data_ptr<uint8_t>(), duq4_torch::stream()));
    return q;
}

// :48 (src/module/quant_tensor.cu:31-57)
inline torch::Tensor sym_dual_quant(const torch::Tensor &x, const torch::Tensor &scale_1, const torch::Tensor &scale_2) {
    duq4_torch::need_cuda_contig("sym_dual_quant", {&x, &scale_1, &scale_2});
    TORCH_CHECK(scale_1.size(0) == x.size(0) && scale_2.size(0) == x.size(0), "sym_dual_quant: scale sizes");
    c10::cuda::CUDAGuard guard(x.device());
    const uint32_t rows = x.size(0), cols = x.size(1), cd = (cols + 1) / 2;
    auto q = torch::empty({rows, cd}, torch::dtype(torch::kUInt8).device(x.device()));
    duq4_torch::ok("sym_dual_quant", duq4_sym_dual_quant(x.data_ptr(), scale_1.data_ptr(), scale_2.data_ptr(), rows, cols, cd,
                                                        q.data_ptr<uint8_t>(), duq4_torch::stream()));
    return q;
}

// :50-53 (src/module/quant_tensor.cu:59-99); bits must be 32
inline torch::Tensor sym_dequant(const torch::Tensor &q, const torch::Tensor &scale_row, const torch::Tensor &scale_col,
                                 const int bits) {
    duq4_torch::need_cuda_contig("sym_dequant", {&q, &scale_row, &scale_col});
    TORCH_CHECK(bits == 32, "Unsupported data type");
    const uint32_t rows = q.size(0), cols = q.size(1);
    TORCH_CHECK(scale_row.size(0) == rows && scale_col.size(0) == cols, "sym_dequant: scale sizes");
    c10::cuda::CUDAGuard guard(q.device());
    auto x = torch::empty({rows, cols}, torch::dtype(torch::kFloat16).device(q.device()));
    duq4_torch::ok("sym_dequant", duq4_sym_dequant(q.data_ptr<int32_t>(), scale_row.data_ptr(), scale_col.data_ptr(), rows, cols,
                                                  x.data_ptr(), duq4_torch::stream()));
    return x;
}

// :55-59 (src/module/quant_tensor.cu:101-148)
inline torch::Tensor sym_dual_dequant(const torch::Tensor &q, const torch::Tensor &scale_row, const torch::Tensor &scale_col_1,
                                      const torch::Tensor &scale_col_2, const int bits) {
    duq4_torch::need_cuda_contig("sym_dual_dequant", {&q, &scale_row, &scale_col_1, &scale_col_2});
    TORCH_CHECK(bits == 32, "Unsupported data type");
    const uint32_t rows = q.size(0), cols = q.size(1);
    c10::cuda::CUDAGuard guard(q.device());
    auto x = torch::empty({rows, cols}, torch::dtype(torch::kFloat16).device(q.device()));
    duq4_torch::ok("sym_dual_dequant", duq4_sym_dual_dequant(q.data_ptr<int32_t>(), scale_row.data_ptr(), scale_col_1.data_ptr(),
                                                            scale_col_2.data_ptr(), rows, cols, x.data_ptr(), duq4_torch::stream()));
    return x;
}

// :61-67 (src/module/quant_tensor.cu:151-161)
class Quantizer4bit : public torch::nn::Module {
public:
    float input_clip_ratio;
    Quantizer4bit(float input_clip_ratio) : input_clip_ratio(input_clip_ratio) {}
    PackedQuantizedTensor forward(torch::Tensor x) {
        x = x.contiguous();
        TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kFloat16, "Quantizer4bit: expected a CUDA fp16 tensor");
        c10::cuda::CUDAGuard guard(x.device());
        auto x2 = x.view({-1, x.size(-1)});
        const uint32_t rows = x2.size(0), cols = x2.size(1), cd = (cols + 1) / 2;
        auto q = torch::empty({rows, cd}, torch::dtype(torch::kUInt8).device(x.device()));
        auto s = torch::empty({rows}, torch::dtype(torch::kFloat16).device(x.device()));
        duq4_torch::ok("Quantizer4bit", duq4_quantize_sym_fused(x2.data_ptr(), rows, cols, input_clip_ratio, q.data_ptr<uint8_t>(),
                                                               s.data_ptr(), duq4_torch::stream()));
        std::vector<int64_t> qshape(x.sizes().begin(), x.sizes().end());
        qshape.back() = cd;
        // the reference's scales are max(|x|, -1).unsqueeze(1)/7: [B,1,S] for x [B,S,K], [R,1] for x [R,K]
        std::vector<int64_t> sshape(x.sizes().begin(), x.sizes().end() - 1);
        sshape.insert(sshape.begin() + (sshape.empty() ? 0 : 1), 1);
        return PackedQuantizedTensor(q.view(qshape), s.view(sshape));
    }
};

// :69-78
class DeQuantizer4bit : torch::nn::Module {
public:
    uint32_t bits = 32;
    DeQuantizer4bit() {}
    DeQuantizer4bit(uint32_t bits) : bits(bits) {}
    torch::Tensor forward(torch::Tensor &x, torch::Tensor &scale_x, torch::Tensor &weight_scale) {
        auto x2 = x.view({-1, x.size(-1)});
        auto y = sym_dequant(x2, scale_x.view(-1), weight_scale.view(-1), (int)bits);
        std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end());
        return y.view(shape);
    }
};

// :80-88: declared empty in the reference as well
class DoubleQuantizer4bit : public torch::nn::Module {};
class DoubleDeQuantizer4bit : public torch::nn::Module {};

// :90 (src/module/quant_tensor.cu:197-206): signed int8 values in [-8,7], [.., K] -> uint8 [.., K/2]
inline torch::Tensor pack_i4(torch::Tensor q) {
    TORCH_CHECK(q.scalar_type() == torch::kInt8, "pack_i4: expected int8");
    TORCH_CHECK(q.ge(-8).logical_and(q.le(7)).all().item<bool>(), "pack_i4: values outside the int4 range");
    auto nib = q.to(torch::kInt16).bitwise_and(0xF).to(torch::kUInt8);
    using namespace torch::indexing;
    return nib.index({"...", Slice(0, None, 2)}).bitwise_or(nib.index({"...", Slice(1, None, 2)}).bitwise_left_shift(4));
}
