// pybind11 module `_CUDA`: the tensor-level operator module of the package, with the function names,
// keyword names, argument checks and return conventions of the reference's compiled extension
// `qlinear4bit._CUDA` (src/export/bindings.cpp:768-932 there; wrappers :10-467), implemented over the C ABI
// of libduq4.so (include/duq4.h). Differences from the reference, all deliberate:
//   * every launch goes to torch's CURRENT stream of the input's device under a CUDAGuard (the reference
//     launches on the legacy default stream whatever the current stream is);
//   * dtypes are checked (the reference reinterprets whatever it is given as fp16 / int32);
//   * batched_matmul works (the reference hands host pointer arrays to the device, bindings.cpp:59-82);
//   * asym_dual_quant returns its tensor (the reference's wrapper falls off the end, bindings.cpp:393-421);
//   * functions the reference does not have are marked "(new)": fused quantizers and the fused linear layer.
// The six FlashInfer KV-cache names of the reference module are outside the W4A4 linear path and absent.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <mutex>
#include <optional>
#include <string>
#include <unordered_map>

#include "../../include/duq4.h"

namespace {

using torch::Tensor;
using OptTensor = std::optional<Tensor>;

struct Arg {
    const Tensor *t;
    const char *name;
    torch::ScalarType dtype = torch::ScalarType::Undefined;   // required element type, when the operator fixes one
};

// What the reference's checkAllContiguous + checkDeviceType + checkAllSameGPU do, on defined tensors only, after the
// element types the operator fixes (a kernel reads every vector as the type it was written for: an fp32 scale
// vector handed over as fp16 would give wrong numbers, not an error). Types are checked first, so a wrong type is
// reported on any machine.
void check_tensors(const char *fn, std::initializer_list<Arg> args) {
    for (const Arg &a : args)
        if (a.t && a.t->defined() && a.dtype != torch::ScalarType::Undefined)
            TORCH_CHECK(a.t->scalar_type() == a.dtype, fn, ": expected ", a.name, " to have dtype ", c10::toString(a.dtype), ", got ",
                        c10::toString(a.t->scalar_type()));
    const Tensor *first = nullptr;
    for (const Arg &a : args) {
        if (!a.t || !a.t->defined()) continue;
        TORCH_CHECK(a.t->is_cuda(), fn, ": expected ", a.name, " to be a CUDA tensor");
        TORCH_CHECK(a.t->is_contiguous(), fn, ": expected ", a.name, " to be contiguous");
        if (!first) first = a.t;
        TORCH_CHECK(a.t->device() == first->device(), fn, ": expected ", a.name, " to be on the same GPU as the first argument");
    }
}
void check_dtype(const char *fn, const Tensor &t, const char *name, torch::ScalarType want) {
    TORCH_CHECK(t.scalar_type() == want, fn, ": expected ", name, " to have dtype ", c10::toString(want), ", got ",
                c10::toString(t.scalar_type()));
}
void check_size(const char *fn, const Tensor &t, const char *name, int64_t dim, int64_t n) {
    TORCH_CHECK(t.dim() > dim && t.size(dim) == n, fn, ": expected ", name, ".size(", dim, ") == ", n);
}
void check_bits(int bits) { TORCH_CHECK(bits == 32, "Unsupported data type"); }
void ok(const char *fn, int status) { TORCH_CHECK(status == 0, fn, " failed with status ", status, ": ", duq4_error_string(status)); }

const Tensor *opt(const OptTensor &o) { return o.has_value() && o->defined() ? &*o : nullptr; }
const void *ptr(const OptTensor &o) { return opt(o) ? (*o).data_ptr() : nullptr; }

// Device guard + the current stream of that device, for the duration of one call.
struct Launch {
    c10::cuda::CUDAGuard guard;
    void *stream;
    explicit Launch(const Tensor &t) : guard(t.device()), stream(at::cuda::getCurrentCUDAStream().stream()) {}
};

int mode_of(const char *fn, const std::string &m) {
    if (m == "sym") return DUQ4_MODE_SYM;
    if (m == "sym_dual") return DUQ4_MODE_SYM_DUAL;
    if (m == "asym") return DUQ4_MODE_ASYM;
    if (m == "asym_dual") return DUQ4_MODE_ASYM_DUAL;
    TORCH_CHECK(false, fn, ": unknown mode '", m, "' (sym, sym_dual, asym, asym_dual)");
    return 0;
}

Tensor empty_like_dev(const Tensor &ref, at::IntArrayRef shape, torch::ScalarType dt) {
    return torch::empty(shape, torch::dtype(dt).device(ref.device()));
}

// ---- GEMMs --------------------------------------------------------------------------------------
// ref: bindings.cpp:10-26
Tensor matmul(const Tensor &A, const Tensor &B) {
    check_tensors("matmul", {{&A, "A"}, {&B, "B"}});
    check_dtype("matmul", A, "A", torch::kUInt8);
    check_dtype("matmul", B, "B", torch::kUInt8);
    const uint32_t M = A.size(0), N = B.size(0), K = A.size(1) * 2;
    TORCH_CHECK(B.size(1) == A.size(1), "matmul: A and B disagree on K");
    auto C = empty_like_dev(A, {M, N}, torch::kInt32);
    Launch l(A);
    ok("matmul", duq4_matmul_4bit(A.data_ptr<uint8_t>(), B.data_ptr<uint8_t>(), M, N, K, C.data_ptr<int32_t>(), l.stream));
    return C;
}
// ref: bindings.cpp:28-44
Tensor matmul_8bit(const Tensor &A, const Tensor &B) {
    check_tensors("matmul_8bit", {{&A, "A"}, {&B, "B"}});
    check_dtype("matmul_8bit", A, "A", torch::kInt8);
    check_dtype("matmul_8bit", B, "B", torch::kInt8);
    const uint32_t M = A.size(0), N = B.size(0), K = A.size(1);
    TORCH_CHECK(B.size(1) == A.size(1), "matmul_8bit: A and B disagree on K");
    auto C = empty_like_dev(A, {M, N}, torch::kInt32);
    Launch l(A);
    ok("matmul_8bit", duq4_matmul_8bit(A.data_ptr<int8_t>(), B.data_ptr<int8_t>(), M, N, K, C.data_ptr<int32_t>(), l.stream));
    return C;
}
// ref: bindings.cpp:46-84. A [b,M,K/2], B [b,N,K/2] -> int32 [b,M,N].
Tensor batched_matmul(const Tensor &A, const Tensor &B) {
    check_tensors("batched_matmul", {{&A, "A"}, {&B, "B"}});
    check_dtype("batched_matmul", A, "A", torch::kUInt8);
    check_dtype("batched_matmul", B, "B", torch::kUInt8);
    TORCH_CHECK(A.dim() == 3 && B.dim() == 3, "batched_matmul: expected 3-D tensors");
    const uint32_t b = A.size(0), M = A.size(1), N = B.size(1), K = A.size(2) * 2;
    check_size("batched_matmul", B, "B", 0, b);
    TORCH_CHECK(B.size(2) == A.size(2), "batched_matmul: A and B disagree on K");
    auto C = empty_like_dev(A, {b, M, N}, torch::kInt32);
    Launch l(A);
    ok("batched_matmul", duq4_batch_matmul_4bit(A.data_ptr<uint8_t>(), B.data_ptr<uint8_t>(), M, N, K, C.data_ptr<int32_t>(), b, l.stream));
    return C;
}

// ---- quantize, scales given ---------------------------------------------------------------------
struct QuantOut {
    uint32_t rows, cols, cd;
    Tensor q;
};
QuantOut quant_out(const char *fn, const Tensor &x) {
    TORCH_CHECK(x.dim() == 2, fn, ": expected x to be 2-D");
    check_dtype(fn, x, "x", torch::kFloat16);
    QuantOut o;
    o.rows = x.size(0);
    o.cols = x.size(1);
    o.cd = (o.cols + 1) / 2;
    o.q = empty_like_dev(x, {o.rows, o.cd}, torch::kUInt8);
    return o;
}
void check_row_vec(const char *fn, const Tensor &v, const char *name, int64_t rows) {
    check_size(fn, v, name, 0, rows);
    check_dtype(fn, v, name, torch::kFloat16);
}
// ref: bindings.cpp:88-105
Tensor sym_quant(const Tensor &x, const Tensor &scale) {
    check_tensors("sym_quant", {{&x, "x"}, {&scale, "scale"}});
    auto o = quant_out("sym_quant", x);
    check_row_vec("sym_quant", scale, "scale", o.rows);
    Launch l(x);
    ok("sym_quant", duq4_sym_quant(x.data_ptr(), scale.data_ptr(), o.rows, o.cols, o.cd, o.q.data_ptr<uint8_t>(), l.stream));
    return o.q;
}
// ref: bindings.cpp:107-127
Tensor sym_dual_quant(const Tensor &x, const Tensor &scale_1, const Tensor &scale_2) {
    check_tensors("sym_dual_quant", {{&x, "x"}, {&scale_1, "scale_1"}, {&scale_2, "scale_2"}});
    auto o = quant_out("sym_dual_quant", x);
    check_row_vec("sym_dual_quant", scale_1, "scale_1", o.rows);
    check_row_vec("sym_dual_quant", scale_2, "scale_2", o.rows);
    Launch l(x);
    ok("sym_dual_quant", duq4_sym_dual_quant(x.data_ptr(), scale_1.data_ptr(), scale_2.data_ptr(), o.rows, o.cols, o.cd,
                                             o.q.data_ptr<uint8_t>(), l.stream));
    return o.q;
}
// ref: bindings.cpp:221-243
Tensor asym_quant(const Tensor &x, const Tensor &scale, const Tensor &zeros) {
    check_tensors("asym_quant", {{&x, "x"}, {&scale, "scale"}, {&zeros, "zeros"}});
    auto o = quant_out("asym_quant", x);
    check_row_vec("asym_quant", scale, "scale", o.rows);
    check_row_vec("asym_quant", zeros, "zeros", o.rows);
    Launch l(x);
    ok("asym_quant", duq4_asym_quant(x.data_ptr(), scale.data_ptr(), zeros.data_ptr(), o.rows, o.cols, o.cd, o.q.data_ptr<uint8_t>(), l.stream));
    return o.q;
}
// ref: bindings.cpp:393-421
Tensor asym_dual_quant(const Tensor &x, const Tensor &scale_1, const Tensor &zeros_1, const Tensor &scale_2, const Tensor &zeros_2) {
    check_tensors("asym_dual_quant", {{&x, "x"}, {&scale_1, "scale_1"}, {&zeros_1, "zeros_1"}, {&scale_2, "scale_2"}, {&zeros_2, "zeros_2"}});
    auto o = quant_out("asym_dual_quant", x);
    check_row_vec("asym_dual_quant", scale_1, "scale_1", o.rows);
    check_row_vec("asym_dual_quant", zeros_1, "zeros_1", o.rows);
    check_row_vec("asym_dual_quant", scale_2, "scale_2", o.rows);
    check_row_vec("asym_dual_quant", zeros_2, "zeros_2", o.rows);
    Launch l(x);
    ok("asym_dual_quant", duq4_asym_dual_quant(x.data_ptr(), scale_1.data_ptr(), zeros_1.data_ptr(), scale_2.data_ptr(), zeros_2.data_ptr(),
                                               o.rows, o.cols, o.cd, o.q.data_ptr<uint8_t>(), l.stream));
    return o.q;
}
// ref: bindings.cpp:245-266. fp32 in, int8 codes in [0,126] out.
Tensor asym_quant_8bit(const Tensor &x, const Tensor &scale, const Tensor &zeros) {
    check_tensors("asym_quant_8bit", {{&x, "x"}, {&scale, "scale"}, {&zeros, "zeros"}});
    TORCH_CHECK(x.dim() == 2, "asym_quant_8bit: expected x to be 2-D");
    check_dtype("asym_quant_8bit", x, "x", torch::kFloat32);
    check_dtype("asym_quant_8bit", scale, "scale", torch::kFloat32);
    check_dtype("asym_quant_8bit", zeros, "zeros", torch::kFloat32);
    check_size("asym_quant_8bit", scale, "scale", 0, x.size(0));
    check_size("asym_quant_8bit", zeros, "zeros", 0, x.size(0));
    auto q = empty_like_dev(x, {x.size(0), x.size(1)}, torch::kInt8);
    Launch l(x);
    ok("asym_quant_8bit", duq4_asym_quant_8bit(x.data_ptr<float>(), scale.data_ptr<float>(), zeros.data_ptr<float>(), x.size(0), x.size(1),
                                               q.data_ptr<int8_t>(), l.stream));
    return q;
}

// ---- fused quantizers (new) -----------------------------------------------------------------------
Tensor row_vec(const Tensor &x, uint32_t rows) { return empty_like_dev(x, {rows}, torch::kFloat16); }

// (new) x fp16 [rows, K] -> (codes uint8 [rows, K/2], scales fp16 [rows]): one kernel for SymQuantizer's
// abs/max/div/mul torch ops plus sym_quant (qlinear4bit/nn/quantizer.py:10-16).
std::tuple<Tensor, Tensor> quantize_sym_fused(const Tensor &x, double clip_ratio) {
    check_tensors("quantize_sym_fused", {{&x, "x", torch::kFloat16}});
    auto o = quant_out("quantize_sym_fused", x);
    auto s = row_vec(x, o.rows);
    Launch l(x);
    ok("quantize_sym_fused", duq4_quantize_sym_fused(x.data_ptr(), o.rows, o.cols, (float)clip_ratio, o.q.data_ptr<uint8_t>(), s.data_ptr(), l.stream));
    return {o.q, s};
}
// (new) -> (codes, scales, zeros); AsymQuantizer (qlinear4bit/nn/quantizer.py:24-35) in one kernel.
std::tuple<Tensor, Tensor, Tensor> quantize_asym_fused(const Tensor &x) {
    check_tensors("quantize_asym_fused", {{&x, "x", torch::kFloat16}});
    auto o = quant_out("quantize_asym_fused", x);
    auto s = row_vec(x, o.rows), z = row_vec(x, o.rows);
    Launch l(x);
    ok("quantize_asym_fused", duq4_quantize_asym_fused(x.data_ptr(), o.rows, o.cols, o.q.data_ptr<uint8_t>(), s.data_ptr(), z.data_ptr(), l.stream));
    return {o.q, s, z};
}
// (new) dual-uniform: one scale for columns < get_dual_quant_col_k(), one for the rest.
std::tuple<Tensor, Tensor, Tensor> quantize_sym_dual_fused(const Tensor &x, double clip_ratio) {
    check_tensors("quantize_sym_dual_fused", {{&x, "x", torch::kFloat16}});
    auto o = quant_out("quantize_sym_dual_fused", x);
    auto s1 = row_vec(x, o.rows), s2 = row_vec(x, o.rows);
    Launch l(x);
    ok("quantize_sym_dual_fused", duq4_quantize_sym_dual_fused(x.data_ptr(), o.rows, o.cols, (float)clip_ratio, o.q.data_ptr<uint8_t>(),
                                                               s1.data_ptr(), s2.data_ptr(), l.stream));
    return {o.q, s1, s2};
}
// (new) -> (codes, scale_1, zeros_1, scale_2, zeros_2)
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> quantize_asym_dual_fused(const Tensor &x) {
    check_tensors("quantize_asym_dual_fused", {{&x, "x", torch::kFloat16}});
    auto o = quant_out("quantize_asym_dual_fused", x);
    auto s1 = row_vec(x, o.rows), z1 = row_vec(x, o.rows), s2 = row_vec(x, o.rows), z2 = row_vec(x, o.rows);
    Launch l(x);
    ok("quantize_asym_dual_fused", duq4_quantize_asym_dual_fused(x.data_ptr(), o.rows, o.cols, o.q.data_ptr<uint8_t>(), s1.data_ptr(),
                                                                 z1.data_ptr(), s2.data_ptr(), z2.data_ptr(), l.stream));
    return {o.q, s1, z1, s2, z2};
}
// (new) SiLU-gated MLP glue in one kernel: gate_up fp16 [rows, 2*I] holds the gate projection in columns
// [0, I) and the up projection in [I, 2I); returns the per-token quantization of h = F.silu(gate) * up
// without storing h: (codes, scales) for "sym", (codes, scales, zeros) for "asym". Codes are packed uint8
// [rows, I/2], or int8 [rows, I] in the GEMM's tensor-core-ready layout when requested.
py::object silu_mul_quantize_fused(const Tensor &gate_up, const std::string &mode, double clip_ratio, bool tensor_core_ready) {
    check_tensors("silu_mul_quantize_fused", {{&gate_up, "gate_up", torch::kFloat16}});
    TORCH_CHECK(gate_up.dim() == 2 && gate_up.size(1) % 2 == 0 && gate_up.scalar_type() == torch::kFloat16,
                "silu_mul_quantize_fused: expected fp16 [rows, 2*I]");
    TORCH_CHECK(mode == "sym" || mode == "asym", "silu_mul_quantize_fused: mode must be 'sym' or 'asym'");
    const uint32_t rows = gate_up.size(0), ld = gate_up.size(1), inter = ld / 2;
    auto q = tensor_core_ready ? empty_like_dev(gate_up, {rows, inter}, torch::kInt8) : empty_like_dev(gate_up, {rows, inter / 2}, torch::kUInt8);
    auto s = row_vec(gate_up, rows);
    Tensor z;
    if (mode == "asym") z = row_vec(gate_up, rows);
    Launch l(gate_up);
    ok("silu_mul_quantize_fused", duq4_silu_mul_quantize_fused(mode_of("silu_mul_quantize_fused", mode), gate_up.data_ptr(), rows, inter, ld, inter,
                                                               (float)clip_ratio, q.data_ptr(), tensor_core_ready ? 1 : 0, s.data_ptr(),
                                                               z.defined() ? z.data_ptr() : nullptr, l.stream));
    if (z.defined()) return py::make_tuple(q, s, z);
    return py::make_tuple(q, s);
}

// ---- dequantize ---------------------------------------------------------------------------------
void check_acc(const char *fn, const Tensor &q, int64_t dims) {
    TORCH_CHECK(q.dim() == dims, fn, ": expected q to be ", dims, "-D");
    check_dtype(fn, q, "q", torch::kInt32);
}
void check_vec(const char *fn, const Tensor &v, const char *name, int64_t dim, int64_t n, torch::ScalarType dt = torch::kFloat16) {
    check_size(fn, v, name, dim, n);
    check_dtype(fn, v, name, dt);
}
// ref: bindings.cpp:130-170
Tensor sym_dequant(const Tensor &q, const Tensor &scale_row, const Tensor &scale_col, int bits) {
    check_tensors("sym_dequant", {{&q, "q"}, {&scale_row, "scale_row"}, {&scale_col, "scale_col"}});
    check_acc("sym_dequant", q, 2);
    const uint32_t rows = q.size(0), cols = q.size(1);
    check_vec("sym_dequant", scale_row, "scale_row", 0, rows);
    check_vec("sym_dequant", scale_col, "scale_col", 0, cols);
    check_bits(bits);
    auto x = empty_like_dev(q, {rows, cols}, torch::kFloat16);
    Launch l(q);
    ok("sym_dequant", duq4_sym_dequant(q.data_ptr<int32_t>(), scale_row.data_ptr(), scale_col.data_ptr(), rows, cols, x.data_ptr(), l.stream));
    return x;
}
// ref: bindings.cpp:172-217
Tensor sym_dual_dequant(const Tensor &q, const Tensor &scale_row, const Tensor &scale_col_1, const Tensor &scale_col_2, int bits) {
    check_tensors("sym_dual_dequant", {{&q, "q"}, {&scale_row, "scale_row"}, {&scale_col_1, "scale_col_1"}, {&scale_col_2, "scale_col_2"}});
    check_acc("sym_dual_dequant", q, 2);
    const uint32_t rows = q.size(0), cols = q.size(1);
    check_vec("sym_dual_dequant", scale_row, "scale_row", 0, rows);
    check_vec("sym_dual_dequant", scale_col_1, "scale_col_1", 0, cols);
    check_vec("sym_dual_dequant", scale_col_2, "scale_col_2", 0, cols);
    check_bits(bits);
    auto x = empty_like_dev(q, {rows, cols}, torch::kFloat16);
    Launch l(q);
    ok("sym_dual_dequant", duq4_sym_dual_dequant(q.data_ptr<int32_t>(), scale_row.data_ptr(), scale_col_1.data_ptr(), scale_col_2.data_ptr(), rows,
                                                 cols, x.data_ptr(), l.stream));
    return x;
}
// ref: bindings.cpp:268-307
Tensor asym_dequant(const Tensor &q, const Tensor &scale_row, const Tensor &zeros_row, const Tensor &scale_col, const Tensor &zeros_col, int bits) {
    check_tensors("asym_dequant", {{&q, "q"}, {&scale_row, "scale_row"}, {&zeros_row, "zeros_row"}, {&scale_col, "scale_col"}, {&zeros_col, "zeros_col"}});
    check_acc("asym_dequant", q, 2);
    const uint32_t rows = q.size(0), cols = q.size(1);
    check_vec("asym_dequant", scale_row, "scale_row", 0, rows);
    check_vec("asym_dequant", zeros_row, "zeros_row", 0, rows);
    check_vec("asym_dequant", scale_col, "scale_col", 0, cols);
    check_vec("asym_dequant", zeros_col, "zeros_col", 0, cols);
    check_bits(bits);
    auto x = empty_like_dev(q, {rows, cols}, torch::kFloat16);
    Launch l(q);
    ok("asym_dequant", duq4_asym_dequant(q.data_ptr<int32_t>(), scale_row.data_ptr(), zeros_row.data_ptr(), scale_col.data_ptr(), zeros_col.data_ptr(),
                                         rows, cols, x.data_ptr(), l.stream));
    return x;
}
// ref: bindings.cpp:423-467
Tensor asym_dual_dequant(const Tensor &q, const Tensor &scale_row, const Tensor &zeros_row, const Tensor &scale_col_1, const Tensor &zeros_col_1,
                         const Tensor &scale_col_2, const Tensor &zeros_col_2, int bits) {
    check_tensors("asym_dual_dequant", {{&q, "q"}, {&scale_row, "scale_row"}, {&zeros_row, "zeros_row"}, {&scale_col_1, "scale_col_1"},
                                        {&zeros_col_1, "zeros_col_1"}, {&scale_col_2, "scale_col_2"}, {&zeros_col_2, "zeros_col_2"}});
    check_acc("asym_dual_dequant", q, 2);
    const uint32_t rows = q.size(0), cols = q.size(1);
    check_vec("asym_dual_dequant", scale_row, "scale_row", 0, rows);
    check_vec("asym_dual_dequant", zeros_row, "zeros_row", 0, rows);
    check_vec("asym_dual_dequant", scale_col_1, "scale_col_1", 0, cols);
    check_vec("asym_dual_dequant", zeros_col_1, "zeros_col_1", 0, cols);
    check_vec("asym_dual_dequant", scale_col_2, "scale_col_2", 0, cols);
    check_vec("asym_dual_dequant", zeros_col_2, "zeros_col_2", 0, cols);
    check_bits(bits);
    auto x = empty_like_dev(q, {rows, cols}, torch::kFloat16);
    Launch l(q);
    ok("asym_dual_dequant", duq4_asym_dual_dequant(q.data_ptr<int32_t>(), scale_row.data_ptr(), zeros_row.data_ptr(), scale_col_1.data_ptr(),
                                                   zeros_col_1.data_ptr(), scale_col_2.data_ptr(), zeros_col_2.data_ptr(), rows, cols, x.data_ptr(),
                                                   l.stream));
    return x;
}
// ref: bindings.cpp:351-391. q [b,rows,cols]; row vectors with size(1) == rows, column vectors with size(1) == cols.
Tensor asym_batch_dequant(const Tensor &q, const Tensor &scale_row, const Tensor &zeros_row, const Tensor &scale_col, const Tensor &zeros_col, int bits) {
    check_tensors("asym_batch_dequant", {{&q, "q"}, {&scale_row, "scale_row"}, {&zeros_row, "zeros_row"}, {&scale_col, "scale_col"}, {&zeros_col, "zeros_col"}});
    check_acc("asym_batch_dequant", q, 3);
    const uint32_t b = q.size(0), rows = q.size(1), cols = q.size(2);
    check_vec("asym_batch_dequant", scale_row, "scale_row", 1, rows);
    check_vec("asym_batch_dequant", zeros_row, "zeros_row", 1, rows);
    check_vec("asym_batch_dequant", scale_col, "scale_col", 1, cols);
    check_vec("asym_batch_dequant", zeros_col, "zeros_col", 1, cols);
    check_bits(bits);
    auto x = empty_like_dev(q, {b, rows, cols}, torch::kFloat16);
    Launch l(q);
    ok("asym_batch_dequant", duq4_asym_batch_dequant(q.data_ptr<int32_t>(), scale_row.data_ptr(), zeros_row.data_ptr(), scale_col.data_ptr(),
                                                     zeros_col.data_ptr(), b, rows, cols, x.data_ptr(), l.stream));
    return x;
}
// ref: bindings.cpp:309-348. fp32 dequant of the 8-bit path.
Tensor asym_dequant_hprec(const Tensor &q, const Tensor &scale_row, const Tensor &zeros_row, const Tensor &scale_col, const Tensor &zeros_col, int bits) {
    check_tensors("asym_dequant_hprec", {{&q, "q"}, {&scale_row, "scale_row"}, {&zeros_row, "zeros_row"}, {&scale_col, "scale_col"}, {&zeros_col, "zeros_col"}});
    check_acc("asym_dequant_hprec", q, 2);
    const uint32_t rows = q.size(0), cols = q.size(1);
    check_vec("asym_dequant_hprec", scale_row, "scale_row", 0, rows, torch::kFloat32);
    check_vec("asym_dequant_hprec", zeros_row, "zeros_row", 0, rows, torch::kFloat32);
    check_vec("asym_dequant_hprec", scale_col, "scale_col", 0, cols, torch::kFloat32);
    check_vec("asym_dequant_hprec", zeros_col, "zeros_col", 0, cols, torch::kFloat32);
    check_bits(bits);
    auto x = empty_like_dev(q, {rows, cols}, torch::kFloat32);
    Launch l(q);
    ok("asym_dequant_hprec", duq4_asym_dequant_hprec(q.data_ptr<int32_t>(), scale_row.data_ptr<float>(), zeros_row.data_ptr<float>(),
                                                     scale_col.data_ptr<float>(), zeros_col.data_ptr<float>(), rows, cols, x.data_ptr<float>(), l.stream));
    return x;
}
// ref: bindings.cpp:471-473
int get_dual_quant_col_k() { return duq4_dual_quant_col_k(); }

// ---- fused linear (new) ---------------------------------------------------------------------------
// Per-channel vectors of an epilogue: fp16, at least N entries ([N] or [N,1]).
void check_col_vec(const char *fn, const OptTensor &v, const char *name, int64_t n) {
    if (!opt(v)) return;
    check_dtype(fn, *v, name, torch::kFloat16);
    TORCH_CHECK(v->numel() == n, fn, ": expected ", name, " to have ", n, " entries, got ", v->numel());
}
duq4_epilogue make_epi(const char *fn, const std::string &mode, int64_t N, const OptTensor &scale_row, const OptTensor &zeros_row,
                       const OptTensor &scale_col_1, const OptTensor &zeros_col_1, const OptTensor &scale_col_2,
                       const OptTensor &zeros_col_2, const OptTensor &bias, int64_t col_offset, int64_t ldo) {
    check_col_vec(fn, scale_col_1, "scale_col_1", N);
    check_col_vec(fn, zeros_col_1, "zeros_col_1", N);
    check_col_vec(fn, scale_col_2, "scale_col_2", N);
    check_col_vec(fn, zeros_col_2, "zeros_col_2", N);
    check_col_vec(fn, bias, "bias", N);
    duq4_epilogue e = {};
    e.mode = mode_of(fn, mode);
    e.col_offset = (uint32_t)col_offset;
    e.scale_row = ptr(scale_row);
    e.zeros_row = ptr(zeros_row);
    e.scale_col_1 = ptr(scale_col_1);
    e.zeros_col_1 = ptr(zeros_col_1);
    e.scale_col_2 = ptr(scale_col_2);
    e.zeros_col_2 = ptr(zeros_col_2);
    e.bias = ptr(bias);
    e.ldo = (uint32_t)ldo;
    return e;
}

// (new) fp16 [M,N] = dequant_mode(A [M,K/2] . W [N,K/2]^T) (+ bias): GEMM, dequant and bias in one kernel; results
// identical to matmul -> *_dequant -> `+ bias` (qlinear4bit/nn/linear.py:42-56 and the other forwards). `out` may be
// a column-slice view of a wider row-major buffer (its row stride is honoured). `next_weights`: packed weights of
// the layer that follows on this stream, a hint that lets the small-M kernels warm L2 with them.
py::object linear_w4a4(const std::string &mode, const Tensor &A, const Tensor &W, const Tensor &scale_row, const OptTensor &zeros_row,
                       const OptTensor &scale_col_1, const OptTensor &zeros_col_1, const OptTensor &scale_col_2,
                       const OptTensor &zeros_col_2, const OptTensor &bias, int64_t col_offset, const OptTensor &out_, bool return_acc,
                       const OptTensor &next_weights) {
    const char *fn = "linear_w4a4";
    constexpr auto F16 = torch::kFloat16;
    check_tensors(fn, {{&A, "A", torch::kUInt8}, {&W, "W", torch::kUInt8}, {&scale_row, "scale_row", F16}, {opt(zeros_row), "zeros_row", F16},
                       {opt(scale_col_1), "scale_col_1", F16}, {opt(zeros_col_1), "zeros_col_1", F16}, {opt(scale_col_2), "scale_col_2", F16},
                       {opt(zeros_col_2), "zeros_col_2", F16}, {opt(bias), "bias", F16}});
    check_dtype(fn, A, "A", torch::kUInt8);
    check_dtype(fn, W, "W", torch::kUInt8);
    TORCH_CHECK(A.dim() == 2 && W.dim() == 2 && W.size(1) == A.size(1), fn, ": A and W disagree on K");
    const int64_t M = A.size(0), N = W.size(0), K = A.size(1) * 2;
    check_vec(fn, scale_row, "scale_row", 0, M);
    if (opt(zeros_row)) check_vec(fn, *zeros_row, "zeros_row", 0, M);
    Tensor out;
    if (opt(out_)) {
        out = *out_;
        TORCH_CHECK(out.is_cuda() && out.device() == A.device() && out.scalar_type() == torch::kFloat16 && out.dim() == 2 && out.size(0) == M &&
                        out.size(1) == N && out.stride(1) == 1,
                    fn, ": out must be fp16 [M,N] with unit column stride on the GPU of A");
    } else {
        out = empty_like_dev(A, {M, N}, torch::kFloat16);
    }
    Tensor acc;
    if (return_acc) acc = empty_like_dev(A, {M, N}, torch::kInt32);
    const int64_t ldo = M > 1 ? out.stride(0) : std::max<int64_t>(out.stride(0), N);
    duq4_epilogue e = make_epi(fn, mode, N, scale_row, zeros_row, scale_col_1, zeros_col_1, scale_col_2, zeros_col_2, bias, col_offset, ldo);
    if (opt(next_weights)) {
        e.next_weights = next_weights->data_ptr();
        e.next_weights_bytes = (uint64_t)next_weights->numel() * next_weights->element_size();
    }
    Launch l(A);
    ok(fn, duq4_linear_w4a4(A.data_ptr<uint8_t>(), W.data_ptr<uint8_t>(), M, N, K, &e, out.data_ptr(), return_acc ? acc.data_ptr<int32_t>() : nullptr,
                            l.stream));
    if (return_acc) return py::make_tuple(out, acc);
    return py::cast(out);
}

// Scratch of linear_w4a4_from_fp16: one tensor per (device, stream), grown on demand. A tensor is only ever used by
// work queued on the stream it was allocated under, so forwards on different streams never share one, and torch's
// caching allocator (which reuses a freed block on its allocation stream only) keeps a replaced tensor's memory
// away from other streams while earlier work may still read it.
struct ScratchKey {
    int dev;
    void *stream;
    bool operator==(const ScratchKey &o) const { return dev == o.dev && stream == o.stream; }
};
struct ScratchKeyHash {
    size_t operator()(const ScratchKey &k) const { return std::hash<void *>()(k.stream) * 31u + (size_t)k.dev; }
};
Tensor scratch_for(const Tensor &x, void *stream, size_t need) {
    static std::mutex mu;
    static std::unordered_map<ScratchKey, Tensor, ScratchKeyHash> *pool = new std::unordered_map<ScratchKey, Tensor, ScratchKeyHash>();
    std::lock_guard<std::mutex> g(mu);
    Tensor &t = (*pool)[ScratchKey{(int)x.device().index(), stream}];
    if (!t.defined() || (size_t)t.numel() < need) t = empty_like_dev(x, {(int64_t)need}, torch::kUInt8);
    return t;
}

// (new) fp16 activations [M,K] -> per-token quantize -> GEMM -> dequant (+ bias) in one library call; the quantized
// activations stay in an internal scratch tensor. Same result as quantizer module + linear_w4a4. `act_mode` defaults
// to the single-scale quantizer of the epilogue's family ("sym" for sym / sym_dual, "asym" otherwise), which is what
// the reference modules pair with each linear variant (qlinear4bit/nn/linear.py:104-115, :239-250).
// `W_prelaid`: optional int8 [N, K] made once from W by weight_prelayout_i8; when given, layers that see more than
// 128 tokens run on it (no in-kernel weight unpack), fewer tokens use the packed W (half the bytes to stream).
Tensor linear_w4a4_from_fp16(const std::string &mode, const Tensor &x, const Tensor &W, const Tensor &scale_col_1, const OptTensor &zeros_col_1,
                             const OptTensor &scale_col_2, const OptTensor &zeros_col_2, const OptTensor &bias, double clip_ratio,
                             const std::optional<std::string> &act_mode_, const OptTensor &W_prelaid) {
    const char *fn = "linear_w4a4_from_fp16";
    constexpr auto F16 = torch::kFloat16;
    check_tensors(fn, {{&x, "x", F16}, {&W, "W", torch::kUInt8}, {&scale_col_1, "scale_col_1", F16}, {opt(zeros_col_1), "zeros_col_1", F16},
                       {opt(scale_col_2), "scale_col_2", F16}, {opt(zeros_col_2), "zeros_col_2", F16}, {opt(bias), "bias", F16},
                       {opt(W_prelaid), "W_prelaid", torch::kInt8}});
    TORCH_CHECK(x.scalar_type() == torch::kFloat16 && x.dim() == 2, fn, ": x must be fp16 [M, K]");
    check_dtype(fn, W, "W", torch::kUInt8);
    const int64_t M = x.size(0), K = x.size(1), N = W.size(0);
    TORCH_CHECK(W.dim() == 2 && W.size(1) * 2 == K, fn, ": x and W disagree on K");
    if (opt(W_prelaid)) {
        check_dtype(fn, *W_prelaid, "W_prelaid", torch::kInt8);
        TORCH_CHECK(W_prelaid->dim() == 2 && W_prelaid->size(0) == N && W_prelaid->size(1) == K, fn, ": W_prelaid must be int8 [N, K]");
    }
    const std::string act_mode = act_mode_.has_value() ? *act_mode_ : ((mode == "sym" || mode == "sym_dual") ? "sym" : "asym");
    duq4_epilogue e = make_epi(fn, mode, N, std::nullopt, std::nullopt, scale_col_1, zeros_col_1, scale_col_2, zeros_col_2, bias, 0, 0);
    auto out = empty_like_dev(x, {M, N}, torch::kFloat16);
    Launch l(x);
    const bool prelaid = opt(W_prelaid) && M > 128;
    const size_t need = prelaid ? duq4_linear_from_fp16_prelaid_workspace_bytes(M, K) : duq4_linear_from_fp16_workspace_bytes(M, K);
    Tensor ws = scratch_for(x, l.stream, need);
    if (prelaid)
        ok(fn, duq4_linear_w4a4_from_fp16_prelaid(x.data_ptr(), W_prelaid->data_ptr<int8_t>(), M, N, K, mode_of(fn, act_mode), (float)clip_ratio, &e,
                                                  out.data_ptr(), ws.data_ptr(), (size_t)ws.numel(), l.stream));
    else
        ok(fn, duq4_linear_w4a4_from_fp16(x.data_ptr(), W.data_ptr<uint8_t>(), M, N, K, mode_of(fn, act_mode), (float)clip_ratio, &e, out.data_ptr(),
                                          ws.data_ptr(), (size_t)ws.numel(), l.stream));
    return out;
}

// (new) One-off re-layout of packed weights uint8 [N, K/2] into the tensor-core-ready int8 [N, K] that
// linear_w4a4_from_fp16(W_prelaid=...) and the library's duq4_linear_w4a4_prelaid read (K % 128 == 0).
Tensor weight_prelayout_i8(const Tensor &W) {
    check_tensors("weight_prelayout_i8", {{&W, "W"}});
    check_dtype("weight_prelayout_i8", W, "W", torch::kUInt8);
    TORCH_CHECK(W.dim() == 2, "weight_prelayout_i8: expected W [N, K/2]");
    const int64_t N = W.size(0), K = W.size(1) * 2;
    auto out = empty_like_dev(W, {N, K}, torch::kInt8);
    Launch l(W);
    ok("weight_prelayout_i8", duq4_weight_prelayout_i8(W.data_ptr<uint8_t>(), N, K, out.data_ptr<int8_t>(), l.stream));
    return out;
}

// (new) SiLU-gated gate/up projection in one launch: W packed [2*I, K/2] = gate rows then up rows, `scale_col` /
// `zeros_col` / `bias` with 2*I entries; returns h fp16 [M, I] equal to F.silu(y[:, :I]) * y[:, I:] for
// y = linear_w4a4(mode, A, W, ...), without writing y. A: packed int4 uint8 [M, K/2] or the tensor-core-ready int8
// [M, K] of silu_mul_quantize_fused. mode: "sym" or "asym". `W_prelaid`: optional int8 [2*I, K] made once from W by
// weight_prelayout_i8; read instead of W when A is int8 and M > 128 (same bits, less work per tile).
Tensor linear_w4a4_gate_up_silu(const std::string &mode, const Tensor &A, const Tensor &W, const Tensor &scale_row, const OptTensor &zeros_row,
                                const OptTensor &scale_col, const OptTensor &zeros_col, const OptTensor &bias, const OptTensor &W_prelaid) {
    const char *fn = "linear_w4a4_gate_up_silu";
    constexpr auto F16 = torch::kFloat16;
    check_tensors(fn, {{&A, "A"}, {&W, "W", torch::kUInt8}, {&scale_row, "scale_row", F16}, {opt(zeros_row), "zeros_row", F16},
                       {opt(scale_col), "scale_col", F16}, {opt(zeros_col), "zeros_col", F16}, {opt(bias), "bias", F16},
                       {opt(W_prelaid), "W_prelaid", torch::kInt8}});
    TORCH_CHECK(mode == "sym" || mode == "asym", fn, ": mode must be 'sym' or 'asym'");
    TORCH_CHECK(A.scalar_type() == torch::kInt8 || A.scalar_type() == torch::kUInt8, fn, ": A must be uint8 (packed) or int8 (tensor-core-ready)");
    check_dtype(fn, W, "W", torch::kUInt8);
    const bool a_is_int8 = A.scalar_type() == torch::kInt8;
    const int64_t M = A.size(0), K = a_is_int8 ? A.size(1) : A.size(1) * 2;
    TORCH_CHECK(W.dim() == 2 && W.size(0) % 2 == 0 && W.size(1) * 2 == K, fn, ": W must be [2*I, K/2]");
    const int64_t inter = W.size(0) / 2;
    check_vec(fn, scale_row, "scale_row", 0, M);
    if (opt(zeros_row)) check_vec(fn, *zeros_row, "zeros_row", 0, M);
    TORCH_CHECK(opt(scale_col), fn, ": scale_col is required");
    duq4_epilogue e = make_epi(fn, mode, 2 * inter, scale_row, zeros_row, scale_col, zeros_col, std::nullopt, std::nullopt, bias, 0, 0);
    auto h = empty_like_dev(A, {M, inter}, torch::kFloat16);
    Launch l(A);
    if (opt(W_prelaid)) {
        check_dtype(fn, *W_prelaid, "W_prelaid", torch::kInt8);
        TORCH_CHECK(W_prelaid->dim() == 2 && W_prelaid->size(0) == 2 * inter && W_prelaid->size(1) == K, fn, ": W_prelaid must be int8 [2*I, K]");
    }
    if (opt(W_prelaid) && a_is_int8 && M > 128)
        ok(fn, duq4_linear_w4a4_gate_up_silu_prelaid(A.data_ptr<int8_t>(), W_prelaid->data_ptr<int8_t>(), M, inter, K, &e, h.data_ptr(), l.stream));
    else
        ok(fn, duq4_linear_w4a4_gate_up_silu(A.data_ptr(), a_is_int8 ? 1 : 0, W.data_ptr<uint8_t>(), M, inter, K, &e, h.data_ptr(), l.stream));
    return h;
}

// (new) batched form: A [b,M,K/2], W [b,N,K/2], row vectors [b,M], column vectors [b,N] (the layout of the
// reference's asym_batch_dequant).
Tensor linear_w4a4_batched(const std::string &mode, const Tensor &A, const Tensor &W, const Tensor &scale_row, const OptTensor &zeros_row,
                           const OptTensor &scale_col_1, const OptTensor &zeros_col_1, const OptTensor &scale_col_2, const OptTensor &zeros_col_2) {
    const char *fn = "linear_w4a4_batched";
    constexpr auto F16 = torch::kFloat16;
    check_tensors(fn, {{&A, "A", torch::kUInt8}, {&W, "W", torch::kUInt8}, {&scale_row, "scale_row", F16}, {opt(zeros_row), "zeros_row", F16},
                       {opt(scale_col_1), "scale_col_1", F16}, {opt(zeros_col_1), "zeros_col_1", F16}, {opt(scale_col_2), "scale_col_2", F16},
                       {opt(zeros_col_2), "zeros_col_2", F16}});
    check_dtype(fn, A, "A", torch::kUInt8);
    check_dtype(fn, W, "W", torch::kUInt8);
    TORCH_CHECK(A.dim() == 3 && W.dim() == 3 && W.size(0) == A.size(0) && W.size(2) == A.size(2), fn, ": expected A [b,M,K/2] and W [b,N,K/2]");
    const int64_t b = A.size(0), M = A.size(1), N = W.size(1), K = A.size(2) * 2;
    check_dtype(fn, scale_row, "scale_row", torch::kFloat16);
    TORCH_CHECK(scale_row.numel() == b * M, fn, ": expected scale_row to have b*M entries");
    if (opt(zeros_row)) {
        check_dtype(fn, *zeros_row, "zeros_row", torch::kFloat16);
        TORCH_CHECK(zeros_row->numel() == b * M, fn, ": expected zeros_row to have b*M entries");
    }
    duq4_epilogue e = make_epi(fn, mode, b * N, scale_row, zeros_row, scale_col_1, zeros_col_1, scale_col_2, zeros_col_2, std::nullopt, 0, 0);
    auto out = empty_like_dev(A, {b, M, N}, torch::kFloat16);
    Launch l(A);
    ok(fn, duq4_linear_w4a4_batched(A.data_ptr<uint8_t>(), W.data_ptr<uint8_t>(), M, N, K, b, &e, out.data_ptr(), nullptr, l.stream));
    return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "W4A4 linear-layer operators for B200 (sm_100a) with the names of the reference's qlinear4bit._CUDA";
    // names, keyword names and order of src/export/bindings.cpp:772-921 of the reference
    m.def("matmul", &matmul, py::arg("A"), py::arg("B"));
    m.def("matmul_8bit", &matmul_8bit, py::arg("A"), py::arg("B"));
    m.def("batched_matmul", &batched_matmul, py::arg("A"), py::arg("B"));
    m.def("sym_quant", &sym_quant, py::arg("x"), py::arg("scale"));
    m.def("sym_dual_quant", &sym_dual_quant, py::arg("x"), py::arg("scale_1"), py::arg("scale_2"));
    m.def("sym_dequant", &sym_dequant, py::arg("q"), py::arg("scale_row"), py::arg("scale_col"), py::arg("bits"));
    m.def("sym_dual_dequant", &sym_dual_dequant, py::arg("q"), py::arg("scale_row"), py::arg("scale_col_1"), py::arg("scale_col_2"), py::arg("bits"));
    m.def("asym_quant", &asym_quant, py::arg("x"), py::arg("scale"), py::arg("zeros"));
    m.def("asym_quant_8bit", &asym_quant_8bit, py::arg("x"), py::arg("scale"), py::arg("zeros"));
    m.def("asym_batch_dequant", &asym_batch_dequant, py::arg("q"), py::arg("scale_row"), py::arg("zeros_row"), py::arg("scale_col"),
          py::arg("zeros_col"), py::arg("bits"));
    m.def("asym_dequant", &asym_dequant, py::arg("q"), py::arg("scale_row"), py::arg("zeros_row"), py::arg("scale_col"), py::arg("zeros_col"),
          py::arg("bits"));
    m.def("asym_dequant_hprec", &asym_dequant_hprec, py::arg("q"), py::arg("scale_row"), py::arg("zeros_row"), py::arg("scale_col"),
          py::arg("zeros_col"), py::arg("bits"));
    m.def("asym_dual_quant", &asym_dual_quant, py::arg("x"), py::arg("scale_1"), py::arg("zeros_1"), py::arg("scale_2"), py::arg("zeros_2"));
    m.def("asym_dual_dequant", &asym_dual_dequant, py::arg("q"), py::arg("scale_row"), py::arg("zeros_row"), py::arg("scale_col_1"),
          py::arg("zeros_col_1"), py::arg("scale_col_2"), py::arg("zeros_col_2"), py::arg("bits"));
    m.def("get_dual_quant_col_k", &get_dual_quant_col_k);
    // (new)
    m.def("quantize_sym_fused", &quantize_sym_fused, py::arg("x"), py::arg("clip_ratio") = 1.0);
    m.def("quantize_asym_fused", &quantize_asym_fused, py::arg("x"));
    m.def("quantize_sym_dual_fused", &quantize_sym_dual_fused, py::arg("x"), py::arg("clip_ratio") = 1.0);
    m.def("quantize_asym_dual_fused", &quantize_asym_dual_fused, py::arg("x"));
    m.def("silu_mul_quantize_fused", &silu_mul_quantize_fused, py::arg("gate_up"), py::arg("mode") = "sym", py::arg("clip_ratio") = 1.0,
          py::arg("tensor_core_ready") = false);
    m.def("linear_w4a4", &linear_w4a4, py::arg("mode"), py::arg("A"), py::arg("W"), py::arg("scale_row"), py::arg("zeros_row") = py::none(),
          py::arg("scale_col_1") = py::none(), py::arg("zeros_col_1") = py::none(), py::arg("scale_col_2") = py::none(),
          py::arg("zeros_col_2") = py::none(), py::arg("bias") = py::none(), py::arg("col_offset") = 0, py::arg("out") = py::none(),
          py::arg("return_acc") = false, py::arg("next_weights") = py::none());
    m.def("linear_w4a4_from_fp16", &linear_w4a4_from_fp16, py::arg("mode"), py::arg("x"), py::arg("W"), py::arg("scale_col_1"),
          py::arg("zeros_col_1") = py::none(), py::arg("scale_col_2") = py::none(), py::arg("zeros_col_2") = py::none(), py::arg("bias") = py::none(),
          py::arg("clip_ratio") = 1.0, py::arg("act_mode") = py::none(), py::arg("W_prelaid") = py::none());
    m.def("weight_prelayout_i8", &weight_prelayout_i8, py::arg("W"));
    m.def("linear_w4a4_gate_up_silu", &linear_w4a4_gate_up_silu, py::arg("mode"), py::arg("A"), py::arg("W"), py::arg("scale_row"),
          py::arg("zeros_row") = py::none(), py::arg("scale_col") = py::none(), py::arg("zeros_col") = py::none(), py::arg("bias") = py::none(),
          py::arg("W_prelaid") = py::none());
    m.def("linear_w4a4_batched", &linear_w4a4_batched, py::arg("mode"), py::arg("A"), py::arg("W"), py::arg("scale_row"),
          py::arg("zeros_row") = py::none(), py::arg("scale_col_1") = py::none(), py::arg("zeros_col_1") = py::none(),
          py::arg("scale_col_2") = py::none(), py::arg("zeros_col_2") = py::none());
}
