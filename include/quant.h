// Reference-named C++ API of the quantize / dequantize launchers: the function names,
// argument orders and types of DUQLinear4bitCUDA's include/quant.h (lines 9-127 there), as
// inline wrappers over the C ABI in duq4.h. Existing C++ callers compile unchanged and
// link against libduq4.so.
//
// Differences a caller can observe: launches go to the legacy default stream exactly as
// in the reference; a rejected argument or a CUDA launch error throws std::runtime_error
// (the reference's quantize launchers report nothing at all).
#pragma once
#include <cuda_fp16.h>

#include <stdexcept>
#include <string>

#include "common.h"
#include "duq4.h"

constexpr int QUANT_COL_K = DUQ4_QUANT_COL_K;  // include/quant.h:5 of the reference
// include/quant.h:7 of the reference: a 128-bit mask with bits 0-4 and 10-14 set. The reference's dual
// asymmetric dequant tests it as `(QUANT_COL_ST << col) & 1`, which is non-zero for output column 0 only;
// the library's epilogues reproduce that outcome (DUQ4_MODE_ASYM_DUAL), the constant is kept for callers.
constexpr __uint128_t QUANT_COL_ST = (((__uint128_t)0x1F) << 0) | (((__uint128_t)0x1F) << 10);

namespace duq4_detail {
inline void check(const char *fn, int status) {
    if (status != 0) throw std::runtime_error(std::string(fn) + ": " + duq4_error_string(status));
}
}  // namespace duq4_detail

// include/quant.h:9-16 of the reference
inline void sym_quant_host(const half *x, const half *scale, uint32_t rows, uint32_t colsSrc, uint32_t colsDst,
                           Int4Storage *q) {
    duq4_detail::check("sym_quant_host", duq4_sym_quant(x, scale, rows, colsSrc, colsDst, q, nullptr));
}
// :19-26
inline void sym_dequant_host(const int32_t *q, const half *scale_row, const half *scale_col, uint32_t rows,
                             uint32_t cols, half *x) {
    duq4_detail::check("sym_dequant_host", duq4_sym_dequant(q, scale_row, scale_col, rows, cols, x, nullptr));
}
// :29-37
inline void sym_dual_quant_host(const half *x, const half *scale_1, const half *scale_2, uint32_t rows,
                                uint32_t colsSrc, uint32_t colsDst, Int4Storage *q) {
    duq4_detail::check("sym_dual_quant_host", duq4_sym_dual_quant(x, scale_1, scale_2, rows, colsSrc, colsDst, q, nullptr));
}
// :40-48
inline void sym_dual_dequant_host(const int32_t *q, const half *scale_row, const half *scale_col_1,
                                  const half *scale_col_2, uint32_t rows, uint32_t cols, half *x) {
    duq4_detail::check("sym_dual_dequant_host",
                       duq4_sym_dual_dequant(q, scale_row, scale_col_1, scale_col_2, rows, cols, x, nullptr));
}
// :49-57
inline void asym_quant_host(const half *x, const half *scale, const half *zeros, uint32_t rows, uint32_t colsSrc,
                            uint32_t colsDst, Int4Storage *q) {
    duq4_detail::check("asym_quant_host", duq4_asym_quant(x, scale, zeros, rows, colsSrc, colsDst, q, nullptr));
}
// :59-68
inline void asym_dequant_host(const int32_t *q, const half *scale_row, const half *zeros_row, const half *scale_col,
                              const half *zeros_col, uint32_t rows, uint32_t cols, half *x) {
    duq4_detail::check("asym_dequant_host",
                       duq4_asym_dequant(q, scale_row, zeros_row, scale_col, zeros_col, rows, cols, x, nullptr));
}
// :70-77
inline void asym_quant_host_8bit(const float *x, const float *scale, const float *zeros, uint32_t rows, uint32_t cols,
                                 int8_t *q) {
    duq4_detail::check("asym_quant_host_8bit", duq4_asym_quant_8bit(x, scale, zeros, rows, cols, q, nullptr));
}
// :79-89
inline void asym_batch_dequant_host(const int32_t *q, const half *scale_row, const half *zeros_row,
                                    const half *scale_col, const half *zeros_col, uint32_t batches, uint32_t rows,
                                    uint32_t cols, half *x) {
    duq4_detail::check("asym_batch_dequant_host", duq4_asym_batch_dequant(q, scale_row, zeros_row, scale_col, zeros_col,
                                                                           batches, rows, cols, x, nullptr));
}
// :92-103. The reference DECLARES (x, scale_1, scale_2, zeros_1, zeros_2) but DEFINES and calls
// (x, scale_1, zeros_1, scale_2, zeros_2) (src/kernels/quant2.cu:141-156, src/export/bindings.cpp:416-419);
// all five are `const half *`, so positional callers get the definition's meaning. Kept.
inline void asym_dual_quant_host(const half *x, const half *scale_1, const half *zeros_1, const half *scale_2,
                                 const half *zeros_2, uint32_t rows, uint32_t colsSrc, uint32_t colsDst,
                                 Int4Storage *q) {
    duq4_detail::check("asym_dual_quant_host",
                       duq4_asym_dual_quant(x, scale_1, zeros_1, scale_2, zeros_2, rows, colsSrc, colsDst, q, nullptr));
}
// :106-117
inline void asym_dual_dequant_host(const int32_t *q, const half *scale_row, const half *zeros_row,
                                   const half *scale_col_1, const half *zeros_col_1, const half *scale_col_2,
                                   const half *zeros_col_2, uint32_t rows, uint32_t cols, half *x) {
    duq4_detail::check("asym_dual_dequant_host",
                       duq4_asym_dual_dequant(q, scale_row, zeros_row, scale_col_1, zeros_col_1, scale_col_2, zeros_col_2,
                                              rows, cols, x, nullptr));
}
// :118-127
inline void asym_dequant_host_hprec(const int32_t *q, const float *scale_row, const float *zeros_row,
                                    const float *scale_col, const float *zeros_col, uint32_t rows, uint32_t cols,
                                    float *x) {
    duq4_detail::check("asym_dequant_host_hprec",
                       duq4_asym_dequant_hprec(q, scale_row, zeros_row, scale_col, zeros_col, rows, cols, x, nullptr));
}
