// Stand-alone dequantizers of an int32 accumulator tensor (HBM-bound, 4 B in + 2 B out per
// element). They exist for callers that keep the reference's three-call sequence
// matmul -> *_dequant -> bias; the fused linear kernels apply the same arithmetic in their
// epilogue and never materialise the int32 tensor. Reference kernels:
// src/kernels/quant.cu:64-97 (sym), :150-188 (asym), :191-239 (batched asym), :282-323
// (fp32 "hprec"); src/kernels/quant2.cu:63-98 (sym dual), :159-208 (asym dual).
#include "duq_common.cuh"
#include "trace_range.h"

namespace duq4 {

// Vector path: each thread turns 8 accumulators (two 128-bit loads) into 8 halves (one
// 128-bit store). Requires cols % 8 == 0 and 16-byte aligned q / x.
__global__ void __launch_bounds__(256) dequant_vec_kernel(const int32_t *__restrict__ q, EpiParams p, uint32_t batches,
                                                          uint32_t rows, uint32_t cols, __half *__restrict__ x) {
    const uint32_t vpr = cols >> 3;
    const size_t total = (size_t)batches * rows * vpr;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t v = (uint32_t)(i % vpr);
        size_t br = i / vpr;  // batch*rows + row
        uint32_t row = (uint32_t)(br % rows);
        uint32_t b = (uint32_t)(br / rows);
        EpiParams pb = p;
        pb.s_row += (size_t)b * p.row_vec_stride;
        if (pb.z_row) pb.z_row += (size_t)b * p.row_vec_stride;
        size_t co = (size_t)b * p.col_vec_stride;
        if (pb.s_col1) pb.s_col1 += co;
        if (pb.z_col1) pb.z_col1 += co;
        if (pb.s_col2) pb.s_col2 += co;
        if (pb.z_col2) pb.z_col2 += co;
        const int4 *src = reinterpret_cast<const int4 *>(q + (br * cols)) + v * 2;
        int4 a0 = __ldg(src), a1 = __ldg(src + 1);
        int acc[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        __half sr = pb.s_row[row];
        __half zr = pb.z_row ? pb.z_row[row] : __ushort_as_half(0);
        uint4 out;
        __half *o = reinterpret_cast<__half *>(&out);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            ColTerms t = load_col_terms(pb, v * 8 + k);
            o[k] = dequant_one(p.mode, acc[k], sr, zr, t);
        }
        reinterpret_cast<uint4 *>(x + br * cols)[v] = out;
    }
}

__global__ void __launch_bounds__(256) dequant_scalar_kernel(const int32_t *__restrict__ q, EpiParams p, uint32_t batches,
                                                             uint32_t rows, uint32_t cols, __half *__restrict__ x) {
    const size_t total = (size_t)batches * rows * cols;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t col = (uint32_t)(i % cols);
        size_t br = i / cols;
        uint32_t row = (uint32_t)(br % rows);
        uint32_t b = (uint32_t)(br / rows);
        EpiParams pb = p;
        size_t co = (size_t)b * p.col_vec_stride;
        if (pb.s_col1) pb.s_col1 += co;
        if (pb.z_col1) pb.z_col1 += co;
        if (pb.s_col2) pb.s_col2 += co;
        if (pb.z_col2) pb.z_col2 += co;
        __half sr = p.s_row[(size_t)b * p.row_vec_stride + row];
        __half zr = p.z_row ? p.z_row[(size_t)b * p.row_vec_stride + row] : __ushort_as_half(0);
        ColTerms t = load_col_terms(pb, col);
        x[i] = dequant_one(p.mode, q[i], sr, zr, t);
    }
}

// fp32 dequant of the 8-bit side path; explicit _rn operations so nothing is contracted.
__global__ void __launch_bounds__(256) dequant_hprec_kernel(const int32_t *__restrict__ q, const float *__restrict__ sr,
                                                            const float *__restrict__ zr, const float *__restrict__ sc,
                                                            const float *__restrict__ zc, uint32_t rows, uint32_t cols,
                                                            float *__restrict__ x) {
    const size_t total = (size_t)rows * cols;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t col = (uint32_t)(i % cols), row = (uint32_t)(i / cols);
        float s = __fmul_rn(sr[row], sc[col]);
        float z = __fadd_rn(zr[row], zc[col]);
        x[i] = __fmul_rn(s, __fsub_rn((float)q[i], z));
    }
}

static int grid_for(size_t items) {
    size_t g = (items + 255) / 256;
    if (g > 148u * 16u) g = 148u * 16u;
    return g ? (int)g : 1;
}

int dequant_launch(const int32_t *q, const EpiParams &p, uint32_t batches, uint32_t rows, uint32_t cols, void *x,
                   cudaStream_t st) {
    if (!q || !x || !p.s_row || !p.s_col1) return DUQ4_ERR_NULL;
    if ((p.mode == DUQ4_MODE_ASYM || p.mode == DUQ4_MODE_ASYM_DUAL) && (!p.z_row || !p.z_col1)) return DUQ4_ERR_NULL;
    if ((p.mode == DUQ4_MODE_SYM_DUAL || p.mode == DUQ4_MODE_ASYM_DUAL) && !p.s_col2) return DUQ4_ERR_NULL;
    if (p.mode == DUQ4_MODE_ASYM_DUAL && !p.z_col2) return DUQ4_ERR_NULL;
    if (batches == 0 || rows == 0 || cols == 0) return DUQ4_OK;
    bool vec = cols % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    if (vec)
        dequant_vec_kernel<<<grid_for((size_t)batches * rows * (cols / 8)), 256, 0, st>>>(q, p, batches, rows, cols, (__half *)x);
    else
        dequant_scalar_kernel<<<grid_for((size_t)batches * rows * cols), 256, 0, st>>>(q, p, batches, rows, cols, (__half *)x);
    return launch_status();
}

static EpiParams make(int mode, const void *sr, const void *zr, const void *sc1, const void *zc1, const void *sc2,
                      const void *zc2) {
    EpiParams p{};
    p.mode = mode;
    p.s_row = (const __half *)sr;
    p.z_row = (const __half *)zr;
    p.s_col1 = (const __half *)sc1;
    p.z_col1 = (const __half *)zc1;
    p.s_col2 = (const __half *)sc2;
    p.z_col2 = (const __half *)zc2;
    return p;
}

}  // namespace duq4

using namespace duq4;

extern "C" {

int duq4_sym_dequant(const int32_t *q, const void *scale_row, const void *scale_col, uint32_t rows, uint32_t cols, void *x,
                     void *stream) {
    DUQ4_TRACE();
    return dequant_launch(q, make(DUQ4_MODE_SYM, scale_row, nullptr, scale_col, nullptr, nullptr, nullptr), 1, rows, cols, x,
                          (cudaStream_t)stream);
}
int duq4_sym_dual_dequant(const int32_t *q, const void *scale_row, const void *scale_col_1, const void *scale_col_2,
                          uint32_t rows, uint32_t cols, void *x, void *stream) {
    DUQ4_TRACE();
    return dequant_launch(q, make(DUQ4_MODE_SYM_DUAL, scale_row, nullptr, scale_col_1, nullptr, scale_col_2, nullptr), 1, rows,
                          cols, x, (cudaStream_t)stream);
}
int duq4_asym_dequant(const int32_t *q, const void *scale_row, const void *zeros_row, const void *scale_col,
                      const void *zeros_col, uint32_t rows, uint32_t cols, void *x, void *stream) {
    DUQ4_TRACE();
    return dequant_launch(q, make(DUQ4_MODE_ASYM, scale_row, zeros_row, scale_col, zeros_col, nullptr, nullptr), 1, rows, cols,
                          x, (cudaStream_t)stream);
}
int duq4_asym_dual_dequant(const int32_t *q, const void *scale_row, const void *zeros_row, const void *scale_col_1,
                           const void *zeros_col_1, const void *scale_col_2, const void *zeros_col_2, uint32_t rows,
                           uint32_t cols, void *x, void *stream) {
    DUQ4_TRACE();
    return dequant_launch(q, make(DUQ4_MODE_ASYM_DUAL, scale_row, zeros_row, scale_col_1, zeros_col_1, scale_col_2, zeros_col_2),
                          1, rows, cols, x, (cudaStream_t)stream);
}
int duq4_asym_batch_dequant(const int32_t *q, const void *scale_row, const void *zeros_row, const void *scale_col,
                            const void *zeros_col, uint32_t batches, uint32_t rows, uint32_t cols, void *x,
                            void *stream) {
    DUQ4_TRACE();
    EpiParams p = make(DUQ4_MODE_ASYM, scale_row, zeros_row, scale_col, zeros_col, nullptr, nullptr);
    p.row_vec_stride = rows;
    p.col_vec_stride = cols;
    return dequant_launch(q, p, batches, rows, cols, x, (cudaStream_t)stream);
}
int duq4_asym_dequant_hprec(const int32_t *q, const float *scale_row, const float *zeros_row, const float *scale_col,
                            const float *zeros_col, uint32_t rows, uint32_t cols, float *x, void *stream) {
    DUQ4_TRACE();
    if (!q || !scale_row || !zeros_row || !scale_col || !zeros_col || !x) return DUQ4_ERR_NULL;
    if (rows == 0 || cols == 0) return DUQ4_OK;
    dequant_hprec_kernel<<<grid_for((size_t)rows * cols), 256, 0, (cudaStream_t)stream>>>(q, scale_row, zeros_row, scale_col,
                                                                                         zeros_col, rows, cols, x);
    return launch_status();
}

}  // extern "C"
