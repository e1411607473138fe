// Pieces of the K-sharded ("row-parallel") W4A4 layer: per-token statistics of a K slice, the fused quantizer with
// the (rank-reduced) statistics given, and the owner's reduce + dequant + gather of the int32 partial accumulators.
// The reference has no multi-GPU code; the arithmetic is that of its quantizer modules (qlinear4bit/nn/quantizer.py:
// 10-16, :24-35), quantize kernels (src/kernels/quant.cu:12-45, :100-132) and dequant kernels (:64-81, :150-169), so
// that the sharded layer equals the unsharded one bit for bit.
#include "duq_common.cuh"
#include "trace_range.h"
#include "quant_device.cuh"

namespace duq4 {

// One CTA of 256 threads per token. MODE: QSYM (stat_a = max|x|) or QASYM (stat_a = min, stat_b = max); NaNs are
// skipped and infinities kept, as the fused quantizers do.
template <int MODE>
__global__ void __launch_bounds__(256) row_stats_kernel(const __half *__restrict__ x, uint32_t rows, uint32_t cols, __half *stat_a,
                                                        __half *stat_b) {
    __shared__ float sm[8][4];
    const uint32_t nvec = cols >> 3;
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)row * cols);
        uint32_t amax = 0;
        __half2 hmx = __float2half2_rn(-INFINITY), hmn = __float2half2_rn(INFINITY);
        for (uint32_t v = threadIdx.x; v < nvec; v += blockDim.x) {
            const uint4 d = __ldg(xr + v);
            const uint32_t w[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (MODE == QASYM) {
                    const __half2 hv = *reinterpret_cast<const __half2 *>(&w[k]);
                    hmx = __hmax2(hmx, hv);
                    hmn = __hmin2(hmn, hv);
                } else {
                    const uint32_t a = w[k] & 0x7FFF7FFFu;
                    amax = __vmaxu2(amax, a & ~__vcmpgtu2(a, 0x7C007C00u));
                }
            }
        }
        Stats st;
        stats_init<MODE>(st);
        if (MODE == QASYM) {
            st.b_hi = fmaxf(__low2float(hmx), __high2float(hmx));
            st.b_lo = fminf(__low2float(hmn), __high2float(hmn));
        } else {
            st.b_hi = __half2float(__ushort_as_half((unsigned short)max(amax & 0xFFFFu, amax >> 16)));
        }
        __syncthreads();   // sm[] of the previous row has been read
        stats_reduce<MODE>(st, sm);
        if (threadIdx.x == 0) {
            if (MODE == QASYM) {
                stat_a[row] = __float2half_rn(st.b_lo);   // exact: the extrema are fp16 values
                stat_b[row] = __float2half_rn(st.b_hi);
            } else {
                stat_a[row] = __float2half_rn(st.b_hi);
            }
        }
    }
}

// The fused quantizer's second half with the statistics given: scale (/ zero-point) from the global statistics, codes
// of this rank's slice as tensor-core-ready int8 (the layout of quant_fused_vec_kernel's out8 branch).
template <int MODE>
__global__ void __launch_bounds__(256) quant_from_stats_i8_kernel(const __half *__restrict__ x, uint32_t rows, uint32_t cols,
                                                                  const __half *__restrict__ stat_a, const __half *__restrict__ stat_b,
                                                                  float clip, uint8_t *__restrict__ q, __half *scale_out, __half *zeros_out) {
    const uint32_t nvec = cols >> 3;
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)row * cols);
        Stats st;
        stats_init<MODE>(st);
        if (MODE == QASYM) {
            st.b_lo = __half2float(stat_a[row]);
            st.b_hi = __half2float(stat_b[row]);
        } else {
            st.b_hi = __half2float(stat_a[row]);
        }
        const RowQ r = rowq_from_stats<MODE>(st, clip);
        if (threadIdx.x == 0) {
            scale_out[row] = r.s1;
            if (MODE == QASYM) zeros_out[row] = r.z1;
        }
        // a slice holding an inf or NaN takes the element-by-element coding path, as in the fused kernel; whether the
        // short path is usable is decided per CTA from the slice it codes (both paths give the same codes on finite data)
        uint32_t am = 0;
        for (uint32_t v = threadIdx.x; v < nvec; v += blockDim.x) {
            const uint4 d = __ldg(xr + v);
            am = __vmaxu2(am, __vmaxu2(__vmaxu2(d.x & 0x7FFF7FFFu, d.y & 0x7FFF7FFFu), __vmaxu2(d.z & 0x7FFF7FFFu, d.w & 0x7FFF7FFFu)));
        }
        const bool special = __syncthreads_or(max(am & 0xFFFFu, am >> 16) >= 0x7C00u);
        const FastQ fq = make_fastq<MODE>(r, special);
        uint8_t *qr = q + (size_t)row * cols;
        for (uint32_t v = threadIdx.x; v < nvec; v += blockDim.x) {
            const uint4 d = __ldg(xr + v);
            const uint32_t w = fq.ok ? code8_fast<MODE>(d, fq) : code8<MODE>(d, v * 8, r);
            const uint32_t off = (v >> 4) * 128 + ((v & 15) >> 2) * 32 + (v & 3) * 4;
            *reinterpret_cast<uint32_t *>(qr + off) = (w << 4) & 0xF0F0F0F0u;
            *reinterpret_cast<uint32_t *>(qr + off + 16) = w & 0xF0F0F0F0u;
        }
    }
}

// Owner's pass: sum of the partial slabs, one dequant, fp16 result to every rank's buffer. A thread handles 8
// consecutive columns of one row.
__global__ void __launch_bounds__(256) reduce_dequant_gather_kernel(const int32_t *__restrict__ slabs, uint32_t n_slabs, size_t slab_stride,
                                                                    uint32_t row0, uint32_t rows, uint32_t N, EpiParams p, __half *out) {
    const uint32_t vec_per_row = N >> 3;
    const size_t total = (size_t)rows * vec_per_row;
    const OutBases ob = out_bases(p, out);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / vec_per_row), c0 = (uint32_t)(i - (size_t)r * vec_per_row) * 8;
        int acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (uint32_t s = 0; s < n_slabs; ++s) {
            const int4 *src = reinterpret_cast<const int4 *>(slabs + s * slab_stride + (size_t)r * N + c0);
            const int4 a = __ldcg(src), b = __ldcg(src + 1);   // written by other GPUs: read through L2
            acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
            acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
        }
        const uint32_t m = row0 + r;
        const __half sr = p.s_row[m];
        const __half zr = p.z_row ? p.z_row[m] : __ushort_as_half(0);
        __align__(16) __half o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const ColTerms t = load_col_terms(p, c0 + j);
            o[j] = dequant_one(p.mode, acc[j], sr, zr, t);
        }
        const size_t off = (size_t)m * p.ldo + c0;
#pragma unroll
        for (int pi = 0; pi < DUQ4_MAX_OUT_PEERS; ++pi)
            if (pi < ob.n) *reinterpret_cast<uint4 *>(ob.base[pi] + off) = *reinterpret_cast<const uint4 *>(o);
    }
}

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace duq4

using namespace duq4;

extern "C" {

int duq4_row_stats(int mode, const void *x, uint32_t rows, uint32_t cols, void *stat_a, void *stat_b, void *stream) {
    DUQ4_TRACE();
    if (!x || !stat_a || (mode == DUQ4_MODE_ASYM && !stat_b)) return DUQ4_ERR_NULL;
    if (mode != DUQ4_MODE_SYM && mode != DUQ4_MODE_ASYM) return DUQ4_ERR_MODE;
    if (rows == 0) return DUQ4_OK;
    if (cols == 0 || cols % 8 != 0) return DUQ4_ERR_SHAPE;
    if (!aligned16(x)) return DUQ4_ERR_ALIGN;
    const uint32_t grid = rows < 148u * 32u ? rows : 148u * 32u;
    if (mode == DUQ4_MODE_SYM)
        row_stats_kernel<QSYM><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half *)x, rows, cols, (__half *)stat_a, (__half *)stat_b);
    else
        row_stats_kernel<QASYM><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half *)x, rows, cols, (__half *)stat_a, (__half *)stat_b);
    return launch_status();
}

int duq4_quantize_i8_from_stats(int mode, const void *x, uint32_t rows, uint32_t cols, const void *stat_a, const void *stat_b,
                                float clip_ratio, int8_t *q_i8, void *scale_out, void *zeros_out, void *stream) {
    DUQ4_TRACE();
    // cols == 0 (a rank without a K slice): only the per-token terms are derived; x and q_i8 may then be NULL
    if ((cols && (!x || !q_i8)) || !stat_a || !scale_out || (mode == DUQ4_MODE_ASYM && (!stat_b || !zeros_out))) return DUQ4_ERR_NULL;
    if (mode != DUQ4_MODE_SYM && mode != DUQ4_MODE_ASYM) return DUQ4_ERR_MODE;
    if (rows == 0) return DUQ4_OK;
    if (cols % 64 != 0) return DUQ4_ERR_SHAPE;
    if (cols && (!aligned16(x) || (reinterpret_cast<uintptr_t>(q_i8) & 3) != 0)) return DUQ4_ERR_ALIGN;
    const uint32_t grid = rows < 148u * 32u ? rows : 148u * 32u;
    if (mode == DUQ4_MODE_SYM)
        quant_from_stats_i8_kernel<QSYM><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half *)x, rows, cols, (const __half *)stat_a,
                                                                               (const __half *)stat_b, clip_ratio, (uint8_t *)q_i8,
                                                                               (__half *)scale_out, (__half *)zeros_out);
    else
        quant_from_stats_i8_kernel<QASYM><<<grid, 256, 0, (cudaStream_t)stream>>>((const __half *)x, rows, cols, (const __half *)stat_a,
                                                                                (const __half *)stat_b, 1.0f, (uint8_t *)q_i8,
                                                                                (__half *)scale_out, (__half *)zeros_out);
    return launch_status();
}

int duq4_reduce_dequant_gather(const int32_t *slabs, uint32_t n_slabs, uint32_t rows_per_slab, uint32_t row0, uint32_t rows, uint32_t N,
                               const duq4_epilogue *epi, void *out, void *stream) {
    DUQ4_TRACE();
    if (!slabs || !epi) return DUQ4_ERR_NULL;
    if (epi->mode < DUQ4_MODE_SYM || epi->mode > DUQ4_MODE_ASYM_DUAL) return DUQ4_ERR_MODE;
    if (rows == 0 || N == 0) return DUQ4_OK;
    if (n_slabs == 0 || rows > rows_per_slab || N % 8 != 0) return DUQ4_ERR_SHAPE;
    const bool asym = epi->mode == DUQ4_MODE_ASYM || epi->mode == DUQ4_MODE_ASYM_DUAL;
    const bool dual = epi->mode == DUQ4_MODE_SYM_DUAL || epi->mode == DUQ4_MODE_ASYM_DUAL;
    if (!epi->scale_row || !epi->scale_col_1 || (asym && (!epi->zeros_row || !epi->zeros_col_1)) || (dual && !epi->scale_col_2) ||
        (epi->mode == DUQ4_MODE_ASYM_DUAL && !epi->zeros_col_2))
        return DUQ4_ERR_NULL;
    if (!out && !epi->n_out_peers) return DUQ4_ERR_NULL;
    if (epi->n_out_peers > DUQ4_MAX_OUT_PEERS) return DUQ4_ERR_SHAPE;
    if (epi->out_rows_per_owner) return DUQ4_ERR_MODE;   // this entry point replicates the rows it owns
    EpiParams p{};
    p.mode = epi->mode;
    p.col_offset = epi->col_offset;
    p.s_row = (const __half *)epi->scale_row;
    p.z_row = asym ? (const __half *)epi->zeros_row : nullptr;
    p.s_col1 = (const __half *)epi->scale_col_1;
    p.z_col1 = (const __half *)epi->zeros_col_1;
    p.s_col2 = (const __half *)epi->scale_col_2;
    p.z_col2 = (const __half *)epi->zeros_col_2;
    p.bias = (const __half *)epi->bias;
    p.ldo = epi->ldo ? epi->ldo : N;
    if (p.ldo < N || p.ldo % 8 != 0) return DUQ4_ERR_SHAPE;
    p.n_peers = epi->n_out_peers;
    for (uint32_t i = 0; i < epi->n_out_peers; ++i) {
        if (!epi->out_peers[i]) return DUQ4_ERR_NULL;
        if (!aligned16(epi->out_peers[i])) return DUQ4_ERR_ALIGN;
        p.peers[i] = (__half *)epi->out_peers[i];
    }
    if (!aligned16(slabs) || (out && !aligned16(out))) return DUQ4_ERR_ALIGN;
    const size_t total = (size_t)rows * (N / 8);
    size_t grid = (total + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    reduce_dequant_gather_kernel<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(slabs, n_slabs, (size_t)rows_per_slab * N, row0, rows, N, p,
                                                                                   (__half *)out);
    return launch_status();
}

}  // extern "C"
