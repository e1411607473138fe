// Per-token int4 activation quantizers (HBM-bound).
//
// Two families:
//   *_given : scales (and zero-points) supplied by the caller -- the reference's
//             sym/asym/sym_dual/asym_dual quantize launchers (src/kernels/quant.cu:12-61,
//             :100-147 and src/kernels/quant2.cu:10-60, :102-156 of the reference).
//   *_fused : row statistics, scale(/zero) computation and coding in ONE pass over x, which
//             replaces the 4-7 torch kernels of the reference's quantizer modules
//             (qlinear4bit/nn/quantizer.py:13, :27-31) plus the quantize launch.
//
// Data movement: 128-bit loads of 8 halves per thread, 32-bit stores of 8 codes; in the
// fused kernels a CTA owns one token and keeps it in registers between the reduction and
// the coding pass, so x is read from HBM exactly once.
#include "duq_common.cuh"
#include "trace_range.h"
#include "quant_device.cuh"

namespace duq4 {

// ---- scales given: vector path (colsSrc % 8 == 0, colsDst == colsSrc/2, aligned) -------
template <int MODE>
__global__ void __launch_bounds__(256) quant_given_vec_kernel(const __half *__restrict__ x, const __half *__restrict__ s1,
                                                              const __half *__restrict__ z1,
                                                              const __half *__restrict__ s2,
                                                              const __half *__restrict__ z2, uint32_t rows,
                                                              uint32_t vec_per_row, uint8_t *__restrict__ q) {
    const size_t total = (size_t)rows * vec_per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t row = (uint32_t)(i / vec_per_row);
        uint32_t v = (uint32_t)(i - (size_t)row * vec_per_row);
        RowQ r = load_rowq<MODE>(s1, z1, s2, z2, row);
        uint4 d = __ldg(reinterpret_cast<const uint4 *>(x) + i);
        reinterpret_cast<uint32_t *>(q)[i] = code8<MODE>(d, v * 8, r);
    }
}

// ---- scales given: generic path, one thread per output byte (any colsSrc / colsDst) ----
template <int MODE>
__global__ void quant_given_scalar_kernel(const __half *__restrict__ x, const __half *__restrict__ s1,
                                          const __half *__restrict__ z1, const __half *__restrict__ s2,
                                          const __half *__restrict__ z2, uint32_t rows, uint32_t colsSrc,
                                          uint32_t colsDst, uint8_t *__restrict__ q) {
    const size_t total = (size_t)rows * colsDst;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t row = (uint32_t)(i / colsDst);
        uint32_t cd = (uint32_t)(i - (size_t)row * colsDst);
        if (cd * 2 >= colsSrc) continue;  // the reference leaves such bytes unwritten
        RowQ r = load_rowq<MODE>(s1, z1, s2, z2, row);
        uint32_t b = 0;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            uint32_t col = cd * 2 + k;
            if (col < colsSrc) b |= (uint32_t)(code_at<MODE>(x[(size_t)row * colsSrc + col], col, r) & 0xF) << (4 * k);
        }
        q[i] = (uint8_t)b;
    }
}

// One CTA (256 threads) per token; the token lives in VPT uint4 registers per thread.
// Requires cols % 8 == 0, cols <= 256*8*VPT, x 16-byte aligned.
// SiLU-gated MLP glue: h = half(half(silu(g)) * u), each step rounded to fp16 the way the torch
// composition `F.silu(gate) * up` rounds it (silu(x) = x / (1 + exp(-x)) evaluated in fp32).
__device__ __forceinline__ uint4 silu_mul8(const uint4 &g, const uint4 &u) {
    uint4 r;
    const __half *hg = reinterpret_cast<const __half *>(&g), *hu = reinterpret_cast<const __half *>(&u);
    __half *hr = reinterpret_cast<__half *>(&r);
#pragma unroll
    for (int k = 0; k < 8; ++k) hr[k] = silu_mul_one(hg[k], hu[k]);
    return r;
}

// SILU = false: the token is x[row, 0:cols] (in_stride = cols). SILU = true: the token is
// silu(x[row, 0:cols]) * x[row, up_off : up_off+cols] of a [rows, in_stride] gate/up tensor, i.e. the
// activation of a SiLU-gated MLP is formed, measured and quantized without ever being stored in fp16.
template <int MODE, int VPT, bool SILU = false, int NT = 256>
__global__ void __launch_bounds__(NT) quant_fused_vec_kernel(const __half *__restrict__ x, uint32_t rows, uint32_t cols,
                                                              float clip, uint8_t *__restrict__ q, __half *s1o,
                                                              __half *z1o, __half *s2o, __half *z2o, bool out8,
                                                              uint32_t in_stride = 0, uint32_t up_off = 0) {
    __shared__ float sm[NT / 32][4];
    const uint32_t nvec = cols >> 3;
    // Programmatic dependent launch (both instructions do nothing unless the launch carries the attribute): the
    // kernel that follows on the stream -- the small-M linear kernel, which streams weights before it needs these
    // codes -- may start right away; this kernel itself touches memory only after the stream's earlier work is done.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)row * (SILU ? in_stride : cols));
        uint4 d[VPT];
        Stats st;
        stats_init<MODE>(st);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            uint32_t v = threadIdx.x + i * NT;
            if (v < nvec) {
                d[i] = __ldg(xr + v);
                if (SILU) d[i] = silu_mul8(d[i], __ldg(xr + (up_off >> 3) + v));
            }
        }
        // Row statistics on the raw bit patterns: for symmetric schemes the integer maximum of
        // (bits & 0x7FFF) IS max|x|; asymmetric ones use fp16x2 min/max. The same integer maximum
        // tells whether the row holds an inf or NaN (>= 0x7C00), which sends it to the slow path.
        constexpr bool kDual = MODE == QSYM_DUAL || MODE == QASYM_DUAL;
        constexpr bool kAsym = MODE == QASYM || MODE == QASYM_DUAL;
        uint32_t am = 0, am_head = 0;
        __half2 hmx = __float2half2_rn(-INFINITY), hmn = __float2half2_rn(INFINITY);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            uint32_t v = threadIdx.x + i * NT;
            if (v < nvec) {
                const uint32_t w[4] = {d[i].x, d[i].y, d[i].z, d[i].w};
                if (kDual && v < 2) {   // columns 0..15 straddle the split at column 10: per element
                    const __half *h = reinterpret_cast<const __half *>(&d[i]);
#pragma unroll
                    for (int k = 0; k < 8; ++k) stats_add<MODE>(st, __half2float(h[k]), v * 8 + k);
#pragma unroll
                    for (int k = 0; k < 4; ++k) am_head = __vmaxu2(am_head, w[k] & 0x7FFF7FFFu);
                } else {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        am = __vmaxu2(am, w[k] & 0x7FFF7FFFu);
                        if (kAsym) {
                            const __half2 hv = *reinterpret_cast<const __half2 *>(&w[k]);
                            hmx = __hmax2(hmx, hv);
                            hmn = __hmin2(hmn, hv);
                        }
                    }
                }
            }
        }
        const uint32_t am16 = max(am & 0xFFFFu, am >> 16), amh16 = max(am_head & 0xFFFFu, am_head >> 16);
        if (kAsym) {
            st.b_hi = fmaxf(st.b_hi, fmaxf(__low2float(hmx), __high2float(hmx)));
            st.b_lo = fminf(st.b_lo, fminf(__low2float(hmn), __high2float(hmn)));
        } else if (am16 < 0x7C00u) {
            st.b_hi = fmaxf(st.b_hi, __half2float(__ushort_as_half((unsigned short)am16)));
        }
        // (also the barrier that protects sm[] against the previous row's readers)
        const bool row_special = __syncthreads_or((am16 >= 0x7C00u) || (amh16 >= 0x7C00u));
        if (row_special) {   // rare: redo the statistics element by element, as the slow path defines them
            stats_init<MODE>(st);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                uint32_t v = threadIdx.x + i * NT;
                if (v < nvec) {
                    const __half *h = reinterpret_cast<const __half *>(&d[i]);
#pragma unroll
                    for (int k = 0; k < 8; ++k) stats_add<MODE>(st, __half2float(h[k]), v * 8 + k);
                }
            }
        }
        stats_reduce<MODE>(st, sm);
        RowQ r = rowq_from_stats<MODE>(st, clip);
        if (threadIdx.x == 0) store_rowq<MODE>(r, row, s1o, z1o, s2o, z2o);
        const FastQ fq = make_fastq<MODE>(r, row_special);
        auto code = [&](const uint4 &dv, uint32_t v) -> uint32_t {
            if (fq.ok && !(kDual && v < 2)) return code8_fast<MODE>(dv, fq);
            return code8<MODE>(dv, v * 8, r);
        };
        if (!out8) {
            uint32_t *qr = reinterpret_cast<uint32_t *>(q + (size_t)row * (cols >> 1));
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                uint32_t v = threadIdx.x + i * NT;
                if (v < nvec) qr[v] = code(d[i], v);
            }
        } else {
            // Tensor-core-ready activations: one int8 (= 16 * code) per element, stored in the K
            // order the GEMM's in-kernel weight unpack produces. Inside each block of 128
            // elements, the low nibbles of 32 consecutive codes form bytes [32c, 32c+16) and the
            // high nibbles bytes [32c+16, 32c+32). The 8 codes of one vector are one packed word w;
            // (w<<4)&0xF0F0F0F0 holds its even elements, w&0xF0F0F0F0 its odd ones.
            uint8_t *qr = q + (size_t)row * cols;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                uint32_t v = threadIdx.x + i * NT;
                if (v < nvec) {
                    uint32_t w = code(d[i], v);
                    uint32_t off = (v >> 4) * 128 + ((v & 15) >> 2) * 32 + (v & 3) * 4;
                    *reinterpret_cast<uint32_t *>(qr + off) = (w << 4) & 0xF0F0F0F0u;
                    *reinterpret_cast<uint32_t *>(qr + off + 16) = w & 0xF0F0F0F0u;
                }
            }
        }
    }
}

// Generic fused path: any cols; two passes over the row (the second one hits L2).
template <int MODE>
__global__ void __launch_bounds__(256) quant_fused_scalar_kernel(const __half *__restrict__ x, uint32_t rows,
                                                                 uint32_t cols, float clip, uint8_t *__restrict__ q,
                                                                 __half *s1o, __half *z1o, __half *s2o, __half *z2o) {
    __shared__ float sm[8][4];
    const uint32_t cd = (cols + 1) >> 1;
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const __half *xr = x + (size_t)row * cols;
        Stats st;
        stats_init<MODE>(st);
        for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) stats_add<MODE>(st, __half2float(xr[c]), c);
        __syncthreads();
        stats_reduce<MODE>(st, sm);
        RowQ r = rowq_from_stats<MODE>(st, clip);
        if (threadIdx.x == 0) store_rowq<MODE>(r, row, s1o, z1o, s2o, z2o);
        for (uint32_t b = threadIdx.x; b < cd; b += blockDim.x) {
            uint32_t out = 0;
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                uint32_t col = b * 2 + k;
                if (col < cols) out |= (uint32_t)(code_at<MODE>(xr[col], col, r) & 0xF) << (4 * k);
            }
            q[(size_t)row * cd + b] = (uint8_t)out;
        }
    }
}

// 8-bit asymmetric quantizer of the reference's side path (src/kernels/quant.cu:245-266):
// fp32 divide, both terms pass through fp16 before the integer rounding.
__global__ void asym_quant8_kernel(const float *__restrict__ x, const float *__restrict__ scale,
                                   const float *__restrict__ zeros, uint32_t rows, uint32_t cols,
                                   int8_t *__restrict__ q) {
    const size_t total = (size_t)rows * cols;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t row = (uint32_t)(i / cols);
        float d = __fdiv_rn(x[i], scale[row]);
        int v = __half2int_rn(__float2half_rn(d)) + __half2int_rn(__float2half_rn(zeros[row]));
        q[i] = (int8_t)clampi(v, 0, kQmaxAsym8);
    }
}

// One-off re-layout of packed int4 weights [rows, K/2] into the tensor-core-ready int8 form [rows, K] that
// duq4_quantize_fused_i8 writes for activations: one int8 = 16 * code per element, K permuted inside 128-blocks.
// Thread = one 32-bit packed word (8 codes).
__global__ void __launch_bounds__(256) prelayout_i8_kernel(const uint32_t *__restrict__ w, uint32_t rows, uint32_t words_per_row,
                                                           uint8_t *__restrict__ out) {
    const size_t total = (size_t)rows * words_per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t row = (uint32_t)(i / words_per_row), v = (uint32_t)(i - (size_t)row * words_per_row);
        const uint32_t word = __ldg(w + i);
        uint8_t *qr = out + (size_t)row * words_per_row * 8;
        const uint32_t off = (v >> 4) * 128 + ((v & 15) >> 2) * 32 + (v & 3) * 4;
        *reinterpret_cast<uint32_t *>(qr + off) = (word << 4) & 0xF0F0F0F0u;
        *reinterpret_cast<uint32_t *>(qr + off + 16) = word & 0xF0F0F0F0u;
    }
}

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int grid_for(size_t work_items, int block) {
    size_t g = (work_items + block - 1) / block;
    const size_t cap = 148 * 16;  // 16 CTAs of 256 threads per SM cover the machine; then grid-stride
    if (g > cap) g = cap;
    if (g == 0) g = 1;
    return (int)g;
}

template <int MODE>
static int launch_given(const void *x, const void *s1, const void *z1, const void *s2, const void *z2, uint32_t rows,
                        uint32_t colsSrc, uint32_t colsDst, uint8_t *q, cudaStream_t st) {
    if (!x || !s1 || !q) return DUQ4_ERR_NULL;
    if ((MODE == QSYM_DUAL || MODE == QASYM_DUAL) && !s2) return DUQ4_ERR_NULL;
    if ((MODE == QASYM || MODE == QASYM_DUAL) && !z1) return DUQ4_ERR_NULL;
    if (MODE == QASYM_DUAL && !z2) return DUQ4_ERR_NULL;
    if (rows == 0 || colsSrc == 0 || colsDst == 0) return DUQ4_OK;  // empty input: nothing to do
    const __half *hx = (const __half *)x, *hs1 = (const __half *)s1, *hz1 = (const __half *)z1,
                 *hs2 = (const __half *)s2, *hz2 = (const __half *)z2;
    if (colsSrc % 8 == 0 && colsDst == colsSrc / 2 && aligned16(x) && (reinterpret_cast<uintptr_t>(q) & 3) == 0) {
        uint32_t vpr = colsSrc / 8;
        quant_given_vec_kernel<MODE><<<grid_for((size_t)rows * vpr, 256), 256, 0, st>>>(hx, hs1, hz1, hs2, hz2, rows, vpr, q);
    } else {
        quant_given_scalar_kernel<MODE><<<grid_for((size_t)rows * colsDst, 256), 256, 0, st>>>(hx, hs1, hz1, hs2, hz2, rows,
                                                                                              colsSrc, colsDst, q);
    }
    return launch_status();
}

template <int MODE>
static int launch_fused(const void *x, uint32_t rows, uint32_t cols, float clip, uint8_t *q, void *s1, void *z1, void *s2,
                        void *z2, cudaStream_t st, bool out8 = false) {
    if (!x || !q || !s1) return DUQ4_ERR_NULL;
    if ((MODE == QSYM_DUAL || MODE == QASYM_DUAL) && !s2) return DUQ4_ERR_NULL;
    if ((MODE == QASYM || MODE == QASYM_DUAL) && !z1) return DUQ4_ERR_NULL;
    if (MODE == QASYM_DUAL && !z2) return DUQ4_ERR_NULL;
    if (rows == 0) return DUQ4_OK;
    if (cols == 0) return DUQ4_ERR_SHAPE;
    const __half *hx = (const __half *)x;
    __half *a = (__half *)s1, *b = (__half *)z1, *c = (__half *)s2, *d = (__half *)z2;
    uint32_t grid = rows < 148u * 32u ? rows : 148u * 32u;
    bool vec = cols % 8 == 0 && aligned16(x) && (reinterpret_cast<uintptr_t>(q) & 3) == 0 && cols <= 256u * 8u * 16u;
    if (out8 && (!vec || cols % 64 != 0)) return DUQ4_ERR_SHAPE;
    // Few tokens (decode): the launch may begin while the stream's previous kernel drains (the kernel waits for it
    // before its first memory access), which takes the launch latency off the layer's critical path.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = rows <= 16 ? 1 : 0;
    const uint32_t zero = 0;
    cudaError_t e;
    if (!vec) {
        quant_fused_scalar_kernel<MODE><<<grid, 256, 0, st>>>(hx, rows, cols, clip, q, a, b, c, d);
        return launch_status();
    } else if (cols <= 256u * 8u * 2u) {
        e = cudaLaunchKernelEx(&cfg, quant_fused_vec_kernel<MODE, 2>, hx, rows, cols, clip, q, a, b, c, d, out8, zero, zero);
    } else if (cols <= 256u * 8u * 4u) {
        e = cudaLaunchKernelEx(&cfg, quant_fused_vec_kernel<MODE, 4>, hx, rows, cols, clip, q, a, b, c, d, out8, zero, zero);
    } else if (cols <= 256u * 8u * 8u) {
        e = cudaLaunchKernelEx(&cfg, quant_fused_vec_kernel<MODE, 8>, hx, rows, cols, clip, q, a, b, c, d, out8, zero, zero);
    } else {
        e = cudaLaunchKernelEx(&cfg, quant_fused_vec_kernel<MODE, 16>, hx, rows, cols, clip, q, a, b, c, d, out8, zero, zero);
    }
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return (int)e;
    }
    return launch_status();
}

// SiLU-gated variant (symmetric / asymmetric single-scale activations).
template <int MODE>
static int launch_silu(const void *gate_up, uint32_t rows, uint32_t inter, uint32_t ld, uint32_t up_off, float clip,
                       uint8_t *q, void *s1, void *z1, cudaStream_t st, bool out8) {
    if (!gate_up || !q || !s1 || (MODE == QASYM && !z1)) return DUQ4_ERR_NULL;
    if (rows == 0) return DUQ4_OK;
    if (inter == 0 || inter % 8 != 0 || ld % 8 != 0 || up_off % 8 != 0 || up_off + inter > ld || inter > 256u * 8u * 16u)
        return DUQ4_ERR_SHAPE;
    if (out8 && inter % 64 != 0) return DUQ4_ERR_SHAPE;
    if (!aligned16(gate_up) || (reinterpret_cast<uintptr_t>(q) & 3) != 0) return DUQ4_ERR_ALIGN;
    const __half *hx = (const __half *)gate_up;
    __half *a = (__half *)s1, *b = (__half *)z1;
    uint32_t grid = rows < 148u * 32u ? rows : 148u * 32u;
    // 512 threads per token: the SiLU evaluation is ALU-heavy, more warps per SM hide it better
    if (inter <= 512u * 8u * 1u)
        quant_fused_vec_kernel<MODE, 1, true, 512><<<grid, 512, 0, st>>>(hx, rows, inter, clip, q, a, b, nullptr, nullptr, out8, ld, up_off);
    else if (inter <= 512u * 8u * 2u)
        quant_fused_vec_kernel<MODE, 2, true, 512><<<grid, 512, 0, st>>>(hx, rows, inter, clip, q, a, b, nullptr, nullptr, out8, ld, up_off);
    else if (inter <= 512u * 8u * 4u)
        quant_fused_vec_kernel<MODE, 4, true, 512><<<grid, 512, 0, st>>>(hx, rows, inter, clip, q, a, b, nullptr, nullptr, out8, ld, up_off);
    else
        quant_fused_vec_kernel<MODE, 8, true, 512><<<grid, 512, 0, st>>>(hx, rows, inter, clip, q, a, b, nullptr, nullptr, out8, ld, up_off);
    return launch_status();
}

// Used by the fused linear entry point (abi.cu).
int quantize_fused_dispatch(int mode, const void *x, uint32_t rows, uint32_t cols, float clip, uint8_t *q, void *s1,
                            void *z1, void *s2, void *z2, cudaStream_t st, bool out8) {
    switch (mode) {
        case QSYM: return launch_fused<QSYM>(x, rows, cols, clip, q, s1, z1, s2, z2, st, out8);
        case QSYM_DUAL: return launch_fused<QSYM_DUAL>(x, rows, cols, clip, q, s1, z1, s2, z2, st, out8);
        case QASYM: return launch_fused<QASYM>(x, rows, cols, clip, q, s1, z1, s2, z2, st, out8);
        case QASYM_DUAL: return launch_fused<QASYM_DUAL>(x, rows, cols, clip, q, s1, z1, s2, z2, st, out8);
        default: return DUQ4_ERR_MODE;
    }
}

}  // namespace duq4

using namespace duq4;

extern "C" {

int duq4_sym_quant(const void *x, const void *scale, uint32_t rows, uint32_t colsSrc, uint32_t colsDst, uint8_t *q,
                   void *stream) {
    DUQ4_TRACE();
    return launch_given<QSYM>(x, scale, nullptr, nullptr, nullptr, rows, colsSrc, colsDst, q, (cudaStream_t)stream);
}
int duq4_sym_dual_quant(const void *x, const void *scale_1, const void *scale_2, uint32_t rows, uint32_t colsSrc,
                        uint32_t colsDst, uint8_t *q, void *stream) {
    DUQ4_TRACE();
    return launch_given<QSYM_DUAL>(x, scale_1, nullptr, scale_2, nullptr, rows, colsSrc, colsDst, q, (cudaStream_t)stream);
}
int duq4_asym_quant(const void *x, const void *scale, const void *zeros, uint32_t rows, uint32_t colsSrc,
                    uint32_t colsDst, uint8_t *q, void *stream) {
    DUQ4_TRACE();
    return launch_given<QASYM>(x, scale, zeros, nullptr, nullptr, rows, colsSrc, colsDst, q, (cudaStream_t)stream);
}
int duq4_asym_dual_quant(const void *x, const void *scale_1, const void *zeros_1, const void *scale_2,
                         const void *zeros_2, uint32_t rows, uint32_t colsSrc, uint32_t colsDst, uint8_t *q,
                         void *stream) {
    DUQ4_TRACE();
    return launch_given<QASYM_DUAL>(x, scale_1, zeros_1, scale_2, zeros_2, rows, colsSrc, colsDst, q, (cudaStream_t)stream);
}
int duq4_asym_quant_8bit(const float *x, const float *scale, const float *zeros, uint32_t rows, uint32_t cols,
                         int8_t *q, void *stream) {
    DUQ4_TRACE();
    if (!x || !scale || !zeros || !q) return DUQ4_ERR_NULL;
    if (rows == 0 || cols == 0) return DUQ4_OK;
    asym_quant8_kernel<<<grid_for((size_t)rows * cols, 256), 256, 0, (cudaStream_t)stream>>>(x, scale, zeros, rows, cols, q);
    return launch_status();
}

int duq4_weight_prelayout_i8(const uint8_t *W, uint32_t N, uint32_t K, int8_t *W_i8, void *stream) {
    DUQ4_TRACE();
    if (!W || !W_i8) return DUQ4_ERR_NULL;
    if (N == 0) return DUQ4_OK;
    if (K == 0 || K % 128 != 0) return DUQ4_ERR_SHAPE;
    if (!aligned16(W) || !aligned16(W_i8)) return DUQ4_ERR_ALIGN;
    prelayout_i8_kernel<<<grid_for((size_t)N * (K / 8), 256), 256, 0, (cudaStream_t)stream>>>((const uint32_t *)W, N, K / 8, (uint8_t *)W_i8);
    return launch_status();
}

int duq4_quantize_fused_i8(int mode, const void *x, uint32_t rows, uint32_t cols, float clip_ratio, int8_t *q_i8,
                           void *scale_1_out, void *zeros_1_out, void *scale_2_out, void *zeros_2_out, void *stream) {
    DUQ4_TRACE();
    return quantize_fused_dispatch(mode, x, rows, cols, clip_ratio, (uint8_t *)q_i8, scale_1_out, zeros_1_out, scale_2_out,
                                   zeros_2_out, (cudaStream_t)stream, true);
}

int duq4_silu_mul_quantize_fused(int mode, const void *gate_up, uint32_t rows, uint32_t inter, uint32_t ld,
                                 uint32_t up_offset, float clip_ratio, void *q, int q_is_int8, void *scale_out,
                                 void *zeros_out, void *stream) {
    DUQ4_TRACE();
    cudaStream_t st = (cudaStream_t)stream;
    if (mode == QSYM)
        return launch_silu<QSYM>(gate_up, rows, inter, ld, up_offset, clip_ratio, (uint8_t *)q, scale_out, nullptr, st, q_is_int8 != 0);
    if (mode == QASYM)
        return launch_silu<QASYM>(gate_up, rows, inter, ld, up_offset, clip_ratio, (uint8_t *)q, scale_out, zeros_out, st, q_is_int8 != 0);
    return DUQ4_ERR_MODE;
}

int duq4_quantize_sym_fused(const void *x, uint32_t rows, uint32_t cols, float clip_ratio, uint8_t *q, void *scale_out,
                            void *stream) {
    DUQ4_TRACE();
    return launch_fused<QSYM>(x, rows, cols, clip_ratio, q, scale_out, nullptr, nullptr, nullptr, (cudaStream_t)stream);
}
int duq4_quantize_asym_fused(const void *x, uint32_t rows, uint32_t cols, uint8_t *q, void *scale_out, void *zeros_out,
                             void *stream) {
    DUQ4_TRACE();
    return launch_fused<QASYM>(x, rows, cols, 1.0f, q, scale_out, zeros_out, nullptr, nullptr, (cudaStream_t)stream);
}
int duq4_quantize_sym_dual_fused(const void *x, uint32_t rows, uint32_t cols, float clip_ratio, uint8_t *q,
                                 void *scale_1_out, void *scale_2_out, void *stream) {
    DUQ4_TRACE();
    return launch_fused<QSYM_DUAL>(x, rows, cols, clip_ratio, q, scale_1_out, nullptr, scale_2_out, nullptr,
                                   (cudaStream_t)stream);
}
int duq4_quantize_asym_dual_fused(const void *x, uint32_t rows, uint32_t cols, uint8_t *q, void *scale_1_out,
                                  void *zeros_1_out, void *scale_2_out, void *zeros_2_out, void *stream) {
    DUQ4_TRACE();
    return launch_fused<QASYM_DUAL>(x, rows, cols, 1.0f, q, scale_1_out, zeros_1_out, scale_2_out, zeros_2_out,
                                    (cudaStream_t)stream);
}

}  // extern "C"
