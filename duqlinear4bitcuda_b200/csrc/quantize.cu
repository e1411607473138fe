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

namespace duq4 {

enum { QSYM = DUQ4_MODE_SYM, QSYM_DUAL = DUQ4_MODE_SYM_DUAL, QASYM = DUQ4_MODE_ASYM, QASYM_DUAL = DUQ4_MODE_ASYM_DUAL };

struct RowQ {  // per-row quantization terms
    __half s1, z1, s2, z2;
    int zi1;  // rn(z1) for the single-scale asymmetric scheme
};

template <int MODE>
__device__ __forceinline__ int code_at(__half x, uint32_t col, const RowQ &r) {
    if (MODE == QSYM) return code_sym(x, r.s1);
    if (MODE == QSYM_DUAL) return code_sym(x, col < kColK ? r.s1 : r.s2);
    if (MODE == QASYM) return code_asym(x, r.s1, r.zi1);
    return code_asym_dual(x, col < kColK ? r.s1 : r.s2, col < kColK ? r.z1 : r.z2);
}

// 8 halves (one uint4) starting at column col0 -> 8 nibbles (one uint32), low nibble first.
template <int MODE>
__device__ __forceinline__ uint32_t code8(const uint4 &v, uint32_t col0, const RowQ &r) {
    const __half *h = reinterpret_cast<const __half *>(&v);
    uint32_t out = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) out |= (uint32_t)(code_at<MODE>(h[i], col0 + i, r) & 0xF) << (4 * i);
    return out;
}

template <int MODE>
__device__ __forceinline__ RowQ load_rowq(const __half *s1, const __half *z1, const __half *s2, const __half *z2,
                                          uint32_t row) {
    RowQ r;
    r.s1 = s1[row];
    r.z1 = r.z2 = r.s2 = __ushort_as_half(0);
    r.zi1 = 0;
    if (MODE == QSYM_DUAL || MODE == QASYM_DUAL) r.s2 = s2[row];
    if (MODE == QASYM || MODE == QASYM_DUAL) r.z1 = z1[row];
    if (MODE == QASYM_DUAL) r.z2 = z2[row];
    if (MODE == QASYM) r.zi1 = __half2int_rn(r.z1);
    return r;
}

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

// ---- fast coding path of the fused kernels -------------------------------------------------
// Same codes as code8<MODE>, far fewer instructions (the fused kernel is otherwise issue-bound,
// not HBM-bound). Valid for a row whose scales are finite and non-zero, whose zero-points are
// finite (|rint(z)| <= 400 for the single-scale asymmetric scheme) and which contains no
// inf/NaN -- everything else takes code8<MODE>.
//   * __hdiv(x, s) is half(rcp.approx.ftz(float(s)) * float(x)) plus a refinement that only
//     fires for quotients below 8.6e-6, which round to the same code either way; the reciprocal
//     is taken once per row with the same instruction.
//   * rounding to integer and clamping happen in fp16x2: adding 1024 + offset to a value already
//     clamped to a 16-wide integer window rounds it to nearest-even exactly like
//     __half2int_rn, and leaves the code in the low four bits of each half.
__device__ __forceinline__ float rcp_approx_ftz(float b) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(b));
    return r;
}
struct FastQ {
    float r1, r2;          // reciprocals of scale set 1 / 2
    __half2 z1, z2;        // zero-point terms, duplicated in both halves (rint(z) for QASYM)
    bool ok;
};
__device__ __forceinline__ bool finite_nonzero(__half h) {
    const unsigned short b = __half_as_ushort(h) & 0x7FFFu;
    return b != 0 && b < 0x7C00u;
}
__device__ __forceinline__ bool finite_h(__half h) { return (__half_as_ushort(h) & 0x7FFFu) < 0x7C00u; }

template <int MODE>
__device__ __forceinline__ FastQ make_fastq(const RowQ &r, bool row_special) {
    FastQ f;
    f.ok = !row_special && finite_nonzero(r.s1);
    f.r1 = rcp_approx_ftz(__half2float(r.s1));
    f.r2 = f.r1;
    f.z1 = f.z2 = __float2half2_rn(0.f);
    if (MODE == QSYM_DUAL || MODE == QASYM_DUAL) {
        f.ok = f.ok && finite_nonzero(r.s2);
        f.r2 = rcp_approx_ftz(__half2float(r.s2));
    }
    if (MODE == QASYM) {
        f.ok = f.ok && finite_h(r.z1) && fabsf(__half2float(r.z1)) <= 400.f;
        f.z1 = __float2half2_rn(rintf(__half2float(r.z1)));
    }
    if (MODE == QASYM_DUAL) {
        f.ok = f.ok && finite_h(r.z1) && finite_h(r.z2);
        f.z1 = __half2half2(r.z1);
        f.z2 = __half2half2(r.z2);
    }
    return f;
}

// One 32-bit word (two halves) -> two codes in bits [0,4) and [16,20).
template <int MODE>
__device__ __forceinline__ uint32_t code2_fast(uint32_t w, float rcp, __half2 z) {
    const __half2 h = *reinterpret_cast<const __half2 *>(&w);
    const float2 f = __half22float2(h);
    const __half2 q = __floats2half2_rn(__fmul_rn(rcp, f.x), __fmul_rn(rcp, f.y));
    __half2 t;
    if (MODE == QSYM || MODE == QSYM_DUAL) {
        const __half2 c = __hmin2(__hmax2(q, __float2half2_rn(-8.f)), __float2half2_rn(6.f));
        t = __hadd2(c, __float2half2_rn(1032.f));            // 0x6400 + (code + 8)
    } else if (MODE == QASYM) {
        const __half2 c = __hmin2(__hmax2(q, __float2half2_rn(-500.f)), __float2half2_rn(500.f));
        const __half2 s = __hadd2(__hadd2(c, __float2half2_rn(1536.f)), z);   // rint(x/s) + rint(z) + 1536
        t = __hmin2(__hmax2(s, __float2half2_rn(1536.f)), __float2half2_rn(1551.f));   // 0x6600 + code
    } else {
        const __half2 c = __hmin2(__hmax2(__hadd2(q, z), __float2half2_rn(0.f)), __float2half2_rn(15.f));
        t = __hadd2(c, __float2half2_rn(1024.f));            // 0x6400 + code
    }
    // each half is 0x6400 (or 0x6600) + code: the code is the low BYTE of the half, the high byte is constant
    return *reinterpret_cast<const uint32_t *>(&t);
}

// 8 halves -> 8 nibbles, low nibble first. col0 >= 16 for the dual schemes (set 2 only).
template <int MODE>
__device__ __forceinline__ uint32_t code8_fast(const uint4 &v, const FastQ &f) {
    const bool dual = MODE == QSYM_DUAL || MODE == QASYM_DUAL;
    const float rcp = dual ? f.r2 : f.r1;
    const __half2 z = dual ? f.z2 : f.z1;
    const uint32_t a = code2_fast<MODE>(v.x, rcp, z), b = code2_fast<MODE>(v.y, rcp, z);
    const uint32_t c = code2_fast<MODE>(v.z, rcp, z), d = code2_fast<MODE>(v.w, rcp, z);
    // Each word holds its two codes in bytes 0 and 2. Gather the four code bytes of two words with one byte
    // permute ([c0, c1, c2, c3], one nibble each), fold odd bytes onto even ones (x | x >> 4 puts c1 into the
    // high nibble of byte 0 and c3 into that of byte 2), and gather the four finished bytes of the two halves.
    const uint32_t ab = __byte_perm(a, b, 0x6420), cd = __byte_perm(c, d, 0x6420);
    uint32_t out = __byte_perm(ab | (ab >> 4), cd | (cd >> 4), 0x6420);
    if (MODE == QSYM || MODE == QSYM_DUAL) out ^= 0x88888888u;   // (code + 8) -> two's complement nibble
    return out;
}

// ---- fused ---------------------------------------------------------------------------
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Row statistics gathered by one thread. Symmetric schemes track max|x| (a: columns < 10
// for the dual scheme, b: the rest / everything); asymmetric ones track min and max.
struct Stats {
    float a_hi, a_lo, b_hi, b_lo;
};
template <int MODE>
__device__ __forceinline__ void stats_init(Stats &s) {
    if (MODE == QSYM || MODE == QSYM_DUAL) {
        s.a_hi = s.b_hi = 0.f;
        s.a_lo = s.b_lo = 0.f;
    } else {
        s.a_hi = s.b_hi = -INFINITY;
        s.a_lo = s.b_lo = INFINITY;
    }
}
template <int MODE>
__device__ __forceinline__ void stats_add(Stats &s, float v, uint32_t col) {
    if (MODE == QSYM) {
        s.b_hi = fmaxf(s.b_hi, fabsf(v));
    } else if (MODE == QSYM_DUAL) {
        if (col < kColK) s.a_hi = fmaxf(s.a_hi, fabsf(v)); else s.b_hi = fmaxf(s.b_hi, fabsf(v));
    } else if (MODE == QASYM) {
        s.b_hi = fmaxf(s.b_hi, v);
        s.b_lo = fminf(s.b_lo, v);
    } else {
        if (col < kColK) { s.a_hi = fmaxf(s.a_hi, v); s.a_lo = fminf(s.a_lo, v); }
        else { s.b_hi = fmaxf(s.b_hi, v); s.b_lo = fminf(s.b_lo, v); }
    }
}

// Block-wide reduction of Stats over 256 threads; result valid in every thread.
template <int MODE>
__device__ __forceinline__ void stats_reduce(Stats &s, float (*sm)[4]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    s.b_hi = warp_max(s.b_hi);
    if (MODE == QSYM_DUAL || MODE == QASYM_DUAL) s.a_hi = warp_max(s.a_hi);
    if (MODE == QASYM || MODE == QASYM_DUAL) s.b_lo = warp_min(s.b_lo);
    if (MODE == QASYM_DUAL) s.a_lo = warp_min(s.a_lo);
    if (lane == 0) { sm[warp][0] = s.a_hi; sm[warp][1] = s.a_lo; sm[warp][2] = s.b_hi; sm[warp][3] = s.b_lo; }
    __syncthreads();
    Stats r;
    stats_init<MODE>(r);
    for (int w = 0; w < nwarp; ++w) {
        r.a_hi = fmaxf(r.a_hi, sm[w][0]);
        r.a_lo = fminf(r.a_lo, sm[w][1]);
        r.b_hi = fmaxf(r.b_hi, sm[w][2]);
        r.b_lo = fminf(r.b_lo, sm[w][3]);
    }
    s = r;
}

// torch semantics of the quantizer modules, each op rounded to fp16 (opmath fp32):
//   sym : scale = half(half(amax) * (1/7)) * clip            (nn/quantizer.py:13)
//   asym: scale = half(half(max - min) * (1/15)); zero = rint(half(-min / scale))   (:27-31)
// torch's CUDA division of an fp16 tensor by a host scalar multiplies by the fp32
// reciprocal; for every fp16 input that equals the correctly rounded quotient by 7 or 15.
__device__ __forceinline__ __half sym_scale(float amax, float clip) {
    __half s = __float2half_rn(amax * (1.0f / 7.0f));
    return __float2half_rn(__half2float(s) * clip);
}
__device__ __forceinline__ void asym_scale_zero(float mn, float mx, __half &s, __half &z) {
    __half d = __float2half_rn(mx - mn);
    s = __float2half_rn(__half2float(d) * (1.0f / 15.0f));
    __half zq = __float2half_rn(__fdiv_rn(-mn, __half2float(s)));
    z = __float2half_rn(rintf(__half2float(zq)));
}

template <int MODE>
__device__ __forceinline__ RowQ rowq_from_stats(const Stats &s, float clip) {
    RowQ r;
    r.s1 = r.s2 = r.z1 = r.z2 = __ushort_as_half(0);
    r.zi1 = 0;
    if (MODE == QSYM) {
        r.s1 = sym_scale(s.b_hi, clip);
    } else if (MODE == QSYM_DUAL) {
        r.s1 = sym_scale(s.a_hi, clip);
        r.s2 = sym_scale(s.b_hi, clip);
    } else if (MODE == QASYM) {
        asym_scale_zero(s.b_lo, s.b_hi, r.s1, r.z1);
        r.zi1 = __half2int_rn(r.z1);
    } else {
        asym_scale_zero(s.a_lo, s.a_hi, r.s1, r.z1);
        asym_scale_zero(s.b_lo, s.b_hi, r.s2, r.z2);
    }
    return r;
}

template <int MODE>
__device__ __forceinline__ void store_rowq(const RowQ &r, uint32_t row, __half *s1, __half *z1, __half *s2, __half *z2) {
    s1[row] = r.s1;
    if (MODE == QSYM_DUAL || MODE == QASYM_DUAL) s2[row] = r.s2;
    if (MODE == QASYM || MODE == QASYM_DUAL) z1[row] = r.z1;
    if (MODE == QASYM_DUAL) z2[row] = r.z2;
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
    if (!vec) {
        quant_fused_scalar_kernel<MODE><<<grid, 256, 0, st>>>(hx, rows, cols, clip, q, a, b, c, d);
    } else if (cols <= 256u * 8u * 2u) {
        quant_fused_vec_kernel<MODE, 2><<<grid, 256, 0, st>>>(hx, rows, cols, clip, q, a, b, c, d, out8);
    } else if (cols <= 256u * 8u * 4u) {
        quant_fused_vec_kernel<MODE, 4><<<grid, 256, 0, st>>>(hx, rows, cols, clip, q, a, b, c, d, out8);
    } else if (cols <= 256u * 8u * 8u) {
        quant_fused_vec_kernel<MODE, 8><<<grid, 256, 0, st>>>(hx, rows, cols, clip, q, a, b, c, d, out8);
    } else {
        quant_fused_vec_kernel<MODE, 16><<<grid, 256, 0, st>>>(hx, rows, cols, clip, q, a, b, c, d, out8);
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
    return launch_given<QSYM>(x, scale, nullptr, nullptr, nullptr, rows, colsSrc, colsDst, q, (cudaStream_t)stream);
}
int duq4_sym_dual_quant(const void *x, const void *scale_1, const void *scale_2, uint32_t rows, uint32_t colsSrc,
                        uint32_t colsDst, uint8_t *q, void *stream) {
    return launch_given<QSYM_DUAL>(x, scale_1, nullptr, scale_2, nullptr, rows, colsSrc, colsDst, q, (cudaStream_t)stream);
}
int duq4_asym_quant(const void *x, const void *scale, const void *zeros, uint32_t rows, uint32_t colsSrc,
                    uint32_t colsDst, uint8_t *q, void *stream) {
    return launch_given<QASYM>(x, scale, zeros, nullptr, nullptr, rows, colsSrc, colsDst, q, (cudaStream_t)stream);
}
int duq4_asym_dual_quant(const void *x, const void *scale_1, const void *zeros_1, const void *scale_2,
                         const void *zeros_2, uint32_t rows, uint32_t colsSrc, uint32_t colsDst, uint8_t *q,
                         void *stream) {
    return launch_given<QASYM_DUAL>(x, scale_1, zeros_1, scale_2, zeros_2, rows, colsSrc, colsDst, q, (cudaStream_t)stream);
}
int duq4_asym_quant_8bit(const float *x, const float *scale, const float *zeros, uint32_t rows, uint32_t cols,
                         int8_t *q, void *stream) {
    if (!x || !scale || !zeros || !q) return DUQ4_ERR_NULL;
    if (rows == 0 || cols == 0) return DUQ4_OK;
    asym_quant8_kernel<<<grid_for((size_t)rows * cols, 256), 256, 0, (cudaStream_t)stream>>>(x, scale, zeros, rows, cols, q);
    return launch_status();
}

int duq4_quantize_fused_i8(int mode, const void *x, uint32_t rows, uint32_t cols, float clip_ratio, int8_t *q_i8,
                           void *scale_1_out, void *zeros_1_out, void *scale_2_out, void *zeros_2_out, void *stream) {
    return quantize_fused_dispatch(mode, x, rows, cols, clip_ratio, (uint8_t *)q_i8, scale_1_out, zeros_1_out, scale_2_out,
                                   zeros_2_out, (cudaStream_t)stream, true);
}

int duq4_silu_mul_quantize_fused(int mode, const void *gate_up, uint32_t rows, uint32_t inter, uint32_t ld,
                                 uint32_t up_offset, float clip_ratio, void *q, int q_is_int8, void *scale_out,
                                 void *zeros_out, void *stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (mode == QSYM)
        return launch_silu<QSYM>(gate_up, rows, inter, ld, up_offset, clip_ratio, (uint8_t *)q, scale_out, nullptr, st, q_is_int8 != 0);
    if (mode == QASYM)
        return launch_silu<QASYM>(gate_up, rows, inter, ld, up_offset, clip_ratio, (uint8_t *)q, scale_out, zeros_out, st, q_is_int8 != 0);
    return DUQ4_ERR_MODE;
}

int duq4_quantize_sym_fused(const void *x, uint32_t rows, uint32_t cols, float clip_ratio, uint8_t *q, void *scale_out,
                            void *stream) {
    return launch_fused<QSYM>(x, rows, cols, clip_ratio, q, scale_out, nullptr, nullptr, nullptr, (cudaStream_t)stream);
}
int duq4_quantize_asym_fused(const void *x, uint32_t rows, uint32_t cols, uint8_t *q, void *scale_out, void *zeros_out,
                             void *stream) {
    return launch_fused<QASYM>(x, rows, cols, 1.0f, q, scale_out, zeros_out, nullptr, nullptr, (cudaStream_t)stream);
}
int duq4_quantize_sym_dual_fused(const void *x, uint32_t rows, uint32_t cols, float clip_ratio, uint8_t *q,
                                 void *scale_1_out, void *scale_2_out, void *stream) {
    return launch_fused<QSYM_DUAL>(x, rows, cols, clip_ratio, q, scale_1_out, nullptr, scale_2_out, nullptr,
                                   (cudaStream_t)stream);
}
int duq4_quantize_asym_dual_fused(const void *x, uint32_t rows, uint32_t cols, uint8_t *q, void *scale_1_out,
                                  void *zeros_1_out, void *scale_2_out, void *zeros_2_out, void *stream) {
    return launch_fused<QASYM_DUAL>(x, rows, cols, 1.0f, q, scale_1_out, zeros_1_out, scale_2_out, zeros_2_out,
                                    (cudaStream_t)stream);
}

}  // extern "C"
