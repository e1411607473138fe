// Device-side pieces of the per-token int4 quantizers, shared by the stand-alone quantize kernels
// (quantize.cu) and the small-M linear kernels that quantize their activations themselves
// (gemv_decode.cu): per-row terms, the operation-by-operation coding path that follows the reference
// kernels (src/kernels/quant.cu:12-45, :100-132; src/kernels/quant2.cu:10-45, :102-139), the short coding
// path, row statistics and the torch-semantics scale / zero-point formulas
// (qlinear4bit/nn/quantizer.py:13, :27-31).
#pragma once
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

// ---- a CTA quantizes its own activations -----------------------------------------------------------------
// Used by the small-M linear kernels: a few tokens x [M, K] (fp16, global memory; they were written by the
// stream's previous kernel and sit in L2) become packed int4 codes in SHARED memory, and the per-token terms
// (scale, zero-point) land in `rowq`; nothing goes back to global memory. Scales, zero-points and codes are
// those of quant_fused_vec_kernel<MODE>, bit for bit: the same statistics (max / min are exact whatever the
// order; NaNs are skipped and infinities kept exactly as that kernel's element-by-element pass does), the same
// scale formulas and the same two coding paths.
//
// The routine sits on the critical path of a kernel that runs for a few microseconds and it runs once per CTA,
// i.e. with cold instruction fetch: it is written for FEW EXECUTED INSTRUCTIONS. All tokens are copied to shared
// memory with asynchronous 16-byte copies (one trip to L2, every copy in flight at once, no registers held);
// statistics and coding then read shared memory in short rolled loops.
//
// Called by the first `nthreads` threads of the CTA (a multiple of 32, at most 256), all of them, with uniform
// arguments. Synchronisation: named barrier 1 over the calling threads; on return every calling thread may read
// all codes and rowq entries. K % 8 == 0, x 16-byte aligned; `raw` (16-byte aligned, M * K * 2 bytes) is staging
// space; code rows are `stride` bytes apart (multiple of 4).
__device__ __forceinline__ void bar_named(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// float <-> unsigned key with the same order (integer warp reductions; -0 sorts below +0 as in fminf / fmaxf)
__device__ __forceinline__ uint32_t f32_key(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float f32_from_key(uint32_t k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k); }

struct TokenQuantScratch {   // shared memory the routine needs besides the staging space and the code rows
    uint32_t part[8][5];     // per-warp partial statistics of the token in work: keys of a_hi, a_lo, b_hi, b_lo; "special" flag
    RowQ rowq[16];           // per-token terms, valid on return
};

template <int MODE>
__device__ __forceinline__ void quantize_tokens_to_smem(const __half *__restrict__ x, uint32_t M, uint32_t K, float clip,
                                                        uint8_t *raw, uint8_t *codes, uint32_t stride, TokenQuantScratch &sc,
                                                        uint32_t nthreads) {
    constexpr bool kDual = MODE == QSYM_DUAL || MODE == QASYM_DUAL;
    constexpr bool kAsym = MODE == QASYM || MODE == QASYM_DUAL;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
    const uint32_t nvec = K >> 3, total = M * nvec;
    const uint32_t raw_s = (uint32_t)__cvta_generic_to_shared(raw);
    const uint4 *x4 = reinterpret_cast<const uint4 *>(x);
    for (uint32_t i = tid; i < total; i += nthreads) cp_async16(raw_s + i * 16u, x4 + i);
    cp_async_wait_all();
    bar_named(1, nthreads);
    const uint4 *r4 = reinterpret_cast<const uint4 *>(raw);
    for (uint32_t m = 0; m < M; ++m) {
        // ---- statistics of this thread's vectors of token m (on the bit patterns: NaNs skipped, infinities kept)
        Stats st;
        stats_init<MODE>(st);
        uint32_t am = 0;                                   // max |bits| of everything, NaNs included: "special" test
        uint32_t amax = 0;                                 // symmetric: max |bits| with NaNs masked out
        __half2 hmx = __float2half2_rn(-INFINITY), hmn = __float2half2_rn(INFINITY);
        for (uint32_t v = tid; v < nvec; v += nthreads) {
            const uint4 d = r4[m * nvec + v];
            const uint32_t w[4] = {d.x, d.y, d.z, d.w};
            if (kDual && v < 2) {   // columns 0..15 straddle the split at column 10: element by element
                const __half *h = reinterpret_cast<const __half *>(&d);
#pragma unroll
                for (int k = 0; k < 8; ++k) stats_add<MODE>(st, __half2float(h[k]), v * 8 + k);
#pragma unroll
                for (int k = 0; k < 4; ++k) am = __vmaxu2(am, w[k] & 0x7FFF7FFFu);
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t a = w[k] & 0x7FFF7FFFu;
                    am = __vmaxu2(am, a);
                    if (kAsym) {
                        const __half2 hv = *reinterpret_cast<const __half2 *>(&w[k]);
                        hmx = __hmax2(hmx, hv);   // a NaN operand is skipped
                        hmn = __hmin2(hmn, hv);
                    } else {
                        amax = __vmaxu2(amax, a & ~__vcmpgtu2(a, 0x7C007C00u));
                    }
                }
            }
        }
        if (kAsym) {
            st.b_hi = fmaxf(st.b_hi, fmaxf(__low2float(hmx), __high2float(hmx)));
            st.b_lo = fminf(st.b_lo, fminf(__low2float(hmn), __high2float(hmn)));
        } else {
            st.b_hi = fmaxf(st.b_hi, __half2float(__ushort_as_half((unsigned short)max(amax & 0xFFFFu, amax >> 16))));
        }
        // ---- warp reduction on order-preserving keys, one shared-memory word per warp and value
        const uint32_t k_bhi = __reduce_max_sync(0xffffffffu, f32_key(st.b_hi));
        uint32_t k_blo = 0, k_ahi = 0, k_alo = 0;
        if (kAsym) k_blo = __reduce_min_sync(0xffffffffu, f32_key(st.b_lo));
        if (kDual) k_ahi = __reduce_max_sync(0xffffffffu, f32_key(st.a_hi));
        if (MODE == QASYM_DUAL) k_alo = __reduce_min_sync(0xffffffffu, f32_key(st.a_lo));
        const uint32_t sp = __reduce_max_sync(0xffffffffu, max(am & 0xFFFFu, am >> 16));
        if (lane == 0) {
            sc.part[warp][0] = k_ahi; sc.part[warp][1] = k_alo; sc.part[warp][2] = k_bhi; sc.part[warp][3] = k_blo;
            sc.part[warp][4] = sp;
        }
        bar_named(1, nthreads);
        // ---- every thread combines the partials, derives the token's terms and codes its own vectors
        uint32_t c_ahi = 0, c_alo = 0xFFFFFFFFu, c_bhi = 0, c_blo = 0xFFFFFFFFu, c_sp = 0;
        for (uint32_t w = 0; w < nwarps; ++w) {
            c_bhi = max(c_bhi, sc.part[w][2]);
            if (kAsym) c_blo = min(c_blo, sc.part[w][3]);
            if (kDual) c_ahi = max(c_ahi, sc.part[w][0]);
            if (MODE == QASYM_DUAL) c_alo = min(c_alo, sc.part[w][1]);
            c_sp = max(c_sp, sc.part[w][4]);
        }
        Stats tot;
        stats_init<MODE>(tot);
        tot.b_hi = f32_from_key(c_bhi);
        if (kAsym) tot.b_lo = f32_from_key(c_blo);
        if (kDual) tot.a_hi = f32_from_key(c_ahi);
        if (MODE == QASYM_DUAL) tot.a_lo = f32_from_key(c_alo);
        const RowQ r = rowq_from_stats<MODE>(tot, clip);
        const FastQ fq = make_fastq<MODE>(r, c_sp >= 0x7C00u);
        if (tid == 0) sc.rowq[m] = r;
        uint32_t *crow = reinterpret_cast<uint32_t *>(codes + (size_t)m * stride);
        for (uint32_t v = tid; v < nvec; v += nthreads) {
            const uint4 d = r4[m * nvec + v];
            crow[v] = (fq.ok && !(kDual && v < 2)) ? code8_fast<MODE>(d, fq) : code8<MODE>(d, v * 8, r);
        }
        bar_named(1, nthreads);   // the partials are free for the next token; this token's codes and terms are visible
    }
}

}  // namespace duq4
