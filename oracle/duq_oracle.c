/*
 * CPU oracle for the W4A4 linear path (quantize -> int4 GEMM -> dequant).
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, in plain C, the arithmetic of the
 * DUQLinear4bitCUDA reference kernels so that the CUDA library can be checked against
 * it. Nothing in the product (the duqlinear4bitcuda_b200 package, libduq4.so) links,
 * loads or calls this file; only the test-suite, the smoke check and the benchmark's
 * CPU-baseline leg do.
 *
 * Parity status: pinned against (a) fixtures generated from the reference's own Python
 * code (tests/golden/, made by tests/golden/make_golden.py) and (b) on a GPU box, the
 * reference's CUDA kernels compiled from their own sources (oracle/_ref, see
 * oracle/Makefile). The reference ships no golden vectors of its own.
 *
 * Every function cites the reference lines it follows (paths relative to the
 * reference project root).
 *
 * fp16 arithmetic: each half operation is computed in float and rounded once to half.
 * For +,-,*,/ this is the correctly rounded half result (24 >= 2*11+2 significand bits),
 * i.e. what mul.f16 / add.f16 / sub.f16 produce on the GPU.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef uint16_t h16;

/* ---- fp16 helpers -------------------------------------------------------------------- */
static inline float h2f(h16 h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }
static inline h16 f2h(float f) { _Float16 v = (_Float16)f; h16 h; memcpy(&h, &v, 2); return h; }
static inline h16 hmul(h16 a, h16 b) { return f2h(h2f(a) * h2f(b)); }
static inline h16 hsub(h16 a, h16 b) { return f2h(h2f(a) - h2f(b)); }
static inline h16 hadd(h16 a, h16 b) { return f2h(h2f(a) + h2f(b)); }

/* float moved by `n` units in the last place (n may be negative); used to bracket the
 * GPU's approximate-reciprocal divide. */
static inline float nudge_f32(float f, int n) {
    if (n == 0 || isnan(f) || isinf(f) || f == 0.0f) return f;
    float target = n > 0 ? copysignf(INFINITY, f) : 0.0f;
    for (int i = 0; i < abs(n); ++i) f = nextafterf(f, target);
    return f;
}

/* __hdiv. Host branch of the CUDA header: half(float(a)/float(b)). The device branch is
 * rcp.approx(b)*a, within ~2 ulp(fp32) of the exact quotient; `nudge` moves the fp32
 * quotient by that many ulps away from (+) or toward (-) zero so a caller can bracket
 * it. (include/cuda_fp16.hpp, __hdiv.) */
static inline h16 hdiv_n(h16 a, h16 b, int nudge) {
    float q = h2f(a) / h2f(b);
    return f2h(nudge_f32(q, nudge));
}

/* __half2int_rn: round-half-even, NaN -> 0, saturating. */
static inline int32_t half2int_rn(h16 h) {
    float f = h2f(h);
    if (isnan(f)) return 0;
    if (f >= 2147483648.0f) return INT32_MAX;
    if (f <= -2147483648.0f) return INT32_MIN;
    return (int32_t)rintf(f); /* default rounding mode = to nearest even */
}
/* __int2half_rn: overflows to +-inf beyond 65504(+16). */
static inline h16 int2half_rn(int32_t v) { return f2h((float)v) ; }
/* note: (float)v rounds to 24 bits first; int -> half via float is still correctly
 * rounded because any int32 needing > 24 bits is far above the half range (-> inf). */

static inline int32_t clampi(int32_t x, int32_t lo, int32_t hi) { return x < lo ? lo : (x > hi ? hi : x); }
static inline int32_t wrap_add(int32_t a, int32_t b) { return (int32_t)((uint32_t)a + (uint32_t)b); }

/* Clamp bounds, include/common.h:53-57. qmax_sym is written (7 - 1e-8) and truncates to 6. */
#define QMIN_SYM (-8)
#define QMAX_SYM (6)
#define QMIN_ASYM (0)
#define QMAX_ASYM (15)
/* include/quant.h:5 */
#define QUANT_COL_K (10)

/* Nibble packing: element 2j in the low nibble, 2j+1 in the high nibble, two's
 * complement. include/int4.h:86-98 (set), qlinear4bit/tools/quantization.py:40-47. */
static inline void set_nibble(uint8_t *b, int i, int32_t v) {
    uint8_t n = (uint8_t)(v & 0xF);
    if (i == 0) *b = (uint8_t)((*b & 0xF0) | n); else *b = (uint8_t)((*b & 0x0F) | (n << 4));
}
static inline int32_t s4_lo(uint8_t b) { int32_t v = b & 0xF; return v >= 8 ? v - 16 : v; }
static inline int32_t s4_hi(uint8_t b) { int32_t v = b >> 4; return v >= 8 ? v - 16 : v; }

/* ---- quantize, scales given ---------------------------------------------------------- */

/* src/kernels/quant.cu:12-45 (sym_quantize_f16_i4_kernel). */
void duqo_sym_quant(const h16 *x, const h16 *scale, uint32_t rows, uint32_t colsSrc,
                    uint32_t colsDst, uint8_t *q, int nudge) {
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t c = 0; c < colsDst; ++c) {
            if (c * 2 >= colsSrc) continue; /* kernel returns without writing */
            uint8_t st = 0;
            for (int i = 0; i < 2; ++i) {
                uint32_t col = c * 2 + i;
                if (col < colsSrc) {
                    h16 d = hdiv_n(x[(size_t)r * colsSrc + col], scale[r], nudge);
                    set_nibble(&st, i, clampi(half2int_rn(d), QMIN_SYM, QMAX_SYM));
                }
            }
            q[(size_t)r * colsDst + c] = st;
        }
}

/* src/kernels/quant2.cu:10-45 (sym_dual_quantize_f16_i4_kernel): scale set 1 for
 * col < QUANT_COL_K, else set 2 (quant2.cu:36). */
void duqo_sym_dual_quant(const h16 *x, const h16 *s1, const h16 *s2, uint32_t rows,
                         uint32_t colsSrc, uint32_t colsDst, uint8_t *q, int nudge) {
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t c = 0; c < colsDst; ++c) {
            if (c * 2 >= colsSrc) continue;
            uint8_t st = 0;
            for (int i = 0; i < 2; ++i) {
                uint32_t col = c * 2 + i;
                if (col < colsSrc) {
                    h16 s = col < QUANT_COL_K ? s1[r] : s2[r];
                    h16 d = hdiv_n(x[(size_t)r * colsSrc + col], s, nudge);
                    set_nibble(&st, i, clampi(half2int_rn(d), QMIN_SYM, QMAX_SYM));
                }
            }
            q[(size_t)r * colsDst + c] = st;
        }
}

/* src/kernels/quant.cu:100-132 (asym_quantize_f16_i4_kernel): rn(x/s) + rn(z), clamp
 * to [0,15] (quant.cu:126). */
void duqo_asym_quant(const h16 *x, const h16 *scale, const h16 *zeros, uint32_t rows,
                     uint32_t colsSrc, uint32_t colsDst, uint8_t *q, int nudge) {
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t c = 0; c < colsDst; ++c) {
            if (c * 2 >= colsSrc) continue;
            uint8_t st = 0;
            for (int i = 0; i < 2; ++i) {
                uint32_t col = c * 2 + i;
                if (col < colsSrc) {
                    h16 d = hdiv_n(x[(size_t)r * colsSrc + col], scale[r], nudge);
                    int32_t v = wrap_add(half2int_rn(d), half2int_rn(zeros[r]));
                    set_nibble(&st, i, clampi(v, QMIN_ASYM, QMAX_ASYM));
                }
            }
            q[(size_t)r * colsDst + c] = st;
        }
}

/* src/kernels/quant2.cu:102-139 (asym_dual_quantize_f16_i4_kernel): rn(x/s + z) with the
 * add in fp16 before rounding (quant2.cu:133); argument order x,s1,z1,s2,z2 as in the
 * definition and its call site (quant2.cu:141-156). */
void duqo_asym_dual_quant(const h16 *x, const h16 *s1, const h16 *z1, const h16 *s2,
                          const h16 *z2, uint32_t rows, uint32_t colsSrc, uint32_t colsDst,
                          uint8_t *q, int nudge) {
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t c = 0; c < colsDst; ++c) {
            if (c * 2 >= colsSrc) continue;
            uint8_t st = 0;
            for (int i = 0; i < 2; ++i) {
                uint32_t col = c * 2 + i;
                if (col < colsSrc) {
                    h16 s = col < QUANT_COL_K ? s1[r] : s2[r];
                    h16 z = col < QUANT_COL_K ? z1[r] : z2[r];
                    h16 d = hdiv_n(x[(size_t)r * colsSrc + col], s, nudge);
                    set_nibble(&st, i, clampi(half2int_rn(hadd(d, z)), QMIN_ASYM, QMAX_ASYM));
                }
            }
            q[(size_t)r * colsDst + c] = st;
        }
}

/* src/kernels/quant.cu:245-266 (asym_quantize_f16_i8_kernel): float divide, both terms
 * pass through half before rounding to int, clamp to [0,126] (quant.cu:241-242). */
void duqo_asym_quant_8bit(const float *x, const float *scale, const float *zeros,
                          uint32_t rows, uint32_t cols, int8_t *q) {
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t c = 0; c < cols; ++c) {
            float d = x[(size_t)r * cols + c] / scale[r];
            int32_t v = wrap_add(half2int_rn(f2h(d)), half2int_rn(f2h(zeros[r])));
            q[(size_t)r * cols + c] = (int8_t)clampi(v, 0, 126);
        }
}

/* ---- per-token scales / zero-points (the torch ops of the quantizer modules) ----------- */

/* qlinear4bit/nn/quantizer.py:13 and src/module/quant_tensor.cu:151-161:
 * scale = half(half(max|x|) / 7) * clip. torch on CUDA divides an fp16 tensor by a host
 * scalar as half(float(a) * (1.0f/7)); identical to half(float(a)/7) for every half a. */
void duqo_sym_scales(const h16 *x, uint32_t rows, uint32_t cols, uint32_t c0, uint32_t c1,
                     float clip, h16 *scale) {
    for (uint32_t r = 0; r < rows; ++r) {
        float amax = 0.0f;
        for (uint32_t c = c0; c < c1 && c < cols; ++c) {
            float v = fabsf(h2f(x[(size_t)r * cols + c]));
            if (v > amax) amax = v;
        }
        h16 s = f2h(amax * (1.0f / 7.0f));
        scale[r] = f2h(h2f(s) * clip);
    }
}

/* qlinear4bit/nn/quantizer.py:27-31: scale = half(half(max - min) / 15);
 * zeros = round_half_even(half(-min / scale)). Columns [c0, c1). */
void duqo_asym_scales_zeros(const h16 *x, uint32_t rows, uint32_t cols, uint32_t c0,
                            uint32_t c1, h16 *scale, h16 *zeros) {
    for (uint32_t r = 0; r < rows; ++r) {
        float mn = INFINITY, mx = -INFINITY;
        for (uint32_t c = c0; c < c1 && c < cols; ++c) {
            float v = h2f(x[(size_t)r * cols + c]);
            if (v < mn) mn = v;
            if (v > mx) mx = v;
        }
        h16 d = f2h(mx - mn);
        h16 s = f2h(h2f(d) * (1.0f / 15.0f));
        h16 zq = f2h(-mn / h2f(s));
        scale[r] = s;
        zeros[r] = f2h(rintf(h2f(zq)));
    }
}

/* ---- integer GEMMs ------------------------------------------------------------------- */

/* src/kernels/gemm.cu:8-43: C[m,n] = sum_k s4(A[m,k]) * s4(B[n,k]), int32, alpha=1 beta=0.
 * The arithmetic itself lives in NVIDIA CUTLASS (device::Gemm<int4b_t,...,Sm80>, an
 * un-vendored submodule of the reference, version unpinned); it is an exact integer
 * contraction, restated here. Both operands are read as signed nibbles. */
void duqo_matmul_4bit(const uint8_t *A, const uint8_t *B, uint32_t M, uint32_t N, uint32_t K,
                      int32_t *C) {
    uint32_t kb = K / 2;
    int8_t *a8 = (int8_t *)malloc((size_t)M * K);
    for (size_t i = 0; i < (size_t)M * kb; ++i) {
        a8[2 * i] = (int8_t)s4_lo(A[i]);
        a8[2 * i + 1] = (int8_t)s4_hi(A[i]);
    }
#pragma omp parallel
    {
        int8_t *b8 = (int8_t *)malloc(K);
#pragma omp for schedule(static)
        for (uint32_t n = 0; n < N; ++n) {
            const uint8_t *br = B + (size_t)n * kb;
            for (uint32_t j = 0; j < kb; ++j) {
                b8[2 * j] = (int8_t)s4_lo(br[j]);
                b8[2 * j + 1] = (int8_t)s4_hi(br[j]);
            }
            for (uint32_t m = 0; m < M; ++m) {
                const int8_t *ar = a8 + (size_t)m * K;
                int32_t acc = 0;
                for (uint32_t k = 0; k < K; ++k) acc += (int32_t)ar[k] * (int32_t)b8[k];
                C[(size_t)m * N + n] = acc;
            }
        }
        free(b8);
    }
    free(a8);
}

/* src/kernels/gemm.cu:46-81: int8 x int8 -> int32. */
void duqo_matmul_8bit(const int8_t *A, const int8_t *B, uint32_t M, uint32_t N, uint32_t K,
                      int32_t *C) {
#pragma omp parallel for schedule(static)
    for (uint32_t n = 0; n < N; ++n)
        for (uint32_t m = 0; m < M; ++m) {
            int32_t acc = 0;
            for (uint32_t k = 0; k < K; ++k)
                acc += (int32_t)A[(size_t)m * K + k] * (int32_t)B[(size_t)n * K + k];
            C[(size_t)m * N + n] = acc;
        }
}

/* src/kernels/gemm.cu:83-117 as intended by src/export/bindings.cpp:46-57:
 * C[b] = A[b] * B[b]^T over contiguous [B,M,K/2], [B,N,K/2]. */
void duqo_batch_matmul_4bit(const uint8_t *A, const uint8_t *B, uint32_t M, uint32_t N,
                            uint32_t K, int32_t *C, uint32_t batch) {
    for (uint32_t b = 0; b < batch; ++b)
        duqo_matmul_4bit(A + (size_t)b * M * (K / 2), B + (size_t)b * N * (K / 2), M, N, K,
                         C + (size_t)b * M * N);
}

/* ---- dequantize ---------------------------------------------------------------------- */

/* src/kernels/quant.cu:64-81: (s_row * s_col) * half(q), each product rounded to half. */
void duqo_sym_dequant(const int32_t *q, const h16 *sr, const h16 *sc, uint32_t rows,
                      uint32_t cols, h16 *x) {
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t c = 0; c < cols; ++c)
            x[(size_t)r * cols + c] =
                hmul(hmul(sr[r], sc[c]), int2half_rn(q[(size_t)r * cols + c]));
}

/* src/kernels/quant2.cu:63-83: column scale set chosen by OUTPUT column < QUANT_COL_K. */
void duqo_sym_dual_dequant(const int32_t *q, const h16 *sr, const h16 *sc1, const h16 *sc2,
                           uint32_t rows, uint32_t cols, uint32_t col0, h16 *x) {
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t c = 0; c < cols; ++c) {
            h16 sc = (c + col0) < QUANT_COL_K ? sc1[c] : sc2[c];
            x[(size_t)r * cols + c] = hmul(hmul(sr[r], sc), int2half_rn(q[(size_t)r * cols + c]));
        }
}

/* src/kernels/quant.cu:150-169: (s_row*s_col) * ((half(q) - z_row) - z_col). */
void duqo_asym_dequant(const int32_t *q, const h16 *sr, const h16 *zr, const h16 *sc,
                       const h16 *zc, uint32_t rows, uint32_t cols, h16 *x) {
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t c = 0; c < cols; ++c) {
            h16 e = int2half_rn(q[(size_t)r * cols + c]);
            x[(size_t)r * cols + c] = hmul(hmul(sr[r], sc[c]), hsub(hsub(e, zr[r]), zc[c]));
        }
}

/* src/kernels/quant2.cu:159-186: set 1 only where ((QUANT_COL_ST << col) & 1) != 0, which
 * holds for output column 0 alone (bit 0 of the mask is set; a left shift clears it). */
void duqo_asym_dual_dequant(const int32_t *q, const h16 *sr, const h16 *zr, const h16 *sc1,
                            const h16 *zc1, const h16 *sc2, const h16 *zc2, uint32_t rows,
                            uint32_t cols, uint32_t col0, h16 *x) {
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t c = 0; c < cols; ++c) {
            int first = (c + col0) == 0;
            h16 sc = first ? sc1[c] : sc2[c];
            h16 zc = first ? zc1[c] : zc2[c];
            h16 e = int2half_rn(q[(size_t)r * cols + c]);
            x[(size_t)r * cols + c] = hmul(hmul(sr[r], sc), hsub(hsub(e, zr[r]), zc));
        }
}

/* src/kernels/quant.cu:191-219: the asym formula per batch, scales at [b*rows+row] and
 * [b*cols+col]. */
void duqo_asym_batch_dequant(const int32_t *q, const h16 *sr, const h16 *zr, const h16 *sc,
                             const h16 *zc, uint32_t batches, uint32_t rows, uint32_t cols,
                             h16 *x) {
    for (uint32_t b = 0; b < batches; ++b)
        duqo_asym_dequant(q + (size_t)b * rows * cols, sr + (size_t)b * rows, zr + (size_t)b * rows,
                          sc + (size_t)b * cols, zc + (size_t)b * cols, rows, cols,
                          x + (size_t)b * rows * cols);
}

/* src/kernels/quant.cu:282-304: fp32 (s_row*s_col) * (float(q) - (z_row + z_col)). */
void duqo_asym_dequant_hprec(const int32_t *q, const float *sr, const float *zr,
                             const float *sc, const float *zc, uint32_t rows, uint32_t cols,
                             float *x) {
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t c = 0; c < cols; ++c) {
            volatile float s = sr[r] * sc[c];
            volatile float z = zr[r] + zc[c];
            volatile float d = (float)q[(size_t)r * cols + c] - z;
            x[(size_t)r * cols + c] = s * d;
        }
}

/* Bias add of the nn modules (qlinear4bit/nn/linear.py:53-54): a separate fp16 add. */
void duqo_add_bias(h16 *x, const h16 *bias, uint32_t rows, uint32_t cols) {
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t c = 0; c < cols; ++c)
            x[(size_t)r * cols + c] = hadd(x[(size_t)r * cols + c], bias[c]);
}

/* Weight preparation, qlinear4bit/nn/linear.py:72-73 with per-row symmetric scales
 * absmax/7 and an explicit clamp to [-8,7] (the benchmark's weight recipe). */
void duqo_weight_sym_quant_pack(const h16 *w, uint32_t N, uint32_t K, h16 *scale, uint8_t *q) {
    for (uint32_t n = 0; n < N; ++n) {
        float amax = 0.0f;
        for (uint32_t k = 0; k < K; ++k) {
            float v = fabsf(h2f(w[(size_t)n * K + k]));
            if (v > amax) amax = v;
        }
        h16 s = f2h(amax / 7.0f);
        scale[n] = s;
        for (uint32_t k = 0; k < K; k += 2) {
            uint8_t st = 0;
            for (int i = 0; i < 2 && k + i < K; ++i) {
                h16 d = f2h(h2f(w[(size_t)n * K + k + i]) / h2f(s));
                set_nibble(&st, i, clampi(half2int_rn(d), -8, 7));
            }
            q[(size_t)n * (K / 2) + k / 2] = st;
        }
    }
}
