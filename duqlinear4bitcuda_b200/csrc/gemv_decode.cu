// Small-M (M <= 16 tokens) W4A4 linear: an HBM-bound pass over the packed weights with the
// dequant in the epilogue. Replaces, for decode shapes, the reference's sequence
// matmul_host_4bit (src/kernels/gemm.cu:8-43, a 128x256 CUTLASS tile that leaves most of
// a B200 idle at M <= 16) + *_dequant_host + bias add.
//
// Shape of the computation ("swap-AB"): the 16 rows of an m16n8k32 int8 MMA are 16 WEIGHT
// rows, its 8 columns are 8 TOKENS. Every weight byte is loaded from HBM exactly once, as
// 128-bit loads, and unpacked in registers:
//     lo = (w << 4) & 0xF0F0F0F0      hi = w & 0xF0F0F0F0
// i.e. each nibble becomes the int8 value 16*s4. Tokens are unpacked the same way, so each
// product carries a factor 256 and the int32 sum is exactly 256x the true accumulator
// (|sum| <= 64*K*256 < 2^31 for K < 131072); the epilogue shifts it back. The order of K
// inside an MMA is a permutation shared by both operands, which a dot product ignores.
//
// A CTA owns 16*R consecutive weight rows; its 8 warps split K and reduce through shared
// memory, so no global scratch is needed and the result does not depend on scheduling.
#include <mma.h>

#include "duq_common.cuh"

namespace duq4 {

constexpr int kGemvWarps = 8;

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t nib_lo(uint32_t w) { return (w << 4) & 0xF0F0F0F0u; }
__device__ __forceinline__ uint32_t nib_hi(uint32_t w) { return w & 0xF0F0F0F0u; }

__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// R  = 16-row weight groups per CTA (1 or 2); TH = token halves (1: M <= 8, 2: M <= 16).
template <int R, int TH>
__global__ void __launch_bounds__(kGemvWarps * 32) gemv_w4a4_kernel(const uint8_t *__restrict__ A,
                                                                    const uint8_t *__restrict__ W, uint32_t M, uint32_t N,
                                                                    uint32_t K, EpiParams p, __half *__restrict__ out,
                                                                    int32_t *__restrict__ acc_out) {
    {   // batched launch: blockIdx.y selects one of the independent problems
        const uint32_t b = blockIdx.y;
        A += (size_t)b * M * (K >> 1);
        W += (size_t)b * N * (K >> 1);
        if (out) out += (size_t)b * M * p.ldo;
        if (acc_out) acc_out += (size_t)b * M * N;
        p = epi_for_batch(p, b);
    }
    __shared__ int red[kGemvWarps][16][16 * R + 1];  // [warp][token][row]; +1 pads the row stride
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t kb = K >> 1;           // bytes per packed row
    const uint32_t nchunk = kb >> 4;      // 16-byte chunks per row
    const uint32_t nstep = (nchunk + 3) >> 2;
    const uint32_t row0 = blockIdx.x * (16 * R);

    int acc[R][TH][4];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int h = 0; h < TH; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[r][h][i] = 0;

    // Row pointers; rows past N are clamped for the loads and dropped at the store.
    const uint4 *wp[R][2];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        uint32_t ra = min(row0 + 16 * r + g, N - 1), rb = min(row0 + 16 * r + g + 8, N - 1);
        wp[r][0] = reinterpret_cast<const uint4 *>(W + (size_t)ra * kb);
        wp[r][1] = reinterpret_cast<const uint4 *>(W + (size_t)rb * kb);
    }
    const uint4 *ap[TH];
    bool aok[TH];
#pragma unroll
    for (int h = 0; h < TH; ++h) {
        uint32_t m = g + 8 * h;
        aok[h] = m < M;
        ap[h] = reinterpret_cast<const uint4 *>(A + (size_t)(aok[h] ? m : 0) * kb);
    }

    constexpr int U = 4;  // k-steps in flight per warp
    for (uint32_t s0 = warp * U; s0 < nstep; s0 += kGemvWarps * U) {
        uint4 wv[U][R][2], av[U][TH];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            uint32_t ch = (s0 + u) * 4 + t;
            bool ok = ch < nchunk;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                wv[u][r][0] = ok ? ldg_stream(wp[r][0] + ch) : make_uint4(0, 0, 0, 0);
                wv[u][r][1] = ok ? ldg_stream(wp[r][1] + ch) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int h = 0; h < TH; ++h) av[u][h] = (ok && aok[h]) ? __ldg(ap[h] + ch) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t *a_[TH];
#pragma unroll
            for (int h = 0; h < TH; ++h) a_[h] = reinterpret_cast<const uint32_t *>(&av[u][h]);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t *w0 = reinterpret_cast<const uint32_t *>(&wv[u][r][0]);
                const uint32_t *w1 = reinterpret_cast<const uint32_t *>(&wv[u][r][1]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t a0 = nib_lo(w0[j]), a1 = nib_lo(w1[j]), a2 = nib_hi(w0[j]), a3 = nib_hi(w1[j]);
#pragma unroll
                    for (int h = 0; h < TH; ++h) mma_s8(acc[r][h], a0, a1, a2, a3, nib_lo(a_[h][j]), nib_hi(a_[h][j]));
                }
            }
        }
    }

    // Cross-warp (split-K) reduction. Fragment element i of acc[r][h]: weight row
    // 16r + g + 8*(i>>1), token 8h + 2t + (i&1).
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int h = 0; h < TH; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) red[warp][8 * h + 2 * t + (i & 1)][16 * r + g + 8 * (i >> 1)] = acc[r][h][i];
    __syncthreads();

    for (uint32_t o = threadIdx.x; o < 16u * R * 8u * TH; o += blockDim.x) {
        uint32_t nl = o % (16 * R), m = o / (16 * R);
        uint32_t n = row0 + nl;
        if (m >= M || n >= N) continue;
        int s = 0;
#pragma unroll
        for (int w = 0; w < kGemvWarps; ++w) s += red[w][m][nl];
        s >>= 8;  // exact: s is a multiple of 256
        if (acc_out) acc_out[(size_t)m * N + n] = s;
        if (p.mode != DUQ4_MODE_NONE) {
            ColTerms ct = load_col_terms(p, n);
            __half zr = p.z_row ? p.z_row[m] : __ushort_as_half(0);
            out[(size_t)m * p.ldo + n] = dequant_one(p.mode, s, p.s_row[m], zr, ct);
        }
    }
}

int gemv_w4a4_launch(const uint8_t *A, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K, uint32_t batch,
                     const EpiParams &p, void *out, int32_t *acc_out, cudaStream_t st) {
    if (((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) != 0) return DUQ4_ERR_ALIGN;
    // Two row groups per CTA halve the token re-reads; one keeps at least ~2 CTAs per SM
    // busy when N is small.
    const bool r2 = (uint64_t)(N / 32) * batch >= 2 * 148;
    const uint32_t rows_per_cta = r2 ? 32 : 16;
    dim3 grid(cdiv(N, rows_per_cta), batch), block(kGemvWarps * 32);
    __half *o = (__half *)out;
    if (M <= 8) {
        if (r2) gemv_w4a4_kernel<2, 1><<<grid, block, 0, st>>>(A, W, M, N, K, p, o, acc_out);
        else gemv_w4a4_kernel<1, 1><<<grid, block, 0, st>>>(A, W, M, N, K, p, o, acc_out);
    } else {
        if (r2) gemv_w4a4_kernel<2, 2><<<grid, block, 0, st>>>(A, W, M, N, K, p, o, acc_out);
        else gemv_w4a4_kernel<1, 2><<<grid, block, 0, st>>>(A, W, M, N, K, p, o, acc_out);
    }
    return launch_status();
}

}  // namespace duq4
