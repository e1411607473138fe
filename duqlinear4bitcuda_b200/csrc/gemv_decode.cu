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
#include <cuda.h>
#include <stdlib.h>

#include "duq_common.cuh"
#include "duq_ptx.cuh"
#include "quant_device.cuh"

namespace duq4 {

constexpr int kGemvWarps = 8;

// Activation quantizer inside the linear kernel (template flag FQ): the kernel receives the fp16 tokens instead of
// packed codes; every CTA quantizes them into its own shared memory (quantize_tokens_to_smem) once its first
// batch of weight loads is in flight, so codes and per-token scales never travel through global memory and the
// layer is ONE launch. Replaces the reference's separate quantize launch (src/kernels/quant.cu:48-61 after the
// torch ops of qlinear4bit/nn/quantizer.py:10-16, :24-35) in front of the GEMM.
struct FusedQ {
    const __half *x;   // fp16 [M, K]
    int act_mode;      // DUQ4_MODE_SYM .. ASYM_DUAL
    float clip;
};
// Shared-memory layout of the FQ variants (dynamic shared memory): scratch, M code rows, then the fp16 staging
// copy of the tokens.
__host__ __device__ constexpr uint32_t fq_code_stride(uint32_t kb) { return kb + 64; }   // +64: the 8 tokens a quarter-warp reads fall into distinct banks
__host__ __device__ constexpr uint32_t fq_scratch_bytes() { return (uint32_t)((sizeof(TokenQuantScratch) + 15) / 16 * 16); }
__host__ __device__ inline uint32_t fq_smem_bytes(uint32_t M, uint32_t kb) {
    return fq_scratch_bytes() + M * fq_code_stride(kb) + M * kb * 4u;
}
__device__ __forceinline__ void fq_quantize(const FusedQ &fq, uint32_t M, uint32_t K, uint8_t *codes, uint32_t stride, TokenQuantScratch &sc) {
    uint8_t *raw = codes + (size_t)M * stride;   // staging copy of the fp16 tokens, behind the code rows
    switch (fq.act_mode) {
        case QSYM: quantize_tokens_to_smem<QSYM>(fq.x, M, K, fq.clip, raw, codes, stride, sc, kGemvWarps * 32); break;
        case QSYM_DUAL: quantize_tokens_to_smem<QSYM_DUAL>(fq.x, M, K, fq.clip, raw, codes, stride, sc, kGemvWarps * 32); break;
        case QASYM: quantize_tokens_to_smem<QASYM>(fq.x, M, K, fq.clip, raw, codes, stride, sc, kGemvWarps * 32); break;
        default: quantize_tokens_to_smem<QASYM_DUAL>(fq.x, M, K, fq.clip, raw, codes, stride, sc, kGemvWarps * 32); break;
    }
}
// 16 bytes of token codes: global memory (read-only path) or the CTA's shared memory
template <bool FQ>
__device__ __forceinline__ uint4 ld_codes(const uint4 *p) {
    if (FQ) return *p;
    return __ldg(p);
}

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Programmatic dependent launch (no-ops unless the launch carries the attribute).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// L2 prefetch of [ptr, ptr + bytes): ptr 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void l2_prefetch_bulk(const void *ptr, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr), "r"(bytes) : "memory");
}
// Next-layer hint: the CTAs of this launch together ask L2 for a window of the next launch's packed
// weights, one contiguous slice per CTA, each when it starts. The window skips the first 12 MiB -- the rows
// the next launch's first wave of CTAs fetches by itself while this launch drains (programmatic dependent
// launch) -- and covers the following 18 MiB, which its later CTAs would otherwise request from a memory
// pipe that has just run dry. Measured on 4096->12288 / 4096->22016 at one token: 6.4 -> 5.7 us and
// 10.6 -> 9.9 us per layer; windows of 8..32 MiB starting at 8..20 MiB all lie within 4 % of that.
constexpr uint64_t kNextSkip = 12ull << 20, kNextLen = 18ull << 20;
__device__ __forceinline__ void prefetch_next_weights(const EpiParams &p, uint32_t cta, uint32_t ncta) {
    if (!p.next_w || p.next_w_bytes <= kNextSkip || (reinterpret_cast<uintptr_t>(p.next_w) & 15) != 0) return;
    uint64_t total = p.next_w_bytes - kNextSkip;
    if (total > kNextLen) total = kNextLen;
    const uint64_t per = ((total + ncta - 1) / ncta + 127) & ~127ull;
    const uint64_t off = (uint64_t)cta * per;
    if (off >= total) return;
    uint64_t n = total - off < per ? total - off : per;
    n &= ~15ull;
    if (n) l2_prefetch_bulk(p.next_w + kNextSkip + off, (uint32_t)n);
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t nib_lo(uint32_t w) { return (w << 4) & 0xF0F0F0F0u; }
__device__ __forceinline__ uint32_t nib_hi(uint32_t w) { return w & 0xF0F0F0F0u; }

__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// R  = 16-row weight groups per CTA (1 or 2); TH = token halves (1: M <= 8, 2: M <= 16); FQ: A is unused and the
// tokens come as fp16 through `fq` (see FusedQ).
template <int R, int TH, bool FQ>
__global__ void __launch_bounds__(kGemvWarps * 32) gemv_w4a4_kernel(const uint8_t *__restrict__ A,
                                                                    const uint8_t *__restrict__ W, uint32_t M, uint32_t N,
                                                                    uint32_t K, EpiParams p, __half *__restrict__ out,
                                                                    int32_t *__restrict__ acc_out, FusedQ fq) {
    extern __shared__ __align__(16) uint8_t fq_smem[];
    TokenQuantScratch &qsc = *reinterpret_cast<TokenQuantScratch *>(fq_smem);
    uint8_t *const qcodes = fq_smem + fq_scratch_bytes();
    const uint32_t kb = K >> 1;           // bytes per packed row
    const uint32_t a_stride = FQ ? fq_code_stride(kb) : kb;
    if (!FQ) {   // batched launch: blockIdx.y selects one of the independent problems
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
        ap[h] = reinterpret_cast<const uint4 *>((FQ ? qcodes : A) + (size_t)(aok[h] ? m : 0) * a_stride);
    }

    // Weights are parameters: with the "static weights" option on, the launch carries the
    // programmatic-serialization attribute and this grid may start while the previous kernel of
    // the stream is still draining. Its first batch of weight loads is issued right away; the
    // activations (and every write) wait for the previous grid. Without the attribute both
    // instructions do nothing.
    pdl_launch_dependents();
    // Per-channel terms of the column this thread will finish (all of a thread's outputs share it):
    // fetched now, so that their DRAM latency runs in parallel with the weight stream instead of
    // extending the CTA's tail. They are parameters like the weights (see duq4_set_static_weights).
    ColTerms ct_mine;
    ct_mine.s = ct_mine.z = ct_mine.b = __ushort_as_half(0);
    ct_mine.has_bias = false;
    {
        const uint32_t n_mine = row0 + (threadIdx.x % (16 * R));
        if (p.mode != DUQ4_MODE_NONE && n_mine < N) ct_mine = load_col_terms(p, n_mine);
    }
    bool waited = false;
    if (FQ) {
        // The tokens are quantized before this thread holds any weight registers; meanwhile L2 is asked for the
        // CTA's weight rows (one bulk prefetch per row), so the DRAM pipe works while the tokens are coded.
        if (threadIdx.x < 16 * R && row0 + threadIdx.x < N && (kb & 15u) == 0)
            l2_prefetch_bulk(W + (size_t)(row0 + threadIdx.x) * kb, kb);
        if (threadIdx.x == 0 && blockIdx.y == 0) prefetch_next_weights(p, blockIdx.x, gridDim.x);
        pdl_wait();
        fq_quantize(fq, M, K, qcodes, a_stride, qsc);   // every warp takes part (named barrier inside)
        waited = true;
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
        }
        if (!waited) {   // the first batch of weight loads is in flight before anything waits
            if (threadIdx.x == 0 && blockIdx.y == 0) prefetch_next_weights(p, blockIdx.x, gridDim.x);
            pdl_wait();
            waited = true;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            uint32_t ch = (s0 + u) * 4 + t;
            bool ok = ch < nchunk;
#pragma unroll
            for (int h = 0; h < TH; ++h) av[u][h] = (ok && aok[h]) ? ld_codes<FQ>(ap[h] + ch) : make_uint4(0, 0, 0, 0);
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

    if (!waited) pdl_wait();   // a warp without a K slice of its own (short rows)
    // Cross-warp (split-K) reduction. Fragment element i of acc[r][h]: weight row
    // 16r + g + 8*(i>>1), token 8h + 2t + (i&1).
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int h = 0; h < TH; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) red[warp][8 * h + 2 * t + (i & 1)][16 * r + g + 8 * (i >> 1)] = acc[r][h][i];
    __syncthreads();

    const bool epi_asym = p.mode == DUQ4_MODE_ASYM || p.mode == DUQ4_MODE_ASYM_DUAL;
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
            __half sr, zr = __ushort_as_half(0);
            if (FQ) {   // the per-token terms this CTA computed itself
                sr = qsc.rowq[m].s1;
                if (epi_asym) zr = qsc.rowq[m].z1;
            } else {
                sr = p.s_row[m];
                if (p.z_row) zr = p.z_row[m];
            }
            const __half v = dequant_one(p.mode, s, sr, zr, ct_mine);   // nl == threadIdx.x % (16*R) for every o of this thread
            const size_t off = (size_t)m * p.ldo + n;
            if (p.n_peers == 0) {
                out[off] = v;
            } else {   // fused all-gather: the same element into every rank's buffer
#pragma unroll
                for (int pi = 0; pi < DUQ4_MAX_OUT_PEERS; ++pi)
                    if (pi < (int)p.n_peers && row_goes_to(p, m, pi)) p.peers[pi][off] = v;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// TMA-streamed variant (used for 9..16 tokens on layers with many rows).
//
// Same arithmetic as gemv_w4a4_kernel, different data movement: a persistent CTA per SM keeps a
// ring of shared-memory stages filled by TMA (one elected thread issues cp.async.bulk.tensor
// copies of [16*R weight rows] x [1 KiB of K], 128B-swizzled), so HBM requests stay in flight
// across row blocks instead of draining at every CTA boundary. Eight consumer warps each own one
// 128-byte K slice of a stage; a ninth warp is the producer. Partial sums of the eight warps meet
// in shared memory once per row block (double-buffered, one named barrier per block).
// Control flow never depends on a failed wait: after a bounded wait expires every remaining
// wait is skipped, all warps still reach every barrier, and the status word is raised.
__device__ int g_gemv_status = 0;

constexpr int kStageKBytes = 1024;   // K bytes per row per stage (8 warps x 128 B)

template <int R>
struct GemvSmem {
    static constexpr int kRows = 16 * R;
    static constexpr int kStageBytes = kRows * kStageKBytes;
    static constexpr int kStages = R == 2 ? 4 : 8;   // 128 KiB of weights in flight per SM (measured: 3 / 4 / 5 / 6 stages of 32 KiB -> 9.8 / 9.6 / 9.8 / 10.4 us on 4096->22016, M=1)
    static constexpr int kRedInts = 2 * kGemvWarps * 16 * (kRows + 1);
    static constexpr int kBytes = 1024 + kStages * kStageBytes + kRedInts * 4 + 2 * kStages * 8 + 16;
};

template <int R, int TH, bool FQ>
__global__ void __launch_bounds__((kGemvWarps + 1) * 32, 1)
gemv_w4a4_tma_kernel(const __grid_constant__ CUtensorMap tmW, const uint8_t *__restrict__ A, uint32_t M, uint32_t N,
                     uint32_t K, uint32_t batch, EpiParams p0, __half *__restrict__ out0, int32_t *__restrict__ acc0, FusedQ fq) {
    using namespace ptx;
    using S = GemvSmem<R>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_flag;
    const uint32_t raw = smem_u32(smem_raw), base = (raw + 1023u) & ~1023u;
    int *red = reinterpret_cast<int *>(smem_raw + (base - raw) + S::kStages * S::kStageBytes);
    const uint32_t bar0 = base + S::kStages * S::kStageBytes + S::kRedInts * 4;
    // FQ: scratch and code rows follow the barriers (S::kBytes leaves 16 spare bytes after them)
    uint8_t *const fq_base = smem_raw + (base - raw) + S::kStages * S::kStageBytes + S::kRedInts * 4 + 2 * S::kStages * 8 + 16;
    TokenQuantScratch &qsc = *reinterpret_cast<TokenQuantScratch *>(fq_base);
    uint8_t *const qcodes = fq_base + fq_scratch_bytes();
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (S::kStages + s); };

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t kb = K >> 1;
    const uint32_t nks = (kb + kStageKBytes - 1) / kStageKBytes;       // stages per row block
    const uint32_t blocks_per_b = (N + S::kRows - 1) / S::kRows;
    const uint32_t units = blocks_per_b * batch;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < S::kStages; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), kGemvWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    volatile int *abortp = &abort_flag;
    pdl_launch_dependents();   // see gemv_w4a4_kernel: weights may stream before the previous grid ends

    if (warp == kGemvWarps) {
        // ---------------- producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            bool hinted = false;
            for (uint32_t u = blockIdx.x; u < units; u += gridDim.x) {
                const uint32_t b = u / blocks_per_b, row0 = (u % blocks_per_b) * S::kRows;
                for (uint32_t ks = 0; ks < nks; ++ks, ++it) {
                    if (!hinted && it == (uint32_t)S::kStages) {   // once this CTA's own ring is full
                        prefetch_next_weights(p0, blockIdx.x, gridDim.x);
                        hinted = true;
                    }
                    const uint32_t s = it % S::kStages, ph = (it / S::kStages) & 1;
                    if (ok) ok = mbar_wait(empty(s), ph ^ 1, abortp, &g_gemv_status, 1);
                    if (!ok) continue;
                    const uint32_t k0 = ks * kStageKBytes;
                    const uint32_t nbox = min(8u, (kb - k0 + 127u) / 128u);   // boxes with any K inside the row
                    mbar_expect_tx(full(s), nbox * 128u * S::kRows);
                    const uint32_t dst = base + s * S::kStageBytes;
                    for (uint32_t j = 0; j < nbox; ++j)
                        tma_load_3d(dst + j * (128u * S::kRows), &tmW, full(s), (int)(k0 + j * 128u), (int)row0, (int)b);
                }
            }
            if (!ok) {  // let copies already issued land before the CTA retires
                uint64_t t0 = globaltimer();
                while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
            }
        }
    } else {
        // ---------------- consumers ----------------
        const int g = lane >> 2, t = lane & 3;
        uint32_t it = 0, lu = 0;
        bool ok = true;
        pdl_wait();   // activations come from the previous grid; outputs may still be read by it
        const uint32_t a_stride = FQ ? fq_code_stride(kb) : kb;
        if (FQ) fq_quantize(fq, M, K, qcodes, a_stride, qsc);   // the producer warp keeps filling the ring meanwhile (one CTA per SM: registers to spare)
        const bool epi_asym = p0.mode == DUQ4_MODE_ASYM || p0.mode == DUQ4_MODE_ASYM_DUAL;
        for (uint32_t u = blockIdx.x; u < units; u += gridDim.x, ++lu) {
            const uint32_t b = u / blocks_per_b, row0 = (u % blocks_per_b) * S::kRows;
            const uint8_t *Ab = FQ ? qcodes : A + (size_t)b * M * kb;
            int acc[R][TH][4];
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int h = 0; h < TH; ++h)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[r][h][i] = 0;

            for (uint32_t ks = 0; ks < nks; ++ks, ++it) {
                const uint32_t s = it % S::kStages, ph = (it / S::kStages) & 1;
                // token slice for this warp's 128 bytes of K: issued before the wait, it does not depend on it
                const uint32_t kbyte = ks * kStageKBytes + warp * 128u + 32u * t;
                const bool kin = kbyte < kb;   // kb is a multiple of 32: in range means the whole 32 bytes are
                uint4 tk[TH][2];
#pragma unroll
                for (int h = 0; h < TH; ++h) {
                    const uint32_t m = g + 8 * h;
                    const bool lok = kin && m < M;
                    const uint4 *ap = reinterpret_cast<const uint4 *>(Ab + (size_t)(lok ? m : 0) * a_stride + (lok ? kbyte : 0));
                    tk[h][0] = lok ? ld_codes<FQ>(ap) : make_uint4(0, 0, 0, 0);
                    tk[h][1] = lok ? ld_codes<FQ>(ap + 1) : make_uint4(0, 0, 0, 0);
                }
                if (ok) ok = mbar_wait(full(s), ph, abortp, &g_gemv_status, 2);
                if (ok && ks * kStageKBytes + warp * 128u < kb) {
                    const uint32_t box = base + s * S::kStageBytes + warp * (128u * S::kRows);
                    const uint32_t c0 = (uint32_t)((2 * t) ^ g) << 4, c1 = (uint32_t)((2 * t + 1) ^ g) << 4;
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const uint32_t ra = box + (16 * r + g) * 128u, rb = ra + 8 * 128u;
                        uint32_t wa[2][4], wb[2][4];
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(wa[0][0]), "=r"(wa[0][1]), "=r"(wa[0][2]), "=r"(wa[0][3]) : "r"(ra + c0));
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(wa[1][0]), "=r"(wa[1][1]), "=r"(wa[1][2]), "=r"(wa[1][3]) : "r"(ra + c1));
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(wb[0][0]), "=r"(wb[0][1]), "=r"(wb[0][2]), "=r"(wb[0][3]) : "r"(rb + c0));
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(wb[1][0]), "=r"(wb[1][1]), "=r"(wb[1][2]), "=r"(wb[1][3]) : "r"(rb + c1));
#pragma unroll
                        for (int q = 0; q < 2; ++q)
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint32_t a0 = nib_lo(wa[q][j]), a1 = nib_lo(wb[q][j]), a2 = nib_hi(wa[q][j]), a3 = nib_hi(wb[q][j]);
#pragma unroll
                                for (int h = 0; h < TH; ++h) {
                                    const uint32_t tw = reinterpret_cast<const uint32_t *>(&tk[h][q])[j];
                                    mma_s8(acc[r][h], a0, a1, a2, a3, nib_lo(tw), nib_hi(tw));
                                }
                            }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty(s));
            }

            // split-K reduction across the eight warps, then the dequant epilogue
            int *rd = red + (lu & 1) * (kGemvWarps * 16 * (S::kRows + 1));
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int h = 0; h < TH; ++h)
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        rd[(warp * 16 + 8 * h + 2 * t + (i & 1)) * (S::kRows + 1) + 16 * r + g + 8 * (i >> 1)] = acc[r][h][i];
            asm volatile("bar.sync 1, %0;" ::"n"(kGemvWarps * 32) : "memory");
            const EpiParams p = epi_for_batch(p0, b);
            for (uint32_t o = threadIdx.x; o < (uint32_t)S::kRows * 8u * TH; o += kGemvWarps * 32) {
                const uint32_t nl = o % S::kRows, m = o / S::kRows, n = row0 + nl;
                if (m >= M || n >= N) continue;
                int sum = 0;
#pragma unroll
                for (int w = 0; w < kGemvWarps; ++w) sum += rd[(w * 16 + m) * (S::kRows + 1) + nl];
                sum >>= 8;  // exact: a multiple of 256
                if (acc0) acc0[((size_t)b * M + m) * N + n] = sum;
                if (p.mode != DUQ4_MODE_NONE) {
                    ColTerms ct = load_col_terms(p, n);
                    __half sr, zr = __ushort_as_half(0);
                    if (FQ) {
                        sr = qsc.rowq[m].s1;
                        if (epi_asym) zr = qsc.rowq[m].z1;
                    } else {
                        sr = p.s_row[m];
                        if (p.z_row) zr = p.z_row[m];
                    }
                    const __half v = dequant_one(p.mode, sum, sr, zr, ct);
                    const size_t off = ((size_t)b * M + m) * p.ldo + n;
                    if (p.n_peers == 0) {
                        out0[off] = v;
                    } else {
#pragma unroll
                        for (int pi = 0; pi < DUQ4_MAX_OUT_PEERS; ++pi)
                            if (pi < (int)p.n_peers && row_goes_to(p, m, pi)) p.peers[pi][off] = v;
                    }
                }
            }
        }
    }
}

int tma_map_bytes_3d(const void *ptr, uint64_t kbytes, uint64_t rows, uint64_t batch, uint32_t box_k, uint32_t box_rows,
                     bool swizzle128, CUtensorMap *out, bool use_cache);

// Set through duq4_set_static_weights(): the caller promises that weight tensors are not
// written by earlier work of the same stream, which lets small-M kernels start fetching them
// while the previous kernel is still finishing.
std::atomic<int> g_static_weights{0};

// Dynamic shared memory above the default 48 KiB needs an opt-in per kernel and device; the FQ variants ask for
// the most they can use once.
constexpr int kFqMaxDynSmem = 160 * 1024;

template <int R, int TH, bool FQ>
static int launch_reg(dim3 grid, const uint8_t *A, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K, const EpiParams &p,
                      __half *out, int32_t *acc_out, cudaStream_t st, const FusedQ &fq) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kGemvWarps * 32);
    cfg.stream = st;
    if (FQ) {
        static DeviceOnce once;
        const int dev = current_device_slot();
        if (dev < 0) return DUQ4_ERR_DEVICE;
        int rc = once.run(dev, [] {
            return (int)cudaFuncSetAttribute(gemv_w4a4_kernel<R, TH, FQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFqMaxDynSmem);
        });
        if (rc) return rc;
        cfg.dynamicSmemBytes = fq_smem_bytes(M, K / 2);
    }
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = g_static_weights.load(std::memory_order_relaxed) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_w4a4_kernel<R, TH, FQ>, A, W, M, N, K, p, out, acc_out, fq);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return (int)e;
    }
    return launch_status();
}

constexpr int kMaxSmemPerCta = 232448;   // 227 KiB
constexpr int kTmaFqMaxDynSmem = kMaxSmemPerCta - 512;   // the kernel also has a few bytes of static shared memory

template <int R, int TH, bool FQ>
static int launch_tma(const uint8_t *A, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K, uint32_t batch,
                      const EpiParams &p, void *out, int32_t *acc_out, cudaStream_t st, int sms, bool cache_maps, const FusedQ &fq) {
    using S = GemvSmem<R>;
    static DeviceOnce once;
    const int dev = current_device_slot();
    if (dev < 0) return DUQ4_ERR_DEVICE;
    int rc = once.run(dev, [] {
        return (int)cudaFuncSetAttribute(gemv_w4a4_tma_kernel<R, TH, FQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FQ ? kTmaFqMaxDynSmem : S::kBytes);
    });
    if (rc) return rc;
    CUtensorMap mw;
    rc = tma_map_bytes_3d(W, K / 2, N, batch, 128, S::kRows, true, &mw, cache_maps);
    if (rc) return rc;
    const uint32_t units = cdiv(N, S::kRows) * batch;
    const uint32_t grid = units < (uint32_t)sms ? units : (uint32_t)sms;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3((kGemvWarps + 1) * 32);
    cfg.dynamicSmemBytes = S::kBytes + (FQ ? fq_smem_bytes(M, K / 2) : 0);
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = g_static_weights.load(std::memory_order_relaxed) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_w4a4_tma_kernel<R, TH, FQ>, mw, A, M, N, K, batch, p, (__half *)out, acc_out, fq);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return (int)e;
    }
    return launch_status();
}

int gemv_status_read(int32_t *out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_gemv_status, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    *out = v;
    if (v != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_gemv_status, &zero, sizeof(int));
    }
    return DUQ4_OK;
}

// ---------------------------------------------------------------------------------------------
// Persistent, double-buffered variant of gemv_w4a4_kernel. Same arithmetic and the same K-split
// over eight warps, but a CTA walks over many 16-row blocks (grid = CTAs that fit on the device
// at once) and keeps TWO batches of weight loads per thread in registers: the loads of batch
// f+1 are issued before batch f is consumed, so the memory pipe never drains at a block
// boundary -- the reduction, barrier and epilogue of one block overlap the next block's loads.
template <int TH, int U>
struct GemvBuf {
    uint4 w[U][2];    // rows g and g+8 of the block, U consecutive k-steps of this warp
    uint4 a[U][TH];   // matching token chunks
    ColTerms ct;      // per-channel terms of this thread's output column (valid in a block's last batch)
};

template <int TH, int U, bool FQ>
__global__ void __launch_bounds__(kGemvWarps * 32, 2)
gemv_w4a4_persist_kernel(const uint8_t *__restrict__ A, const uint8_t *__restrict__ W, uint32_t M, uint32_t N, uint32_t K,
                         uint32_t batch, EpiParams p0, __half *__restrict__ out0, int32_t *__restrict__ acc0, FusedQ fq) {
    extern __shared__ __align__(16) uint8_t fq_smem[];
    TokenQuantScratch &qsc = *reinterpret_cast<TokenQuantScratch *>(fq_smem);
    uint8_t *const qcodes = fq_smem + fq_scratch_bytes();
    __shared__ int red[2][kGemvWarps][16][17];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t kb = K >> 1, nchunk = kb >> 4, nstep = (nchunk + 3) >> 2;
    const uint32_t nb = (nstep + kGemvWarps * U - 1) / (kGemvWarps * U);   // batches per row block
    const uint32_t blocks_per_b = (N + 15) / 16, units = blocks_per_b * batch;
    const uint32_t my_units = blockIdx.x < units ? (units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const uint32_t total = my_units * nb;

    auto unit_of = [&](uint32_t f) { return blockIdx.x + (f / nb) * gridDim.x; };
    auto issue_w = [&](GemvBuf<TH, U> &buf, uint32_t f) {
        const uint32_t unit = unit_of(f), bi = f % nb;
        const uint32_t b = unit / blocks_per_b, row0 = (unit % blocks_per_b) * 16;
        const uint8_t *Wb = W + (size_t)b * N * kb;
        const uint4 *r0 = reinterpret_cast<const uint4 *>(Wb + (size_t)min(row0 + g, N - 1) * kb);
        const uint4 *r1 = reinterpret_cast<const uint4 *>(Wb + (size_t)min(row0 + g + 8, N - 1) * kb);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t ch = ((bi * kGemvWarps + warp) * U + u) * 4 + t;
            const bool ok = ch < nchunk;
            buf.w[u][0] = ok ? ldg_stream(r0 + ch) : make_uint4(0, 0, 0, 0);
            buf.w[u][1] = ok ? ldg_stream(r1 + ch) : make_uint4(0, 0, 0, 0);
        }
        // The epilogue's per-channel terms ride with the block's last batch of weight loads, so that
        // their DRAM latency is hidden like the weights' (they are parameters too).
        const uint32_t n_mine = row0 + (threadIdx.x & 15);
        if (bi == nb - 1 && p0.mode != DUQ4_MODE_NONE && n_mine < N) buf.ct = load_col_terms(epi_for_batch(p0, b), n_mine);
    };
    const uint32_t a_stride = FQ ? fq_code_stride(kb) : kb;
    const bool epi_asym = p0.mode == DUQ4_MODE_ASYM || p0.mode == DUQ4_MODE_ASYM_DUAL;
    auto issue_a = [&](GemvBuf<TH, U> &buf, uint32_t f) {
        const uint32_t unit = unit_of(f), bi = f % nb;
        const uint8_t *Ab = FQ ? qcodes : A + (size_t)(unit / blocks_per_b) * M * kb;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t ch = ((bi * kGemvWarps + warp) * U + u) * 4 + t;
#pragma unroll
            for (int h = 0; h < TH; ++h) {
                const uint32_t m = g + 8 * h;
                const bool ok = ch < nchunk && m < M;
                buf.a[u][h] = ok ? ld_codes<FQ>(reinterpret_cast<const uint4 *>(Ab + (size_t)m * a_stride) + ch) : make_uint4(0, 0, 0, 0);
            }
        }
    };

    int acc[TH][4];
#pragma unroll
    for (int h = 0; h < TH; ++h)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[h][i] = 0;

    auto consume = [&](const GemvBuf<TH, U> &buf, uint32_t f) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t *w0 = reinterpret_cast<const uint32_t *>(&buf.w[u][0]);
            const uint32_t *w1 = reinterpret_cast<const uint32_t *>(&buf.w[u][1]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t a0 = nib_lo(w0[j]), a1 = nib_lo(w1[j]), a2 = nib_hi(w0[j]), a3 = nib_hi(w1[j]);
#pragma unroll
                for (int h = 0; h < TH; ++h) {
                    const uint32_t tw = reinterpret_cast<const uint32_t *>(&buf.a[u][h])[j];
                    mma_s8(acc[h], a0, a1, a2, a3, nib_lo(tw), nib_hi(tw));
                }
            }
        }
        if (f % nb != nb - 1) return;
        // last batch of a row block: split-K reduction over the eight warps, dequant, store
        const uint32_t ui = f / nb, unit = unit_of(f);
        const uint32_t b = unit / blocks_per_b, row0 = (unit % blocks_per_b) * 16;
        int(*rd)[16][17] = red[ui & 1];
#pragma unroll
        for (int h = 0; h < TH; ++h)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                rd[warp][8 * h + 2 * t + (i & 1)][g + 8 * (i >> 1)] = acc[h][i];
                acc[h][i] = 0;
            }
        __syncthreads();   // one barrier per block; red[] alternates so the next block's writers cannot overtake readers
        const uint32_t o = threadIdx.x;
        if (o < 16u * 8u * TH) {
            const uint32_t nl = o & 15, m = o >> 4, n = row0 + nl;
            if (m < M && n < N) {
                int sum = 0;
#pragma unroll
                for (int w = 0; w < kGemvWarps; ++w) sum += rd[w][m][nl];
                sum >>= 8;   // exact: a multiple of 256
                const EpiParams p = epi_for_batch(p0, b);
                if (acc0) acc0[((size_t)b * M + m) * N + n] = sum;
                if (p.mode != DUQ4_MODE_NONE) {
                    __half sr, zr = __ushort_as_half(0);
                    if (FQ) {
                        sr = qsc.rowq[m].s1;
                        if (epi_asym) zr = qsc.rowq[m].z1;
                    } else {
                        sr = p.s_row[m];
                        if (p.z_row) zr = p.z_row[m];
                    }
                    const __half v = dequant_one(p.mode, sum, sr, zr, buf.ct);   // nl == threadIdx.x & 15
                    const size_t off = ((size_t)b * M + m) * p.ldo + n;
                    if (p.n_peers == 0) {
                        out0[off] = v;
                    } else {
#pragma unroll
                        for (int pi = 0; pi < DUQ4_MAX_OUT_PEERS; ++pi)
                            if (pi < (int)p.n_peers && row_goes_to(p, m, pi)) p.peers[pi][off] = v;
                    }
                }
            }
        }
    };

    pdl_launch_dependents();
    GemvBuf<TH, U> b0, b1;
    if (total > 0) issue_w(b0, 0);   // weights are parameters: fetched before the previous grid has finished
    if (FQ && total > 1) issue_w(b1, 1);   // FQ: the wait below is followed by the token quantizer, so both batches fly meanwhile
    if (threadIdx.x == 0) prefetch_next_weights(p0, blockIdx.x, gridDim.x);
    if (FQ) {
        // While the tokens are quantized this CTA holds one batch of weight loads in registers; L2 is asked for the
        // rest of its first row blocks (one bulk prefetch per weight row) so that the DRAM pipe keeps working.
        constexpr uint32_t kAhead = 3;   // row blocks
        const uint32_t r = threadIdx.x & 15, j = threadIdx.x >> 4;
        if (j < kAhead && j < my_units && (kb & 15u) == 0) {
            const uint32_t unit = blockIdx.x + j * gridDim.x;
            const uint32_t b = unit / blocks_per_b, row = (unit % blocks_per_b) * 16 + r;
            if (row < N) l2_prefetch_bulk(W + ((size_t)b * N + row) * kb, kb);
        }
    }
    pdl_wait();                      // activations / outputs belong to the stream's earlier work
    if (FQ) fq_quantize(fq, M, K, qcodes, a_stride, qsc);
    if (total > 0) issue_a(b0, 0);
    if (FQ && total > 1) issue_a(b1, 1);
    for (uint32_t f = 0; f < total; f += 2) {
        if (f + 1 < total && !(FQ && f == 0)) { issue_w(b1, f + 1); issue_a(b1, f + 1); }
        consume(b0, f);
        if (f + 1 >= total) break;
        if (f + 2 < total) { issue_w(b0, f + 2); issue_a(b0, f + 2); }
        consume(b1, f + 1);
    }
}

template <int TH, int U, bool FQ>
static int launch_persist(const uint8_t *A, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K, uint32_t batch,
                          const EpiParams &p, void *out, int32_t *acc_out, cudaStream_t st, int sms, const FusedQ &fq) {
    const uint32_t units = cdiv(N, 16) * batch;
    uint32_t grid = 2u * (uint32_t)sms;
    if (grid > units) grid = units;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kGemvWarps * 32);
    cfg.stream = st;
    if (FQ) {
        static DeviceOnce once;
        const int dev = current_device_slot();
        if (dev < 0) return DUQ4_ERR_DEVICE;
        int rc = once.run(dev, [] {
            return (int)cudaFuncSetAttribute(gemv_w4a4_persist_kernel<TH, U, FQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFqMaxDynSmem);
        });
        if (rc) return rc;
        cfg.dynamicSmemBytes = fq_smem_bytes(M, K / 2);
    }
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = g_static_weights.load(std::memory_order_relaxed) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_w4a4_persist_kernel<TH, U, FQ>, A, W, M, N, K, batch, p, (__half *)out, acc_out, fq);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return (int)e;
    }
    return launch_status();
}

// Kernel choice for M <= 16 tokens. FQ = the tokens arrive as fp16 (`fq`, A unused, batch 1) and the kernel
// quantizes them itself.
template <bool FQ>
static int gemv_dispatch(const uint8_t *A, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K, uint32_t batch,
                         const EpiParams &p, void *out, int32_t *acc_out, cudaStream_t st, bool cache_maps, const FusedQ &fq) {
    const int sms = sm_count_current_device();
    static const int force = [] {
        const char *e = getenv("DUQ4_GEMV_VARIANT");   // debug: 0 = one-shot register kernel, 1 = TMA-streamed kernel, 3 = persistent register kernel
        return e ? atoi(e) : -1;
    }();
    // Measured on B200 (cold weights, CUDA-graph chain of layers, us per layer; one-shot / persistent / TMA):
    //   4096->22016: M=1 10.9/10.8/10.4, M=16 16.9/15.6/14.3     4096->4096: M=1 2.9/2.9/3.7, M=16 4.8/4.1/5.0
    //   11008->4096: M=1 7.1/6.3/7.1,   M=16 10.0/8.2/9.8
    // -> TMA-streamed for > 8 tokens on layers with >= 2 32-row blocks per SM; persistent when a row block
    //    needs more than one batch of loads per warp (long K) or for > 8 tokens; one-shot otherwise.
    const bool big_n = (uint64_t)cdiv(N, 32) * batch >= 2ull * sms;
    const bool long_k = (K / 2 / 64) > (uint32_t)(kGemvWarps * 4);
    // ... and for any token count on the largest layers (>= 4 32-row blocks per SM; 4096->22016 at M=1 with the
    //    next-layer hint: 9.8 us TMA-streamed vs 10.1 us one-shot, while 4096->12288 is 6.15 vs 5.8)
    const bool huge_n = (uint64_t)cdiv(N, 32) * batch >= 4ull * sms;
    // FQ (one token in practice): the TMA-streamed kernel whenever the layer has two row blocks per SM -- its ring keeps
    // 128 KiB of weights per SM in flight while the token is quantized (4096->12288: 7.2 us against 7.7 us persistent)
    bool use_tma = force >= 0 ? force == 1 : (K / 2 >= 2048 && big_n && (FQ || M > 8 || huge_n));
    const bool two = (uint64_t)cdiv(N, 32) * batch >= 2ull * sms;
    // FQ: the code rows must fit beside the TMA ring
    if (FQ && use_tma && (two ? GemvSmem<2>::kBytes : GemvSmem<1>::kBytes) + fq_smem_bytes(M, K / 2) > (uint32_t)kTmaFqMaxDynSmem) use_tma = false;
    // FQ: every CTA quantizes the tokens once, so only the persistent kernels (a CTA per SM or two, not a CTA per
    // 16 rows) carry it: measured on 4096->12288 at one token, 13.2 us with 768 one-shot CTAs.
    const bool persist = force >= 0 ? (force == 3 || (force == 1 && !use_tma) || (FQ && force == 0)) : (!use_tma && (FQ || long_k || M > 8));
    if (persist) {
        if (M <= 8) return launch_persist<1, 4, FQ>(A, W, M, N, K, batch, p, out, acc_out, st, sms, fq);
        return launch_persist<2, 2, FQ>(A, W, M, N, K, batch, p, out, acc_out, st, sms, fq);
    }
    if (use_tma) {
        if (M <= 8) return two ? launch_tma<2, 1, FQ>(A, W, M, N, K, batch, p, out, acc_out, st, sms, cache_maps, fq)
                               : launch_tma<1, 1, FQ>(A, W, M, N, K, batch, p, out, acc_out, st, sms, cache_maps, fq);
        return two ? launch_tma<2, 2, FQ>(A, W, M, N, K, batch, p, out, acc_out, st, sms, cache_maps, fq)
                   : launch_tma<1, 2, FQ>(A, W, M, N, K, batch, p, out, acc_out, st, sms, cache_maps, fq);
    }
    // Up to 8 tokens: 16-row CTAs (three per SM) -- more, smaller CTAs keep the weight stream smoother
    // across CTA boundaries than 32-row ones (4096->22016, M=1: 10.3 vs 10.8 us). 9..16 tokens: two row
    // groups per CTA halve the token re-reads when there are enough rows to fill the SMs.
    const bool r2 = M > 8 && (uint64_t)(N / 32) * batch >= 2 * 148;
    const uint32_t rows_per_cta = r2 ? 32 : 16;
    dim3 grid(cdiv(N, rows_per_cta), batch);
    __half *o = (__half *)out;
    if (M <= 8) return r2 ? launch_reg<2, 1, FQ>(grid, A, W, M, N, K, p, o, acc_out, st, fq) : launch_reg<1, 1, FQ>(grid, A, W, M, N, K, p, o, acc_out, st, fq);
    return r2 ? launch_reg<2, 2, FQ>(grid, A, W, M, N, K, p, o, acc_out, st, fq) : launch_reg<1, 2, FQ>(grid, A, W, M, N, K, p, o, acc_out, st, fq);
}

int gemv_w4a4_launch(const uint8_t *A, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K, uint32_t batch,
                     const EpiParams &p, void *out, int32_t *acc_out, cudaStream_t st, bool cache_maps) {
    if (((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) != 0) return DUQ4_ERR_ALIGN;
    return gemv_dispatch<false>(A, W, M, N, K, batch, p, out, acc_out, st, cache_maps, FusedQ{});
}

// True when gemv_w4a4_from_fp16_launch should take the layer. Measured (B200, cold weights, graph chain of layers,
// us per layer at 1 / 2 / 4 / 8 tokens; single launch | quantizer launch + linear launch with programmatic overlap):
//   4096->12288  7.2  9.2 10.9 17.3 |  7.8  8.3  8.5  8.5      4096->4096   4.0  5.6  7.4 12.5 | 4.2 4.3 4.4 4.6
//   4096->22016 10.3 11.2 13.2 24.0 | 11.5 11.4 12.2 13.8      11008->4096  8.3 10.5   -    -  | 8.0 8.1 8.3 8.5
// Every CTA repeats the quantization, so the single launch pays off for ONE token only (where it also halves the
// host-side launch work); from two tokens on the separate quantizer, started early by programmatic dependent
// launch, is faster. The tokens' staging copy and code rows have to fit into shared memory beside what the kernels
// already hold, and the asynchronous copies need 16-byte aligned rows.
bool gemv_fused_quant_fits(const void *x, uint32_t M, uint32_t K) {
    static const uint32_t max_m = [] {   // debug override of the token count up to which the single-launch route is taken
        const char *e = getenv("DUQ4_FUSEQ_MAX_M");
        const int v = e ? atoi(e) : 1;
        return (uint32_t)(v < 0 ? 0 : (v > 16 ? 16 : v));
    }();
    return M >= 1 && M <= max_m && K % 64 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && fq_smem_bytes(M, K / 2) <= 96u * 1024u;
}

// M <= 16 tokens given as fp16: ONE launch that quantizes the tokens per CTA and runs the layer. p.s_row / p.z_row
// are ignored (the kernel uses the per-token terms it computes; set 1 for the dual-uniform schemes).
int gemv_w4a4_from_fp16_launch(const void *x, int act_mode, float clip, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K,
                               const EpiParams &p, void *out, cudaStream_t st, bool cache_maps) {
    if ((reinterpret_cast<uintptr_t>(W) & 15) != 0) return DUQ4_ERR_ALIGN;
    if (!gemv_fused_quant_fits(x, M, K)) return DUQ4_ERR_SHAPE;
    FusedQ fq{(const __half *)x, act_mode, clip};
    return gemv_dispatch<true>(nullptr, W, M, N, K, 1, p, out, nullptr, st, cache_maps, fq);
}

}  // namespace duq4
