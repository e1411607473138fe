// Pieces shared by the tensor-core GEMM kernels (1-CTA tiles in gemm_tc.cu, CTA-pair tiles in
// gemm_tc2.cu): tcgen05 / TMEM wrappers, operand descriptors, kernel arguments and the
// dequantizing epilogue of one 128-row accumulator slab.
#pragma once
#include "duq_common.cuh"
#include "duq_ptx.cuh"

namespace duq4 {
namespace tc {

using namespace ptx;

constexpr int kEpiWarps = 4;   // epilogue warps per CTA (one per TMEM lane quadrant)

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 16 bytes to the same offset of every rank's buffer through the NVLink switch: `mc_addr` is an address inside
// an NVLS multicast mapping, 16-byte aligned.
__device__ __forceinline__ void multimem_st16(void *mc_addr, const uint4 &v) {
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}

// K-major, 128-byte-swizzled operand descriptor: rows of 128 bytes, 8-row groups 1024 bytes
// apart (stride byte offset), version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;               // leading byte offset (unused for swizzled K-major): 1
    d |= (uint64_t)(1024u >> 4) << 32;    // stride byte offset
    d |= (uint64_t)1 << 46;               // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;               // SWIZZLE_128B
    return d;
}
// kind::i8 instruction descriptor: D = s32, A = B = signed int8, both K-major, no saturation.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ uint32_t nib_lo(uint32_t w) { return (w << 4) & 0xF0F0F0F0u; }
__device__ __forceinline__ uint32_t nib_hi(uint32_t w) { return w & 0xF0F0F0F0u; }

struct Args {
    uint32_t M, N, K, batch;  // K in elements
    uint32_t tiles_m, tiles_n;
    uint32_t bn;              // CTA-pair kernel only: accumulator columns per tile (multiple of 32, <= 256)
    uint32_t a_rows;          // rows of the A buffer the tensor map may read (>= M; the extra rows are never stored)
    uint32_t band_rows;       // CTA-pair kernel only: row blocks per band of the tile order (see the kernel)
    uint32_t acc_fits_22;     // 1 = every accumulator of this launch is at most 2^22 in magnitude (see dequant16)
    uint32_t gate_up;         // CTA-pair kernel only: 0, or I = width of a SiLU-gated gate/up projection (W has 2*I rows)
    // CTA-pair kernel only, K-split of the last, partly filled round of tiles: the last sk_tiles tiles are each
    // computed by sk_group pairs (a K range each); the pairs exchange int32 partial tiles through sk_scratch and signal
    // sk_counters[tile slot] once per epilogue warp; up to four of them reduce and store a column range each.
    uint32_t sk_tiles, sk_group;
    int32_t *sk_scratch;
    unsigned int *sk_counters;
    EpiParams epi;
    __half *out;
    int32_t *acc_out;
};


// Column terms (scale, zero, bias) of the tile's BN columns into the calling warp's private
// shared-memory copy. Each epilogue warp keeps its own copy so that the epilogue warps never
// have to meet at a barrier (one a warp could miss when the CTA is leaving early).
// `pb` comes in as the launch's parameters and leaves adjusted to batch `b`.
template <int BN>
__device__ __forceinline__ void epi_stage_colterms(const Args &a, EpiParams &pb, uint32_t b, uint32_t n0, int lane, __half *cs,
                                                   __half *cz, __half *cb, int c_lo = 0, int c_hi = BN) {
    // c_lo / c_hi: the tile columns the calling warp will use (a warp that shares a tile by columns stages its part only)
    const int mode = a.epi.mode;
    __syncwarp();  // previous tile's readers are done
    if (mode != DUQ4_MODE_NONE) {
        size_t co = (size_t)b * pb.col_vec_stride;
        if (pb.s_col1) pb.s_col1 += co;
        if (pb.z_col1) pb.z_col1 += co;
        if (pb.s_col2) pb.s_col2 += co;
        if (pb.z_col2) pb.z_col2 += co;
        if (pb.bias) pb.bias += co;
        // all loads first, then the stores: with a store between them every load would wait for the one before it
        // (a chain of BN/32 trips to L2 per tile, on the critical path of a tile's epilogue)
        ColTerms t[BN / 32];
#pragma unroll
        for (int i = 0; i < BN / 32; ++i) {
            const int c = lane + 32 * i;
            const uint32_t n = n0 + c;
            t[i].s = t[i].z = t[i].b = __ushort_as_half(0);
            if (c >= c_lo && c < c_hi && n < a.N) t[i] = load_col_terms(pb, n);
        }
#pragma unroll
        for (int i = 0; i < BN / 32; ++i) {
            const int c = lane + 32 * i;
            if (c >= c_lo && c < c_hi) {
                cs[c] = t[i].s;
                cz[c] = t[i].z;
                cb[c] = t[i].b;
            }
        }
    }
    __syncwarp();
}

// One warp's 32 rows of a 128-row accumulator slab: TMEM -> (>> shift) -> optional int32 store ->
// fp16 dequant (+ bias) -> global / peer memory. `m_base` is the global row of the slab's first
// row, `tmem_acc` the TMEM address (lane 0) of the accumulator's first column.
// fp16 dequant of one row's 16 accumulators of a chunk, two columns per instruction: the reference arithmetic
// (one rounding per fp16 operation, explicit .rn forms so that nothing is contracted into an fma), straight-line code
// for the compiler to interleave -- an epilogue warp is alone on its scheduler, so instruction-level parallelism is all
// the latency hiding it gets. ASYM / BIAS are compile-time so that no per-element branch splits the block.
// FASTCVT: |accumulator| <= 2^22, so int -> float is an integer add and a float subtract (exact) instead of the
// quarter-rate conversion instruction; float -> fp16 then rounds once, as the direct int -> fp16 conversion does.
template <bool ASYM, bool BIAS, bool FASTCVT>
__device__ __forceinline__ void dequant16(const uint32_t (&v)[16], __half sr, __half zr, const __half *cs, const __half *cz,
                                          const __half *cb, __half2 (&o)[8]) {
    const __half2 sr2 = __half2half2(sr), zr2 = __half2half2(zr);
    const uint4 s4a = *reinterpret_cast<const uint4 *>(cs), s4b = *reinterpret_cast<const uint4 *>(cs + 8);
    const __half2 *s2a = reinterpret_cast<const __half2 *>(&s4a), *s2b = reinterpret_cast<const __half2 *>(&s4b);
    uint4 z4a = make_uint4(0, 0, 0, 0), z4b = z4a, b4a = z4a, b4b = z4a;
    if (ASYM) { z4a = *reinterpret_cast<const uint4 *>(cz); z4b = *reinterpret_cast<const uint4 *>(cz + 8); }
    if (BIAS) { b4a = *reinterpret_cast<const uint4 *>(cb); b4b = *reinterpret_cast<const uint4 *>(cb + 8); }
    const __half2 *z2a = reinterpret_cast<const __half2 *>(&z4a), *z2b = reinterpret_cast<const __half2 *>(&z4b);
    const __half2 *b2a = reinterpret_cast<const __half2 *>(&b4a), *b2b = reinterpret_cast<const __half2 *>(&b4b);
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        __half2 e;
        if (FASTCVT) {
            const float f0 = __int_as_float(0x4B400000 + (int)v[2 * p]) - 12582912.0f;
            const float f1 = __int_as_float(0x4B400000 + (int)v[2 * p + 1]) - 12582912.0f;
            e = __floats2half2_rn(f0, f1);
        } else {
            e = __halves2half2(__int2half_rn((int)v[2 * p]), __int2half_rn((int)v[2 * p + 1]));
        }
        const __half2 sc = p < 4 ? s2a[p] : s2b[p - 4];
        const __half2 ss = __hmul2_rn(sr2, sc);
        __half2 val;
        if (ASYM) {
            const __half2 zc = p < 4 ? z2a[p] : z2b[p - 4];
            val = __hmul2_rn(ss, __hsub2_rn(__hsub2_rn(e, zr2), zc));
        } else {
            val = __hmul2_rn(ss, e);
        }
        if (BIAS) val = __hadd2_rn(val, p < 4 ? b2a[p] : b2b[p - 4]);
        o[p] = val;
    }
}

// K-split of a tile over a group of CTA pairs (see the pair kernel): what one call of epi_store_tile does with the
// partial-sum slabs. A slab (128 x BN int32) is private to the warps that exchange it -- the same lane quadrant of
// the same CTA of each pair of the group -- so it is laid out for their access pattern: element (chunk ch, group of
// four columns j4, lane, 4 ints), i.e. every 128-bit access of a warp covers 512 contiguous bytes.
struct SplitK {
    int32_t *out = nullptr;        // phase 1: the raw accumulators of every chunk OUTSIDE [keep_b, keep_e) go to this slab; nothing else happens
    int keep_b = 0, keep_e = 0;
    const int32_t *add = nullptr;  // phase 2: slabs add + c * stride, c in [0, n) except `skip`, are added to the accumulators
    uint32_t n = 0;
    int skip = -1;
    size_t stride = 0;
    int ch_b = 0, ch_e = -1;       // phase 2 handles the chunks [ch_b, ch_e) only (ch_e < 0: up to the tile's end)
};

template <int BN, bool STAGED>
__device__ __forceinline__ void epi_store_tile(const Args &a, const EpiParams &pb, uint32_t b, uint32_t m_base, uint32_t n0,
                                   uint32_t tmem_acc, int quad, int lane, uint32_t shift, const __half *cs,
                                   const __half *cz, const __half *cb, uint8_t *stg, int nch = BN / 16, const SplitK sk = SplitK(),
                                   int ch_lo = 0, int ch_hi = -1) {
    // ch_lo / ch_hi: the chunks [ch_lo, ch_hi) of the tile that the calling warp handles (a multiple of four chunks at the
    // lower end; ch_hi < 0: up to the tile's end) -- several warps of one TMEM lane quadrant can share a tile by columns
    // nch: 16-column chunks of the accumulator that belong to this tile (tiles narrower than BN)
    const uint32_t n_end = min(a.N, n0 + 16u * (uint32_t)nch);   // first column not written by this tile
    const int mode = a.epi.mode;
    const uint32_t m = m_base + quad * 32 + lane;
    const bool row_ok = m < a.M;
    __half sr = __ushort_as_half(0), zr = __ushort_as_half(0);
    if (row_ok && mode != DUQ4_MODE_NONE) {
        sr = pb.s_row[(size_t)b * pb.row_vec_stride + m];
        if (pb.z_row) zr = pb.z_row[(size_t)b * pb.row_vec_stride + m];
    }
    const bool has_bias = pb.bias != nullptr;
    const bool asym = mode == DUQ4_MODE_ASYM || mode == DUQ4_MODE_ASYM_DUAL;
    const size_t ooff = ((size_t)b * a.M + m) * pb.ldo + n0;
    int32_t *arow = a.acc_out ? a.acc_out + ((size_t)b * a.M + m) * a.N + n0 : nullptr;
    if (pb.n_acc_owners && row_ok) {   // K-sharded layer: the partial sums of row m go to the rank that owns row m
        const uint32_t owner = m / pb.acc_rows_per_owner, r = m - owner * pb.acc_rows_per_owner;
        int32_t *base = pb.acc_owners[0];
#pragma unroll
        for (int o = 1; o < DUQ4_MAX_OUT_PEERS; ++o)
            if (owner == (uint32_t)o) base = pb.acc_owners[o];
        arow = base + ((size_t)pb.acc_slot * pb.acc_rows_per_owner + r) * a.N + n0;
    }
    const OutBases ob = out_bases(pb, a.out);
    uintptr_t obits = 0;
#pragma unroll
    for (int pi = 0; pi < DUQ4_MAX_OUT_PEERS; ++pi)
        if (pi < ob.n) obits |= reinterpret_cast<uintptr_t>(ob.base[pi]);
    const bool vec_ok = ((pb.ldo & 7u) == 0) && ((obits & 15u) == 0);
    __half *const mc = (STAGED && vec_ok && (reinterpret_cast<uintptr_t>(pb.mc_out) & 15u) == 0) ? pb.mc_out : nullptr;
    const bool avec_ok = ((a.N & 3u) == 0) && ((reinterpret_cast<uintptr_t>(a.acc_out) & 15u) == 0);   // owner buffers: alignment checked by the host
    const uint32_t taddr = tmem_acc + ((uint32_t)(quad * 32) << 16);
    const int w_hi = (ch_hi < 0 || ch_hi > nch) ? nch : ch_hi;
    const int ch_first = sk.out ? ch_lo : max(ch_lo, sk.ch_b), ch_last = (sk.out || sk.ch_e < 0) ? w_hi : min(w_hi, sk.ch_e);
    // first chunk at or after `c` that this call handles (phase 1 of a K-split skips the chunks the pair reduces itself)
    auto next_chunk = [&](int c) {
        if (sk.out && c >= sk.keep_b && c < sk.keep_e) c = sk.keep_e;
        return c < ch_last ? c : ch_last;
    };
    // the TMEM load of a chunk is issued while the chunk before it is processed
    uint32_t vn[16];
    int ch = next_chunk(ch_first);
    if (ch < ch_last) {
        __syncwarp();  // tcgen05.ld is warp-collective
        tmem_ld16(taddr + ch * 16, vn);
    }
#pragma unroll 1
    for (; ch < ch_last; ch = next_chunk(ch + 1)) {
        uint32_t v[16];
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = vn[j];
        {
            const int nx = next_chunk(ch + 1);
            if (nx < ch_last) {
                __syncwarp();
                tmem_ld16(taddr + nx * 16, vn);
            }
        }
        const uint32_t c0 = ch * 16;
        if (sk.out) {   // K-split tile, phase 1: raw accumulators to the scratch slab
            int4 *dst = reinterpret_cast<int4 *>(sk.out) + ((size_t)(ch * 4 + quad) * 4) * 32 + lane;
#pragma unroll
            for (int j = 0; j < 16; j += 4) dst[(j >> 2) * 32] = make_int4((int)v[j], (int)v[j + 1], (int)v[j + 2], (int)v[j + 3]);
            continue;
        }
        for (uint32_t c = 0; c < sk.n;) {   // K-split tile, phase 2: add the other pairs' partial sums, two slabs at a time
            if ((int)c == sk.skip) { ++c; continue; }
            uint32_t c1 = c + 1;
            if ((int)c1 == sk.skip) ++c1;
            const bool two = c1 < sk.n;
            const int4 *s0 = reinterpret_cast<const int4 *>(sk.add + c * sk.stride) + ((size_t)(ch * 4 + quad) * 4) * 32 + lane;
            const int4 *s1 = two ? reinterpret_cast<const int4 *>(sk.add + c1 * sk.stride) + ((size_t)(ch * 4 + quad) * 4) * 32 + lane : s0;
            int4 t0[4], t1[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                t0[q] = __ldcg(s0 + q * 32);
                t1[q] = two ? __ldcg(s1 + q * 32) : make_int4(0, 0, 0, 0);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                v[4 * q] += (uint32_t)(t0[q].x + t1[q].x); v[4 * q + 1] += (uint32_t)(t0[q].y + t1[q].y);
                v[4 * q + 2] += (uint32_t)(t0[q].z + t1[q].z); v[4 * q + 3] += (uint32_t)(t0[q].w + t1[q].w);
            }
            c = c1 + 1;
        }
        const bool col_any = n0 + c0 < n_end;
        const bool full = n0 + c0 + 16 <= n_end;
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = (uint32_t)(((int)v[j]) >> shift);
        if (STAGED && pb.n_acc_owners) {
            // K-sharded layer: partial sums to the owners of the rows. Staged like the fp16 output so that what crosses
            // NVLink are 128-byte row segments: lane = row writes its 16 ints (64 bytes) of this chunk; after two chunks
            // (32 columns) the warp reads the block back, four rows of 128 bytes per store instruction.
            int4 *mine = reinterpret_cast<int4 *>(stg + lane * 144 + (ch & 1) * 64);
#pragma unroll
            for (int j = 0; j < 16; j += 4) mine[j >> 2] = make_int4((int)v[j], (int)v[j + 1], (int)v[j + 2], (int)v[j + 3]);
            if ((ch & 1) == 1 || ch == ch_last - 1) {
                __syncwarp();
                const uint32_t g0 = (uint32_t)(ch >> 1) * 32 + (lane & 7) * 4;   // first column of this lane's 4 ints (tile-relative)
                const bool second_half = (lane & 7) >= 4;                        // columns of the odd chunk of the pair
                const bool have = n0 + g0 + 4 <= n_end && !(second_half && (ch & 1) == 0);
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const uint32_t r = it * 4 + (lane >> 3);
                    const uint32_t mr = m_base + quad * 32 + r;
                    if (mr >= a.M || !have) continue;
                    const uint32_t owner = mr / pb.acc_rows_per_owner, ro = mr - owner * pb.acc_rows_per_owner;
                    int32_t *base = pb.acc_owners[0];
#pragma unroll
                    for (int o = 1; o < DUQ4_MAX_OUT_PEERS; ++o)
                        if (owner == (uint32_t)o) base = pb.acc_owners[o];
                    *reinterpret_cast<int4 *>(base + ((size_t)pb.acc_slot * pb.acc_rows_per_owner + ro) * a.N + n0 + g0) =
                        *reinterpret_cast<const int4 *>(stg + r * 144 + (lane & 7) * 16);
                }
                __syncwarp();
            }
            if (mode == DUQ4_MODE_NONE) continue;
        } else if (arow && row_ok && col_any) {
            if (full && avec_ok) {
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                    *reinterpret_cast<int4 *>(arow + c0 + j) = make_int4((int)v[j], (int)v[j + 1], (int)v[j + 2], (int)v[j + 3]);
            } else {
                for (int j = 0; j < 16; ++j)
                    if (n0 + c0 + j < n_end) arow[c0 + j] = (int)v[j];
            }
        }
        if (mode == DUQ4_MODE_NONE) continue;
        __align__(16) __half2 o2[8];
        {
            const __half *csp = cs + c0, *czp = cz + c0, *cbp = cb + c0;
            const bool fast = a.acc_fits_22 != 0;
            if (asym) {
                if (has_bias) { if (fast) dequant16<true, true, true>(v, sr, zr, csp, czp, cbp, o2); else dequant16<true, true, false>(v, sr, zr, csp, czp, cbp, o2); }
                else          { if (fast) dequant16<true, false, true>(v, sr, zr, csp, czp, cbp, o2); else dequant16<true, false, false>(v, sr, zr, csp, czp, cbp, o2); }
            } else {
                if (has_bias) { if (fast) dequant16<false, true, true>(v, sr, zr, csp, czp, cbp, o2); else dequant16<false, true, false>(v, sr, zr, csp, czp, cbp, o2); }
                else          { if (fast) dequant16<false, false, true>(v, sr, zr, csp, czp, cbp, o2); else dequant16<false, false, false>(v, sr, zr, csp, czp, cbp, o2); }
            }
        }
        const __half *o = reinterpret_cast<const __half *>(o2);
        if (!STAGED) {
            if (!row_ok || !col_any) continue;
#pragma unroll
            for (int pi = 0; pi < DUQ4_MAX_OUT_PEERS; ++pi) {
                if (pi >= ob.n) break;
                if (!row_goes_to(pb, m, pi)) continue;
                __half *orow = ob.base[pi] + ooff;
                if (full && vec_ok) {
                    *reinterpret_cast<uint4 *>(orow + c0) = *reinterpret_cast<const uint4 *>(&o[0]);
                    *reinterpret_cast<uint4 *>(orow + c0 + 8) = *reinterpret_cast<const uint4 *>(&o[8]);
                } else {
                    for (int j = 0; j < 16; ++j)
                        if (n0 + c0 + j < n_end) orow[c0 + j] = o[j];
                }
            }
            continue;
        }
        // staged: lane = row writes its 32 bytes; after four chunks (64 columns) the warp
        // reads the block back as 128-byte row segments, four rows per store instruction
        *reinterpret_cast<uint4 *>(stg + lane * 144 + (ch & 3) * 32) = *reinterpret_cast<const uint4 *>(&o[0]);
        *reinterpret_cast<uint4 *>(stg + lane * 144 + (ch & 3) * 32 + 16) = *reinterpret_cast<const uint4 *>(&o[8]);
        if ((ch & 3) != 3 && ch != ch_last - 1) continue;   // flush every 64 columns and at the end of the range
        __syncwarp();
        const uint32_t g0 = (uint32_t)(ch >> 2) * 64 + (lane & 7) * 8;   // first column of this lane's 8 (tile-relative)
        const bool seg_full = n0 + g0 + 8 <= n_end;
        if (ob.n == 1 && !mc && vec_ok && pb.out_rows_per_owner == 0 && m_base + quad * 32 + 32 <= a.M && n0 + (uint32_t)(ch >> 2) * 64 + 64 <= n_end &&
            (ch & 3) == 3) {
            // the common case -- one destination, a whole 32 x 64 block inside the matrix: all eight reads, then all eight
            // stores, no per-segment decisions
            uint4 seg[8];
#pragma unroll
            for (int it = 0; it < 8; ++it) seg[it] = *reinterpret_cast<const uint4 *>(stg + (it * 4 + (lane >> 3)) * 144 + (lane & 7) * 16);
            __half *dst = ob.base[0] + ((size_t)b * a.M + m_base + quad * 32 + (lane >> 3)) * pb.ldo + n0 + g0;
            const size_t step = (size_t)4 * pb.ldo;
#pragma unroll
            for (int it = 0; it < 8; ++it) *reinterpret_cast<uint4 *>(dst + it * step) = seg[it];
            __syncwarp();   // the block is free for the next 64 columns
            continue;
        }
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const uint32_t r = it * 4 + (lane >> 3);
            const uint32_t mr = m_base + quad * 32 + r;
            if (mr >= a.M || n0 + g0 >= n_end) continue;
            const uint4 seg = *reinterpret_cast<const uint4 *>(stg + r * 144 + (lane & 7) * 16);
            const size_t off = ((size_t)b * a.M + mr) * pb.ldo + n0 + g0;
            if (mc && seg_full) {   // one store; the switch delivers it to every rank's buffer
                multimem_st16(mc + off, seg);
                continue;
            }
#pragma unroll
            for (int pi = 0; pi < DUQ4_MAX_OUT_PEERS; ++pi) {
                if (pi >= ob.n) break;
                if (!row_goes_to(pb, mr, pi)) continue;
                if (seg_full && vec_ok) {
                    *reinterpret_cast<uint4 *>(ob.base[pi] + off) = seg;
                } else {
                    const __half *hs = reinterpret_cast<const __half *>(&seg);
                    for (int j = 0; j < 8; ++j)
                        if (n0 + g0 + j < n_end) ob.base[pi][off + j] = hs[j];
                }
            }
        }
        __syncwarp();   // the block is free for the next 64 columns
    }
}

}  // namespace tc
}  // namespace duq4
