// CTA-pair (cta_group::2) variant of the tensor-core W4A4 GEMM, for pre-unpacked activations
// (A int8 [M,K] as written by the fused quantizer, W packed int4 [N,K/2]).
//
// Two CTAs on neighbouring SMs (a cluster of 2, no multicast loads) compute one 256 x 256 tile:
// CTA r of the pair holds rows [128r, 128r+128) of A and rows [128r, 128r+128) of the tile's W
// block. One thread of the even ("leader") CTA issues tcgen05.mma.cta_group::2 with M = 256,
// N = 256: each SM multiplies its own 128 A rows with the whole W block, half of which it reads
// from its partner's shared memory. Compared with the single-CTA 128 x 256 tile every CTA
// unpacks, stores and serves only HALF of the W block per unit of MMA work, which is what the
// single-CTA kernel is limited by (shared-memory bandwidth shared between the unpack and the
// MMA operand reads).
//
// Synchronisation (all waits bounded, see duq_ptx.cuh):
//   pk_full/pk_empty[s]  local : TMA of the packed W half  <->  unpack warps
//   up_full[u]   LEADER's only : 1 arrival + 32 KiB of TMA bytes (both CTAs' A tiles, their copies
//                                 carry .cta_group::2 and signal the leader's barrier) and one
//                                 arrival per unpack warp of BOTH CTAs  ->  MMA issuer
//   up_empty[u]  local, both   : tcgen05.commit by the leader into each CTA's barrier
//   acc_full[b]  local, both   : tcgen05.commit after a tile's last MMA
//   acc_empty[b] LEADER's only : one arrival per epilogue warp of BOTH CTAs
#include <cuda.h>

#include "duq_common.cuh"
#include "duq_ptx.cuh"
#include "gemm_tc_shared.cuh"

namespace duq4 {

__device__ int g_tc2_status = 0;

int tma_map_bytes_3d(const void *ptr, uint64_t kbytes, uint64_t rows, uint64_t batch, uint32_t box_k, uint32_t box_rows,
                     bool swizzle128, CUtensorMap *out, bool use_cache);

namespace tc2 {

using namespace ptx;
using namespace tc;

constexpr int BMH = 128;   // A rows per CTA (half of the pair's 256)
constexpr int BNH = 128;   // W rows per CTA at the full tile width (half of the pair's 256)
constexpr int BN = 256;    // accumulator columns at the full tile width; a launch may use narrower tiles
                           // (Args::bn, a multiple of 32) when that fills the last wave of tiles better
constexpr int BKE = 128;   // K elements per stage
// Warp roles: TMA-W producer, MMA issuer, EPI epilogue warps, UWN unpack warps, A producer -- 15 warps.
// The plain GEMM uses 4 epilogue + 8 unpack warps. The SiLU-gated gate/up variant (GU) turns that
// around, 8 + 4: its epilogue evaluates exp and an IEEE divide per output and needs the issue
// slots, while its W unpack (int8 activations need none) is light. Two epilogue warps then share
// a TMEM lane quadrant and split the tile's hidden channels between them.
constexpr int kThreads2 = 32 * 15;
constexpr int kUnpackedStage = (BMH + BNH) * BKE;   // 32 KiB: A tile then W half, both 128B-swizzled int8
constexpr int kStageOutWarp = 32 * 144;
// APK = activations arrive packed (int4, the reference's format) and are unpacked here too;
// otherwise they arrive as the quantizer's tensor-core-ready int8 and go straight into the MMA ring.
// WI8 = the weights arrive pre-laid-out as int8 as well (duq4_weight_prelayout_i8: 16 * code, K permuted like
// the activations): both operands go straight from TMA into the MMA ring and the unpack warps have nothing to do.
// Twice the weight bytes from HBM / L2, no shared-memory unpack traffic -- the measured alternative to the
// in-kernel unpack.
// STG = the epilogue stages its fp16 rows through shared memory and stores 128-byte row segments (what crosses NVLink
// well, and what the multicast and owner-routed stores need). A launch on pre-laid-out weights whose result stays on
// this GPU runs without: each lane stores its own row's 32 bytes per chunk (whole sectors in local memory) and the
// staging area pays for a sixth ring stage -- 98 vs 104 us at 512 tokens, 150 vs 155 at 1024, no difference from 2048 on.
template <bool APK, bool GU = false, bool WI8 = false, bool STG = true>
struct Cfg2 {
    static_assert(STG || (WI8 && !GU), "only the plain kernel on pre-laid-out weights has an unstaged form");
    // Epilogue warps / unpack warps. A tile's epilogue on FOUR warps (one per TMEM lane quadrant, alone on its
    // scheduler, every TMEM load -> dequant -> store chain exposed) takes 13 us -- measured with one-k-step problems --
    // against 17.7 us of MMA work per tile at K = 8192 and 8.8 us at K = 4096: hidden at the first, the limit at the
    // second. Where the unpack warps have little or nothing to do (gate/up variant, pre-laid-out weights) eight
    // warps share the epilogue, two per quadrant, half of the tile's columns each.
    static constexpr int EPI = (GU || WI8) ? 8 : 4;
    static constexpr int UWN = (GU || WI8) ? 4 : 8;
    static constexpr int kColTerms = EPI * 3 * BN * 2;
    // Ring depths. A packed stage is refilled by a TMA copy that takes about a microsecond to land
    // (L2 / HBM latency) while a k-step of MMA work takes 0.3-0.4 us, so the packed ring has to
    // cover ~3 k-steps of latency plus the stage being unpacked: with 3 stages the kernel ran at
    // (copy latency / 3) per k-step whatever the tile width.
    static constexpr int NPK = WI8 ? 1 : (GU ? (APK ? 3 : 5) : (APK ? 4 : 5));
    static constexpr int NUP = WI8 ? (STG ? 5 : 6) : ((APK || GU) ? 4 : 5);
    static constexpr int kPackedStage = WI8 ? 0 : (APK ? BMH + BNH : BNH) * (BKE / 2);   // 16 / 8 KiB; none without an unpack
    static constexpr int kStageOut = STG ? EPI * kStageOutWarp : 0;
    static constexpr int kSmem = 1024 + NUP * kUnpackedStage + NPK * kPackedStage + kColTerms + kStageOut + 512;
    static_assert(kSmem <= 232448, "exceeds the shared memory of a CTA");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_addr`'s counterpart in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait on a barrier that receives arrivals from the partner CTA (cluster-scope acquire).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag, int code) {
    uint64_t t0 = 0;
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_cluster(bar, parity)) return true;
        if ((it & 0xFFu) == 0) {
            if (*abort_flag) return false;
            uint64_t now = globaltimer();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > kPtxWaitLimitNs) {
                *abort_flag = 1;
                atomicCAS(&g_tc2_status, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma2_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on ONE barrier (shared::cluster address, either CTA of the pair) once every MMA issued
// so far by this thread has completed in both CTAs.
__device__ __forceinline__ void umma2_commit(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
// A-tile copy of either CTA: data lands in the issuing CTA's shared memory, the byte count is
// credited to the LEADER's barrier.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, uint32_t leader_bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(leader_bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// Epilogue of the SiLU-gated gate/up projection. The tile's accumulator holds, for the same 128
// hidden channels j = j0 .. j0+127, the gate pre-activations in columns [0,128) and the up
// projections in columns [128,256) (the two CTAs of the pair loaded their W halves from the gate
// rows and from the up rows). One warp's 32 rows: both halves are dequantized to fp16 exactly as the
// plain epilogue would write them, h = half(half(silu(g)) * u) is formed in registers and only h
// [M, I] goes to memory -- the fp16 gate/up tensor never exists.
__device__ __forceinline__ void epi_store_tile_gate_up(const Args &a, const EpiParams &pb, uint32_t m_base, uint32_t j0,
                                                       uint32_t tmem_acc, int quad, int lane, const __half *cs,
                                                       const __half *cz, const __half *cb, uint8_t *stg, int ch_begin,
                                                       int ch_end) {
    const int mode = a.epi.mode;
    const uint32_t inter = a.gate_up;
    const uint32_t m = m_base + quad * 32 + lane;
    const bool row_ok = m < a.M;
    __half sr = __ushort_as_half(0), zr = __ushort_as_half(0);
    if (row_ok) {
        sr = pb.s_row[m];
        if (pb.z_row) zr = pb.z_row[m];
    }
    const bool has_bias = pb.bias != nullptr;
    const bool asym = mode == DUQ4_MODE_ASYM;
    const OutBases ob = out_bases(pb, a.out);
    uintptr_t obits = 0;
#pragma unroll
    for (int pi = 0; pi < DUQ4_MAX_OUT_PEERS; ++pi)
        if (pi < ob.n) obits |= reinterpret_cast<uintptr_t>(ob.base[pi]);
    const bool vec_ok = ((pb.ldo & 7u) == 0) && ((obits & 15u) == 0);
    const uint32_t taddr = tmem_acc + ((uint32_t)(quad * 32) << 16);
    // Dequant with the plain epilogue's routine (two columns per instruction, every lane of hmul2 / hsub2 / hadd2 rounds
    // like the scalar _rn form, so the values equal the plain epilogue's), one call for the chunk's 16 gate columns and
    // one for its 16 up columns.
    auto deq16 = [&](uint32_t (&v)[16], int c, __half2 (&o2)[8]) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = (uint32_t)(((int)v[j]) >> 8);   // accumulators are 256 x the true sums
        const bool fast = a.acc_fits_22 != 0;
        if (asym) {
            if (has_bias) { if (fast) tc::dequant16<true, true, true>(v, sr, zr, cs + c, cz + c, cb + c, o2); else tc::dequant16<true, true, false>(v, sr, zr, cs + c, cz + c, cb + c, o2); }
            else          { if (fast) tc::dequant16<true, false, true>(v, sr, zr, cs + c, cz + c, cb + c, o2); else tc::dequant16<true, false, false>(v, sr, zr, cs + c, cz + c, cb + c, o2); }
        } else {
            if (has_bias) { if (fast) tc::dequant16<false, true, true>(v, sr, zr, cs + c, cz + c, cb + c, o2); else tc::dequant16<false, true, false>(v, sr, zr, cs + c, cz + c, cb + c, o2); }
            else          { if (fast) tc::dequant16<false, false, true>(v, sr, zr, cs + c, cz + c, cb + c, o2); else tc::dequant16<false, false, false>(v, sr, zr, cs + c, cz + c, cb + c, o2); }
        }
    };
#pragma unroll 1
    for (int ch = ch_begin; ch < ch_end; ++ch) {   // 16-channel chunks of the tile's 128 hidden channels (a multiple of 4 of them)
        uint32_t vg[16], vu[16];
        __syncwarp();  // tcgen05.ld is warp-collective
        tmem_ld16(taddr + ch * 16, vg);
        tmem_ld16(taddr + 128 + ch * 16, vu);
        tmem_ld_wait();
        const int c0 = ch * 16;
        __align__(16) __half o[16];
        __half2 g2[8], u2[8];
        deq16(vg, c0, g2);
        deq16(vu, 128 + c0, u2);
        // h = half(half(silu(g)) * u) as silu_mul_one forms it, in stages over the 16 elements so that the sixteen
        // exponentials (branch-free) can be interleaved by the compiler before the divides (one block each)
        float xs[16], ds[16];
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            const float2 x2 = __half22float2(g2[p]);
            xs[2 * p] = x2.x;
            xs[2 * p + 1] = x2.y;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) ds[j] = 1.0f + expf(-xs[j]);
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            const __half2 s2 = __floats2half2_rn(__fdiv_rn(xs[2 * p], ds[2 * p]), __fdiv_rn(xs[2 * p + 1], ds[2 * p + 1]));
            *reinterpret_cast<__half2 *>(&o[2 * p]) = __hmul2_rn(s2, u2[p]);
        }
        *reinterpret_cast<uint4 *>(stg + lane * 144 + (ch & 3) * 32) = *reinterpret_cast<const uint4 *>(&o[0]);
        *reinterpret_cast<uint4 *>(stg + lane * 144 + (ch & 3) * 32 + 16) = *reinterpret_cast<const uint4 *>(&o[8]);
        if ((ch & 3) != 3) continue;
        __syncwarp();
        const uint32_t g0 = (uint32_t)(ch >> 2) * 64 + (lane & 7) * 8;   // first hidden channel of this lane's 8 (tile-relative)
        const bool seg_full = j0 + g0 + 8 <= inter;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const uint32_t r = it * 4 + (lane >> 3);
            const uint32_t mr = m_base + quad * 32 + r;
            if (mr >= a.M || j0 + g0 >= inter) continue;
            const uint4 seg = *reinterpret_cast<const uint4 *>(stg + r * 144 + (lane & 7) * 16);
            const size_t off = (size_t)mr * pb.ldo + j0 + g0;
#pragma unroll
            for (int pi = 0; pi < DUQ4_MAX_OUT_PEERS; ++pi) {
                if (pi >= ob.n) break;
                if (seg_full && vec_ok) {
                    *reinterpret_cast<uint4 *>(ob.base[pi] + off) = seg;
                } else {
                    const __half *hs = reinterpret_cast<const __half *>(&seg);
                    for (int j = 0; j < 8; ++j)
                        if (j0 + g0 + j < inter) ob.base[pi][off + j] = hs[j];
                }
            }
        }
        __syncwarp();   // the block is free for the next 64 channels
    }
}

template <bool APK, bool GU, bool WI8, bool STG>
__global__ void __launch_bounds__(kThreads2, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Args a) {
    static_assert(!WI8 || !APK, "pre-laid-out weights go with int8 activations");
    using C2 = Cfg2<APK, GU, WI8, STG>;
    constexpr int NPK = C2::NPK, NUP = C2::NUP, kPackedStage = C2::kPackedStage;
    constexpr int EPI = C2::EPI, UW = C2::UWN, kColTerms = C2::kColTerms;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gbase = smem_raw + (base - raw);
    const uint32_t up0 = base;
    const uint32_t pk0 = up0 + NUP * kUnpackedStage;
    const uint32_t ct_off = NUP * kUnpackedStage + NPK * kPackedStage;
    __half *colterms = reinterpret_cast<__half *>(gbase + ct_off);
    uint8_t *stage_out = gbase + ct_off + kColTerms;
    const uint32_t bar0 = base + ct_off + kColTerms + C2::kStageOut;
    auto pk_full = [&](int s) { return bar0 + 8u * s; };
    auto pk_empty = [&](int s) { return bar0 + 8u * (8 + s); };
    auto up_full = [&](int s) { return bar0 + 8u * (16 + s); };
    auto up_empty = [&](int s) { return bar0 + 8u * (22 + s); };
    auto acc_full = [&](int s) { return bar0 + 8u * (28 + s); };
    auto acc_empty = [&](int s) { return bar0 + 8u * (30 + s); };
    const uint32_t drain_bar = bar0 + 8u * 32;
    static_assert(NPK <= 8 && NUP <= 6, "barrier map");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const uint32_t pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const uint32_t num_tiles = a.tiles_m * a.tiles_n * a.batch;   // tiles of 256 x 256
    const uint32_t ksteps = (a.K + BKE - 1) / BKE;
    const uint32_t bn = a.bn, bnh = bn >> 1;   // this launch's tile width and each CTA's share of the W block
    constexpr int kLastWarp = 2 + EPI + UW;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < 8; ++s) {
            mbar_init(pk_full(s), 1);
            mbar_init(pk_empty(s), UW);
        }
        for (int s = 0; s < 6; ++s) {
            mbar_init(up_full(s), WI8 ? 1 : (APK ? 0 : 1) + 2 * UW);
            mbar_init(up_empty(s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(acc_full(s), 1);
            mbar_init(acc_empty(s), 2 * EPI);
        }
        mbar_init(drain_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // the same warp of both CTAs performs the paired allocation
        tmem_alloc2(smem_u32(&tmem_base_slot), 512);
        tmem_relinquish2();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers are initialised before anyone arrives remotely
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abortp = &abort_flag;

    // Work list of this pair: its tiles of the full rounds (tile = pair, pair + npairs, ... below dp_tiles), then --
    // when the launch splits its last, partly filled round along K -- one K range of one of the remaining tiles.
    struct Work {
        uint32_t tile, k0, k1;
        int sk_rank;        // -1: whole tile; >= 0: K-split tile, this pair's place in the group that shares it
        uint32_t sk_slot;
    };
    const uint32_t dp_tiles = num_tiles - a.sk_tiles;
    const uint32_t n_dp = pair < dp_tiles ? (dp_tiles - pair + npairs - 1) / npairs : 0;
    auto work_at = [&](uint32_t i, Work &w) -> bool {
        if (i < n_dp) {
            w.tile = pair + i * npairs; w.k0 = 0; w.k1 = ksteps; w.sk_rank = -1; w.sk_slot = 0;
            return true;
        }
        if (i == n_dp && pair < a.sk_tiles * a.sk_group) {
            const uint32_t g = pair / a.sk_group, r = pair % a.sk_group;
            w.tile = dp_tiles + g; w.k0 = r * ksteps / a.sk_group; w.k1 = (r + 1) * ksteps / a.sk_group;
            w.sk_rank = (int)r; w.sk_slot = g;
            return true;
        }
        return false;
    };
    // Tile order: row block fastest inside bands of a.band_rows row blocks, bands one after the other. Consecutive tiles
    // -- the ones the pairs work on at the same time -- then share a few weight tiles and the activations of one band
    // (16 row blocks of K = 8192: 33 MB), which stay in L2 beside the streaming weights and results; with all 32 row
    // blocks of an 8192-token problem in one band the activations were evicted between column tiles.
    const uint32_t kBandRows = a.band_rows;
    auto tile_coords = [&](uint32_t tile, uint32_t &b, uint32_t &tm, uint32_t &tn) {
        const uint32_t per_b = a.tiles_m * a.tiles_n;
        b = tile / per_b;
        const uint32_t r = tile % per_b;
        const uint32_t per_band = kBandRows * a.tiles_n;
        const uint32_t band = r / per_band, rb = r % per_band;
        const uint32_t rows_here = min(kBandRows, a.tiles_m - band * kBandRows);
        tn = rb / rows_here;
        tm = band * kBandRows + rb % rows_here;
    };

    if (warp == 0) {
        // ---------------- TMA producer: this CTA's half of the packed W block ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            Work w;
            for (uint32_t wi = 0; ok && work_at(wi, w); ++wi) {
                uint32_t b, tm, tn;
                tile_coords(w.tile, b, tm, tn);
                for (uint32_t ks = w.k0; ks < w.k1; ++ks, ++it) {
                    if (WI8) {   // this CTA's half of the int8 W block straight into the MMA ring, credited to the leader
                        const uint32_t u = it % NUP, uph = (it / NUP) & 1;
                        if (!(ok = mbar_wait(up_empty(u), uph ^ 1, abortp, &g_tc2_status, 1))) break;
                        // gate/up mode: the leader's half comes from the gate rows, the partner's from the up rows
                        const uint32_t wrow8 = a.gate_up ? (rank ? a.gate_up : 0u) + tn * 128u : tn * bn + rank * bnh;
                        tma_load_3d_pair(up0 + u * kUnpackedStage + BMH * BKE, &tmB, mapa(up_full(u), 0), ks * BKE, wrow8, b);
                        continue;
                    }
                    const uint32_t s = it % NPK, ph = (it / NPK) & 1;
                    if (!(ok = mbar_wait(pk_empty(s), ph ^ 1, abortp, &g_tc2_status, 1))) break;
                    mbar_expect_tx(pk_full(s), ((APK ? BMH : 0) + bnh) * (BKE / 2));
                    uint32_t dst = pk0 + s * kPackedStage;
                    if (APK) {
                        tma_load_3d(dst, &tmA, pk_full(s), ks * (BKE / 2), tm * 256 + rank * BMH, b);
                        dst += BMH * (BKE / 2);
                    }
                    // gate/up mode: the leader's half comes from the gate rows, the partner's from the up rows
                    const uint32_t wrow = a.gate_up ? (rank ? a.gate_up : 0u) + tn * 128u : tn * bn + rank * bnh;
                    tma_load_3d(dst, &tmB, pk_full(s), ks * (BKE / 2), wrow, b);
                }
            }
            if (!ok) {
                uint64_t t0 = globaltimer();
                while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
            }
        }
    } else if (!APK && warp == kLastWarp) {
        // ---------------- TMA producer: this CTA's 128 rows of A, credited to the leader ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            Work w;
            for (uint32_t wi = 0; ok && work_at(wi, w); ++wi) {
                uint32_t b, tm, tn;
                tile_coords(w.tile, b, tm, tn);
                for (uint32_t ks = w.k0; ks < w.k1; ++ks, ++it) {
                    const uint32_t u = it % NUP, uph = (it / NUP) & 1;
                    if (!(ok = mbar_wait(up_empty(u), uph ^ 1, abortp, &g_tc2_status, 7))) break;
                    if (rank == 0) mbar_expect_tx(up_full(u), 2 * BMH * BKE + (WI8 ? 2 * bnh * BKE : 0));   // both CTAs' A tiles (and int8 W halves)
                    tma_load_3d_pair(up0 + u * kUnpackedStage, &tmA, mapa(up_full(u), 0), ks * BKE, tm * 256 + rank * BMH, b);
                }
            }
            if (!ok) {
                uint64_t t0 = globaltimer();
                while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = make_idesc(256, (int)bn);
            uint32_t it = 0, lt = 0;
            bool ok = true, issued = false;
            Work w;
            for (uint32_t wi = 0; ok && work_at(wi, w); ++wi, ++lt) {
                const uint32_t buf = lt & 1, aph = (lt >> 1) & 1;
                if (!(ok = mbar_wait_cluster(acc_empty(buf), aph ^ 1, abortp, 2))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (uint32_t ks = w.k0; ks < w.k1; ++ks, ++it) {
                    const uint32_t u = it % NUP, ph = (it / NUP) & 1;
                    if (!(ok = mbar_wait_cluster(up_full(u), ph, abortp, 3))) break;
                    tc_fence_after();
                    const uint32_t sa = up0 + u * kUnpackedStage, sb = sa + BMH * BKE;
                    const uint64_t da = make_desc(sa), db = make_desc(sb);
#pragma unroll
                    for (int kk = 0; kk < BKE / 32; ++kk)
                        umma2_i8(d_tmem, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, ((ks - w.k0) | kk) != 0);
                    issued = true;
                    umma2_commit(up_empty(u));            // this CTA's stage ...
                    umma2_commit(mapa(up_empty(u), 1));   // ... and the partner's
                }
                if (ok) {
                    umma2_commit(acc_full(buf));
                    umma2_commit(mapa(acc_full(buf), 1));
                }
            }
            if (!ok && issued) {
                umma2_commit(drain_bar);
                uint64_t t0 = globaltimer();
                while (!mbar_try(drain_bar, 0) && globaltimer() - t0 < kPtxWaitLimitNs) __nanosleep(1000);
            }
        }
    } else if (warp < 2 + EPI) {
        // ---------------- epilogue: this CTA's 128 rows of the tile ----------------
        const int quad = warp & 3;
        uint32_t lt = 0;
        bool ok = true;
        Work w;
        for (uint32_t wi = 0; ok && work_at(wi, w); ++wi, ++lt) {
            uint32_t b, tm, tn;
            tile_coords(w.tile, b, tm, tn);
            const uint32_t buf = lt & 1, aph = (lt >> 1) & 1;
            const uint32_t n0 = tn * bn;
            EpiParams pb = a.epi;
            __half *cs = colterms + (warp - 2) * 3 * BN, *cz = cs + BN, *cb = cz + BN;
            // with eight epilogue warps the two warps of a lane quadrant take the chunks [0, 8) and [8, end) of the tile
            const int wch_lo = (EPI == 8 && warp >= 6) ? 8 : 0, wch_hi = (EPI == 8 && warp < 6) ? 8 : -1;
            if (GU) {
                // per-channel terms of the tile's 128 gate columns, then of its 128 up columns; this warp's hidden
                // channels only, all loads before the first store (see epi_stage_colterms)
                __syncwarp();
                const int hc_lo = ((warp - 2) >> 2) * 64, hc_hi = hc_lo + 64;
                ColTerms t[BN / 32];
#pragma unroll
                for (int i = 0; i < BN / 32; ++i) {
                    const int c = lane + 32 * i;
                    const uint32_t j = tn * 128u + (uint32_t)(c & 127);
                    t[i].s = t[i].z = t[i].b = __ushort_as_half(0);
                    if ((c & 127) >= hc_lo && (c & 127) < hc_hi && j < a.gate_up) t[i] = load_col_terms(pb, (c < 128 ? 0u : a.gate_up) + j);
                }
#pragma unroll
                for (int i = 0; i < BN / 32; ++i) {
                    const int c = lane + 32 * i;
                    if ((c & 127) >= hc_lo && (c & 127) < hc_hi) {
                        cs[c] = t[i].s;
                        cz[c] = t[i].z;
                        cb[c] = t[i].b;
                    }
                }
                __syncwarp();
            } else {
                epi_stage_colterms<BN>(a, pb, b, n0, lane, cs, cz, cb, wch_lo * 16, wch_hi < 0 ? BN : wch_hi * 16);
            }
            if (!(ok = mbar_wait(acc_full(buf), aph, abortp, &g_tc2_status, 4))) break;
            tc_fence_after();
            if (GU)   // warps 2..5 take hidden channels [0,64) of the tile, warps 6..9 [64,128)
                epi_store_tile_gate_up(a, pb, tm * 256 + rank * BMH, tn * 128u, tmem_base + buf * BN, quad, lane, cs, cz, cb,
                                       stage_out + (warp - 2) * kStageOutWarp, ((warp - 2) >> 2) * 4, ((warp - 2) >> 2) * 4 + 4);
            else if (w.sk_rank < 0)
                epi_store_tile<BN, STG>(a, pb, b, tm * 256 + rank * BMH, n0, tmem_base + buf * BN, quad, lane, 8, cs, cz, cb,
                                         stage_out + (warp - 2) * kStageOutWarp, (int)(bn >> 4), tc::SplitK(), wch_lo, wch_hi);
            else {
                // K-split tile: the G pairs of the group hold partial sums over their K ranges. Reduce-scatter through
                // L2: the first R = min(G, 4) pairs each own a range of the tile's 16-column chunks (multiples of four
                // chunks, so that the output staging below flushes whole 64-column groups). Phase 1: every pair writes
                // the chunks it does not own to its slab -- [tile slot][pair of the group][CTA of the pair][128 rows][BN]
                // int32 -- and arrives. Phase 2: an owning pair waits for the whole group, adds the other pairs' slabs to
                // its own accumulators for its chunks, dequantizes and stores them. The adds are exact, so the result
                // does not depend on the split.
                const uint32_t G = a.sk_group, R = G < 4 ? G : 4;
                const int nch = (int)(bn >> 4);
                const int cpr = 4 * ((nch + 4 * (int)R - 1) / (4 * (int)R));
                const int r = w.sk_rank;
                const int own_b = r < (int)R ? min(nch, r * cpr) : 0, own_e = r < (int)R ? min(nch, (r + 1) * cpr) : 0;
                const size_t slab = (size_t)BMH * BN;
                int32_t *slot0 = a.sk_scratch + (size_t)w.sk_slot * G * 2 * slab;
                tc::SplitK p1;
                p1.out = slot0 + ((size_t)r * 2 + rank) * slab;
                p1.keep_b = own_b; p1.keep_e = own_e;
                epi_store_tile<BN, STG>(a, pb, b, tm * 256 + rank * BMH, n0, tmem_base + buf * BN, quad, lane, 8, cs, cz, cb,
                                         stage_out + (warp - 2) * kStageOutWarp, nch, p1, wch_lo, wch_hi);
                __threadfence();   // this lane's partial sums are visible device-wide before the arrival below
                __syncwarp();
                unsigned int *cw = a.sk_counters + w.sk_slot;
                if (lane == 0) atomicAdd(cw, 1u);
                if (own_e > own_b) {
                    // bounded wait for the 2 x EPI epilogue warps of each of the G pairs
                    const unsigned int want = G * 2 * EPI;
                    bool arrived = false;
                    uint64_t t0 = 0;
                    for (uint32_t spin = 1; !arrived; ++spin) {
                        unsigned int v;
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(cw) : "memory");
                        arrived = v >= want;
                        if (arrived || (spin & 0x3Fu) != 0) continue;
                        if (*abortp) break;
                        const uint64_t now = globaltimer();
                        if (t0 == 0) t0 = now;
                        else if (now - t0 > kPtxWaitLimitNs) {
                            *abortp = 1;
                            atomicCAS(&g_tc2_status, 0, 8);
                            break;
                        }
                    }
                    if (!(ok = arrived)) break;
                    tc::SplitK p2;
                    p2.add = slot0 + (size_t)rank * slab;
                    p2.n = G; p2.skip = r; p2.stride = 2 * slab;
                    p2.ch_b = own_b; p2.ch_e = own_e;
                    epi_store_tile<BN, STG>(a, pb, b, tm * 256 + rank * BMH, n0, tmem_base + buf * BN, quad, lane, 8, cs, cz, cb,
                                             stage_out + (warp - 2) * kStageOutWarp, nch, p2, wch_lo, wch_hi);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa(acc_empty(buf), 0));
        }
    } else if (!WI8 && warp < kLastWarp) {
        // ---------------- unpack warps: this CTA's packed W half (and packed A rows) -> swizzled int8 ----------------
        const int ut = (warp - 2 - EPI) * 32 + lane;
        const int kChunks = (int)((APK ? BMH + bnh : bnh) * 4);   // 16-byte chunks of packed rows in a stage
        constexpr uint32_t kDstOff = APK ? 0 : BMH * BKE;
        uint32_t it = 0;
        bool ok = true;
        Work w;
        for (uint32_t wi = 0; ok && work_at(wi, w); ++wi) {
            for (uint32_t ks = w.k0; ks < w.k1; ++ks, ++it) {
                const uint32_t s = it % NPK, ph = (it / NPK) & 1;
                const uint32_t u = it % NUP, uph = (it / NUP) & 1;
                if (!(ok = mbar_wait(pk_full(s), ph, abortp, &g_tc2_status, 5))) break;
                if (!(ok = mbar_wait(up_empty(u), uph ^ 1, abortp, &g_tc2_status, 6))) break;
                const uint32_t src = pk0 + s * kPackedStage, dst = up0 + u * kUnpackedStage + kDstOff;
#pragma unroll 2
                for (int idx = ut; idx < kChunks; idx += UW * 32) {
                    uint32_t w0, w1, w2, w3;
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3)
                                 : "r"(src + idx * 16));
                    const uint32_t row = idx >> 2, c = idx & 3, sw = row & 7;
                    const uint32_t rowaddr = dst + row * 128;
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(rowaddr + (((2 * c) ^ sw) << 4)),
                                 "r"(nib_lo(w0)), "r"(nib_lo(w1)), "r"(nib_lo(w2)), "r"(nib_lo(w3))
                                 : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(rowaddr + (((2 * c + 1) ^ sw) << 4)),
                                 "r"(nib_hi(w0)), "r"(nib_hi(w1)), "r"(nib_hi(w2)), "r"(nib_hi(w3))
                                 : "memory");
                }
                fence_proxy_async();   // generic-proxy writes -> the pair's MMA (async proxy); the cluster-scope release of the arrive below publishes them to the partner
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(pk_empty(s));
                    mbar_arrive_cluster(mapa(up_full(u), 0));
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the partner has finished with this CTA's shared memory and its own TMEM
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc2(tmem_base, 512);
    }
}

}  // namespace tc2

// Tile width for a launch. Tiles are handed out round-robin to a fixed number of CTA pairs, so the
// launch takes ceil(tiles / pairs) rounds. Measured on B200, a round of 224-wide tiles takes 0.98 of
// a round of 256-wide tiles and 192-wide ones 0.94 (the MMA time hardly shrinks with the width), so
// a narrower tile only pays where it does not add a round: it then trims the round time a little
// and spreads a nearly empty last round over more pairs (e.g. N = 8192: 32 -> 37 tile columns,
// M = 2048: 256 tiles = 3.46 rounds -> 296 tiles = exactly 4 rounds of cheaper tiles).
// DUQ4_TC_BN pins a width (multiple of 32; tests and experiments).
static uint32_t pick_tile_width(uint32_t tiles_m, uint32_t N, uint32_t batch, uint32_t pairs) {
    static const int forced = [] {
        const char *e = getenv("DUQ4_TC_BN");
        const int v = e ? atoi(e) : 0;
        return (v < 32 || v > 256 || v % 32 != 0) ? 0 : v;
    }();
    if (forced) return (uint32_t)forced;
    auto rounds = [&](uint32_t bn) { return ((uint64_t)tiles_m * cdiv(N, bn) * batch + pairs - 1) / pairs; };
    return rounds(224) <= rounds(256) ? 224u : 256u;
}

// Scratch the K-split of a launch's last round may use: partial int32 tiles of at most one round of pairs, plus the
// arrival counters (the first 1 KiB).
constexpr size_t kSkCounterBytes = 1024;
size_t gemm_tc2_split_scratch_bytes() { return kSkCounterBytes + (size_t)148 / 2 * 256 * 256 * sizeof(int32_t); }

template <bool APK, bool GU = false, bool WI8 = false, bool STG = true>
static int launch2(const void *A, const void *B, uint32_t M, uint32_t N, uint32_t K, uint32_t batch, const EpiParams &p,
                   void *out, int32_t *acc_out, cudaStream_t st, uint32_t gate_up = 0, bool cache_maps = true,
                   void *sk_scratch = nullptr, size_t sk_bytes = 0) {
    using namespace tc2;
    constexpr int kSmem2 = Cfg2<APK, GU, WI8, STG>::kSmem;
    auto *kernel = gemm_tc2_kernel<APK, GU, WI8, STG>;
    if (((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) != 0) return DUQ4_ERR_ALIGN;
    if (K >= 131072u) return DUQ4_ERR_SHAPE;
    static DeviceOnce once;
    static std::atomic<int> pairs_of[64];
    const int dev = current_device_slot();
    if (dev < 0) return DUQ4_ERR_DEVICE;
    int orc = once.run(dev, [&] {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem2);
        if (e != cudaSuccess) return (int)e;
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3(2 * 148);
        q.blockDim = dim3(kThreads2);
        q.dynamicSmemBytes = kSmem2;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        q.attrs = at;
        q.numAttrs = 1;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, kernel, &q);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            n = 0;
        }
        pairs_of[dev].store(n, std::memory_order_relaxed);
        return 0;
    });
    if (orc) return orc;
    const int max_pairs = pairs_of[dev].load(std::memory_order_relaxed);
    if (max_pairs < 1) return DUQ4_ERR_DEVICE;
    tc::Args a{};
    a.M = M; a.N = N; a.K = K; a.batch = batch;
    a.epi = p;
    a.out = (__half *)out;
    a.acc_out = acc_out;
    a.tiles_m = cdiv(M, 256);
    a.acc_fits_22 = (uint64_t)K * 64 <= (1u << 22) ? 1u : 0u;   // |int4 x int4| <= 64 per term
    // row blocks per band of the tile order; measured on 8192 tokens: K = 8192 -> 3652 / 3806 / 3804 / 3616 TOPS with bands of
    // 4 / 8 / 16 / 32, K = 28672 -> 3459 / 3552 / 3389 / 3301
    a.band_rows = K > 16384 ? 8 : 16;
    a.gate_up = gate_up;   // N is then the width I of h; W has 2*I rows, tiles are 256 rows x 128 hidden channels
    // 256-wide tiles for peer output too: a 224-wide tile starts on a 448-byte boundary, so its 128-byte row
    // segments straddle 128-byte lines of the destination -- harmless in local HBM (whole 32-byte sectors),
    // two packets instead of one per segment over NVLink (fused gather at 4 GPUs: 0.457 vs 0.381 ms)
    a.bn = (gate_up || p.n_peers > 1) ? 256u : pick_tile_width(a.tiles_m, N, batch, (uint32_t)max_pairs);
    a.tiles_n = gate_up ? cdiv(N, 128) : cdiv(N, a.bn);
    CUtensorMap ma, mb;
    int rc = APK ? tma_map_bytes_3d(A, K / 2, M, batch, BKE / 2, BMH, false, &ma, cache_maps)
                 : tma_map_bytes_3d(A, K, M, batch, BKE, BMH, true, &ma, cache_maps);
    if (rc) return rc;
    rc = WI8 ? tma_map_bytes_3d(B, K, gate_up ? 2ull * N : N, batch, BKE, a.bn / 2, true, &mb, cache_maps)
             : tma_map_bytes_3d(B, K / 2, gate_up ? 2ull * N : N, batch, BKE / 2, a.bn / 2, false, &mb, cache_maps);
    if (rc) return rc;
    const uint32_t tiles = a.tiles_m * a.tiles_n * batch;
    uint32_t pairs = tiles < (uint32_t)max_pairs ? tiles : (uint32_t)max_pairs;
    // K-split of the last, partly filled round (needs caller scratch): T tiles are left after the full rounds; when
    // they occupy at most half of the pairs, each is computed by G pairs, a K range each, and up to four pairs of the
    // group each add the others' partial sums for a quarter of the tile's columns before their epilogue (a
    // reduce-scatter through L2). The round then costs about 1/G of a tile (plus the partial tiles' trip through L2)
    // instead of a whole one: 8192 -> 28672 at 512 tokens is 224 tiles on 74 pairs,
    // 3 rounds + 2 tiles; the 2 tiles are split eight ways instead of taking a fourth round.
    a.sk_tiles = a.sk_group = 0;
    if (!GU && sk_scratch && (reinterpret_cast<uintptr_t>(sk_scratch) & 255) == 0) {
        const uint32_t T = tiles % (uint32_t)max_pairs;
        uint32_t G = T ? (uint32_t)max_pairs / T : 0;
        if (G > 8) G = 8;
        const uint32_t ksteps = cdiv(K, (uint32_t)BKE);
        while (G >= 2 && ksteps < 4 * G) --G;   // every K range keeps at least four pipeline stages of work
        const size_t need = kSkCounterBytes + (size_t)T * G * 256 * 256 * sizeof(int32_t);
        if (T && G >= 2 && T * sizeof(unsigned int) <= kSkCounterBytes && need <= sk_bytes) {
            a.sk_tiles = T;
            a.sk_group = G;
            a.sk_counters = (unsigned int *)sk_scratch;
            a.sk_scratch = (int32_t *)((uint8_t *)sk_scratch + kSkCounterBytes);
            const uint32_t busy = tiles - T >= (uint32_t)max_pairs ? (uint32_t)max_pairs : T * G;   // full rounds use every pair
            pairs = busy;
            cudaError_t me = cudaMemsetAsync(sk_scratch, 0, kSkCounterBytes, st);
            if (me != cudaSuccess) return (int)me;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(kThreads2);
    cfg.dynamicSmemBytes = kSmem2;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ma, mb, a);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return (int)e;
    }
    return launch_status();
}

// A: int8 pre-unpacked [batch, M, K] (a_packed = false) or packed int4 [batch, M, K/2]; W packed
// [batch, N, K/2]. Returns DUQ4_ERR_DEVICE when the device cannot co-schedule CTA pairs (the
// caller then uses the single-CTA kernel).
int gemm_tc2_launch(bool a_packed, const void *A, const void *B, uint32_t M, uint32_t N, uint32_t K, uint32_t batch,
                    const EpiParams &p, void *out, int32_t *acc_out, cudaStream_t st, bool cache_maps) {
    return a_packed ? launch2<true>(A, B, M, N, K, batch, p, out, acc_out, st, 0, cache_maps)
                    : launch2<false>(A, B, M, N, K, batch, p, out, acc_out, st, 0, cache_maps);
}

// Both operands int8 in the tensor-core-ready layout (A from duq4_quantize_fused_i8, W from
// duq4_weight_prelayout_i8). DUQ4_ERR_DEVICE when the device cannot co-schedule CTA pairs.
int gemm_tc2_launch_prelaid(const void *A, const void *W_i8, uint32_t M, uint32_t N, uint32_t K, const EpiParams &p, void *out,
                            int32_t *acc_out, cudaStream_t st, void *sk_scratch, size_t sk_bytes) {
    // results that stay on this GPU need no staged row segments (see Cfg2)
    if (p.n_peers == 0 && p.n_acc_owners == 0)
        return launch2<false, false, true, false>(A, W_i8, M, N, K, 1, p, out, acc_out, st, 0, true, sk_scratch, sk_bytes);
    return launch2<false, false, true>(A, W_i8, M, N, K, 1, p, out, acc_out, st, 0, true, sk_scratch, sk_bytes);
}

// SiLU-gated gate/up projection: W packed [2*I, K/2] (gate rows, then up rows), per-channel vectors of
// length 2*I, h_out fp16 [M, I] = silu(gate) * up of the dequantized projections.
int gemm_tc2_launch_gate_up(bool a_packed, const void *A, const void *W, uint32_t M, uint32_t inter, uint32_t K,
                            const EpiParams &p, void *h_out, cudaStream_t st) {
    return a_packed ? launch2<true, true>(A, W, M, inter, K, 1, p, h_out, nullptr, st, inter)
                    : launch2<false, true>(A, W, M, inter, K, 1, p, h_out, nullptr, st, inter);
}

// The same on pre-laid-out int8 weights (W_i8 [2*I, K], see duq4_weight_prelayout_i8) and int8 activations.
int gemm_tc2_launch_gate_up_prelaid(const void *A, const void *W_i8, uint32_t M, uint32_t inter, uint32_t K, const EpiParams &p, void *h_out,
                                    cudaStream_t st) {
    return launch2<false, true, true>(A, W_i8, M, inter, K, 1, p, h_out, nullptr, st, inter);
}

int tc2_status_read(int32_t *out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc2_status, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    *out = v;
    if (v != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_tc2_status, &zero, sizeof(int));
    }
    return DUQ4_OK;
}

}  // namespace duq4
