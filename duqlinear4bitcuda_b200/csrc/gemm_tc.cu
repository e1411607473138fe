// Tensor-core integer GEMM for sm_100a: C[M,N] = A[M,K] * B[N,K]^T with the dequant epilogue.
//
// Replaces the reference's CUTLASS Sm80 GEMMs (src/kernels/gemm.cu:8-43 int4, :46-81 int8,
// :83-117 batched) and, when an epilogue mode is given, the dequant launch and bias add
// that follow them in the module forwards (qlinear4bit/nn/linear.py:42-56 etc.).
//
// Blackwell has no 4-bit integer MMA, so the int4 path is:
//   TMA (cp.async.bulk.tensor, no multicast) : packed int4 tiles  -> shared memory
//   unpack warps                             : nibble -> int8 (value 16*s4), written in the
//                                              K-major 128B-swizzled layout UMMA expects
//   one thread                               : tcgen05.mma.kind::i8, int32 accumulators in TMEM
//   epilogue warps                           : tcgen05.ld -> (>>8) -> fp16 dequant -> global
// Both operands carry the factor 16, so accumulators are exactly 256x the true sums and the
// epilogue shifts them back (|sum| <= 64*K*256 < 2^31 for K < 131072, checked by the host).
// Inside a 128-element K block the unpack permutes K (low nibbles of a 16-byte packed chunk
// form one 16-byte int8 chunk, high nibbles the next); A and B share the permutation.
// The int8 path (matmul_8bit) lets TMA write the swizzled tiles directly and skips the unpack.
//
// Persistent kernel: one CTA per SM walks tiles in M-fastest order (CTAs running together
// share B tiles and all of A through L2). TMEM holds two accumulator buffers so the
// epilogue of tile i overlaps the main loop of tile i+1. Every mbarrier wait is bounded
// (1 s of %globaltimer); on expiry the CTA raises a status word and leaves in order.
#include <cuda.h>
#include <stdlib.h>

#include <mutex>
#include <unordered_map>

#include "duq_common.cuh"
#include "duq_ptx.cuh"
#include "gemm_tc_shared.cuh"

namespace duq4 {

__device__ int g_tc_status = 0;  // 0 = ok, else code of the wait that expired

namespace tc {

using namespace ptx;

constexpr int BM = 128;          // rows of A per tile = TMEM lanes
constexpr int BK = 128;          // K elements per pipeline stage (= one 128-byte swizzle row of int8)
// Operand formats of one launch.
constexpr int MODE_I8 = 0;     // A and B int8: TMA writes the swizzled tiles, no unpack
constexpr int MODE_I4 = 1;     // A and B packed int4: both unpacked in shared memory
constexpr int MODE_A8B4 = 2;   // A already unpacked in HBM (int8 = 16*s4, K permuted per 128-block
                               // exactly as the in-kernel unpack permutes it), B packed int4
// warps: 0 TMA producer, 1 MMA issuer, 2..5 epilogue, 6..6+UW-1 unpack, last: second TMA producer (A of MODE_A8B4)
__host__ __device__ constexpr int threads_for(int uw) { return 32 * (2 + kEpiWarps + uw + 1); }
constexpr uint64_t kWaitLimitNs = kPtxWaitLimitNs;

template <int MODE, int BN, int UW_, int NPK_, int NUP_>
struct Cfg {
    static constexpr int UW = UW_;
    static constexpr int kPackedStage = MODE == MODE_I4 ? (BM + BN) * (BK / 2) : (MODE == MODE_A8B4 ? BN * (BK / 2) : 0);
    static constexpr int kUnpackedStage = (BM + BN) * BK;
    static constexpr int NPK = MODE == MODE_I8 ? 1 : NPK_;   // packed-tile ring (TMA -> unpack warps)
    static constexpr int NUP = NUP_;                          // swizzled int8 ring (-> MMA)
    static_assert(NPK <= 8 && NUP <= 6, "barrier map holds 8 packed and 6 unpacked stages");
    static constexpr int kColTerms = kEpiWarps * 3 * BN * 2;  // per epilogue warp: (scale, zero, bias) x BN halves
    // Output staging (per epilogue warp 32 rows x 64 fp16, rows padded to 144 bytes): lets the
    // epilogue turn its one-row-per-lane registers into 128-byte row segments before they go to
    // global or peer memory. Only where the rings leave room (not in MODE_I4).
    static constexpr bool kStaged = MODE != MODE_I4;
    static constexpr int kStageOutWarp = 32 * 144;
    static constexpr int kStageOut = kStaged ? kEpiWarps * kStageOutWarp : 0;
    static constexpr int kSmem = 1024 /*align slack*/ + NUP * kUnpackedStage + NPK * kPackedStage + kColTerms + kStageOut + 512 /*barriers*/;
    static_assert(kSmem <= 232448, "exceeds the 227 KiB of shared memory a CTA can have");
    // two accumulator buffers; the allocation must be a power of two >= 32 columns
    static constexpr int kTmemCols = 2 * BN <= 32 ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));
};

template <int MODE, int BN, int UW, int NPK_, int NUP_>
__global__ void __launch_bounds__(threads_for(UW), 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                     const __grid_constant__ CUtensorMap tmB, const Args a) {
    using C = Cfg<MODE, BN, UW, NPK_, NUP_>;
    constexpr bool INT4 = MODE != MODE_I8;
    constexpr int kUnpackWarps = UW;
    constexpr int kLastWarp = 2 + kEpiWarps + UW;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *gbase = smem_raw + (base - raw);
    const uint32_t up0 = base;                                   // unpacked stages (1024-aligned each)
    const uint32_t pk0 = up0 + C::NUP * C::kUnpackedStage;       // packed stages
    const uint32_t ct_off = C::NUP * C::kUnpackedStage + C::NPK * C::kPackedStage;
    __half *colterms = reinterpret_cast<__half *>(gbase + ct_off);
    uint8_t *stage_out = gbase + ct_off + C::kColTerms;
    const uint32_t bar0 = base + ct_off + C::kColTerms + C::kStageOut;
    // barrier map (8 bytes each)
    auto pk_full = [&](int s) { return bar0 + 8u * s; };
    auto pk_empty = [&](int s) { return bar0 + 8u * (8 + s); };
    auto up_full = [&](int s) { return bar0 + 8u * (16 + s); };
    auto up_empty = [&](int s) { return bar0 + 8u * (22 + s); };
    auto acc_full = [&](int s) { return bar0 + 8u * (28 + s); };
    auto acc_empty = [&](int s) { return bar0 + 8u * (30 + s); };
    const uint32_t drain_bar = bar0 + 8u * 32;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t num_tiles = a.tiles_m * a.tiles_n * a.batch;
    const uint32_t ksteps = (a.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < 8; ++s) {
            mbar_init(pk_full(s), 1);
            mbar_init(pk_empty(s), kUnpackWarps);
        }
        for (int s = 0; s < 6; ++s) {
            mbar_init(up_full(s), MODE == MODE_I8 ? 1 : (MODE == MODE_I4 ? kUnpackWarps : kUnpackWarps + 1));
            mbar_init(up_empty(s), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(acc_full(s), 1);
            mbar_init(acc_empty(s), kEpiWarps);
        }
        mbar_init(drain_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abortp = &abort_flag;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;  // global stage counter
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                uint32_t per_b = a.tiles_m * a.tiles_n;
                uint32_t b = tile / per_b, r = tile % per_b;
                uint32_t tn = r / a.tiles_m, tm = r % a.tiles_m;
                for (uint32_t ks = 0; ks < ksteps; ++ks, ++it) {
                    if (MODE == MODE_I4) {
                        uint32_t s = it % C::NPK, ph = (it / C::NPK) & 1;
                        if (!(ok = mbar_wait(pk_empty(s), ph ^ 1, abortp, &g_tc_status, 1))) break;
                        uint32_t dst = pk0 + s * C::kPackedStage;
                        mbar_expect_tx(pk_full(s), C::kPackedStage);
                        tma_load_3d(dst, &tmA, pk_full(s), ks * (BK / 2), tm * BM, b);
                        tma_load_3d(dst + BM * (BK / 2), &tmB, pk_full(s), ks * (BK / 2), tn * BN, b);
                    } else if (MODE == MODE_A8B4) {
                        uint32_t s = it % C::NPK, ph = (it / C::NPK) & 1;
                        if (!(ok = mbar_wait(pk_empty(s), ph ^ 1, abortp, &g_tc_status, 1))) break;
                        mbar_expect_tx(pk_full(s), C::kPackedStage);
                        tma_load_3d(pk0 + s * C::kPackedStage, &tmB, pk_full(s), ks * (BK / 2), tn * BN, b);
                    } else {
                        uint32_t s = it % C::NUP, ph = (it / C::NUP) & 1;
                        if (!(ok = mbar_wait(up_empty(s), ph ^ 1, abortp, &g_tc_status, 1))) break;
                        uint32_t dst = up0 + s * C::kUnpackedStage;
                        mbar_expect_tx(up_full(s), C::kUnpackedStage);
                        tma_load_3d(dst, &tmA, up_full(s), ks * BK, tm * BM, b);
                        tma_load_3d(dst + BM * BK, &tmB, up_full(s), ks * BK, tn * BN, b);
                    }
                }
            }
            if (!ok) {  // give copies already in flight time to land before the CTA retires
                uint64_t t0 = globaltimer();
                while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
            }
        }
    } else if (MODE == MODE_A8B4 && warp == kLastWarp) {
        // ---------------- second TMA producer: pre-unpacked A straight into the MMA ring ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                uint32_t per_b = a.tiles_m * a.tiles_n;
                uint32_t b = tile / per_b, r = tile % per_b;
                uint32_t tm = r % a.tiles_m;
                for (uint32_t ks = 0; ks < ksteps; ++ks, ++it) {
                    uint32_t u = it % C::NUP, uph = (it / C::NUP) & 1;
                    if (!(ok = mbar_wait(up_empty(u), uph ^ 1, abortp, &g_tc_status, 7))) break;
                    mbar_expect_tx(up_full(u), BM * BK);
                    tma_load_3d(up0 + u * C::kUnpackedStage, &tmA, up_full(u), ks * BK, tm * BM, b);
                }
            }
            if (!ok) {
                uint64_t t0 = globaltimer();
                while (globaltimer() - t0 < 200000ull) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN);
            uint32_t it = 0, lt = 0;
            bool ok = true, issued = false;
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++lt) {
                uint32_t buf = lt & 1, aph = (lt >> 1) & 1;
                if (!(ok = mbar_wait(acc_empty(buf), aph ^ 1, abortp, &g_tc_status, 2))) break;
                tc_fence_after();
                uint32_t d_tmem = tmem_base + buf * BN;
                for (uint32_t ks = 0; ks < ksteps; ++ks, ++it) {
                    uint32_t s = it % C::NUP, ph = (it / C::NUP) & 1;
                    if (!(ok = mbar_wait(up_full(s), ph, abortp, &g_tc_status, 3))) break;
                    tc_fence_after();
                    uint32_t sa = up0 + s * C::kUnpackedStage, sb = sa + BM * BK;
                    uint64_t da = make_desc(sa), db = make_desc(sb);
#pragma unroll
                    for (int kk = 0; kk < BK / 32; ++kk)
                        umma_i8(d_tmem, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, (ks | kk) != 0);
                    issued = true;
                    umma_commit(up_empty(s));  // frees the stage once these MMAs have read it
                }
                if (ok) umma_commit(acc_full(buf));
            }
            if (!ok && issued) {  // aborting: let issued MMAs finish before TMEM is released
                umma_commit(drain_bar);
                uint64_t t0 = globaltimer();
                while (!mbar_try(drain_bar, 0) && globaltimer() - t0 < kWaitLimitNs) __nanosleep(1000);
            }
        }
    } else if (warp < 2 + kEpiWarps) {
        // ---------------- epilogue ----------------
        const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
        const uint32_t shift = INT4 ? 8 : 0;
        uint32_t lt = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++lt) {
            uint32_t per_b = a.tiles_m * a.tiles_n;
            uint32_t b = tile / per_b, r = tile % per_b;
            uint32_t tn = r / a.tiles_m, tm = r % a.tiles_m;
            uint32_t buf = lt & 1, aph = (lt >> 1) & 1;
            const uint32_t n0 = tn * BN;
            EpiParams pb = a.epi;
            __half *cs = colterms + (warp - 2) * 3 * BN, *cz = cs + BN, *cb = cz + BN;
            epi_stage_colterms<BN>(a, pb, b, n0, lane, cs, cz, cb);
            if (!(ok = mbar_wait(acc_full(buf), aph, abortp, &g_tc_status, 4))) break;
            tc_fence_after();

            epi_store_tile<BN, C::kStaged>(a, pb, b, tm * BM, n0, tmem_base + buf * BN, quad, lane, shift, cs, cz, cb,
                                           stage_out + (warp - 2) * C::kStageOutWarp);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(buf));
        }
    } else if (INT4 && warp < kLastWarp) {
        // ---------------- unpack warps: packed int4 -> swizzled int8 ----------------
        const int ut = (warp - 2 - kEpiWarps) * 32 + lane;
        constexpr int kRows = MODE == MODE_I4 ? BM + BN : BN;   // packed rows per stage
        constexpr int kChunks = kRows * 4;                      // 16-byte packed chunks per stage
        constexpr uint32_t kDstOff = MODE == MODE_I4 ? 0 : BM * BK;  // MODE_A8B4 fills the B half only
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            for (uint32_t ks = 0; ks < ksteps; ++ks, ++it) {
                uint32_t s = it % C::NPK, ph = (it / C::NPK) & 1;
                uint32_t u = it % C::NUP, uph = (it / C::NUP) & 1;
                if (!(ok = mbar_wait(pk_full(s), ph, abortp, &g_tc_status, 5))) break;
                if (!(ok = mbar_wait(up_empty(u), uph ^ 1, abortp, &g_tc_status, 6))) break;
                const uint32_t src = pk0 + s * C::kPackedStage, dst = up0 + u * C::kUnpackedStage + kDstOff;
#pragma unroll 4
                for (int idx = ut; idx < kChunks; idx += kUnpackWarps * 32) {
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
                fence_proxy_async();  // make the generic-proxy writes visible to the MMA (async proxy)
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(pk_empty(s));
                    mbar_arrive(up_full(u));
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// ---- host side ------------------------------------------------------------------------
typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                             const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeFn)p;
    });
    return fn;
}

struct MapKey {
    const void *ptr;
    uint64_t kbytes, rows, batch;
    uint32_t box_k, box_rows, swizzle;
    bool operator==(const MapKey &o) const {
        return ptr == o.ptr && kbytes == o.kbytes && rows == o.rows && batch == o.batch && box_k == o.box_k &&
               box_rows == o.box_rows && swizzle == o.swizzle;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey &k) const {
        size_t h = std::hash<const void *>()(k.ptr);
        auto mix = [&](uint64_t v) { h ^= std::hash<uint64_t>()(v) + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
        mix(k.kbytes); mix(k.rows); mix(k.batch); mix(k.box_k); mix(k.box_rows); mix(k.swizzle);
        return h;
    }
};

// Byte tensor [batch, rows, kbytes] (kbytes contiguous); box = [1, box_rows, box_k].
static int get_map(const void *ptr, uint64_t kbytes, uint64_t rows, uint64_t batch, uint32_t box_k, uint32_t box_rows,
                   bool swizzle128, CUtensorMap *out, bool use_cache = true) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    if (!out) {   // diagnostic query: number of cached descriptors
        std::lock_guard<std::mutex> g(mu);
        return (int)cache.size();
    }
    MapKey key{ptr, kbytes, rows, batch, box_k, box_rows, swizzle128 ? 1u : 0u};
    if (use_cache) {
        std::lock_guard<std::mutex> g(mu);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *out = it->second;
            return DUQ4_OK;
        }
    }
    EncodeFn fn = encode_fn();
    if (!fn) return DUQ4_ERR_DEVICE;
    cuuint64_t dims[3] = {kbytes, rows, batch};
    cuuint64_t strides[2] = {kbytes, kbytes * rows};
    cuuint32_t box[3] = {box_k, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return DUQ4_ERR_SHAPE;
    if (use_cache) {
        std::lock_guard<std::mutex> g(mu);
        if (cache.size() > 4096) cache.clear();
        cache[key] = m;
    }
    *out = m;
    return DUQ4_OK;
}

}  // namespace tc

// use_cache = false: the descriptor is encoded into *out for this call only (nothing is looked up or kept,
// so the host heap is not touched).
int tma_map_bytes_3d(const void *ptr, uint64_t kbytes, uint64_t rows, uint64_t batch, uint32_t box_k, uint32_t box_rows,
                      bool swizzle128, CUtensorMap *out, bool use_cache) {
    return tc::get_map(ptr, kbytes, rows, batch, box_k, box_rows, swizzle128, out, use_cache);
}

// Entries currently held by the descriptor cache (diagnostic).
int tma_map_cache_entries() { return tc::get_map(nullptr, 0, 0, 0, 0, 0, false, nullptr, true); }

namespace tc {

static int sm_count() { return sm_count_current_device(); }

template <int MODE, int BN, int UW, int NPK_, int NUP_>
static int launch(const void *A, const void *B, const Args &args, cudaStream_t st, bool cache_maps) {
    using C = Cfg<MODE, BN, UW, NPK_, NUP_>;
    static DeviceOnce once;
    const int dev = current_device_slot();
    if (dev < 0) return DUQ4_ERR_DEVICE;
    int orc = once.run(dev, [] {
        return (int)cudaFuncSetAttribute(gemm_tc_kernel<MODE, BN, UW, NPK_, NUP_>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kSmem);
    });
    if (orc) return orc;
    const bool a_packed = MODE == MODE_I4, b_packed = MODE != MODE_I8;
    CUtensorMap ma, mb;
    int rc = get_map(A, a_packed ? args.K / 2 : args.K, args.a_rows > args.M ? args.a_rows : args.M, args.batch, a_packed ? BK / 2 : BK, BM, !a_packed, &ma, cache_maps);
    if (rc) return rc;
    rc = get_map(B, b_packed ? args.K / 2 : args.K, args.N, args.batch, b_packed ? BK / 2 : BK, BN, !b_packed, &mb, cache_maps);
    if (rc) return rc;
    uint32_t tiles = args.tiles_m * args.tiles_n * args.batch;
    uint32_t grid = tiles < (uint32_t)sm_count() ? tiles : (uint32_t)sm_count();
    gemm_tc_kernel<MODE, BN, UW, NPK_, NUP_><<<grid, threads_for(UW), C::kSmem, st>>>(ma, mb, args);
    return launch_status();
}

// Debug override of the pipeline shape (DUQ4_TC_VARIANT=0..2); unset = the tuned default.
static int variant() {
    static const int v = [] {
        const char *e = getenv("DUQ4_TC_VARIANT");
        const int x = e ? atoi(e) : 1;
        return (x < 0 || x > 2) ? 1 : x;
    }();
    return v;
}

}  // namespace tc

int gemm_tc2_launch(bool a_packed, const void *A, const void *B, uint32_t M, uint32_t N, uint32_t K, uint32_t batch,
                    const EpiParams &p, void *out, int32_t *acc_out, cudaStream_t st, bool cache_maps);

// CTA-pair tiles for large int4 problems: DUQ4_TC_PAIR=0/1 overrides the default (on).
static bool pair_tiles() {
    static const bool v = [] {
        const char *e = getenv("DUQ4_TC_PAIR");
        return e ? (atoi(e) != 0) : true;
    }();
    return v;
}

// A [batch,M,K] x B [batch,N,K]^T. mode: tc::MODE_I8 / MODE_I4 / MODE_A8B4 (see above).
// a_rows: rows the A buffer really has (0 = M). A caller that owns a larger buffer lets the tensor map cover it, so
// that the A tile of a launch with few tokens is read in-bounds instead of zero-filled (batch must be 1 then).
int gemm_tc_launch(int mode, const void *A, const void *B, uint32_t M, uint32_t N, uint32_t K, uint32_t batch,
                   const EpiParams &p, void *out, int32_t *acc_out, cudaStream_t st, bool cache_maps, uint32_t a_rows) {
    using namespace tc;
    if (((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) != 0) return DUQ4_ERR_ALIGN;
    if (mode != MODE_I8 && K >= 131072u) return DUQ4_ERR_SHAPE;  // 256x-scaled accumulators must fit int32
    Args a{};
    a.M = M; a.N = N; a.K = K; a.batch = batch;
    a.a_rows = (batch == 1 && a_rows > M) ? a_rows : M;
    a.epi = p;
    a.out = (__half *)out;
    a.acc_out = acc_out;
    a.tiles_m = cdiv(M, BM);
    a.acc_fits_22 = (uint64_t)K * (mode == MODE_I8 ? 16384u : 64u) <= (1u << 22) ? 1u : 0u;   // |term| <= 128 * 128 or 8 * 8
    // 256-wide tiles halve the A-operand shared-memory traffic per MMA; fall back to 128
    // when that would leave most SMs without a tile.
    const bool wide = (uint64_t)a.tiles_m * cdiv(N, 256) * batch >= 120 || N > 128 * 148;
    a.tiles_n = cdiv(N, wide ? 256 : 128);
    const int v = variant();
    if (mode == MODE_I8) return wide ? launch<MODE_I8, 256, 4, 1, 4>(A, B, a, st, cache_maps) : launch<MODE_I8, 128, 4, 1, 6>(A, B, a, st, cache_maps);
    const bool pair_ok = pair_tiles() && (uint64_t)cdiv(M, 256) * cdiv(N, 256) * batch >= 60;
    if (mode == MODE_I4) {
        if (pair_ok) {
            int rc = gemm_tc2_launch(true, A, B, M, N, K, batch, p, out, acc_out, st, cache_maps);
            if (rc != DUQ4_ERR_DEVICE) return rc;   // no CTA pairs on this device: single-CTA tiles below
        }
        if (!wide) return launch<MODE_I4, 128, 8, 4, 4>(A, B, a, st, cache_maps);
        if (v == 0) return launch<MODE_I4, 256, 4, 4, 2>(A, B, a, st, cache_maps);
        if (v == 2) return launch<MODE_I4, 256, 8, 4, 2>(A, B, a, st, cache_maps);
        return launch<MODE_I4, 256, 8, 3, 3>(A, B, a, st, cache_maps);
    }
    if ((mode == MODE_A8B4 || mode == MODE_I4) && a.tiles_m == 1) {
        // At most 128 tokens: every tile streams its own block of W exactly once and there is one row of
        // tiles, so 256-wide tiles (pairs or not) would leave SMs idle and take two rounds on the others
        // (4096 -> 22016 at 64 tokens: 36.8 us). Narrow tiles give (nearly) every SM exactly one; choose the
        // width that minimises the bytes the busiest SM streams, ties to the wider tile (fewer re-reads of
        // the activations). Measured 23.2 us for that layer; a packed ring of 256-byte-per-row boxes, 4 or
        // 12 unpack warps and a deeper or shallower operand ring all measured the same or worse.
        const uint32_t sms = (uint32_t)sm_count();
        uint32_t best_bn = 0;
        uint64_t best = ~0ull;
        for (uint32_t bn : {160u, 128u, 96u, 64u}) {
            const uint64_t rounds = ((uint64_t)cdiv(N, bn) * batch + sms - 1) / sms;
            if (rounds * bn < best) { best = rounds * bn; best_bn = bn; }
        }
        a.tiles_n = cdiv(N, best_bn);
        if (mode == MODE_I4) {   // packed activations (the reference's format): both operands unpacked in the CTA
            switch (best_bn) {
                case 160: return launch<MODE_I4, 160, 8, 4, 3>(A, B, a, st, cache_maps);
                case 128: return launch<MODE_I4, 128, 8, 4, 4>(A, B, a, st, cache_maps);
                case 96: return launch<MODE_I4, 96, 8, 4, 4>(A, B, a, st, cache_maps);
                default: return launch<MODE_I4, 64, 8, 4, 4>(A, B, a, st, cache_maps);
            }
        }
        switch (best_bn) {
            case 160: return launch<MODE_A8B4, 160, 8, 8, 3>(A, B, a, st, cache_maps);
            case 128: return launch<MODE_A8B4, 128, 8, 8, 4>(A, B, a, st, cache_maps);
            case 96: return launch<MODE_A8B4, 96, 8, 8, 4>(A, B, a, st, cache_maps);
            default: return launch<MODE_A8B4, 64, 8, 8, 4>(A, B, a, st, cache_maps);
        }
    }
    if (mode == MODE_A8B4) {
        if (pair_ok) {
            int rc = gemm_tc2_launch(false, A, B, M, N, K, batch, p, out, acc_out, st, cache_maps);
            if (rc != DUQ4_ERR_DEVICE) return rc;   // no CTA pairs on this device: single-CTA tiles below
        }
        if (!wide) return launch<MODE_A8B4, 128, 8, 4, 4>(A, B, a, st, cache_maps);
        if (v == 0) return launch<MODE_A8B4, 256, 8, 3, 3>(A, B, a, st, cache_maps);
        if (v == 2) return launch<MODE_A8B4, 256, 10, 3, 3>(A, B, a, st, cache_maps);
        return launch<MODE_A8B4, 256, 12, 3, 3>(A, B, a, st, cache_maps);
    }
    return DUQ4_ERR_MODE;
}

int tc_status_read(cudaStream_t st, int32_t *out) {
    cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return (int)e;
    int v = 0;
    e = cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    *out = v;
    if (v != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
    }
    return DUQ4_OK;
}

}  // namespace duq4
