// Shared device/host helpers for libduq4 (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>

#include "../../include/duq4.h"

namespace duq4 {

// Clamp bounds of the reference (include/common.h:53-57 there). The symmetric upper bound
// is written `(7 - 1e-8)` in the reference and truncates to 6; codes must match it.
constexpr int kQminSym = -8;
constexpr int kQmaxSym = 6;
constexpr int kQminAsym = 0;
constexpr int kQmaxAsym = 15;
constexpr int kQmaxAsym8 = 126;  // src/kernels/quant.cu:241-242 of the reference
constexpr uint32_t kColK = DUQ4_QUANT_COL_K;

__host__ __device__ inline uint32_t cdiv(uint32_t a, uint32_t b) { return (a + b - 1) / b; }

inline int launch_status() {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) (void)cudaGetLastError();
    return (int)e;
}

// Per-device one-time launch set-up (function attributes are per device): `done[dev]` flags for
// up to 64 devices, one array per kernel instantiation. Returns the current device or -1.
inline int current_device_slot() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    return dev;
}

// Once-per-device host set-up that any number of host threads may reach at the same time (function
// attributes, occupancy queries): the first caller on a device runs `f` under a lock, later callers see
// the published flag. `f` returns 0 on success; a failure is returned and the set-up retried next time.
struct DeviceOnce {
    std::mutex mu;
    std::atomic<int> done[64];
    DeviceOnce() { for (auto &d : done) d.store(0, std::memory_order_relaxed); }
    template <class F>
    int run(int dev, F &&f) {
        if (done[dev].load(std::memory_order_acquire)) return 0;
        std::lock_guard<std::mutex> g(mu);
        if (done[dev].load(std::memory_order_relaxed)) return 0;
        const int rc = f();
        if (rc == 0) done[dev].store(1, std::memory_order_release);
        return rc;
    }
};

// SM count of the device that is current (queried once per device; 148 if the query fails).
inline int sm_count_current_device() {
    static std::atomic<int> n[64];   // zero-initialised
    const int dev = current_device_slot();
    if (dev < 0) return 148;
    int v = n[dev].load(std::memory_order_relaxed);
    if (v <= 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        n[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return max(lo, min(hi, v)); }

// One symmetric code: clamp(rn(x / s), -8, 6). __hdiv is the same intrinsic the reference
// kernel calls, so codes agree bit for bit with it.
__device__ __forceinline__ int code_sym(__half x, __half s) {
    return clampi(__half2int_rn(__hdiv(x, s)), kQminSym, kQmaxSym);
}
// Asymmetric, single scale: rn(x/s) + rn(z).
__device__ __forceinline__ int code_asym(__half x, __half s, int zi) {
    return clampi(__half2int_rn(__hdiv(x, s)) + zi, kQminAsym, kQmaxAsym);
}
// Asymmetric, dual scheme: rn(x/s + z), the add rounded to fp16 first.
__device__ __forceinline__ int code_asym_dual(__half x, __half s, __half z) {
    return clampi(__half2int_rn(__hadd_rn(__hdiv(x, s), z)), kQminAsym, kQmaxAsym);
}

// Epilogue parameters as the kernels see them.
struct EpiParams {
    int mode;
    uint32_t col_offset;
    const __half *s_row, *z_row, *s_col1, *z_col1, *s_col2, *z_col2, *bias;
    uint32_t ldo;
    // batched launches: element strides between consecutive problems
    uint32_t row_vec_stride, col_vec_stride;
    // Fused all-gather: when n_peers > 0 every output element is stored into each of these
    // buffers (same layout and offsets in all of them; peer-mapped device pointers, this rank's
    // own buffer included) instead of the single `out` pointer.
    uint32_t n_peers;
    __half *peers[DUQ4_MAX_OUT_PEERS];
    // L2 prefetch hint (small-M kernels): packed weights of the next launch on the stream
    const uint8_t *next_w;
    uint64_t next_w_bytes;
    // NVLS multicast address of the result buffer (see duq4_epilogue.out_multicast), or null
    __half *mc_out;
    // K-sharded layers: int32 partial accumulators go to the owner of each row block (see duq4_epilogue.acc_owners)
    uint32_t n_acc_owners, acc_rows_per_owner, acc_slot;
    int32_t *acc_owners[DUQ4_MAX_OUT_PEERS];
    // fused gather with row routing: > 0 = row m of the launch is stored only into peers[m / out_rows_per_owner]
    uint32_t out_rows_per_owner;
};
// Does row m of a launch go to output buffer pi? (every buffer without row routing)
__device__ __forceinline__ bool row_goes_to(const EpiParams &p, uint32_t m, int pi) {
    return p.out_rows_per_owner == 0 || m / p.out_rows_per_owner == (uint32_t)pi;
}

// Output bases of a launch: the peer list if there is one, else the plain `out` pointer.
struct OutBases {
    __half *base[DUQ4_MAX_OUT_PEERS];
    int n;
};
__device__ __forceinline__ OutBases out_bases(const EpiParams &p, __half *out) {
    OutBases o;
    if (p.n_peers) {
        o.n = (int)p.n_peers;
#pragma unroll
        for (int i = 0; i < DUQ4_MAX_OUT_PEERS; ++i) o.base[i] = p.peers[i];
    } else {
        o.n = out ? 1 : 0;
        o.base[0] = out;
#pragma unroll
        for (int i = 1; i < DUQ4_MAX_OUT_PEERS; ++i) o.base[i] = nullptr;
    }
    return o;
}

// Epilogue operands of problem `b` of a batched launch.
__host__ __device__ inline EpiParams epi_for_batch(EpiParams p, uint32_t b) {
    size_t ro = (size_t)b * p.row_vec_stride, co = (size_t)b * p.col_vec_stride;
    if (p.s_row) p.s_row += ro;
    if (p.z_row) p.z_row += ro;
    if (p.s_col1) p.s_col1 += co;
    if (p.z_col1) p.z_col1 += co;
    if (p.s_col2) p.s_col2 += co;
    if (p.z_col2) p.z_col2 += co;
    if (p.bias) p.bias += co;
    return p;
}

// Column-side operands of one output column, resolved once per column.
struct ColTerms {
    __half s, z, b;
    bool has_bias;
};

__device__ __forceinline__ ColTerms load_col_terms(const EpiParams &p, uint32_t c) {
    ColTerms t;
    t.z = __ushort_as_half(0);
    t.b = __ushort_as_half(0);
    t.s = __ushort_as_half(0);
    uint32_t gc = c + p.col_offset;
    switch (p.mode) {
        case DUQ4_MODE_SYM: t.s = p.s_col1[c]; break;
        case DUQ4_MODE_SYM_DUAL: t.s = gc < kColK ? p.s_col1[c] : p.s_col2[c]; break;
        case DUQ4_MODE_ASYM: t.s = p.s_col1[c]; t.z = p.z_col1[c]; break;
        case DUQ4_MODE_ASYM_DUAL:
            t.s = gc == 0 ? p.s_col1[c] : p.s_col2[c];
            t.z = gc == 0 ? p.z_col1[c] : p.z_col2[c];
            break;
        default: break;
    }
    t.has_bias = p.bias != nullptr;
    if (t.has_bias) t.b = p.bias[c];
    return t;
}

// SiLU-gated MLP glue for one element: h = half(half(silu(g)) * u), each step rounded to fp16 the way
// the torch composition `F.silu(gate) * up` rounds it (silu(x) = x / (1 + exp(-x)) evaluated in fp32).
__device__ __forceinline__ __half silu_mul_one(__half g, __half u) {
    const float x = __half2float(g);
    const __half s = __float2half_rn(__fdiv_rn(x, 1.0f + expf(-x)));
    return __hmul_rn(s, u);
}

// The reference dequant arithmetic, one rounding per fp16 operation, explicit .rn forms so
// that no multiply is contracted into an fma with the bias add:
//   sym : (s_row * s_col) * half(acc)
//   asym: (s_row * s_col) * ((half(acc) - z_row) - z_col)
__device__ __forceinline__ __half dequant_one(int mode, int acc, __half sr, __half zr, const ColTerms &t) {
    __half e = __int2half_rn(acc);
    __half ss = __hmul_rn(sr, t.s);
    __half v;
    if (mode == DUQ4_MODE_ASYM || mode == DUQ4_MODE_ASYM_DUAL)
        v = __hmul_rn(ss, __hsub_rn(__hsub_rn(e, zr), t.z));
    else
        v = __hmul_rn(ss, e);
    if (t.has_bias) v = __hadd_rn(v, t.b);
    return v;
}

}  // namespace duq4
