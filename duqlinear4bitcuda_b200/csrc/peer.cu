// Device-side barrier across the ranks of an N-sharded layer (one process per GPU), used around the fused
// all-gather of the GEMM epilogue. Flags live in memory every rank maps (peer-mapped device memory); plain
// system-scope stores and loads over NVLink, no multicast. Every wait is bounded.
#include "duq_common.cuh"
#include "duq_ptx.cuh"

namespace duq4 {

__device__ int g_peer_status = 0;   // 0 = ok, 1 = a barrier wait ran out

struct PeerFlags {
    unsigned long long *of_rank[DUQ4_MAX_OUT_PEERS];
};

// One CTA of 32 threads; thread t < world talks to rank t.
__global__ void peer_barrier_kernel(PeerFlags f, uint32_t world, uint32_t rank, unsigned long long epoch, unsigned long long limit_ns) {
    const uint32_t t = threadIdx.x;
    if (t >= world) return;
    // everything this rank's stream did before the barrier (this GPU's stores into peers' buffers included)
    // is ordered before the flag a peer will observe
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(f.of_rank[t] + rank), "l"(epoch) : "memory");
    const unsigned long long *mine = f.of_rank[rank] + t;
    const uint64_t t0 = ptx::globaltimer();
    for (uint32_t it = 1;; ++it) {
        unsigned long long v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(mine) : "memory");
        if (v >= epoch) break;
        if ((it & 63u) == 0) {
            if (ptx::globaltimer() - t0 > limit_ns) {   // the peer did not arrive in time: report and leave
                atomicCAS(&g_peer_status, 0, 1);
                break;
            }
            __nanosleep(200);
        }
    }
    asm volatile("fence.acq_rel.sys;" ::: "memory");
}

int peer_status_read(int32_t *out) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_peer_status, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    *out = v;
    if (v != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(int));
    }
    return DUQ4_OK;
}

}  // namespace duq4

using namespace duq4;

extern "C" int duq4_peer_barrier(const void *const *flag_ptrs, uint32_t world, uint32_t rank, uint64_t epoch, uint64_t timeout_ns,
                                 void *stream) {
    if (!flag_ptrs) return DUQ4_ERR_NULL;
    if (world == 0 || world > DUQ4_MAX_OUT_PEERS || rank >= world || epoch == 0) return DUQ4_ERR_SHAPE;
    PeerFlags f{};
    for (uint32_t i = 0; i < world; ++i) {
        if (!flag_ptrs[i]) return DUQ4_ERR_NULL;
        if ((reinterpret_cast<uintptr_t>(flag_ptrs[i]) & 7) != 0) return DUQ4_ERR_ALIGN;
        f.of_rank[i] = (unsigned long long *)flag_ptrs[i];
    }
    const unsigned long long limit = timeout_ns ? timeout_ns : ptx::kPtxWaitLimitNs;
    peer_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, world, rank, (unsigned long long)epoch, limit);
    return launch_status();
}
