// Host-buffer entry point of the W4A4 linear layer.
//
// duq4_linear_w4a4_from_fp16_host takes activations and output in HOST memory and overlaps the
// three legs of the job over row chunks of the token matrix:
//
//     upload stream   : x chunk c+1  host -> device
//     caller's stream : quantize + GEMM + dequant of chunk c        (duq4_linear_w4a4_from_fp16)
//     download stream : out chunk c-1 device -> host
//
// The output is 3.5x larger than the input for the layers this library targets (N > K), so the
// download leg bounds the call; the upload and the arithmetic hide behind it. The two helper
// streams fork from the caller's stream at entry and join it before the call returns, so the
// call is ordered like a single piece of work on that stream.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/duq4.h"

namespace {

constexpr int kMaxDevices = 64;
constexpr uint32_t kMaxChunks = 64;

struct PipeState {
    bool ready = false;
    cudaStream_t up = nullptr, down = nullptr;
    cudaEvent_t fork = nullptr, join_down = nullptr;
    cudaEvent_t uploaded[kMaxChunks] = {}, computed[kMaxChunks] = {};
};

std::mutex g_mu;        // guards creation of g_state entries
std::mutex g_call_mu;   // held while one call enqueues: its record/wait pairs on the shared events stay paired
PipeState g_state[kMaxDevices];

// Streams and events of the device that is current, created on first use.
int pipe_state(PipeState **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return DUQ4_ERR_DEVICE;
    std::lock_guard<std::mutex> g(g_mu);
    PipeState &s = g_state[dev];
    if (!s.ready) {
        // built in a local copy and published only when complete; a failure destroys what was made
        PipeState t;
        auto fail = [&t](cudaError_t err) {
            if (t.up) cudaStreamDestroy(t.up);
            if (t.down) cudaStreamDestroy(t.down);
            if (t.fork) cudaEventDestroy(t.fork);
            if (t.join_down) cudaEventDestroy(t.join_down);
            for (uint32_t i = 0; i < kMaxChunks; ++i) {
                if (t.uploaded[i]) cudaEventDestroy(t.uploaded[i]);
                if (t.computed[i]) cudaEventDestroy(t.computed[i]);
            }
            return (int)err;
        };
        if ((e = cudaStreamCreateWithFlags(&t.up, cudaStreamNonBlocking)) != cudaSuccess) return fail(e);
        if ((e = cudaStreamCreateWithFlags(&t.down, cudaStreamNonBlocking)) != cudaSuccess) return fail(e);
        if ((e = cudaEventCreateWithFlags(&t.fork, cudaEventDisableTiming)) != cudaSuccess) return fail(e);
        if ((e = cudaEventCreateWithFlags(&t.join_down, cudaEventDisableTiming)) != cudaSuccess) return fail(e);
        for (uint32_t i = 0; i < kMaxChunks; ++i) {
            if ((e = cudaEventCreateWithFlags(&t.uploaded[i], cudaEventDisableTiming)) != cudaSuccess) return fail(e);
            if ((e = cudaEventCreateWithFlags(&t.computed[i], cudaEventDisableTiming)) != cudaSuccess) return fail(e);
        }
        t.ready = true;
        s = t;
    }
    *out = &s;
    return DUQ4_OK;
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Rows per chunk: the caller's value rounded up to the GEMM's 256-row tile, or about a sixteenth
// of the job (the pipeline's fill time is one chunk's upload + arithmetic); never more than
// kMaxChunks chunks.
uint32_t pick_chunk_rows(uint32_t M, uint32_t chunk_rows) {
    uint64_t r = chunk_rows ? chunk_rows : (M + 15) / 16;
    r = (r + 255) / 256 * 256;
    const uint64_t least = ((uint64_t)M + kMaxChunks - 1) / kMaxChunks;
    if (r < least) r = (least + 255) / 256 * 256;
    if (r > M) r = M;
    return (uint32_t)r;
}

}  // namespace

extern "C" {

size_t duq4_linear_host_staging_bytes(uint32_t M, uint32_t N, uint32_t K, uint32_t chunk_rows) {
    if (M == 0 || N == 0 || K == 0) return 0;
    const uint32_t rows = pick_chunk_rows(M, chunk_rows);
    return align_up((size_t)M * K * 2, 256) + align_up((size_t)M * N * 2, 256) +
           align_up(duq4_linear_from_fp16_workspace_bytes(rows, K), 256);
}

int duq4_linear_w4a4_from_fp16_host(const void *x_host, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K,
                                    int act_mode, float clip_ratio, const duq4_epilogue *epi, void *out_host,
                                    uint32_t chunk_rows, void *staging, size_t staging_bytes, void *stream) {
    if (!x_host || !W || !epi || !out_host) return DUQ4_ERR_NULL;
    if (epi->n_out_peers != 0) return DUQ4_ERR_MODE;   // the result goes to host memory, not to peers
    if (M == 0 || N == 0) return DUQ4_OK;
    if (K == 0 || K % 64 != 0) return DUQ4_ERR_SHAPE;
    const uint64_t ldo = epi->ldo ? epi->ldo : N;
    if (ldo < N) return DUQ4_ERR_SHAPE;
    if (!staging || (reinterpret_cast<uintptr_t>(staging) & 255) != 0 ||
        staging_bytes < duq4_linear_host_staging_bytes(M, N, K, chunk_rows))
        return DUQ4_ERR_WORKSPACE;
    PipeState *ps = nullptr;
    int rc = pipe_state(&ps);
    if (rc) return rc;

    const uint32_t rows = pick_chunk_rows(M, chunk_rows);
    const uint32_t chunks = (M + rows - 1) / rows;
    uint8_t *x_dev = (uint8_t *)staging;
    uint8_t *o_dev = x_dev + align_up((size_t)M * K * 2, 256);
    uint8_t *ws = o_dev + align_up((size_t)M * N * 2, 256);
    const size_t ws_bytes = duq4_linear_from_fp16_workspace_bytes(rows, K);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    std::lock_guard<std::mutex> enqueue_lock(g_call_mu);
#define DUQ4_TRY(call)                     \
    do {                                   \
        e = (call);                        \
        if (e != cudaSuccess) return (int)e; \
    } while (0)

    // fork: earlier work of the caller's stream may still use the staging area
    DUQ4_TRY(cudaEventRecord(ps->fork, st));
    DUQ4_TRY(cudaStreamWaitEvent(ps->up, ps->fork, 0));
    DUQ4_TRY(cudaStreamWaitEvent(ps->down, ps->fork, 0));
    for (uint32_t c = 0; c < chunks; ++c) {
        const uint32_t r0 = c * rows, nr = (M - r0 < rows) ? M - r0 : rows;
        DUQ4_TRY(cudaMemcpyAsync(x_dev + (size_t)r0 * K * 2, (const uint8_t *)x_host + (size_t)r0 * K * 2,
                                 (size_t)nr * K * 2, cudaMemcpyHostToDevice, ps->up));
        DUQ4_TRY(cudaEventRecord(ps->uploaded[c], ps->up));
    }
    duq4_epilogue dev_epi = *epi;
    dev_epi.ldo = N;   // the device copy of the output is dense; the row pitch is applied by the download
    for (uint32_t c = 0; c < chunks; ++c) {
        const uint32_t r0 = c * rows, nr = (M - r0 < rows) ? M - r0 : rows;
        DUQ4_TRY(cudaStreamWaitEvent(st, ps->uploaded[c], 0));
        rc = duq4_linear_w4a4_from_fp16(x_dev + (size_t)r0 * K * 2, W, nr, N, K, act_mode, clip_ratio, &dev_epi,
                                        o_dev + (size_t)r0 * N * 2, ws, ws_bytes, stream);
        if (rc) break;   // still join the helper streams below
        DUQ4_TRY(cudaEventRecord(ps->computed[c], st));
        DUQ4_TRY(cudaStreamWaitEvent(ps->down, ps->computed[c], 0));
        uint8_t *dst = (uint8_t *)out_host + (size_t)r0 * ldo * 2;
        if (ldo == N)
            DUQ4_TRY(cudaMemcpyAsync(dst, o_dev + (size_t)r0 * N * 2, (size_t)nr * N * 2, cudaMemcpyDeviceToHost, ps->down));
        else
            DUQ4_TRY(cudaMemcpy2DAsync(dst, ldo * 2, o_dev + (size_t)r0 * N * 2, (size_t)N * 2, (size_t)N * 2, nr,
                                       cudaMemcpyDeviceToHost, ps->down));
    }
    // join: the caller's stream continues after the last download (and after every upload, which
    // matters only on the error path -- on success each upload was already waited for)
    DUQ4_TRY(cudaStreamWaitEvent(st, ps->uploaded[chunks - 1], 0));
    DUQ4_TRY(cudaEventRecord(ps->join_down, ps->down));
    DUQ4_TRY(cudaStreamWaitEvent(st, ps->join_down, 0));
#undef DUQ4_TRY
    return rc;
}

}  // extern "C"
