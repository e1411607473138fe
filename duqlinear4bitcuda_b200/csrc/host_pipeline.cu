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
// download leg bounds the call; the upload and the arithmetic hide behind it. The helper
// streams fork from the caller's stream at entry and join it before the call returns, so the
// call is ordered like a single piece of work on that stream.
//
// Two relatives share the machinery (run_pipeline):
//   duq4_linear_w4a4_from_fp16_to_host   activations already on the device (e.g. gathered from the ranks' row
//                                        slices over NVLink), result to host memory: arithmetic of chunk c overlaps
//                                        the download of chunk c-1;
//   duq4_linear_w4a4_from_fp16_to_peers  N-sharded layer whose [M, N] result is replicated on every rank: the GEMM
//                                        of chunk c writes this rank's column block into its OWN result buffer and the
//                                        copy engines push chunk c-1 to the other ranks' buffers (2-D peer copies over
//                                        NVLink, one helper stream per peer) -- the all-gather runs on the copy
//                                        engines, overlapped with the arithmetic, instead of as stores of the epilogue.
//
// duq4_linear_w4a4_from_fp16_to_host_rows (run_rows_pipeline) is the N-sharded job whose result goes back to ONE host
// buffer, delivered as contiguous rows instead of as column blocks whose 1/G-row pieces interleave in every host row
// (2-D copies of 7 KiB rows reach 49 - 54 GB/s on a link that moves contiguous data at 57 GB/s). The ranks first
// exchange over NVLink (idle in such a job): the epilogue of each rank's GEMM stores row m of a chunk only into the buffer of the rank that
// owns row m (out_rows_per_owner), a rank barrier makes the chunk complete, and every rank downloads the contiguous
// full-width rows it owns while the next chunk is computed.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/duq4.h"
#include "trace_range.h"

namespace {

constexpr int kMaxDevices = 64;
constexpr uint32_t kMaxChunks = 64;

constexpr int kMaxPeers = DUQ4_MAX_OUT_PEERS;

struct PipeState {
    bool ready = false;
    cudaStream_t up = nullptr, down = nullptr;
    cudaStream_t peer[kMaxPeers] = {};
    cudaEvent_t fork = nullptr, join_down = nullptr;
    cudaEvent_t join_peer[kMaxPeers] = {};
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
            for (int i = 0; i < kMaxPeers; ++i) {
                if (t.peer[i]) cudaStreamDestroy(t.peer[i]);
                if (t.join_peer[i]) cudaEventDestroy(t.join_peer[i]);
            }
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
        for (int i = 0; i < kMaxPeers; ++i) {
            if ((e = cudaStreamCreateWithFlags(&t.peer[i], cudaStreamNonBlocking)) != cudaSuccess) return fail(e);
            if ((e = cudaEventCreateWithFlags(&t.join_peer[i], cudaEventDisableTiming)) != cudaSuccess) return fail(e);
        }
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

// Where a chunk's fp16 result goes.
struct Sink {
    void *host = nullptr;          // host sink: base of the [M, ldo] host result (first column of this call's block)
    void *const *peers = nullptr;  // peer sink: every rank's [M, ldo] device buffer at this block's first column, own included
    uint32_t n_peers = 0, self = 0;
};

size_t pipeline_staging_bytes(bool x_on_host, bool host_sink, bool prelaid, uint32_t M, uint32_t N, uint32_t K, uint32_t rows) {
    return (x_on_host ? align_up((size_t)M * K * 2, 256) : 0) + (host_sink ? align_up((size_t)M * N * 2, 256) : 0) +
           align_up(prelaid ? duq4_linear_from_fp16_prelaid_workspace_bytes(rows, K) : duq4_linear_from_fp16_workspace_bytes(rows, K), 256);
}

int run_pipeline(const void *x, bool x_on_host, const void *W, bool prelaid, uint32_t M, uint32_t N, uint32_t K, int act_mode,
                 float clip_ratio, const duq4_epilogue *epi, const Sink &sink, uint32_t chunk_rows, void *staging, size_t staging_bytes,
                 void *stream) {
    const bool host_sink = sink.host != nullptr;
    if (!x || !W || !epi || (!host_sink && (!sink.peers || sink.n_peers == 0))) return DUQ4_ERR_NULL;
    if (M == 0 || N == 0) return DUQ4_OK;
    if (K == 0 || K % 64 != 0 || (prelaid && K % 128 != 0)) return DUQ4_ERR_SHAPE;
    const uint64_t ldo = epi->ldo ? epi->ldo : N;
    if (ldo < N) return DUQ4_ERR_SHAPE;
    if (!host_sink && (sink.n_peers > (uint32_t)kMaxPeers || sink.self >= sink.n_peers)) return DUQ4_ERR_SHAPE;
    const uint32_t rows = pick_chunk_rows(M, chunk_rows);
    if (!staging || (reinterpret_cast<uintptr_t>(staging) & 255) != 0 ||
        staging_bytes < pipeline_staging_bytes(x_on_host, host_sink, prelaid, M, N, K, rows))
        return DUQ4_ERR_WORKSPACE;
    PipeState *ps = nullptr;
    int rc = pipe_state(&ps);
    if (rc) return rc;

    const uint32_t chunks = (M + rows - 1) / rows;
    uint8_t *cur = (uint8_t *)staging;
    uint8_t *x_dev = x_on_host ? cur : (uint8_t *)const_cast<void *>(x);
    if (x_on_host) cur += align_up((size_t)M * K * 2, 256);
    uint8_t *o_dev = host_sink ? cur : nullptr;
    if (host_sink) cur += align_up((size_t)M * N * 2, 256);
    uint8_t *ws = cur;
    const size_t ws_bytes = prelaid ? duq4_linear_from_fp16_prelaid_workspace_bytes(rows, K) : duq4_linear_from_fp16_workspace_bytes(rows, K);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    std::lock_guard<std::mutex> enqueue_lock(g_call_mu);
#define DUQ4_TRY(call)                     \
    do {                                   \
        e = (call);                        \
        if (e != cudaSuccess) return (int)e; \
    } while (0)

    // fork: earlier work of the caller's stream may still use the staging area / the result buffers
    DUQ4_TRY(cudaEventRecord(ps->fork, st));
    if (x_on_host) DUQ4_TRY(cudaStreamWaitEvent(ps->up, ps->fork, 0));
    if (host_sink) DUQ4_TRY(cudaStreamWaitEvent(ps->down, ps->fork, 0));
    if (!host_sink)
        for (uint32_t p = 0; p < sink.n_peers; ++p)
            if (p != sink.self) DUQ4_TRY(cudaStreamWaitEvent(ps->peer[p], ps->fork, 0));
    if (x_on_host) {
        for (uint32_t c = 0; c < chunks; ++c) {
            const uint32_t r0 = c * rows, nr = (M - r0 < rows) ? M - r0 : rows;
            DUQ4_TRY(cudaMemcpyAsync(x_dev + (size_t)r0 * K * 2, (const uint8_t *)x + (size_t)r0 * K * 2, (size_t)nr * K * 2,
                                     cudaMemcpyHostToDevice, ps->up));
            DUQ4_TRY(cudaEventRecord(ps->uploaded[c], ps->up));
        }
    }
    duq4_epilogue dev_epi = *epi;
    dev_epi.n_out_peers = 0;
    dev_epi.out_multicast = nullptr;
    if (host_sink) dev_epi.ldo = N;   // the device copy of the output is dense; the row pitch is applied by the download
    for (uint32_t c = 0; c < chunks; ++c) {
        const uint32_t r0 = c * rows, nr = (M - r0 < rows) ? M - r0 : rows;
        if (x_on_host) DUQ4_TRY(cudaStreamWaitEvent(st, ps->uploaded[c], 0));
        uint8_t *o_chunk = host_sink ? o_dev + (size_t)r0 * N * 2 : (uint8_t *)sink.peers[sink.self] + (size_t)r0 * ldo * 2;
        rc = prelaid ? duq4_linear_w4a4_from_fp16_prelaid(x_dev + (size_t)r0 * K * 2, (const int8_t *)W, nr, N, K, act_mode, clip_ratio, &dev_epi,
                                                          o_chunk, ws, ws_bytes, stream)
                     : duq4_linear_w4a4_from_fp16(x_dev + (size_t)r0 * K * 2, (const uint8_t *)W, nr, N, K, act_mode, clip_ratio, &dev_epi, o_chunk,
                                                  ws, ws_bytes, stream);
        if (rc) break;   // still join the helper streams below
        DUQ4_TRY(cudaEventRecord(ps->computed[c], st));
        if (host_sink) {
            DUQ4_TRY(cudaStreamWaitEvent(ps->down, ps->computed[c], 0));
            uint8_t *dst = (uint8_t *)sink.host + (size_t)r0 * ldo * 2;
            if (ldo == N)
                DUQ4_TRY(cudaMemcpyAsync(dst, o_chunk, (size_t)nr * N * 2, cudaMemcpyDeviceToHost, ps->down));
            else
                DUQ4_TRY(cudaMemcpy2DAsync(dst, ldo * 2, o_chunk, (size_t)N * 2, (size_t)N * 2, nr, cudaMemcpyDeviceToHost, ps->down));
        } else {
            // this chunk of the block to every other rank, starting with the next rank so that the ranks' copies fan
            // out over different destinations at any one time
            for (uint32_t k = 1; k < sink.n_peers; ++k) {
                const uint32_t p = (sink.self + k) % sink.n_peers;
                DUQ4_TRY(cudaStreamWaitEvent(ps->peer[p], ps->computed[c], 0));
                DUQ4_TRY(cudaMemcpy2DAsync((uint8_t *)sink.peers[p] + (size_t)r0 * ldo * 2, ldo * 2, o_chunk, ldo * 2, (size_t)N * 2, nr,
                                           cudaMemcpyDeviceToDevice, ps->peer[p]));
            }
        }
    }
    // join: the caller's stream continues after the last copy (and after every upload, which matters only on the
    // error path -- on success each upload was already waited for)
    if (x_on_host) DUQ4_TRY(cudaStreamWaitEvent(st, ps->uploaded[chunks - 1], 0));
    if (host_sink) {
        DUQ4_TRY(cudaEventRecord(ps->join_down, ps->down));
        DUQ4_TRY(cudaStreamWaitEvent(st, ps->join_down, 0));
    } else {
        for (uint32_t p = 0; p < sink.n_peers; ++p) {
            if (p == sink.self) continue;
            DUQ4_TRY(cudaEventRecord(ps->join_peer[p], ps->peer[p]));
            DUQ4_TRY(cudaStreamWaitEvent(st, ps->join_peer[p], 0));
        }
    }
#undef DUQ4_TRY
    return rc;
}

// See the file comment. `bases[i]`: row 0, column 0 of rank i's [M, ldo] exchange buffer.
int run_rows_pipeline(const void *x, const void *W, bool prelaid, uint32_t M, uint32_t N, uint32_t K, int act_mode, float clip_ratio,
                      const duq4_epilogue *epi, uint32_t col_begin, uint32_t self, const void *const *flags, uint64_t *epoch_io,
                      uint64_t timeout_ns, void *out_host, uint32_t chunk_rows, void *staging, size_t staging_bytes, void *stream) {
    if (!x || !epi || !flags || !epoch_io || !out_host || (N && !W)) return DUQ4_ERR_NULL;
    const uint32_t G = epi->n_out_peers;
    if (G == 0 || G > (uint32_t)kMaxPeers || self >= G) return DUQ4_ERR_SHAPE;
    for (uint32_t i = 0; i < G; ++i)
        if (!epi->out_peers[i] || !flags[i]) return DUQ4_ERR_NULL;
    if (epi->out_multicast || epi->out_rows_per_owner) return DUQ4_ERR_MODE;   // the routing is chosen here, per chunk
    const uint64_t ldo = epi->ldo;
    if (ldo == 0 || (uint64_t)col_begin + N > ldo) return DUQ4_ERR_SHAPE;
    if (M == 0) return DUQ4_OK;
    if (K == 0 || K % 64 != 0 || (prelaid && K % 128 != 0)) return DUQ4_ERR_SHAPE;
    const uint32_t rows = pick_chunk_rows(M, chunk_rows);
    const size_t ws_bytes = N == 0 ? 0 : (prelaid ? duq4_linear_from_fp16_prelaid_workspace_bytes(rows, K) : duq4_linear_from_fp16_workspace_bytes(rows, K));
    if (N && (!staging || (reinterpret_cast<uintptr_t>(staging) & 255) != 0 || staging_bytes < ws_bytes)) return DUQ4_ERR_WORKSPACE;
    PipeState *ps = nullptr;
    int rc = pipe_state(&ps);
    if (rc) return rc;
    const uint32_t chunks = (M + rows - 1) / rows;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    uint64_t epoch = *epoch_io;
    std::lock_guard<std::mutex> enqueue_lock(g_call_mu);
#define DUQ4_TRY(call)                       \
    do {                                     \
        e = (call);                          \
        if (e != cudaSuccess) { *epoch_io = epoch; return (int)e; } \
    } while (0)
    // every rank has finished with the previous contents of the exchange buffers (its own download included: that
    // joined the caller's stream) before anybody stores into them
    if ((rc = duq4_peer_barrier(flags, G, self, ++epoch, timeout_ns, stream)) != 0) { *epoch_io = epoch; return rc; }
    DUQ4_TRY(cudaEventRecord(ps->fork, st));
    DUQ4_TRY(cudaStreamWaitEvent(ps->down, ps->fork, 0));
    for (uint32_t c = 0; c < chunks; ++c) {
        const uint32_t r0 = c * rows, nr = (M - r0 < rows) ? M - r0 : rows;
        const uint32_t sub = (nr + G - 1) / G;   // rows of this chunk per owner
        if (N && rc == 0) {
            duq4_epilogue ce = *epi;
            for (uint32_t i = 0; i < G; ++i) ce.out_peers[i] = (uint8_t *)epi->out_peers[i] + ((size_t)r0 * ldo + col_begin) * 2;
            ce.out_rows_per_owner = sub;
            const uint8_t *xc = (const uint8_t *)x + (size_t)r0 * K * 2;
            rc = prelaid ? duq4_linear_w4a4_from_fp16_prelaid(xc, (const int8_t *)W, nr, N, K, act_mode, clip_ratio, &ce, nullptr, staging, ws_bytes, stream)
                         : duq4_linear_w4a4_from_fp16(xc, (const uint8_t *)W, nr, N, K, act_mode, clip_ratio, &ce, nullptr, staging, ws_bytes, stream);
        }
        // the barriers are kept on the error path too, so that the other ranks are not left waiting for this one
        const int brc = duq4_peer_barrier(flags, G, self, ++epoch, timeout_ns, stream);
        if (brc && !rc) rc = brc;
        if (rc) continue;
        const uint64_t m0 = (uint64_t)r0 + (uint64_t)self * sub, m1 = (m0 + sub < (uint64_t)r0 + nr) ? m0 + sub : (uint64_t)r0 + nr;
        if (m1 <= m0) continue;
        DUQ4_TRY(cudaEventRecord(ps->computed[c], st));
        DUQ4_TRY(cudaStreamWaitEvent(ps->down, ps->computed[c], 0));
        DUQ4_TRY(cudaMemcpyAsync((uint8_t *)out_host + m0 * ldo * 2, (const uint8_t *)epi->out_peers[self] + m0 * ldo * 2, (m1 - m0) * ldo * 2,
                                 cudaMemcpyDeviceToHost, ps->down));
    }
    DUQ4_TRY(cudaEventRecord(ps->join_down, ps->down));
    DUQ4_TRY(cudaStreamWaitEvent(st, ps->join_down, 0));
#undef DUQ4_TRY
    *epoch_io = epoch;
    return rc;
}

}  // namespace

extern "C" {

size_t duq4_linear_host_staging_bytes(uint32_t M, uint32_t N, uint32_t K, uint32_t chunk_rows) {
    if (M == 0 || N == 0 || K == 0) return 0;
    return pipeline_staging_bytes(true, true, false, M, N, K, pick_chunk_rows(M, chunk_rows));
}

int duq4_linear_w4a4_from_fp16_host(const void *x_host, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K, int act_mode,
                                    float clip_ratio, const duq4_epilogue *epi, void *out_host, uint32_t chunk_rows, void *staging,
                                    size_t staging_bytes, void *stream) {
    DUQ4_TRACE();
    if (!out_host) return DUQ4_ERR_NULL;
    if (epi && epi->n_out_peers != 0) return DUQ4_ERR_MODE;   // the result goes to host memory, not to peers
    Sink sink;
    sink.host = out_host;
    return run_pipeline(x_host, true, W, false, M, N, K, act_mode, clip_ratio, epi, sink, chunk_rows, staging, staging_bytes, stream);
}

size_t duq4_linear_pipeline_staging_bytes(int to_host, int w_is_prelaid, uint32_t M, uint32_t N, uint32_t K, uint32_t chunk_rows) {
    if (M == 0 || N == 0 || K == 0) return 0;
    return pipeline_staging_bytes(false, to_host != 0, w_is_prelaid != 0, M, N, K, pick_chunk_rows(M, chunk_rows));
}

int duq4_linear_w4a4_from_fp16_to_host(const void *x, const void *W, int w_is_prelaid, uint32_t M, uint32_t N, uint32_t K, int act_mode,
                                       float clip_ratio, const duq4_epilogue *epi, void *out_host, uint32_t chunk_rows, void *staging,
                                       size_t staging_bytes, void *stream) {
    DUQ4_TRACE();
    if (!out_host) return DUQ4_ERR_NULL;
    if (epi && epi->n_out_peers != 0) return DUQ4_ERR_MODE;
    Sink sink;
    sink.host = out_host;
    return run_pipeline(x, false, W, w_is_prelaid != 0, M, N, K, act_mode, clip_ratio, epi, sink, chunk_rows, staging, staging_bytes, stream);
}

int duq4_linear_w4a4_from_fp16_to_peers(const void *x, const void *W, int w_is_prelaid, uint32_t M, uint32_t N, uint32_t K, int act_mode,
                                        float clip_ratio, const duq4_epilogue *epi, uint32_t self_index, uint32_t chunk_rows, void *staging,
                                        size_t staging_bytes, void *stream) {
    DUQ4_TRACE();
    if (!epi) return DUQ4_ERR_NULL;
    if (epi->n_out_peers == 0 || epi->n_out_peers > DUQ4_MAX_OUT_PEERS) return DUQ4_ERR_SHAPE;
    for (uint32_t i = 0; i < epi->n_out_peers; ++i)
        if (!epi->out_peers[i]) return DUQ4_ERR_NULL;
    Sink sink;
    sink.peers = epi->out_peers;
    sink.n_peers = epi->n_out_peers;
    sink.self = self_index;
    return run_pipeline(x, false, W, w_is_prelaid != 0, M, N, K, act_mode, clip_ratio, epi, sink, chunk_rows, staging, staging_bytes, stream);
}

int duq4_linear_w4a4_from_fp16_to_host_rows(const void *x, const void *W, int w_is_prelaid, uint32_t M, uint32_t N, uint32_t K, int act_mode,
                                            float clip_ratio, const duq4_epilogue *epi, uint32_t col_begin, uint32_t self_index,
                                            const void *const *barrier_flags, uint64_t *barrier_epoch, uint64_t barrier_timeout_ns,
                                            void *out_host, uint32_t chunk_rows, void *staging, size_t staging_bytes, void *stream) {
    DUQ4_TRACE();
    return run_rows_pipeline(x, W, w_is_prelaid != 0, M, N, K, act_mode, clip_ratio, epi, col_begin, self_index, barrier_flags, barrier_epoch,
                             barrier_timeout_ns, out_host, chunk_rows, staging, staging_bytes, stream);
}

}  // extern "C"
