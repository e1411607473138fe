// extern "C" entry points for the GEMMs and the fused linear layer, plus library metadata.
// Argument checking happens here, before any launch; the kernels live in gemv_decode.cu
// (M <= 16, HBM-bound) and gemm_tc.cu (tcgen05 tensor cores).
#include <mutex>

#include "duq_common.cuh"
#include "trace_range.h"

namespace duq4 {
int gemv_w4a4_launch(const uint8_t *A, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K, uint32_t batch,
                     const EpiParams &p, void *out, int32_t *acc_out, cudaStream_t st, bool cache_maps = true);
int tma_map_cache_entries();
bool gemv_fused_quant_fits(const void *x, uint32_t M, uint32_t K);
int gemv_w4a4_from_fp16_launch(const void *x, int act_mode, float clip, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K,
                               const EpiParams &p, void *out, cudaStream_t st, bool cache_maps);
int gemm_tc_launch(int mode, const void *A, const void *B, uint32_t M, uint32_t N, uint32_t K, uint32_t batch,
                   const EpiParams &p, void *out, int32_t *acc_out, cudaStream_t st, bool cache_maps = true,
                   uint32_t a_rows = 0);
int gemm_tc2_launch_gate_up(bool a_packed, const void *A, const void *W, uint32_t M, uint32_t inter, uint32_t K,
                            const EpiParams &p, void *h_out, cudaStream_t st);
int gemm_tc2_launch_prelaid(const void *A, const void *W_i8, uint32_t M, uint32_t N, uint32_t K, const EpiParams &p, void *out,
                            int32_t *acc_out, cudaStream_t st, void *sk_scratch = nullptr, size_t sk_bytes = 0);
size_t gemm_tc2_split_scratch_bytes();
int gemm_tc2_launch_gate_up_prelaid(const void *A, const void *W_i8, uint32_t M, uint32_t inter, uint32_t K, const EpiParams &p, void *h_out,
                                    cudaStream_t st);
int tc_status_read(cudaStream_t st, int32_t *out);
int gemv_status_read(int32_t *out);
int peer_status_read(int32_t *out);
int tc2_status_read(int32_t *out);
extern std::atomic<int> g_static_weights;
int quantize_fused_dispatch(int mode, const void *x, uint32_t rows, uint32_t cols, float clip, uint8_t *q, void *s1,
                            void *z1, void *s2, void *z2, cudaStream_t st, bool out8);

constexpr uint32_t kSmallM = 16;  // at or below this many tokens the layer is weight-bandwidth bound

// `rows`: row count of the call when the entry point supports row routing of the fused gather
// (out_rows_per_owner), -1 when it does not.
static int check_epi(const duq4_epilogue *e, uint32_t N, bool need_row, EpiParams *p, int64_t rows = -1) {
    *p = EpiParams{};
    if (!e) {
        p->mode = DUQ4_MODE_NONE;
        p->ldo = N;
        return DUQ4_OK;
    }
    if (e->mode < DUQ4_MODE_NONE || e->mode > DUQ4_MODE_ASYM_DUAL) return DUQ4_ERR_MODE;
    p->mode = e->mode;
    p->col_offset = e->col_offset;
    p->s_row = (const __half *)e->scale_row;
    p->z_row = (const __half *)e->zeros_row;
    p->s_col1 = (const __half *)e->scale_col_1;
    p->z_col1 = (const __half *)e->zeros_col_1;
    p->s_col2 = (const __half *)e->scale_col_2;
    p->z_col2 = (const __half *)e->zeros_col_2;
    p->bias = (const __half *)e->bias;
    p->ldo = e->ldo ? e->ldo : N;
    if (p->ldo < N) return DUQ4_ERR_SHAPE;
    if (e->n_out_peers > DUQ4_MAX_OUT_PEERS) return DUQ4_ERR_SHAPE;
    p->n_peers = e->n_out_peers;
    for (uint32_t i = 0; i < e->n_out_peers; ++i) {
        if (!e->out_peers[i]) return DUQ4_ERR_NULL;
        p->peers[i] = (__half *)e->out_peers[i];
    }
    p->mc_out = e->n_out_peers ? (__half *)e->out_multicast : nullptr;
    if (e->out_rows_per_owner) {
        if (e->n_out_peers == 0 || e->out_multicast || rows < 0) return DUQ4_ERR_MODE;
        if ((int64_t)e->n_out_peers * e->out_rows_per_owner < rows) return DUQ4_ERR_SHAPE;
        p->out_rows_per_owner = e->out_rows_per_owner;
    }
    if (e->n_acc_owners) {
        if (e->n_acc_owners > DUQ4_MAX_OUT_PEERS || e->acc_rows_per_owner == 0 || e->acc_slot >= e->n_acc_owners || (N & 3u) != 0)
            return DUQ4_ERR_SHAPE;
        if (e->mode != DUQ4_MODE_NONE) return DUQ4_ERR_MODE;   // the dequant runs once, on the summed accumulators
        p->n_acc_owners = e->n_acc_owners;
        p->acc_rows_per_owner = e->acc_rows_per_owner;
        p->acc_slot = e->acc_slot;
        for (uint32_t i = 0; i < e->n_acc_owners; ++i) {
            if (!e->acc_owners[i]) return DUQ4_ERR_NULL;
            if ((reinterpret_cast<uintptr_t>(e->acc_owners[i]) & 15) != 0) return DUQ4_ERR_ALIGN;
            p->acc_owners[i] = e->acc_owners[i];
        }
    }
    p->next_w = (const uint8_t *)e->next_weights;
    p->next_w_bytes = e->next_weights ? e->next_weights_bytes : 0;
    if (e->mode == DUQ4_MODE_NONE) return DUQ4_OK;
    const bool asym = e->mode == DUQ4_MODE_ASYM || e->mode == DUQ4_MODE_ASYM_DUAL;
    const bool dual = e->mode == DUQ4_MODE_SYM_DUAL || e->mode == DUQ4_MODE_ASYM_DUAL;
    if (need_row && (!p->s_row || (asym && !p->z_row))) return DUQ4_ERR_NULL;
    if (!p->s_col1 || (asym && !p->z_col1)) return DUQ4_ERR_NULL;
    if (dual && (!p->s_col2 || (e->mode == DUQ4_MODE_ASYM_DUAL && !p->z_col2))) return DUQ4_ERR_NULL;
    if (!asym) p->z_row = nullptr;
    return DUQ4_OK;
}

static int linear_dispatch(const uint8_t *A, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K, uint32_t batch,
                           const EpiParams &p, void *out, int32_t *acc_out, cudaStream_t st, bool cache_maps = true) {
    if (!A || !W) return DUQ4_ERR_NULL;
    if (p.mode != DUQ4_MODE_NONE && !out && !p.n_peers) return DUQ4_ERR_NULL;
    if (p.mode == DUQ4_MODE_NONE && !acc_out) return DUQ4_ERR_NULL;
    if (M == 0 || N == 0 || batch == 0) return DUQ4_OK;
    if (K == 0 || K % 64 != 0) return DUQ4_ERR_SHAPE;
    if (M <= kSmallM) return gemv_w4a4_launch(A, W, M, N, K, batch, p, out, acc_out, st, cache_maps);
    return gemm_tc_launch(1 /* both operands packed int4 */, A, W, M, N, K, batch, p, out, acc_out, st, cache_maps);
}

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace duq4

using namespace duq4;

extern "C" {

const char *duq4_version(void) { return "duq4-b200 0.1 (sm_100a)"; }

const char *duq4_error_string(int status) {
    switch (status) {
        case DUQ4_OK: return "ok";
        case DUQ4_ERR_NULL: return "a required pointer is NULL";
        case DUQ4_ERR_SHAPE: return "unsupported shape (zero, not a required multiple, or too large)";
        case DUQ4_ERR_MODE: return "unknown quantizer/epilogue mode";
        case DUQ4_ERR_WORKSPACE: return "workspace missing, too small or misaligned";
        case DUQ4_ERR_ALIGN: return "pointer not 16-byte aligned";
        case DUQ4_ERR_DEVICE: return "device or driver does not provide what the kernel needs";
        case DUQ4_ERR_TIMEOUT: return "a bounded device-side wait expired";
        case DUQ4_ERR_TOO_LARGE: return "problem needs more scratch than the library's built-in scratch array holds";
        default: return status > 0 ? cudaGetErrorString((cudaError_t)status) : "unknown duq4 status";
    }
}

int duq4_dual_quant_col_k(void) { return DUQ4_QUANT_COL_K; }

int duq4_tensor_map_cache_entries(void) { return tma_map_cache_entries(); }

int duq4_set_static_weights(int on) {
    return g_static_weights.exchange(on ? 1 : 0);
}

int duq4_matmul_4bit(const uint8_t *A, const uint8_t *B, uint32_t M, uint32_t N, uint32_t K, int32_t *C, void *stream) {
    DUQ4_TRACE();
    EpiParams p{};
    p.mode = DUQ4_MODE_NONE;
    p.ldo = N;
    return linear_dispatch(A, B, M, N, K, 1, p, nullptr, C, (cudaStream_t)stream);
}

int duq4_matmul_8bit(const int8_t *A, const int8_t *B, uint32_t M, uint32_t N, uint32_t K, int32_t *C, void *stream) {
    DUQ4_TRACE();
    if (!A || !B || !C) return DUQ4_ERR_NULL;
    if (M == 0 || N == 0) return DUQ4_OK;
    if (K == 0 || K % 16 != 0) return DUQ4_ERR_SHAPE;
    EpiParams p{};
    p.mode = DUQ4_MODE_NONE;
    p.ldo = N;
    return gemm_tc_launch(0 /* int8 operands */, A, B, M, N, K, 1, p, nullptr, C, (cudaStream_t)stream);
}

int duq4_batch_matmul_4bit(const uint8_t *A, const uint8_t *B, uint32_t M, uint32_t N, uint32_t K, int32_t *C,
                           uint32_t batch_count, void *stream) {
    DUQ4_TRACE();
    EpiParams p{};
    p.mode = DUQ4_MODE_NONE;
    p.ldo = N;
    return linear_dispatch(A, B, M, N, K, batch_count, p, nullptr, C, (cudaStream_t)stream);
}

int duq4_linear_w4a4(const uint8_t *A, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K, const duq4_epilogue *epi,
                     void *out, int32_t *acc_out, void *stream) {
    DUQ4_TRACE();
    EpiParams p;
    int rc = check_epi(epi, N, true, &p, M);
    if (rc) return rc;
    return linear_dispatch(A, W, M, N, K, 1, p, out, acc_out, (cudaStream_t)stream);
}

int duq4_linear_w4a4_batched(const uint8_t *A, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K, uint32_t batch_count,
                             const duq4_epilogue *epi, void *out, int32_t *acc_out, void *stream) {
    DUQ4_TRACE();
    EpiParams p;
    int rc = check_epi(epi, N, true, &p);
    if (rc) return rc;
    if (p.ldo != N) return DUQ4_ERR_SHAPE;  // batched outputs are dense [batch, M, N]
    p.row_vec_stride = M;
    p.col_vec_stride = N;
    return linear_dispatch(A, W, M, N, K, batch_count, p, out, acc_out, (cudaStream_t)stream);
}

int duq4_linear_w4a4_preunpacked(const int8_t *A_i8, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K,
                                 const duq4_epilogue *epi, void *out, int32_t *acc_out, void *stream) {
    DUQ4_TRACE();
    EpiParams p;
    int rc = check_epi(epi, N, true, &p, M);
    if (rc) return rc;
    if (!A_i8 || !W) return DUQ4_ERR_NULL;
    if (p.mode != DUQ4_MODE_NONE && !out && !p.n_peers) return DUQ4_ERR_NULL;
    if (p.mode == DUQ4_MODE_NONE && !acc_out && !p.n_acc_owners) return DUQ4_ERR_NULL;
    if (M == 0 || N == 0) return DUQ4_OK;
    if (K == 0 || K % 64 != 0) return DUQ4_ERR_SHAPE;
    if (p.n_acc_owners && (uint64_t)p.n_acc_owners * p.acc_rows_per_owner < M) return DUQ4_ERR_SHAPE;
    return gemm_tc_launch(2 /* A pre-unpacked int8, W packed int4 */, A_i8, W, M, N, K, 1, p, out, acc_out, (cudaStream_t)stream);
}

size_t duq4_gemm_split_scratch_bytes(void) { return gemm_tc2_split_scratch_bytes(); }

int duq4_linear_w4a4_prelaid(const int8_t *A_i8, const int8_t *W_i8, uint32_t M, uint32_t N, uint32_t K, const duq4_epilogue *epi,
                             void *out, int32_t *acc_out, void *split_scratch, size_t split_scratch_bytes, void *stream) {
    DUQ4_TRACE();
    EpiParams p;
    int rc = check_epi(epi, N, true, &p, M);
    if (rc) return rc;
    if (!A_i8 || !W_i8) return DUQ4_ERR_NULL;
    if (p.mode != DUQ4_MODE_NONE && !out && !p.n_peers) return DUQ4_ERR_NULL;
    if (p.mode == DUQ4_MODE_NONE && !acc_out && !p.n_acc_owners) return DUQ4_ERR_NULL;
    if (M == 0 || N == 0) return DUQ4_OK;
    if (K == 0 || K % 128 != 0) return DUQ4_ERR_SHAPE;
    if (p.n_acc_owners && (uint64_t)p.n_acc_owners * p.acc_rows_per_owner < M) return DUQ4_ERR_SHAPE;
    if (((reinterpret_cast<uintptr_t>(A_i8) | reinterpret_cast<uintptr_t>(W_i8)) & 15) != 0) return DUQ4_ERR_ALIGN;
    return gemm_tc2_launch_prelaid(A_i8, W_i8, M, N, K, p, out, acc_out, (cudaStream_t)stream, split_scratch, split_scratch_bytes);
}

int duq4_linear_w4a4_gate_up_silu(const void *A, int a_is_int8, const uint8_t *W, uint32_t M, uint32_t inter, uint32_t K,
                                  const duq4_epilogue *epi, void *h_out, void *stream) {
    DUQ4_TRACE();
    if (!A || !W || !epi) return DUQ4_ERR_NULL;
    if (epi->mode != DUQ4_MODE_SYM && epi->mode != DUQ4_MODE_ASYM) return DUQ4_ERR_MODE;   // the dual selectors go by output column
    EpiParams p;
    int rc = check_epi(epi, inter, true, &p);   // ldo defaults to the width of h
    if (rc) return rc;
    if (!h_out && !p.n_peers) return DUQ4_ERR_NULL;
    if (M == 0 || inter == 0) return DUQ4_OK;
    if (K == 0 || K % 64 != 0 || inter > 0x7FFFFFFFu) return DUQ4_ERR_SHAPE;
    return gemm_tc2_launch_gate_up(a_is_int8 == 0, A, W, M, inter, K, p, h_out, (cudaStream_t)stream);
}

int duq4_linear_w4a4_gate_up_silu_prelaid(const int8_t *A_i8, const int8_t *W_i8, uint32_t M, uint32_t inter, uint32_t K,
                                          const duq4_epilogue *epi, void *h_out, void *stream) {
    DUQ4_TRACE();
    if (!A_i8 || !W_i8 || !epi) return DUQ4_ERR_NULL;
    if (epi->mode != DUQ4_MODE_SYM && epi->mode != DUQ4_MODE_ASYM) return DUQ4_ERR_MODE;
    EpiParams p;
    int rc = check_epi(epi, inter, true, &p);
    if (rc) return rc;
    if (!h_out && !p.n_peers) return DUQ4_ERR_NULL;
    if (M == 0 || inter == 0) return DUQ4_OK;
    if (K == 0 || K % 128 != 0 || inter > 0x7FFFFFFFu) return DUQ4_ERR_SHAPE;
    if (((reinterpret_cast<uintptr_t>(A_i8) | reinterpret_cast<uintptr_t>(W_i8)) & 15) != 0) return DUQ4_ERR_ALIGN;
    return gemm_tc2_launch_gate_up_prelaid(A_i8, W_i8, M, inter, K, p, h_out, (cudaStream_t)stream);
}

// Scratch layout of duq4_linear_w4a4_from_fp16: activation codes, then four fp16 vectors [M]
// (scale_1, zeros_1, scale_2, zeros_2), each region 256-byte aligned. M <= 16 stores packed
// codes [M, K/2]; larger M stores tensor-core-ready int8 codes [M, K].
// 17..31 tokens: the int8 code buffer is sized for 32 rows, so that the GEMM's A tiles read 32 in-bounds rows
// (rows >= M hold whatever the scratch held; their accumulators are never stored). Measured on 4096->22016:
// 34 us with the tensor map ending at row M, 25 us with 32 rows.
static uint32_t code_rows(uint32_t M) { return (M > kSmallM && M < 32) ? 32 : M; }
static size_t codes_bytes(uint32_t M, uint32_t K) { return M <= kSmallM ? (size_t)M * (K / 2) : (size_t)code_rows(M) * K; }

size_t duq4_linear_from_fp16_workspace_bytes(uint32_t M, uint32_t K) {
    return align_up(codes_bytes(M, K), 256) + 4 * align_up((size_t)M * 2, 256);
}

int duq4_linear_w4a4_from_fp16(const void *x, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K, int act_mode,
                               float clip_ratio, const duq4_epilogue *epi, void *out, void *workspace,
                               size_t workspace_bytes, void *stream) {
    DUQ4_TRACE();
    if (!x || !W || !epi || (!out && !epi->n_out_peers)) return DUQ4_ERR_NULL;
    if (act_mode < DUQ4_MODE_SYM || act_mode > DUQ4_MODE_ASYM_DUAL) return DUQ4_ERR_MODE;
    if (M == 0 || N == 0) return DUQ4_OK;
    if (K == 0 || K % 64 != 0) return DUQ4_ERR_SHAPE;
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0 ||
        workspace_bytes < duq4_linear_from_fp16_workspace_bytes(M, K))
        return DUQ4_ERR_WORKSPACE;
    EpiParams p;
    int rc = check_epi(epi, N, false, &p, M);
    if (rc) return rc;
    if (p.mode == DUQ4_MODE_NONE) return DUQ4_ERR_MODE;
    uint8_t *ws = (uint8_t *)workspace;
    uint8_t *codes = ws;
    size_t off = align_up(codes_bytes(M, K), 256), vec = align_up((size_t)M * 2, 256);
    const bool small = M <= kSmallM;
    void *s1 = ws + off, *z1 = ws + off + vec, *s2 = ws + off + 2 * vec, *z2 = ws + off + 3 * vec;
    cudaStream_t st = (cudaStream_t)stream;
    const bool epi_asym = p.mode == DUQ4_MODE_ASYM || p.mode == DUQ4_MODE_ASYM_DUAL;
    const bool act_asym = act_mode == DUQ4_MODE_ASYM || act_mode == DUQ4_MODE_ASYM_DUAL;
    if (epi_asym && !act_asym) return DUQ4_ERR_MODE;  // an asymmetric epilogue needs per-token zero-points
    // up to 16 tokens: ONE launch -- every CTA of the small-M kernel quantizes the tokens into its own shared
    // memory; codes and per-token scales never reach the workspace
    if (small && gemv_fused_quant_fits(x, M, K)) return gemv_w4a4_from_fp16_launch(x, act_mode, clip_ratio, W, M, N, K, p, out, st, true);
    rc = quantize_fused_dispatch(act_mode, x, M, K, clip_ratio, codes, s1, z1, s2, z2, st, !small);
    if (rc) return rc;
    p.s_row = (const __half *)s1;
    p.z_row = epi_asym ? (const __half *)z1 : nullptr;
    if (small) return linear_dispatch(codes, W, M, N, K, 1, p, out, nullptr, st);
    return gemm_tc_launch(2 /* A pre-unpacked int8, W packed int4 */, codes, W, M, N, K, 1, p, out, nullptr, st, true, code_rows(M));
}

size_t duq4_linear_from_fp16_prelaid_workspace_bytes(uint32_t M, uint32_t K);

int duq4_linear_w4a4_from_fp16_prelaid(const void *x, const int8_t *W_i8, uint32_t M, uint32_t N, uint32_t K, int act_mode,
                                       float clip_ratio, const duq4_epilogue *epi, void *out, void *workspace,
                                       size_t workspace_bytes, void *stream) {
    DUQ4_TRACE();
    if (!x || !W_i8 || !epi || (!out && !epi->n_out_peers)) return DUQ4_ERR_NULL;
    if (act_mode < DUQ4_MODE_SYM || act_mode > DUQ4_MODE_ASYM_DUAL) return DUQ4_ERR_MODE;
    if (M == 0 || N == 0) return DUQ4_OK;
    if (K == 0 || K % 128 != 0) return DUQ4_ERR_SHAPE;
    const size_t cbytes = align_up((size_t)M * K, 256), vec = align_up((size_t)M * 2, 256);
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0 || workspace_bytes < duq4_linear_from_fp16_prelaid_workspace_bytes(M, K))
        return DUQ4_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(W_i8) & 15) != 0) return DUQ4_ERR_ALIGN;
    EpiParams p;
    int rc = check_epi(epi, N, false, &p, M);
    if (rc) return rc;
    if (p.mode == DUQ4_MODE_NONE) return DUQ4_ERR_MODE;
    const bool epi_asym = p.mode == DUQ4_MODE_ASYM || p.mode == DUQ4_MODE_ASYM_DUAL;
    const bool act_asym = act_mode == DUQ4_MODE_ASYM || act_mode == DUQ4_MODE_ASYM_DUAL;
    if (epi_asym && !act_asym) return DUQ4_ERR_MODE;
    uint8_t *ws = (uint8_t *)workspace;
    void *s1 = ws + cbytes, *z1 = ws + cbytes + vec, *s2 = ws + cbytes + 2 * vec, *z2 = ws + cbytes + 3 * vec;
    cudaStream_t st = (cudaStream_t)stream;
    rc = quantize_fused_dispatch(act_mode, x, M, K, clip_ratio, ws, s1, z1, s2, z2, st, true);
    if (rc) return rc;
    p.s_row = (const __half *)s1;
    p.z_row = epi_asym ? (const __half *)z1 : nullptr;
    return gemm_tc2_launch_prelaid(ws, W_i8, M, N, K, p, out, nullptr, st, ws + cbytes + 4 * vec, gemm_tc2_split_scratch_bytes());
}

size_t duq4_linear_from_fp16_prelaid_workspace_bytes(uint32_t M, uint32_t K) {
    return align_up((size_t)M * K, 256) + 4 * align_up((size_t)M * 2, 256) + gemm_tc2_split_scratch_bytes();
}

// ---- scratch held inside the library ------------------------------------------------------
// duq4_linear_w4a4_from_fp16_static keeps its intermediate (activation codes and per-token
// scales / zero-points) in this array instead of caller memory. The array is part of the
// library image: every GPU on which the library's kernels get loaded carries its own copy
// until the process exits. Inside host code the name `g_static_scratch` is only a handle for
// the runtime, never a device address: the address used in launches is the one
// cudaGetSymbolAddress returns for the device that is current at the time of the query.
static __device__ __align__(256) unsigned char g_static_scratch[DUQ4_STATIC_SCRATCH_BYTES];

static int static_scratch_address(void **out) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static void *addr[kMaxDevices] = {};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return DUQ4_ERR_DEVICE;
    std::lock_guard<std::mutex> g(mu);
    if (!addr[dev]) {  // first use on this device: resolve the symbol with this device current
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p || (reinterpret_cast<uintptr_t>(p) & 255) != 0) return DUQ4_ERR_WORKSPACE;
        addr[dev] = p;
    }
    *out = addr[dev];
    return DUQ4_OK;
}

int duq4_linear_w4a4_from_fp16_static(const void *x, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K, int act_mode,
                                      float clip_ratio, const duq4_epilogue *epi, void *out, void *stream) {
    if (!x || !W || !out || !epi) return DUQ4_ERR_NULL;
    if (act_mode < DUQ4_MODE_SYM || act_mode > DUQ4_MODE_ASYM_DUAL) return DUQ4_ERR_MODE;
    if (M == 0 || N == 0) return DUQ4_OK;
    if (K == 0 || K % 64 != 0) return DUQ4_ERR_SHAPE;
    if (duq4_linear_from_fp16_workspace_bytes(M, K) > (size_t)DUQ4_STATIC_SCRATCH_BYTES) return DUQ4_ERR_TOO_LARGE;
    EpiParams p;
    int rc = check_epi(epi, N, false, &p);
    if (rc) return rc;
    if (p.mode == DUQ4_MODE_NONE) return DUQ4_ERR_MODE;
    const bool epi_asym = p.mode == DUQ4_MODE_ASYM || p.mode == DUQ4_MODE_ASYM_DUAL;
    const bool act_asym = act_mode == DUQ4_MODE_ASYM || act_mode == DUQ4_MODE_ASYM_DUAL;
    if (epi_asym && !act_asym) return DUQ4_ERR_MODE;
    void *base = nullptr;
    rc = static_scratch_address(&base);
    if (rc) return rc;
    uint8_t *ws = (uint8_t *)base;
    const size_t off = align_up(codes_bytes(M, K), 256), vec = align_up((size_t)M * 2, 256);
    const bool small = M <= kSmallM;
    void *s1 = ws + off, *z1 = ws + off + vec, *s2 = ws + off + 2 * vec, *z2 = ws + off + 3 * vec;
    cudaStream_t st = (cudaStream_t)stream;
    // up to 16 tokens: one launch that needs no scratch at all (see duq4_linear_w4a4_from_fp16)
    if (small && gemv_fused_quant_fits(x, M, K)) return gemv_w4a4_from_fp16_launch(x, act_mode, clip_ratio, W, M, N, K, p, out, st, false);
    // Nothing in the scratch has to start at zero: the quantizer overwrites every code byte and
    // every per-token vector entry the GEMM reads before the GEMM reads it.
    rc = quantize_fused_dispatch(act_mode, x, M, K, clip_ratio, ws, s1, z1, s2, z2, st, !small);
    if (rc) return rc;
    p.s_row = (const __half *)s1;
    p.z_row = epi_asym ? (const __half *)z1 : nullptr;
    // tensor maps are encoded on the stack for this call (cache_maps = false on every path: small-M TMA kernel,
    // single-CTA and CTA-pair tensor-core kernels): no cache lookup or insertion, no host heap use
    if (small) return linear_dispatch(ws, W, M, N, K, 1, p, out, nullptr, st, false);
    return gemm_tc_launch(2 /* A pre-unpacked int8, W packed int4 */, ws, W, M, N, K, 1, p, out, nullptr, st, false, code_rows(M));
}

int duq4_last_device_status(void *stream, int32_t *status_out) {
    if (!status_out) return DUQ4_ERR_NULL;
    int32_t a = 0, b = 0;
    int rc = tc_status_read((cudaStream_t)stream, &a);   // synchronises the stream
    if (rc) return rc;
    rc = gemv_status_read(&b);
    if (rc) return rc;
    int32_t c = 0;
    rc = tc2_status_read(&c);
    if (rc) return rc;
    int32_t d = 0;
    rc = peer_status_read(&d);
    if (rc) return rc;
    // 1..9: tensor-core GEMM wait, 101..: small-M kernel wait, 201..: CTA-pair GEMM wait, 301: peer barrier wait
    *status_out = a ? a : (b ? 100 + b : (c ? 200 + c : (d ? 300 + d : 0)));
    return DUQ4_OK;
}

}  // extern "C"
