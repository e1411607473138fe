/*
 * duq4.h -- C ABI of libduq4.so, the sm_100a (B200) W4A4 linear-layer library.
 *
 * One entry point per host launcher of the DUQLinear4bitCUDA reference
 * (include/quant.h and include/gemm.h of that project; cited per function below as
 * "ref:"), plus fused entry points the reference does not have. Conventions:
 *
 *   - every pointer is a DEVICE pointer unless the comment says otherwise; the caller
 *     owns every buffer; nothing here allocates device memory;
 *   - "fp16" buffers are IEEE binary16 (CUDA `half`), passed as `const void *`;
 *   - packed int4 tensors are uint8, row-major [rows, K/2]; element 2j sits in the LOW
 *     nibble of byte j, element 2j+1 in the HIGH nibble, two's complement
 *     (ref: include/int4.h:86-98, qlinear4bit/tools/quantization.py:40-47);
 *   - the trailing `stream` is a cudaStream_t (NULL = legacy default stream, which is
 *     what every launch of the reference uses);
 *   - return value: 0 = ok, < 0 = argument rejected before any launch (DUQ4_ERR_*),
 *     > 0 = a cudaError_t reported by the launch.
 *   - all functions may be called from several host threads at once (on different streams or
 *     devices); the process-wide state is a mutex-guarded cache of TMA descriptors keyed by
 *     (pointer, shape), once-per-device kernel set-up guarded the same way, the atomic
 *     duq4_set_static_weights flag, the scratch array of the _static entry point (shared by all
 *     its calls on a GPU -- see there), and two helper streams per device that the _host entry
 *     point creates on first use.
 *   - tracing: every entry point that can launch work (all but the _static one and the metadata
 *     getters) opens an NVTX range named after itself in the NVTX domain "duq4" for the duration of
 *     the host call; a timeline tool attached through NVTX sees one range per call.
 */
#ifndef DUQ4_H_
#define DUQ4_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DUQ4_OK 0
#define DUQ4_ERR_NULL (-1)        /* a required pointer is NULL */
#define DUQ4_ERR_SHAPE (-2)       /* a dimension is zero, not a multiple the kernel needs, or too large */
#define DUQ4_ERR_MODE (-3)        /* unknown epilogue / quantizer mode */
#define DUQ4_ERR_WORKSPACE (-4)   /* workspace missing, too small or misaligned */
#define DUQ4_ERR_ALIGN (-5)       /* a pointer is not aligned as required */
#define DUQ4_ERR_DEVICE (-6)      /* not an sm_100 device / driver entry point unavailable */
#define DUQ4_ERR_TIMEOUT (-7)     /* a bounded device-side wait gave up (see duq4_last_device_status) */
#define DUQ4_ERR_TOO_LARGE (-8)   /* duq4_linear_w4a4_from_fp16_static: scratch need exceeds DUQ4_STATIC_SCRATCH_BYTES */

/* Column split of the dual-uniform schemes (ref: include/quant.h:5, QUANT_COL_K). */
#define DUQ4_QUANT_COL_K 10

#ifndef DUQ4_MAX_OUT_PEERS
#define DUQ4_MAX_OUT_PEERS 8
#endif

/* Quantizer / dequantizer variants. */
#define DUQ4_MODE_NONE 0       /* no dequant: int32 accumulators only */
#define DUQ4_MODE_SYM 1        /* ref: sym_quant_host / sym_dequant_host */
#define DUQ4_MODE_SYM_DUAL 2   /* ref: sym_dual_quant_host / sym_dual_dequant_host */
#define DUQ4_MODE_ASYM 3       /* ref: asym_quant_host / asym_dequant_host */
#define DUQ4_MODE_ASYM_DUAL 4  /* ref: asym_dual_quant_host / asym_dual_dequant_host */

const char *duq4_version(void);
const char *duq4_error_string(int status);
/* Value exported by the reference's pybind module as get_dual_quant_col_k()
 * (ref: src/export/bindings.cpp:471-473). */
int duq4_dual_quant_col_k(void);
/* Number of TMA descriptors the library's cache holds at the moment (diagnostic; the cache lives on
 * the host heap, is keyed by (pointer, shape) and is emptied when it passes 4096 entries). No reference
 * counterpart. */
int duq4_tensor_map_cache_entries(void);

/* Process-wide promise about WEIGHT-side operands (the second matrix of the linear / matmul entry
 * points and the per-output-channel vectors of the epilogue: scale_col_*, zeros_col_*, bias):
 * on != 0 states that they are never written by earlier work queued on the same stream (they
 * are parameters, uploaded and synchronised before use). The small-M (M <= 16) kernels are then
 * launched with programmatic stream serialization and start streaming weights and per-channel
 * vectors while the preceding kernel of the stream is still finishing; activations, per-token
 * scales and all outputs still wait for it. Off by default (full stream ordering). Returns the
 * previous value. No reference counterpart. */
int duq4_set_static_weights(int on);

/* ---- quantize, scales (and zero-points) supplied by the caller ------------------------ */

/* ref: include/quant.h:9-16 sym_quant_host -> src/kernels/quant.cu:12-61.
 * q = clamp(rn(x / scale[row]), -8, 6) packed two per byte; colsDst = ceil(colsSrc/2). */
int duq4_sym_quant(const void *x, const void *scale, uint32_t rows, uint32_t colsSrc,
                   uint32_t colsDst, uint8_t *q, void *stream);
/* ref: include/quant.h:29-37 sym_dual_quant_host -> src/kernels/quant2.cu:10-60.
 * Columns < 10 use scale_1[row], the rest scale_2[row]. */
int duq4_sym_dual_quant(const void *x, const void *scale_1, const void *scale_2, uint32_t rows,
                        uint32_t colsSrc, uint32_t colsDst, uint8_t *q, void *stream);
/* ref: include/quant.h:49-57 asym_quant_host -> src/kernels/quant.cu:100-147.
 * q = clamp(rn(x/scale[row]) + rn(zeros[row]), 0, 15). */
int duq4_asym_quant(const void *x, const void *scale, const void *zeros, uint32_t rows,
                    uint32_t colsSrc, uint32_t colsDst, uint8_t *q, void *stream);
/* ref: include/quant.h:92-103 asym_dual_quant_host -> src/kernels/quant2.cu:102-156.
 * q = clamp(rn(x/s + z), 0, 15), (s,z) = set 1 for columns < 10 else set 2. Argument
 * order follows the reference's DEFINITION (x, s1, z1, s2, z2), which is also how its
 * binding calls it; the reference header lists (s1, s2, z1, z2). */
int duq4_asym_dual_quant(const void *x, const void *scale_1, const void *zeros_1,
                         const void *scale_2, const void *zeros_2, uint32_t rows,
                         uint32_t colsSrc, uint32_t colsDst, uint8_t *q, void *stream);
/* ref: include/quant.h:70-77 asym_quant_host_8bit -> src/kernels/quant.cu:245-279.
 * fp32 in; q = clamp(rn(half(x/s)) + rn(half(z)), 0, 126) as int8. */
int duq4_asym_quant_8bit(const float *x, const float *scale, const float *zeros, uint32_t rows,
                         uint32_t cols, int8_t *q, void *stream);

/* ---- fused per-token quantize: statistics, scale(/zero) and codes in one pass --------- */
/* No single reference function; each replaces the torch ops of a quantizer module plus
 * the quantize launch (ref: qlinear4bit/nn/quantizer.py:10-16 SymQuantizer,
 * :24-35 AsymQuantizer; src/module/quant_tensor.cu:151-161 Quantizer4bit::forward).
 * x fp16 [rows, cols], cols even; q uint8 [rows, cols/2]; scale/zeros fp16 [rows] out.
 * Dual variants compute one (scale[,zero]) over columns [0,10) and one over [10,cols). */
int duq4_quantize_sym_fused(const void *x, uint32_t rows, uint32_t cols, float clip_ratio,
                            uint8_t *q, void *scale_out, void *stream);
int duq4_quantize_asym_fused(const void *x, uint32_t rows, uint32_t cols, uint8_t *q,
                             void *scale_out, void *zeros_out, void *stream);
int duq4_quantize_sym_dual_fused(const void *x, uint32_t rows, uint32_t cols, float clip_ratio,
                                 uint8_t *q, void *scale_1_out, void *scale_2_out, void *stream);
int duq4_quantize_asym_dual_fused(const void *x, uint32_t rows, uint32_t cols, uint8_t *q,
                                  void *scale_1_out, void *zeros_1_out, void *scale_2_out,
                                  void *zeros_2_out, void *stream);

/* Fused quantizer writing TENSOR-CORE-READY activations for duq4_linear_w4a4_preunpacked:
 * q_i8 [rows, cols] holds one int8 = 16 * code per element (the nibble in the high four bits),
 * and inside every block of 128 columns the elements are permuted the way the GEMM's own
 * in-kernel int4 unpack permutes them (position 32c+b <- column 32c+2b, position 32c+16+b <-
 * column 32c+2b+1, b in [0,16), c in [0,4)). The buffer is an opaque operand of that GEMM, not
 * a format of the reference. mode is DUQ4_MODE_SYM/SYM_DUAL/ASYM/ASYM_DUAL; outputs a mode
 * does not produce may be NULL. cols % 64 == 0. No reference counterpart: it removes the
 * activation half of the shared-memory unpack work from the GEMM. */
int duq4_quantize_fused_i8(int mode, const void *x, uint32_t rows, uint32_t cols, float clip_ratio,
                           int8_t *q_i8, void *scale_1_out, void *zeros_1_out, void *scale_2_out,
                           void *zeros_2_out, void *stream);

/* Glue of a SiLU-gated MLP block (gate/up GEMM -> SiLU(gate)*up -> requantize -> down GEMM), no
 * reference counterpart (the reference has no MLP module; a user composes its Linear modules with
 * torch's silu and multiply). gate_up is fp16 [rows, ld]; the token fed to the quantizer is
 *     h[r, j] = half( half(silu(gate_up[r, j])) * gate_up[r, up_offset + j] ),   j in [0, inter),
 * with silu evaluated in fp32 -- bit for bit what `F.silu(gate) * up` yields in fp16 -- and is
 * quantized per token exactly as duq4_quantize_{sym,asym}_fused would quantize a stored h, but h
 * never goes to memory. mode: DUQ4_MODE_SYM or DUQ4_MODE_ASYM. q receives packed codes
 * [rows, inter/2] (q_is_int8 = 0) or tensor-core-ready int8 [rows, inter] (q_is_int8 != 0, see
 * duq4_quantize_fused_i8). inter, ld and up_offset must be multiples of 8 (64 for int8 output). */
int duq4_silu_mul_quantize_fused(int mode, const void *gate_up, uint32_t rows, uint32_t inter, uint32_t ld,
                                 uint32_t up_offset, float clip_ratio, void *q, int q_is_int8,
                                 void *scale_out, void *zeros_out, void *stream);

/* ---- dequantize an int32 accumulator tensor ------------------------------------------- */

/* ref: include/quant.h:19-26 sym_dequant_host -> src/kernels/quant.cu:64-97.
 * x = (scale_row[r] * scale_col[c]) * half(q), every product rounded to fp16. */
int duq4_sym_dequant(const int32_t *q, const void *scale_row, const void *scale_col,
                     uint32_t rows, uint32_t cols, void *x, void *stream);
/* ref: include/quant.h:40-48 sym_dual_dequant_host -> src/kernels/quant2.cu:63-98.
 * scale_col = scale_col_1[c] for output column c < 10, else scale_col_2[c]. */
int duq4_sym_dual_dequant(const int32_t *q, const void *scale_row, const void *scale_col_1,
                          const void *scale_col_2, uint32_t rows, uint32_t cols, void *x,
                          void *stream);
/* ref: include/quant.h:59-68 asym_dequant_host -> src/kernels/quant.cu:150-188.
 * x = (s_row*s_col) * ((half(q) - z_row) - z_col). */
int duq4_asym_dequant(const int32_t *q, const void *scale_row, const void *zeros_row,
                      const void *scale_col, const void *zeros_col, uint32_t rows, uint32_t cols,
                      void *x, void *stream);
/* ref: include/quant.h:106-117 asym_dual_dequant_host -> src/kernels/quant2.cu:159-208.
 * Column set 1 is used for output column 0 only (the reference's selector
 * `(QUANT_COL_ST << col) & 1`), set 2 elsewhere. */
int duq4_asym_dual_dequant(const int32_t *q, const void *scale_row, const void *zeros_row,
                           const void *scale_col_1, const void *zeros_col_1,
                           const void *scale_col_2, const void *zeros_col_2, uint32_t rows,
                           uint32_t cols, void *x, void *stream);
/* ref: include/quant.h:79-89 asym_batch_dequant_host -> src/kernels/quant.cu:191-239.
 * q [batches, rows, cols]; row vectors [batches, rows], column vectors [batches, cols]. */
int duq4_asym_batch_dequant(const int32_t *q, const void *scale_row, const void *zeros_row,
                            const void *scale_col, const void *zeros_col, uint32_t batches,
                            uint32_t rows, uint32_t cols, void *x, void *stream);
/* ref: include/quant.h:118-127 asym_dequant_host_hprec -> src/kernels/quant.cu:282-323.
 * fp32: x = (s_row*s_col) * (float(q) - (z_row + z_col)). */
int duq4_asym_dequant_hprec(const int32_t *q, const float *scale_row, const float *zeros_row,
                            const float *scale_col, const float *zeros_col, uint32_t rows,
                            uint32_t cols, float *x, void *stream);

/* ---- integer GEMMs, C[M,N] = A[M,K] * B[N,K]^T, int32 out ----------------------------- */

/* ref: include/gemm.h:5-12 matmul_host_4bit -> src/kernels/gemm.cu:8-43 (CUTLASS Sm80
 * int4 tensor-op GEMM). A, B packed signed int4; K % 64 == 0 (the reference asserts
 * packed-K % 32 == 0, qlinear4bit/tools/tensor_utils.py:52). */
int duq4_matmul_4bit(const uint8_t *A, const uint8_t *B, uint32_t M, uint32_t N, uint32_t K,
                     int32_t *C, void *stream);
/* ref: include/gemm.h:14-21 matmul_host_8bit -> src/kernels/gemm.cu:46-81. K % 16 == 0. */
int duq4_matmul_8bit(const int8_t *A, const int8_t *B, uint32_t M, uint32_t N, uint32_t K,
                     int32_t *C, void *stream);
/* ref: include/gemm.h:23-31 batch_matmul_host_4bit -> src/kernels/gemm.cu:83-117, with
 * the contiguous layout its binding builds (src/export/bindings.cpp:46-57):
 * A [batch, M, K/2], B [batch, N, K/2] -> C [batch, M, N]. The reference passes HOST
 * arrays of pointers to a device kernel and does not work; this one does. */
int duq4_batch_matmul_4bit(const uint8_t *A, const uint8_t *B, uint32_t M, uint32_t N,
                           uint32_t K, int32_t *C, uint32_t batch_count, void *stream);

/* ---- fused linear layer: int4 GEMM with the dequant (and bias) in its epilogue -------- */

/* What the GEMM epilogue applies. Column vectors are indexed by the LOCAL column
 * c in [0, N); `col_offset` is the global index of local column 0 and only enters the
 * dual-uniform selectors (c + col_offset < 10, c + col_offset == 0), so that an
 * N-sharded layer gives the same result as the unsharded one. */
typedef struct duq4_epilogue {
    int32_t mode;            /* DUQ4_MODE_* */
    uint32_t col_offset;
    const void *scale_row;   /* fp16 [M]   per-token scales              (all modes but NONE) */
    const void *zeros_row;   /* fp16 [M]   per-token zero-points         (ASYM, ASYM_DUAL)    */
    const void *scale_col_1; /* fp16 [N]   per-output-channel scales                           */
    const void *zeros_col_1; /* fp16 [N]                                 (ASYM, ASYM_DUAL)    */
    const void *scale_col_2; /* fp16 [N]                                 (SYM_DUAL, ASYM_DUAL) */
    const void *zeros_col_2; /* fp16 [N]                                 (ASYM_DUAL)          */
    const void *bias;        /* fp16 [N] or NULL; added last as a separate fp16 add
                                (ref: qlinear4bit/nn/linear.py:53-54)                          */
    uint32_t ldo;            /* row stride of `out` in elements; 0 means N */
    /* Fused all-gather for N-sharded layers (optional, no reference counterpart): with
     * n_out_peers > 0 the kernel stores every output element into EACH of out_peers[0..n) at the
     * offset it would use in `out` (which is then ignored and may be NULL). The pointers are
     * device addresses valid on the launching GPU: its own buffer and peer-mapped buffers of the
     * other ranks (CUDA IPC / VMM / torch symmetric memory), all [M, ldo] with identical layout;
     * point each at this shard's first column. Plain st.global over NVLink; the caller
     * synchronises the ranks before anyone reads the gathered result. */
    uint32_t n_out_peers;
    void *out_peers[8];
    /* Optional hint for chains of small-M (M <= 16) layers: device pointer and size of the packed
     * weights the NEXT launch on this stream will read. The kernel asks the L2 cache to fetch part of
     * that range while its own last CTAs drain, so the next layer does not start on a cold memory
     * pipe. Purely a performance hint: the bytes are never read or written by this launch, results
     * do not depend on it. NULL / 0 = none. Ignored by the tensor-core kernels. */
    const void *next_weights;
    uint64_t next_weights_bytes;
    /* Fused all-gather through the NVLink switch (optional, with n_out_peers > 0): the MULTICAST address
     * of the same [M, ldo] result buffer (an NVLS multicast mapping that spans all ranks, as CUDA's
     * multicast objects / torch symmetric memory provide), pointing at this shard's first column like the
     * out_peers entries. Full 16-byte row segments then leave the GPU ONCE (multimem.st) and the switch
     * replicates them into every rank's buffer, instead of one store per peer; ragged edges still go
     * through out_peers. NULL = plain peer stores. Tensor-core kernels only. */
    void *out_multicast;
    /* K-sharded ("row-parallel") layers (optional, no reference counterpart): every rank computes int32 PARTIAL
     * accumulators over its K slice; with n_acc_owners > 0 the tensor-core kernel stores the partial of row m
     * into the buffer of the rank that owns row m -- acc_owners[m / acc_rows_per_owner], an int32 array
     * [n_acc_owners][acc_rows_per_owner][N] (peer-mapped like out_peers, 16-byte aligned, N % 4 == 0), slab
     * acc_slot = this rank -- instead of `acc_out`, with mode DUQ4_MODE_NONE. The owner then adds the slabs and
     * dequantizes once (duq4_reduce_dequant_gather). Plain st.global over NVLink. */
    uint32_t n_acc_owners;
    uint32_t acc_rows_per_owner;
    uint32_t acc_slot;
    int32_t *acc_owners[8];
    /* Row routing of the fused gather (optional, with n_out_peers > 0): 0 = every row goes to every buffer of
     * out_peers (the replicated result above). R > 0 = row m of this call is stored ONLY into
     * out_peers[m / R] (n_out_peers * R >= M): after all ranks' launches, buffer o holds rows [o*R, (o+1)*R) of the
     * full-width result and nothing else -- an all-to-all written by the epilogue, which is what a job needs whose
     * result leaves the GPUs again (each rank downloads the contiguous rows it owns; see
     * duq4_linear_w4a4_from_fp16_to_host_rows). out_multicast must be NULL. */
    uint32_t out_rows_per_owner;
} duq4_epilogue;

/* out[M,N] fp16 = dequant(A[M,K/2] x W[N,K/2]^T) (+ bias); replaces the three launches
 * matmul + *_dequant + bias add of the reference's module forwards
 * (ref: qlinear4bit/nn/linear.py:42-56, :104-115, :167-176, :239-250;
 *  src/module/linear.cu:108-153, :200-246). `acc_out` (int32 [M,N], row stride N) is
 * optional and receives the exact accumulators. M <= 16 runs the HBM-bound small-M
 * kernel, larger M the tcgen05 tensor-core kernel. K % 64 == 0. */
int duq4_linear_w4a4(const uint8_t *A, const uint8_t *W, uint32_t M, uint32_t N, uint32_t K,
                     const duq4_epilogue *epi, void *out, int32_t *acc_out, void *stream);

/* Same layer with the activations given as the int8 buffer written by duq4_quantize_fused_i8
 * (always the tensor-core kernel, any M >= 1). Results are identical to duq4_linear_w4a4 on
 * the packed codes of the same activations. */
int duq4_linear_w4a4_preunpacked(const int8_t *A_i8, const uint8_t *W, uint32_t M, uint32_t N,
                                 uint32_t K, const duq4_epilogue *epi, void *out, int32_t *acc_out,
                                 void *stream);

/* Weight pre-layout (optional, no reference counterpart: a one-off int8 pre-unpack of W):
 * duq4_weight_prelayout_i8 turns packed weights W [N, K/2] into W_i8 [N, K] in the tensor-core-ready form of
 * duq4_quantize_fused_i8 (int8 = 16 * code, K permuted inside 128-blocks; K % 128 == 0; twice the bytes), once per
 * weight tensor. duq4_linear_w4a4_prelaid then runs the layer with BOTH operands in that form on the CTA-pair
 * tensor-core kernel with no in-kernel unpack (any M >= 1; DUQ4_ERR_DEVICE where CTA pairs cannot be scheduled).
 * Results are identical to duq4_linear_w4a4_preunpacked on the packed weights. The packed format stays the
 * format of record (state_dict); a caller derives W_i8 lazily and keeps it beside the packed tensor.
 * split_scratch (optional; NULL / 0 = none): device memory, 256-byte aligned, duq4_gemm_split_scratch_bytes()
 * bytes. With it, a launch whose tile count leaves a partly filled last round on the GPU's CTA pairs splits
 * those tiles along K over the idle pairs (int32 partial tiles meet in the scratch and are added before the
 * dequant -- exact, so the results do not change); without it every tile is computed by one pair. The call
 * clears the few bytes it needs to start from zero; calls sharing one scratch must not overlap on the GPU. */
int duq4_weight_prelayout_i8(const uint8_t *W, uint32_t N, uint32_t K, int8_t *W_i8, void *stream);
size_t duq4_gemm_split_scratch_bytes(void);
int duq4_linear_w4a4_prelaid(const int8_t *A_i8, const int8_t *W_i8, uint32_t M, uint32_t N, uint32_t K,
                             const duq4_epilogue *epi, void *out, int32_t *acc_out, void *split_scratch,
                             size_t split_scratch_bytes, void *stream);
/* duq4_linear_w4a4_from_fp16 on pre-laid-out weights: fused quantizer (tensor-core-ready int8 codes into the
 * workspace) + duq4_linear_w4a4_prelaid; the route for layers that see many tokens at a time (prefill). Same
 * arguments and results as duq4_linear_w4a4_from_fp16 except that W_i8 is the output of duq4_weight_prelayout_i8
 * and K % 128 == 0, and the workspace need is duq4_linear_from_fp16_prelaid_workspace_bytes(M, K): codes and
 * per-token vectors plus about 19 MiB in which the kernel splits the last, partly filled round of tiles along K
 * (partial int32 tiles of up to 74 CTA pairs), so that a launch whose tile count is just above a multiple of the
 * pair count does not pay a whole extra round. */
size_t duq4_linear_from_fp16_prelaid_workspace_bytes(uint32_t M, uint32_t K);
int duq4_linear_w4a4_from_fp16_prelaid(const void *x, const int8_t *W_i8, uint32_t M, uint32_t N, uint32_t K, int act_mode,
                                       float clip_ratio, const duq4_epilogue *epi, void *out, void *workspace,
                                       size_t workspace_bytes, void *stream);

/* Batched form: A [batch,M,K/2], W [batch,N,K/2], out [batch,M,N]; the epilogue's row
 * vectors are [batch,M] and its column vectors [batch,N] (the layout of the reference's
 * asym_batch_dequant, src/kernels/quant.cu:211-218). */
int duq4_linear_w4a4_batched(const uint8_t *A, const uint8_t *W, uint32_t M, uint32_t N,
                             uint32_t K, uint32_t batch_count, const duq4_epilogue *epi,
                             void *out, int32_t *acc_out, void *stream);

/* Bytes of caller-provided scratch duq4_linear_w4a4_from_fp16 needs for [M,K] tokens. */
size_t duq4_linear_from_fp16_workspace_bytes(uint32_t M, uint32_t K);

/* x fp16 [M,K] -> per-token quantize (act_mode: DUQ4_MODE_*, scales computed on the fly
 * as in the fused quantizers) -> GEMM -> dequant. epi->scale_row / zeros_row are ignored
 * and replaced by the computed ones, which live in `workspace` (256-byte aligned, at
 * least duq4_linear_from_fp16_workspace_bytes(M,K)). For ASYM_DUAL/SYM_DUAL activation
 * modes the epilogue uses set 1 of the computed row scales, as the reference modules do
 * (they only ever carry one row-scale vector, qlinear4bit/tools/tensor_utils.py:20-27).
 * Launches: ONE token runs as a single kernel -- each CTA of the weight-streaming kernel quantizes the token into
 * its own shared memory once its first weight loads are in flight, and the workspace is left untouched (K up to
 * about 38000). Everything else is two launches (fused quantizer into the workspace, then the linear kernel); for
 * up to 16 tokens the quantizer is launched with programmatic stream serialization, so it is already resident
 * when the stream's previous kernel ends, and -- with duq4_set_static_weights(1) -- the linear kernel streams its
 * first weights while the quantizer runs. The results do not depend on which route is taken. */
int duq4_linear_w4a4_from_fp16(const void *x, const uint8_t *W, uint32_t M, uint32_t N,
                               uint32_t K, int act_mode, float clip_ratio,
                               const duq4_epilogue *epi, void *out, void *workspace,
                               size_t workspace_bytes, void *stream);

/* Capacity of the scratch array built into the library (2 MiB per GPU that loads it). */
#define DUQ4_STATIC_SCRATCH_BYTES (2u << 20)

/* duq4_linear_w4a4_from_fp16 for callers that have no device memory to lend and may not
 * allocate any: it takes no workspace argument and makes no allocation of any kind (no
 * cudaMalloc/cudaFree, no pooled or library allocator, no host heap: the TMA descriptors of the
 * call are encoded on the stack and the descriptor cache is neither consulted nor extended, on
 * every kernel the call can route to). Typical callers: a
 * plugin running inside a serving process whose allocator has already claimed the whole GPU
 * (a cudaMalloc there fails or stalls the device), code on a latency path where an allocation's
 * implicit device synchronisation is not acceptable, and small embedders that only own their
 * input and output tensors. This entry point has NO counterpart in the reference project.
 *
 * The intermediate (activation codes + per-token scales / zero-points) lives in a fixed array
 * inside the library image, DUQ4_STATIC_SCRATCH_BYTES per GPU, resident on every GPU that loads
 * the library until the process exits. Consequences:
 *   - size limit: duq4_linear_from_fp16_workspace_bytes(M, K) must not exceed
 *     DUQ4_STATIC_SCRATCH_BYTES (all M <= 16 decode shapes up to K = 131008 fit; e.g. M = 256 at
 *     K = 8192 is just over). Larger problems are rejected with DUQ4_ERR_TOO_LARGE before any
 *     launch; use duq4_linear_w4a4_from_fp16 with your own workspace for those.
 *   - one array per GPU shared by ALL calls: two calls that can overlap on the same GPU
 *     (different streams, or different host threads without ordering) race on it and produce
 *     garbage. Serialise them on one stream or with events.
 *   - the array keeps whatever the previous call left; every byte a call reads is written by
 *     that same call first, so no clearing is needed between calls.
 *   - the first call on each GPU looks up the array's device address (cudaGetSymbolAddress, with
 *     that GPU current) and remembers it; make that first call outside any stream capture.
 * Arguments, modes, results and status codes otherwise equal duq4_linear_w4a4_from_fp16. */
int duq4_linear_w4a4_from_fp16_static(const void *x, const uint8_t *W, uint32_t M, uint32_t N,
                                      uint32_t K, int act_mode, float clip_ratio,
                                      const duq4_epilogue *epi, void *out, void *stream);

/* SiLU-gated gate/up projection of an MLP in one launch: W packed [2*inter, K/2] holds the gate rows
 * followed by the up rows (the fused weight a user of the reference builds by concatenating the two
 * Linear4bit weights), per-channel vectors of `epi` have 2*inter entries in the same order, and
 *     h_out[m, j] = half( half(silu(g[m, j])) * u[m, j] ),   g = layer output column j, u = column inter + j,
 * i.e. exactly what `F.silu(y[:, :inter]) * y[:, inter:]` gives on the fp16 output y of
 * duq4_linear_w4a4 -- but y is never written: the CTA pair computing a tile loads one half of its
 * W block from the gate rows and the other from the up rows, and the epilogue combines them.
 * A: activations, packed int4 [M, K/2] (a_is_int8 = 0) or the tensor-core-ready int8 [M, K] of
 * duq4_quantize_fused_i8 (a_is_int8 = 1). epi->mode: DUQ4_MODE_SYM or DUQ4_MODE_ASYM (the dual
 * schemes select by output column and are rejected); epi->scale_row (/zeros_row) per token;
 * epi->ldo = row pitch of h_out (0 = inter). Needs a device that co-schedules CTA pairs
 * (DUQ4_ERR_DEVICE otherwise). No reference counterpart: the reference has Linear modules only
 * (qlinear4bit/nn/linear.py), an MLP is composed by its user. */
int duq4_linear_w4a4_gate_up_silu(const void *A, int a_is_int8, const uint8_t *W, uint32_t M,
                                  uint32_t inter, uint32_t K, const duq4_epilogue *epi,
                                  void *h_out, void *stream);

/* The same on pre-laid-out weights: W_i8 int8 [2*inter, K] = duq4_weight_prelayout_i8 of the fused gate/up weight,
 * A_i8 the tensor-core-ready activations; K % 128 == 0. Same results. */
int duq4_linear_w4a4_gate_up_silu_prelaid(const int8_t *A_i8, const int8_t *W_i8, uint32_t M, uint32_t inter, uint32_t K,
                                          const duq4_epilogue *epi, void *h_out, void *stream);

/* The same layer with the activations and the result in HOST memory (what a caller holds when
 * the reference module is fed from the CPU side; ref: src/module/linear.cu:108-153 moves nothing
 * itself, torch's .to(device) / .cpu() around it do). x_host [M, K] fp16 and out_host
 * [M, epi->ldo or N] fp16 are host pointers -- page-locked memory lets the copies overlap the
 * arithmetic, pageable memory works but serialises. W and the per-channel vectors of `epi` are
 * device pointers as everywhere else; epi->n_out_peers must be 0. The tokens are cut into chunks
 * of `chunk_rows` rows (0 = about a sixteenth of M; rounded up to a multiple of 256, at most 64
 * chunks) and upload, quantize + GEMM + dequant, and download of successive chunks run on three
 * streams; the helper streams fork from `stream` at entry and join it at the end, so later work
 * on `stream` sees out_host complete. `staging` is DEVICE memory, 256-byte aligned, of at least
 * duq4_linear_host_staging_bytes(M, N, K, chunk_rows) bytes (device copies of x and of the
 * result plus one chunk's quantizer scratch). Results equal duq4_linear_w4a4_from_fp16 bit for
 * bit (chunking by rows changes nothing: every stage is per token). No reference counterpart. */
size_t duq4_linear_host_staging_bytes(uint32_t M, uint32_t N, uint32_t K, uint32_t chunk_rows);
int duq4_linear_w4a4_from_fp16_host(const void *x_host, const uint8_t *W, uint32_t M, uint32_t N,
                                    uint32_t K, int act_mode, float clip_ratio,
                                    const duq4_epilogue *epi, void *out_host, uint32_t chunk_rows,
                                    void *staging, size_t staging_bytes, void *stream);

/* Relatives of the host-buffer entry point, same chunked pipeline (no reference counterpart). W is the packed
 * weight tensor (w_is_prelaid = 0) or the int8 re-layout of duq4_weight_prelayout_i8 (w_is_prelaid != 0).
 * `staging`: device memory, 256-byte aligned, duq4_linear_pipeline_staging_bytes(to_host, w_is_prelaid, M, N, K,
 * chunk_rows) bytes.
 *   _to_host : x fp16 [M, K] is already on the DEVICE (e.g. each rank uploaded a row slice of a host-resident
 *              input and the slices were all-gathered over NVLink), the result goes to HOST memory out_host
 *              [M, epi->ldo or N]; the arithmetic of a chunk overlaps the download of the previous one.
 *   _to_peers: N-sharded layer with a replicated result. epi->out_peers[0..n) are every rank's [M, epi->ldo]
 *              device buffers at this shard's first column (as for the fused all-gather) and self_index names
 *              the entry that is this rank's own buffer. The GEMM of a chunk writes the block into the OWN
 *              buffer; copy engines then push the chunk to the other ranks (2-D peer copies on one helper
 *              stream per peer) while the next chunk is computed. epi->out_multicast is ignored. The caller
 *              brackets the call with duq4_peer_barrier as for the fused all-gather. */
size_t duq4_linear_pipeline_staging_bytes(int to_host, int w_is_prelaid, uint32_t M, uint32_t N, uint32_t K, uint32_t chunk_rows);
int duq4_linear_w4a4_from_fp16_to_host(const void *x, const void *W, int w_is_prelaid, uint32_t M, uint32_t N, uint32_t K,
                                       int act_mode, float clip_ratio, const duq4_epilogue *epi, void *out_host,
                                       uint32_t chunk_rows, void *staging, size_t staging_bytes, void *stream);
int duq4_linear_w4a4_from_fp16_to_peers(const void *x, const void *W, int w_is_prelaid, uint32_t M, uint32_t N, uint32_t K,
                                        int act_mode, float clip_ratio, const duq4_epilogue *epi, uint32_t self_index,
                                        uint32_t chunk_rows, void *staging, size_t staging_bytes, void *stream);

/* N-sharded layer whose activations are on the device and whose ONE result [M, epi->ldo] lives in HOST memory
 * that every rank can write (no reference counterpart). Rank `self_index` of G = epi->n_out_peers holds the
 * weights of columns [col_begin, col_begin + N) (N may be 0: the rank then only takes part in the exchange).
 * epi->out_peers[i] is row 0, column 0 of rank i's [M, epi->ldo] device exchange buffer (peer-mapped, as for the
 * fused all-gather; epi->ldo is the full width and must be given; out_multicast NULL). Per row chunk: quantize +
 * GEMM + dequant, whose epilogue stores row m only into the buffer of the rank that owns it (1/G of the chunk's
 * rows each, out_rows_per_owner) -- the column blocks cross NVLink instead of interleaving on the host --, a rank
 * barrier (duq4_peer_barrier on `barrier_flags`, epochs *barrier_epoch + 1 ... ; the last epoch used is written
 * back), then the download of the contiguous full-width rows this rank owns into out_host, overlapped with the
 * next chunk. Every rank calls it with the same M, K, epi->ldo, chunk_rows. The call joins its helper stream
 * into `stream` before it returns; the host result is complete when every rank's stream has finished.
 * `staging`: duq4_linear_pipeline_staging_bytes(0, w_is_prelaid, M, N, K, chunk_rows) bytes of device memory.
 * Same bits as the unsharded layer. A rank whose barrier wait runs out records status 301. */
int duq4_linear_w4a4_from_fp16_to_host_rows(const void *x, const void *W, int w_is_prelaid, uint32_t M, uint32_t N, uint32_t K,
                                            int act_mode, float clip_ratio, const duq4_epilogue *epi, uint32_t col_begin,
                                            uint32_t self_index, const void *const *barrier_flags, uint64_t *barrier_epoch,
                                            uint64_t barrier_timeout_ns, void *out_host, uint32_t chunk_rows, void *staging,
                                            size_t staging_bytes, void *stream);

/* ---- K-sharded (row-parallel) layer: pieces of one fused forward per rank (no reference counterpart) ----
 * The column-parallel gate/up projection of a tensor-parallel MLP leaves each rank with its own K slice of the
 * down projection's input. Bit-exactness with the unsharded layer: row statistics are exact reductions, the GEMM is
 * an exact integer contraction, and ONE dequant runs on the summed accumulators.
 *   duq4_row_stats             per-token statistics of this rank's slice x [rows, cols]: DUQ4_MODE_SYM -> stat_a =
 *                              max|x| ; DUQ4_MODE_ASYM -> stat_a = min, stat_b = max (fp16 [rows]; NaNs skipped as
 *                              in the fused quantizers). The caller reduces them over the ranks (max / min).
 *   duq4_quantize_i8_from_stats  the fused quantizer with the statistics GIVEN (the reduced ones): scale (and
 *                              zero-point) by the quantizer modules' formulas, codes of the slice as
 *                              tensor-core-ready int8 (see duq4_quantize_fused_i8); writes scale_out / zeros_out.
 *                              cols == 0 (a rank without a K slice) only derives the per-token terms.
 *   (GEMM)                     duq4_linear_w4a4_preunpacked / _prelaid with epi->mode = DUQ4_MODE_NONE and
 *                              epi->acc_owners: partial accumulators to the owners of the row blocks.
 *   duq4_reduce_dequant_gather after a rank barrier: this rank adds the n_slabs partial slabs of the rows it owns
 *                              ([n_slabs][rows_owned_max][N] int32, its own acc_owners buffer), dequantizes
 *                              (epi->mode, scale_row / zeros_row indexed by GLOBAL row, per-channel vectors, bias)
 *                              rows [row0, row0 + rows) and stores the fp16 result into every buffer of
 *                              epi->out_peers ([M, epi->ldo], n_out_peers >= 1) or into `out`. */
int duq4_row_stats(int mode, const void *x, uint32_t rows, uint32_t cols, void *stat_a, void *stat_b, void *stream);
int duq4_quantize_i8_from_stats(int mode, const void *x, uint32_t rows, uint32_t cols, const void *stat_a, const void *stat_b,
                                float clip_ratio, int8_t *q_i8, void *scale_out, void *zeros_out, void *stream);
int duq4_reduce_dequant_gather(const int32_t *slabs, uint32_t n_slabs, uint32_t rows_per_slab, uint32_t row0, uint32_t rows,
                               uint32_t N, const duq4_epilogue *epi, void *out, void *stream);

/* Device-side barrier across the ranks of an N-sharded layer, on `stream` (no reference counterpart; it
 * brackets the fused all-gather: "everybody has consumed the previous result" / "everybody's block has
 * landed"). flag_ptrs: HOST array of `world` device addresses, entry r = rank r's flag array of `world`
 * uint64 slots, zero-initialised, mapped into this process (its own and peer-mapped, like out_peers).
 * The kernel makes this rank's earlier work on the stream visible system-wide, writes `epoch` into slot
 * [rank] of every rank's array and waits until its own slots all hold a value >= epoch. `epoch` must grow
 * by one per barrier (start at 1; all ranks count alike). The wait is BOUNDED: after timeout_ns (0 = one
 * second) the kernel gives up, records code 301 in the device status word (duq4_last_device_status) and
 * returns, so a rank that never arrives costs a time-out, not a hung GPU. One launch of one CTA. */
int duq4_peer_barrier(const void *const *flag_ptrs, uint32_t world, uint32_t rank, uint64_t epoch,
                      uint64_t timeout_ns, void *stream);

/* Device-side status word of the most recent tensor-core GEMM on the current device:
 * 0 = no bounded wait expired. Reads back 4 bytes (synchronises the stream given). */
int duq4_last_device_status(void *stream, int32_t *status_out /* host pointer */);

#ifdef __cplusplus
}
#endif
#endif /* DUQ4_H_ */
