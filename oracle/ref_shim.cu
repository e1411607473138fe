/*
 * extern "C" shim over the reference's own host launchers, so that the test-suite can
 * call the reference CUDA kernels (compiled from the reference's sources, in place) on a
 * GPU box through ctypes. TEST INFRASTRUCTURE ONLY; built by oracle/Makefile into
 * oracle/_ref/libduq_ref.so, never linked into the product.
 *
 * Each wrapper forwards to one function of the reference's include/quant.h or
 * include/gemm.h and returns the CUDA status after a device synchronise. The reference
 * launches on the legacy default stream and reports nothing itself.
 */
#include <quant.h>
#include <gemm.h>

static int done() {
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaGetLastError();
    return (int)e;
}

extern "C" {

int ref_sym_quant(const void *x, const void *scale, uint32_t rows, uint32_t colsSrc,
                  uint32_t colsDst, void *q) {
    sym_quant_host((const half *)x, (const half *)scale, rows, colsSrc, colsDst, (Int4Storage *)q);
    return done();
}
int ref_sym_dual_quant(const void *x, const void *s1, const void *s2, uint32_t rows,
                       uint32_t colsSrc, uint32_t colsDst, void *q) {
    sym_dual_quant_host((const half *)x, (const half *)s1, (const half *)s2, rows, colsSrc, colsDst,
                        (Int4Storage *)q);
    return done();
}
int ref_asym_quant(const void *x, const void *scale, const void *zeros, uint32_t rows,
                   uint32_t colsSrc, uint32_t colsDst, void *q) {
    asym_quant_host((const half *)x, (const half *)scale, (const half *)zeros, rows, colsSrc,
                    colsDst, (Int4Storage *)q);
    return done();
}
/* The definition takes (x, s1, z1, s2, z2) while the header declares (x, s1, s2, z1, z2);
 * the types agree, so the call below binds to the definition's order. */
int ref_asym_dual_quant(const void *x, const void *s1, const void *z1, const void *s2,
                        const void *z2, uint32_t rows, uint32_t colsSrc, uint32_t colsDst, void *q) {
    asym_dual_quant_host((const half *)x, (const half *)s1, (const half *)z1, (const half *)s2,
                         (const half *)z2, rows, colsSrc, colsDst, (Int4Storage *)q);
    return done();
}
int ref_asym_quant_8bit(const float *x, const float *scale, const float *zeros, uint32_t rows,
                        uint32_t cols, int8_t *q) {
    asym_quant_host_8bit(x, scale, zeros, rows, cols, q);
    return done();
}
int ref_sym_dequant(const int32_t *q, const void *sr, const void *sc, uint32_t rows, uint32_t cols,
                    void *x) {
    sym_dequant_host(q, (const half *)sr, (const half *)sc, rows, cols, (half *)x);
    return done();
}
int ref_sym_dual_dequant(const int32_t *q, const void *sr, const void *sc1, const void *sc2,
                         uint32_t rows, uint32_t cols, void *x) {
    sym_dual_dequant_host(q, (const half *)sr, (const half *)sc1, (const half *)sc2, rows, cols,
                          (half *)x);
    return done();
}
int ref_asym_dequant(const int32_t *q, const void *sr, const void *zr, const void *sc,
                     const void *zc, uint32_t rows, uint32_t cols, void *x) {
    asym_dequant_host(q, (const half *)sr, (const half *)zr, (const half *)sc, (const half *)zc, rows,
                      cols, (half *)x);
    return done();
}
int ref_asym_dual_dequant(const int32_t *q, const void *sr, const void *zr, const void *sc1,
                          const void *zc1, const void *sc2, const void *zc2, uint32_t rows,
                          uint32_t cols, void *x) {
    asym_dual_dequant_host(q, (const half *)sr, (const half *)zr, (const half *)sc1,
                           (const half *)zc1, (const half *)sc2, (const half *)zc2, rows, cols,
                           (half *)x);
    return done();
}
int ref_asym_batch_dequant(const int32_t *q, const void *sr, const void *zr, const void *sc,
                           const void *zc, uint32_t batches, uint32_t rows, uint32_t cols, void *x) {
    asym_batch_dequant_host(q, (const half *)sr, (const half *)zr, (const half *)sc,
                            (const half *)zc, batches, rows, cols, (half *)x);
    return done();
}
int ref_asym_dequant_hprec(const int32_t *q, const float *sr, const float *zr, const float *sc,
                           const float *zc, uint32_t rows, uint32_t cols, float *x) {
    asym_dequant_host_hprec(q, sr, zr, sc, zc, rows, cols, x);
    return done();
}
int ref_matmul_4bit(const void *A, const void *B, uint32_t M, uint32_t N, uint32_t K, int32_t *C) {
    try {
        matmul_host_4bit((const Int4Storage *)A, (const Int4Storage *)B, M, N, K, C);
    } catch (...) {
        return -1;
    }
    return done();
}
int ref_matmul_8bit(const int8_t *A, const int8_t *B, uint32_t M, uint32_t N, uint32_t K,
                    int32_t *C) {
    try {
        matmul_host_8bit(A, B, M, N, K, C);
    } catch (...) {
        return -1;
    }
    return done();
}

}  // extern "C"
