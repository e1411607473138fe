// Reference-named C++ API of the integer GEMMs: the names and signatures of
// DUQLinear4bitCUDA's include/gemm.h (lines 5-31 there) as inline wrappers over the C ABI.
// Launches go to the legacy default stream, as in the reference; failures throw
// std::runtime_error (the reference throws from CHECK_CUTLASS, include/cutools.cuh:24-29).
#pragma once
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

#include "common.h"
#include "duq4.h"

namespace duq4_detail {
inline void check_gemm(const char *fn, int status) {
    if (status != 0) throw std::runtime_error(std::string(fn) + ": " + duq4_error_string(status));
}
}  // namespace duq4_detail

// include/gemm.h:5-12 of the reference: C[M,N] = A[M,K/2 bytes] * B[N,K/2 bytes]^T, int32.
inline void matmul_host_4bit(const Int4Storage *A, const Int4Storage *B, uint32_t M, uint32_t N, uint32_t K, int32_t *C) {
    duq4_detail::check_gemm("matmul_host_4bit", duq4_matmul_4bit(A, B, M, N, K, C, nullptr));
}
// :14-21
inline void matmul_host_8bit(const int8_t *A, const int8_t *B, uint32_t M, uint32_t N, uint32_t K, int32_t *C) {
    duq4_detail::check_gemm("matmul_host_8bit", duq4_matmul_8bit(A, B, M, N, K, C, nullptr));
}
// :23-31. A, B, C are HOST arrays of `batch_count` device pointers, as the reference's
// binding builds them (src/export/bindings.cpp:59-71). The reference forwards those host arrays
// to a device kernel, which cannot work; here equally spaced problems (the only layout its
// binding produces) go out as one batched launch, anything else as one launch per problem.
inline void batch_matmul_host_4bit(const Int4Storage **A, const Int4Storage **B, uint32_t M, uint32_t N, uint32_t K,
                                   int32_t **C, uint32_t batch_count) {
    if (batch_count == 0) return;
    const size_t sa = (size_t)M * (K / 2), sb = (size_t)N * (K / 2), sc = (size_t)M * N;
    bool dense = true;
    for (uint32_t i = 1; i < batch_count && dense; ++i)
        dense = A[i] == A[0] + i * sa && B[i] == B[0] + i * sb && C[i] == C[0] + i * sc;
    if (dense) {
        duq4_detail::check_gemm("batch_matmul_host_4bit", duq4_batch_matmul_4bit(A[0], B[0], M, N, K, C[0], batch_count, nullptr));
        return;
    }
    for (uint32_t i = 0; i < batch_count; ++i)
        duq4_detail::check_gemm("batch_matmul_host_4bit", duq4_matmul_4bit(A[i], B[i], M, N, K, C[i], nullptr));
}
