// Argument block shared by the GEMM entry points and the kernel instantiations.
#pragma once
#include "common.cuh"

namespace sgnn {

// Arguments of one GEMM, C[M,N] = op(A) op(B) + beta C, as the instantiations take them.
struct GemmCall {
    const float *A;
    int64_t lda;
    const float *B;
    int64_t ldb;
    float *C;
    int64_t ldc;
    int M, N, K;
    float beta;
    void *workspace;
    size_t workspace_bytes;
    cudaStream_t stream;
};

// Defined in gemm_bf16x9_nt.cu / gemm_bf16x9_tn.cu.  `query` != nullptr: only report the workspace size.
int gemm_bf16x9_nt(const GemmCall &c, size_t *query);  // A[M,K] row-major, B[N,K] row-major
int gemm_bf16x9_tn(const GemmCall &c, size_t *query);  // A[K,M] row-major, B[K,N] row-major; split along K
// The same kernels with the six leading cross products only (SGNN_GEMM_SIX_PRODUCTS).
int gemm_bf16x6_nt(const GemmCall &c, size_t *query);
int gemm_bf16x6_tn(const GemmCall &c, size_t *query);

}  // namespace sgnn
