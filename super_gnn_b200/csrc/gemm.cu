// C-ABI entry points of the dense fp32 GEMM (tensor cores, fp32 accuracy by splitting every operand into
// three bf16 terms).  The kernels live in gemm_bf16x9_nt.cu / gemm_bf16x9_tn.cu; this file validates and
// dispatches.
#include "gemm_call.cuh"

using namespace sgnn;

static int check_shape(int op, int64_t M, int64_t N, int64_t K, const char *what)
{
    const int base = op & ~SGNN_GEMM_SIX_PRODUCTS;
    SGNN_REQUIRE(base == SGNN_GEMM_NT || base == SGNN_GEMM_TN, SGNN_ERR_INVALID_ARGUMENT,
                 "%s: op must be SGNN_GEMM_NT or SGNN_GEMM_TN, optionally or-ed with SGNN_GEMM_SIX_PRODUCTS", what);
    SGNN_REQUIRE(M >= 0 && N >= 0 && K > 0, SGNN_ERR_INVALID_ARGUMENT, "%s: M, N must be >= 0 and K > 0", what);
    SGNN_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31), SGNN_ERR_TOO_LARGE, "%s: M, N, K must be below 2^31",
                 what);
    return SGNN_OK;
}

static int dispatch(int op, const GemmCall &c, size_t *query)
{
    const bool six = (op & SGNN_GEMM_SIX_PRODUCTS) != 0;
    if ((op & ~SGNN_GEMM_SIX_PRODUCTS) == SGNN_GEMM_NT) return six ? gemm_bf16x6_nt(c, query) : gemm_bf16x9_nt(c, query);
    return six ? gemm_bf16x6_tn(c, query) : gemm_bf16x9_tn(c, query);
}

extern "C" SGNN_API int sgnn_gemm_f32_workspace_bytes(int op, int64_t M, int64_t N, int64_t K, size_t *bytes)
{
    int rc = check_shape(op, M, N, K, "sgnn_gemm_f32_workspace_bytes");
    if (rc) return rc;
    SGNN_REQUIRE(bytes != nullptr, SGNN_ERR_INVALID_ARGUMENT, "sgnn_gemm_f32_workspace_bytes: null result pointer");
    *bytes = 0;
    if (M == 0 || N == 0) return SGNN_OK;
    // the leading dimensions do not enter the size: pass the packed ones
    const bool nt = (op & ~SGNN_GEMM_SIX_PRODUCTS) == SGNN_GEMM_NT;
    GemmCall c{nullptr, nt ? K : M, nullptr, nt ? K : N, nullptr, N, (int)M, (int)N, (int)K, 0.f, nullptr, 0, nullptr};
    return dispatch(op, c, bytes);
}

extern "C" SGNN_API int sgnn_gemm_f32(int op, const float *d_A, int64_t lda, const float *d_B, int64_t ldb, float *d_C,
                                      int64_t ldc, int64_t M, int64_t N, int64_t K, float beta, void *d_workspace,
                                      size_t workspace_bytes, void *stream)
{
    int rc = check_shape(op, M, N, K, "sgnn_gemm_f32");
    if (rc) return rc;
    if (M == 0 || N == 0) return SGNN_OK;
    SGNN_REQUIRE(d_A && d_B && d_C, SGNN_ERR_INVALID_ARGUMENT, "sgnn_gemm_f32: null pointer");
    const bool nt = (op & ~SGNN_GEMM_SIX_PRODUCTS) == SGNN_GEMM_NT;
    const int64_t min_lda = nt ? K : M, min_ldb = nt ? K : N;
    SGNN_REQUIRE(lda >= min_lda && ldb >= min_ldb && ldc >= N, SGNN_ERR_INVALID_ARGUMENT,
                 "sgnn_gemm_f32: leading dimension shorter than a row (lda=%lld ldb=%lld ldc=%lld)", (long long)lda,
                 (long long)ldb, (long long)ldc);
    SGNN_REQUIRE(lda % 4 == 0 && ldb % 4 == 0 && ldc % 4 == 0 && aligned16(d_A) && aligned16(d_B) && aligned16(d_C),
                 SGNN_ERR_INVALID_ARGUMENT, "sgnn_gemm_f32: rows must start on 16-byte boundaries");
    SGNN_REQUIRE(beta == beta, SGNN_ERR_INVALID_ARGUMENT, "sgnn_gemm_f32: beta is NaN");
    GemmCall c{d_A, lda, d_B, ldb, d_C, ldc, (int)M, (int)N, (int)K, beta, d_workspace, workspace_bytes, (cudaStream_t)stream};
    return dispatch(op, c, nullptr);
}
