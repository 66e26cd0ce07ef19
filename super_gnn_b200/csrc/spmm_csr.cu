// C ABI entry points of the CSR SpMM (fp32 operand and packed wire-format operand).
#include "spmm_core.cuh"

namespace sgnn {

__global__ void csr_row_stats_kernel(const int64_t *__restrict__ rowptr, int64_t M, unsigned long long *stats)
{
    unsigned long long mx = 0, empty = 0;
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < M; r += (int64_t)gridDim.x * blockDim.x) {
        const unsigned long long d = (unsigned long long)(rowptr[r + 1] - rowptr[r]);
        mx = d > mx ? d : mx;
        empty += (d == 0);
    }
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long m2 = __shfl_xor_sync(FULL, mx, o);
        mx = m2 > mx ? m2 : mx;
        empty += __shfl_xor_sync(FULL, empty, o);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicMax(stats, mx);
        atomicAdd(stats + 1, empty);
    }
}

// Structural check of a CSR matrix on the device: counts what the SpMM kernels would trust blindly.
// flags[0]: rows whose end lies before their start; flags[1]: column indices outside [0, K);
// flags[2]: rowptr[0] != 0; flags[3]: rowptr[M] != nnz.  Counts only: nothing traps, nothing is dereferenced
// through a bad index.
__global__ void csr_check_kernel(const int64_t *__restrict__ rowptr, const int *__restrict__ col, int64_t M, int64_t K,
                                 int64_t nnz, unsigned long long *flags)
{
    unsigned long long bad_rows = 0, bad_cols = 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (int64_t r = t0; r < M; r += stride) bad_rows += (rowptr[r + 1] < rowptr[r]);
    for (int64_t e = t0; e < nnz; e += stride) bad_cols += ((unsigned long long)(unsigned)col[e] >= (unsigned long long)K) || col[e] < 0;
    for (int o = 16; o > 0; o >>= 1) {
        bad_rows += __shfl_xor_sync(FULL, bad_rows, o);
        bad_cols += __shfl_xor_sync(FULL, bad_cols, o);
    }
    if ((threadIdx.x & 31) == 0) {
        if (bad_rows) atomicAdd(flags, bad_rows);
        if (bad_cols) atomicAdd(flags + 1, bad_cols);
    }
    if (t0 == 0) {
        if (rowptr[0] != 0) atomicAdd(flags + 2, 1ULL);
        if (rowptr[M] != nnz) atomicAdd(flags + 3, 1ULL);
    }
}

static int check_csr(const int64_t *rowptr, const int32_t *col, int64_t nnz, int64_t M, int64_t K, int64_t N,
                     const float *Y, int64_t ldy)
{
    SGNN_REQUIRE(M >= 0 && K >= 0 && N >= 0 && nnz >= 0, SGNN_ERR_INVALID_ARGUMENT,
                 "spmm: negative size (M=%lld K=%lld N=%lld nnz=%lld)", (long long)M, (long long)K, (long long)N,
                 (long long)nnz);
    SGNN_REQUIRE(rowptr != nullptr, SGNN_ERR_INVALID_ARGUMENT, "spmm: rowptr is null");
    SGNN_REQUIRE(nnz == 0 || col != nullptr, SGNN_ERR_INVALID_ARGUMENT, "spmm: col is null");
    SGNN_REQUIRE(M == 0 || N == 0 || Y != nullptr, SGNN_ERR_INVALID_ARGUMENT, "spmm: Y is null");
    SGNN_REQUIRE(ldy >= N, SGNN_ERR_INVALID_ARGUMENT, "spmm: ldy (%lld) < N (%lld)", (long long)ldy, (long long)N);
    SGNN_REQUIRE(K <= 2147483647LL && N <= (1 << 24), SGNN_ERR_TOO_LARGE,
                 "spmm: K must fit int32 and N <= 2^24 (K=%lld N=%lld)", (long long)K, (long long)N);
    SGNN_REQUIRE(nnz == 0 || K > 0, SGNN_ERR_INVALID_ARGUMENT, "spmm: nonzeros but K == 0");
    return SGNN_OK;
}

}  // namespace sgnn

using namespace sgnn;

static int spmm_f32(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val, int64_t nnz,
                    const float *d_X, int64_t ldx, float *d_Y, int64_t ldy, int64_t M, int64_t K, int64_t N,
                    int accumulate, int algo, const float *d_row_scale, const float *d_col_scale, void *stream,
                    int64_t nnz_begin);

extern "C" SGNN_API int sgnn_spmm_csr_f32(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val, int64_t nnz,
                                 const float *d_X, int64_t ldx, float *d_Y, int64_t ldy, int64_t M, int64_t K,
                                 int64_t N, int accumulate, int algo, const float *d_row_scale,
                                 const float *d_col_scale, void *stream)
{
    return spmm_f32(d_rowptr, d_col, d_val, nnz, d_X, ldx, d_Y, ldy, M, K, N, accumulate, algo, d_row_scale,
                    d_col_scale, stream, 0);
}

extern "C" SGNN_API int sgnn_spmm_csr_rows_f32(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val,
                                               int64_t nnz_begin, int64_t nnz, const float *d_X, int64_t ldx,
                                               float *d_Y, int64_t ldy, int64_t M, int64_t K, int64_t N,
                                               int accumulate, int algo, const float *d_row_scale,
                                               const float *d_col_scale, void *stream)
{
    SGNN_REQUIRE(nnz_begin >= 0, SGNN_ERR_INVALID_ARGUMENT, "spmm (row range): negative nnz_begin");
    return spmm_f32(d_rowptr, d_col, d_val, nnz, d_X, ldx, d_Y, ldy, M, K, N, accumulate, algo, d_row_scale,
                    d_col_scale, stream, nnz_begin);
}

static int spmm_f32(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val, int64_t nnz,
                    const float *d_X, int64_t ldx, float *d_Y, int64_t ldy, int64_t M, int64_t K, int64_t N,
                    int accumulate, int algo, const float *d_row_scale, const float *d_col_scale, void *stream,
                    int64_t nnz_begin)
{
    int rc = check_csr(d_rowptr, d_col, nnz, M, K, N, d_Y, ldy);
    if (rc != SGNN_OK) return rc;
    SGNN_REQUIRE(nnz == 0 || N == 0 || d_X != nullptr, SGNN_ERR_INVALID_ARGUMENT, "spmm: X is null");
    SGNN_REQUIRE(ldx >= N, SGNN_ERR_INVALID_ARGUMENT, "spmm: ldx (%lld) < N (%lld)", (long long)ldx, (long long)N);
    SGNN_REQUIRE(ldx <= (1 << 30), SGNN_ERR_TOO_LARGE, "spmm: ldx must not exceed 2^30 elements");
    SGNN_REQUIRE(algo >= SGNN_SPMM_AUTO && algo <= SGNN_SPMM_NNZ_SPLIT_STAGED, SGNN_ERR_INVALID_ARGUMENT,
                 "spmm: unknown algo %d", algo);
    const bool vec4 = (N % 4 == 0) && (ldx % 4 == 0) && (ldy % 4 == 0) && aligned16(d_X) && aligned16(d_Y);
    if (d_col_scale != nullptr) {
        DenseSrcT<true, true> src{d_X, (int)ldx, d_col_scale};
        return spmm_dispatch<DenseSrcT<true, true>>(src, 0, d_rowptr, d_col, d_val, nnz, d_Y, ldy, M, N, accumulate,
                                                    algo, vec4, d_row_scale, (cudaStream_t)stream, nnz_begin);
    }
    if (d_val != nullptr) {
        DenseSrcT<true> src{d_X, (int)ldx, nullptr};
        return spmm_dispatch<DenseSrcT<true>>(src, 0, d_rowptr, d_col, d_val, nnz, d_Y, ldy, M, N, accumulate, algo,
                                              vec4, d_row_scale, (cudaStream_t)stream, nnz_begin);
    }
    DenseSrcT<false> src{d_X, (int)ldx, nullptr};
    return spmm_dispatch<DenseSrcT<false>>(src, 0, d_rowptr, d_col, d_val, nnz, d_Y, ldy, M, N, accumulate, algo, vec4,
                                           d_row_scale, (cudaStream_t)stream, nnz_begin);
}

extern "C" SGNN_API int sgnn_spmm_csr_dequant_f32(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val,
                                         int64_t nnz, const uint8_t *d_packed, const float *d_params,
                                         const uint16_t *d_params_bf16, int64_t R, int64_t F,
                                         const int32_t *d_work_range, int P, int bits, float *d_Y, int64_t ldy,
                                         int64_t M, int algo, const float *d_row_scale, void *stream)
{
    int rc = check_csr(d_rowptr, d_col, nnz, M, R, F, d_Y, ldy);
    if (rc != SGNN_OK) return rc;
    SGNN_REQUIRE(bits == 2 || bits == 4 || bits == 8, SGNN_ERR_INVALID_ARGUMENT, "spmm_dequant: bits must be 2, 4 or 8 (got %d)", bits);
    SGNN_REQUIRE(P >= 1 && P <= SGNN_MAX_PEERS, SGNN_ERR_TOO_LARGE, "spmm_dequant: P=%d outside [1, %d]", P, SGNN_MAX_PEERS);
    SGNN_REQUIRE(d_work_range != nullptr, SGNN_ERR_INVALID_ARGUMENT, "spmm_dequant: work_range is null");
    SGNN_REQUIRE((d_params != nullptr) != (d_params_bf16 != nullptr), SGNN_ERR_INVALID_ARGUMENT,
                 "spmm_dequant: give exactly one of params (fp32) and params_bf16");
    SGNN_REQUIRE(nnz == 0 || F == 0 || d_packed != nullptr, SGNN_ERR_INVALID_ARGUMENT, "spmm_dequant: packed is null");
    SGNN_REQUIRE(algo >= SGNN_SPMM_AUTO && algo <= SGNN_SPMM_NNZ_SPLIT, SGNN_ERR_INVALID_ARGUMENT,
                 "spmm_dequant: unknown algo %d", algo);
    const bool vec4 = (F % 4 == 0) && (ldy % 4 == 0) && aligned16(d_Y) &&
                      ((reinterpret_cast<uintptr_t>(d_packed) & 3u) == 0);
    SGNN_REQUIRE(R <= (1LL << 28), SGNN_ERR_TOO_LARGE, "spmm_dequant: at most 2^28 packed operand rows");
    if (d_val != nullptr) {
        PackedSrcT<true> src{d_packed, (int)F, d_params, d_params_bf16, d_work_range, P, bits};
        return spmm_dispatch<PackedSrcT<true>>(src, PackedSrcT<true>::smem_bytes(P), d_rowptr, d_col, d_val, nnz, d_Y,
                                               ldy, M, F, /*accumulate=*/1, algo, vec4, d_row_scale, (cudaStream_t)stream);
    }
    PackedSrcT<false> src{d_packed, (int)F, d_params, d_params_bf16, d_work_range, P, bits};
    return spmm_dispatch<PackedSrcT<false>>(src, PackedSrcT<false>::smem_bytes(P), d_rowptr, d_col, d_val, nnz, d_Y,
                                            ldy, M, F, /*accumulate=*/1, algo, vec4, d_row_scale, (cudaStream_t)stream);
}

template <int BITS>
static int spmm_rowcodes(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val, int64_t nnz,
                         const uint8_t *d_codes, const float *d_params, const uint16_t *d_params_bf16, int64_t F,
                         float *d_Y, int64_t ldy, int64_t M, int algo, const float *d_row_scale, cudaStream_t s)
{
    const int nv = rowcodes_nv(F);
    const int lognv = nv == 4 ? 2 : (nv == 2 ? 1 : 0);
    if (d_val != nullptr) {
        RowCodesSrcT<true, BITS> src{d_codes, (int)(F * BITS / 8), lognv, d_params, d_params_bf16};
        return spmm_dispatch<RowCodesSrcT<true, BITS>>(src, 0, d_rowptr, d_col, d_val, nnz, d_Y, ldy, M, F,
                                                       /*accumulate=*/1, algo, /*vec4=*/true, d_row_scale, s);
    }
    RowCodesSrcT<false, BITS> src{d_codes, (int)(F * BITS / 8), lognv, d_params, d_params_bf16};
    return spmm_dispatch<RowCodesSrcT<false, BITS>>(src, 0, d_rowptr, d_col, d_val, nnz, d_Y, ldy, M, F,
                                                    /*accumulate=*/1, algo, /*vec4=*/true, d_row_scale, s);
}

extern "C" SGNN_API int sgnn_spmm_csr_dequant_rowcodes_f32(const int64_t *d_rowptr, const int32_t *d_col,
                                                           const float *d_val, int64_t nnz, const uint8_t *d_codes,
                                                           const float *d_params, const uint16_t *d_params_bf16,
                                                           int64_t R, int64_t F, int bits, float *d_Y, int64_t ldy,
                                                           int64_t M, int algo, const float *d_row_scale, void *stream)
{
    int rc = check_csr(d_rowptr, d_col, nnz, M, R, F, d_Y, ldy);
    if (rc != SGNN_OK) return rc;
    SGNN_REQUIRE(bits == 2 || bits == 4 || bits == 8, SGNN_ERR_INVALID_ARGUMENT,
                 "spmm_dequant_rowcodes: bits must be 2, 4 or 8 (got %d)", bits);
    SGNN_REQUIRE((d_params != nullptr) != (d_params_bf16 != nullptr), SGNN_ERR_INVALID_ARGUMENT,
                 "spmm_dequant_rowcodes: give exactly one of params (fp32) and params_bf16");
    SGNN_REQUIRE(algo >= SGNN_SPMM_AUTO && algo <= SGNN_SPMM_NNZ_SPLIT, SGNN_ERR_INVALID_ARGUMENT,
                 "spmm_dequant_rowcodes: unknown algo %d", algo);
    if (M == 0 || F == 0 || nnz == 0) return SGNN_OK;
    SGNN_REQUIRE(rowcodes_width_ok(F), SGNN_ERR_UNSUPPORTED,
                 "spmm_dequant_rowcodes: the row-codes layout needs F %% 4 == 0 and F <= 128, F == 256 or F == 512 (F=%lld)",
                 (long long)F);
    SGNN_REQUIRE(d_codes != nullptr, SGNN_ERR_INVALID_ARGUMENT, "spmm_dequant_rowcodes: codes is null");
    SGNN_REQUIRE((ldy % 4 == 0) && aligned16(d_Y), SGNN_ERR_INVALID_ARGUMENT,
                 "spmm_dequant_rowcodes: rows of Y must be 16-byte aligned");
    SGNN_REQUIRE(reinterpret_cast<uintptr_t>(d_codes) % (size_t)(bits / 2) == 0, SGNN_ERR_INVALID_ARGUMENT,
                 "spmm_dequant_rowcodes: the code buffer must be aligned to %d bytes", bits / 2);
    SGNN_REQUIRE(R * (F * bits / 8) <= 2147483647LL * 64, SGNN_ERR_TOO_LARGE, "spmm_dequant_rowcodes: operand too large");
    cudaStream_t s = (cudaStream_t)stream;
    if (bits == 8) return spmm_rowcodes<8>(d_rowptr, d_col, d_val, nnz, d_codes, d_params, d_params_bf16, F, d_Y, ldy, M, algo, d_row_scale, s);
    if (bits == 4) return spmm_rowcodes<4>(d_rowptr, d_col, d_val, nnz, d_codes, d_params, d_params_bf16, F, d_Y, ldy, M, algo, d_row_scale, s);
    return spmm_rowcodes<2>(d_rowptr, d_col, d_val, nnz, d_codes, d_params, d_params_bf16, F, d_Y, ldy, M, algo, d_row_scale, s);
}

extern "C" SGNN_API int sgnn_csr_check(const int64_t *d_rowptr, const int32_t *d_col, int64_t M, int64_t K, int64_t nnz,
                                       int64_t *d_flags, void *stream)
{
    SGNN_REQUIRE(M >= 0 && K >= 0 && nnz >= 0, SGNN_ERR_INVALID_ARGUMENT, "csr_check: negative size");
    SGNN_REQUIRE(d_rowptr != nullptr && d_flags != nullptr, SGNN_ERR_INVALID_ARGUMENT, "csr_check: null pointer");
    SGNN_REQUIRE(nnz == 0 || d_col != nullptr, SGNN_ERR_INVALID_ARGUMENT, "csr_check: col is null");
    const int64_t work = M > nnz ? M : nnz;
    int64_t blocks = ceil_div(work > 0 ? work : 1, 256);
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    csr_check_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(d_rowptr, d_col, M, K, nnz,
                                                                          reinterpret_cast<unsigned long long *>(d_flags));
    SGNN_LAUNCH_OK("csr_check_kernel");
    return SGNN_OK;
}

extern "C" SGNN_API int sgnn_csr_row_stats(const int64_t *d_rowptr, int64_t M, int64_t *d_stats, void *stream)
{
    SGNN_REQUIRE(M >= 0, SGNN_ERR_INVALID_ARGUMENT, "row_stats: negative M");
    SGNN_REQUIRE(d_rowptr != nullptr && d_stats != nullptr, SGNN_ERR_INVALID_ARGUMENT, "row_stats: null pointer");
    if (M == 0) return SGNN_OK;
    int64_t blocks = ceil_div(M, 256);
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    csr_row_stats_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        d_rowptr, M, reinterpret_cast<unsigned long long *>(d_stats));
    SGNN_LAUNCH_OK("csr_row_stats_kernel");
    return SGNN_OK;
}
