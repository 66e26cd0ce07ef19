// CSR transpose on the device (set-up code, run once per matrix): CSR of A^T with rows in
// ascending order inside every column.  A stable radix sort of the nonzeros by column does
// the permutation (CUB, from the CUDA toolkit); the histogram, the row expansion and the
// gather of the permuted values are small kernels of our own.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include "common.cuh"

namespace sgnn {

constexpr int kTrThreads = 256;

// A column index outside [0, K) (malformed input) is skipped instead of counted: it would land outside `counts`.
__global__ void tr_histogram_kernel(const int *__restrict__ col, int64_t nnz, int64_t K,
                                    unsigned long long *__restrict__ counts)
{
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < nnz; e += (int64_t)gridDim.x * blockDim.x) {
        const unsigned c = (unsigned)col[e];
        if ((int64_t)c < K) atomicAdd(counts + c, 1ULL);
    }
}

// row id of every nonzero and the identity permutation
__global__ void tr_expand_rows_kernel(const int64_t *__restrict__ rowptr, int64_t M, int *__restrict__ row_of,
                                      int *__restrict__ perm)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = (int64_t)gridDim.x * (kTrThreads / 32);
    for (int64_t r = (int64_t)blockIdx.x * (kTrThreads / 32) + (threadIdx.x >> 5); r < M; r += warps_total) {
        const int64_t b = rowptr[r], e = rowptr[r + 1];
        for (int64_t i = b + lane; i < e; i += 32) {
            row_of[i] = (int)r;
            perm[i] = (int)i;
        }
    }
}

__global__ void tr_permute_kernel(const int *__restrict__ perm, const int *__restrict__ row_of,
                                  const float *__restrict__ val, int64_t nnz, int *__restrict__ row_T,
                                  float *__restrict__ val_T)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nnz; i += (int64_t)gridDim.x * blockDim.x) {
        const int p = perm[i];
        row_T[i] = row_of[p];
        if (val) val_T[i] = val[p];
    }
}

static size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

struct TrLayout {
    size_t keys_out, perm_in, perm_out, row_of, counts, cub, total;
    size_t cub_bytes;
};

static int tr_layout(int64_t K, int64_t nnz, TrLayout &L)
{
    size_t sort_bytes = 0, scan_bytes = 0;
    int end_bit = 1;
    while (end_bit < 32 && ((int64_t)1 << end_bit) < K) ++end_bit;
    cudaError_t e = cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, (const int *)nullptr, (int *)nullptr,
                                                    (const int *)nullptr, (int *)nullptr, nnz, 0, end_bit);
    if (e != cudaSuccess) return SGNN_ERR_CUDA;
    e = cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, (const unsigned long long *)nullptr,
                                      (unsigned long long *)nullptr, K + 1);
    if (e != cudaSuccess) return SGNN_ERR_CUDA;
    L.cub_bytes = sort_bytes > scan_bytes ? sort_bytes : scan_bytes;
    size_t o = 0;
    L.keys_out = o; o += align_up((size_t)nnz * 4);
    L.perm_in = o; o += align_up((size_t)nnz * 4);
    L.perm_out = o; o += align_up((size_t)nnz * 4);
    L.row_of = o; o += align_up((size_t)nnz * 4);
    L.counts = o; o += align_up((size_t)(K + 1) * 8);
    L.cub = o; o += align_up(L.cub_bytes);
    L.total = o + 256;
    return SGNN_OK;
}

}  // namespace sgnn

using namespace sgnn;

extern "C" SGNN_API size_t sgnn_csr_transpose_workspace_bytes(int64_t M, int64_t K, int64_t nnz)
{
    (void)M;
    if (K < 0 || nnz < 0 || nnz > 2147483647LL) return 0;
    TrLayout L;
    if (tr_layout(K, nnz, L) != SGNN_OK) return 0;
    return L.total;
}

extern "C" SGNN_API int sgnn_csr_transpose(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val, int64_t M,
                                  int64_t K, int64_t nnz, int64_t *d_colptr, int32_t *d_row_T, float *d_val_T,
                                  void *d_workspace, size_t workspace_bytes, void *stream)
{
    SGNN_REQUIRE(M >= 0 && K >= 0 && nnz >= 0, SGNN_ERR_INVALID_ARGUMENT, "csr_transpose: negative size");
    SGNN_REQUIRE(nnz <= 2147483647LL && M <= 2147483647LL && K <= 2147483647LL, SGNN_ERR_TOO_LARGE,
                 "csr_transpose: M, K and nnz must fit int32");
    SGNN_REQUIRE(d_rowptr && d_colptr, SGNN_ERR_INVALID_ARGUMENT, "csr_transpose: null pointer");
    SGNN_REQUIRE(nnz == 0 || (d_col && d_row_T), SGNN_ERR_INVALID_ARGUMENT, "csr_transpose: null index pointer");
    SGNN_REQUIRE(d_val == nullptr || nnz == 0 || d_val_T != nullptr, SGNN_ERR_INVALID_ARGUMENT,
                 "csr_transpose: val given but val_T is null");
    SGNN_REQUIRE(nnz == 0 || K > 0, SGNN_ERR_INVALID_ARGUMENT, "csr_transpose: nonzeros but K == 0");
    cudaStream_t s = (cudaStream_t)stream;
    TrLayout L;
    SGNN_REQUIRE(tr_layout(K, nnz, L) == SGNN_OK, SGNN_ERR_CUDA, "csr_transpose: workspace query failed");
    SGNN_REQUIRE(d_workspace != nullptr && workspace_bytes >= L.total, SGNN_ERR_WORKSPACE,
                 "csr_transpose: workspace of %zu bytes needed, %zu given", L.total, workspace_bytes);
    char *ws = reinterpret_cast<char *>((reinterpret_cast<uintptr_t>(d_workspace) + 255) & ~(uintptr_t)255);
    int *keys_out = reinterpret_cast<int *>(ws + L.keys_out);
    int *perm_in = reinterpret_cast<int *>(ws + L.perm_in);
    int *perm_out = reinterpret_cast<int *>(ws + L.perm_out);
    int *row_of = reinterpret_cast<int *>(ws + L.row_of);
    unsigned long long *counts = reinterpret_cast<unsigned long long *>(ws + L.counts);
    void *cub_ws = ws + L.cub;

    const int64_t cap = (int64_t)sm_count() * 16;
    auto blocks_for = [&](int64_t n) {
        int64_t b = ceil_div(n > 0 ? n : 1, kTrThreads);
        return (unsigned)(b > cap ? cap : b);
    };
    // column histogram -> colptr (exclusive scan over K+1 entries, the last one zero)
    SGNN_CUDA_OK(cudaMemsetAsync(counts, 0, (size_t)(K + 1) * 8, s));
    if (nnz > 0) {
        tr_histogram_kernel<<<blocks_for(nnz), kTrThreads, 0, s>>>(d_col, nnz, K, counts);
        SGNN_LAUNCH_OK("tr_histogram_kernel");
    }
    size_t cb = L.cub_bytes;
    SGNN_CUDA_OK(cub::DeviceScan::ExclusiveSum(cub_ws, cb, counts, reinterpret_cast<unsigned long long *>(d_colptr),
                                               K + 1, s));
    if (nnz == 0) return SGNN_OK;
    tr_expand_rows_kernel<<<blocks_for(M * 32), kTrThreads, 0, s>>>(d_rowptr, M, row_of, perm_in);
    SGNN_LAUNCH_OK("tr_expand_rows_kernel");
    int end_bit = 1;
    while (end_bit < 32 && ((int64_t)1 << end_bit) < K) ++end_bit;
    cb = L.cub_bytes;
    SGNN_CUDA_OK(cub::DeviceRadixSort::SortPairs(cub_ws, cb, d_col, keys_out, perm_in, perm_out, nnz, 0, end_bit, s));
    tr_permute_kernel<<<blocks_for(nnz), kTrThreads, 0, s>>>(perm_out, row_of, d_val, nnz, d_row_T, d_val_T);
    SGNN_LAUNCH_OK("tr_permute_kernel");
    return SGNN_OK;
}

// ---------------------------------------------------------------------------
// Transpose without any allocation.  The scratch lives in a static device array, so this
// entry point can serve callers that must not allocate: a process whose whole device memory
// is owned by a framework's pool (nothing left for a raw cudaMalloc), or a real-time loop in
// which an allocation (an implicit device synchronisation) is not acceptable.
// ---------------------------------------------------------------------------
namespace sgnn {

constexpr size_t kStaticScratchBytes = 48u << 20;  // 48 MiB, held by every GPU that loads the library
static __device__ __align__(256) unsigned char g_transpose_scratch[kStaticScratchBytes];

// Device address of the scratch on each device.  In host code `g_transpose_scratch` is only a
// stand-in for the symbol, not a device address; the address is asked for once per device.
static void *g_scratch_addr[64] = {nullptr};

static int static_scratch(void **out)
{
    int dev = 0;
    SGNN_CUDA_OK(cudaGetDevice(&dev));
    SGNN_REQUIRE(dev >= 0 && dev < 64, SGNN_ERR_UNSUPPORTED, "csr_transpose_noalloc: device index %d not supported", dev);
    if (g_scratch_addr[dev] == nullptr) {
        void *p = nullptr;
        SGNN_CUDA_OK(cudaGetSymbolAddress(&p, g_transpose_scratch));
        SGNN_REQUIRE(p != nullptr, SGNN_ERR_CUDA, "csr_transpose_noalloc: no device address for the static scratch");
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return SGNN_OK;
}

}  // namespace sgnn

extern "C" SGNN_API int sgnn_csr_transpose_noalloc(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val,
                                                   int64_t M, int64_t K, int64_t nnz, int64_t *d_colptr,
                                                   int32_t *d_row_T, float *d_val_T, void *stream)
{
    SGNN_REQUIRE(M >= 0 && K >= 0 && nnz >= 0, SGNN_ERR_INVALID_ARGUMENT, "csr_transpose_noalloc: negative size");
    SGNN_REQUIRE(nnz <= SGNN_TRANSPOSE_NOALLOC_MAX_NNZ, SGNN_ERR_TOO_LARGE,
                 "csr_transpose_noalloc: nnz = %lld exceeds the static scratch limit of %lld nonzeros; "
                 "use sgnn_csr_transpose with a workspace",
                 (long long)nnz, (long long)SGNN_TRANSPOSE_NOALLOC_MAX_NNZ);
    SGNN_REQUIRE(K <= SGNN_TRANSPOSE_NOALLOC_MAX_COLS, SGNN_ERR_TOO_LARGE,
                 "csr_transpose_noalloc: K = %lld exceeds the static scratch limit of %lld columns; "
                 "use sgnn_csr_transpose with a workspace",
                 (long long)K, (long long)SGNN_TRANSPOSE_NOALLOC_MAX_COLS);
    TrLayout L;
    SGNN_REQUIRE(tr_layout(K, nnz, L) == SGNN_OK, SGNN_ERR_CUDA, "csr_transpose_noalloc: workspace query failed");
    SGNN_REQUIRE(L.total <= kStaticScratchBytes, SGNN_ERR_TOO_LARGE,
                 "csr_transpose_noalloc: %zu bytes of scratch needed, %zu available", L.total, kStaticScratchBytes);
    void *scratch = nullptr;
    int rc = static_scratch(&scratch);
    if (rc != SGNN_OK) return rc;
    // the counters inside the scratch are zeroed by the transpose itself on every call
    return sgnn_csr_transpose(d_rowptr, d_col, d_val, M, K, nnz, d_colptr, d_row_T, d_val_T, scratch,
                              kStaticScratchBytes, stream);
}
