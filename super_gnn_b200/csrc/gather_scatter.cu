// Row gather and scatter-add of boundary rows (sm_100a): pure HBM-bound row copies.
// A warp moves one row, 16 bytes per lane per step when rows are 16-byte aligned.
#include "common.cuh"

namespace sgnn {

constexpr int kGsThreads = 256;

template <bool VEC4, bool SCATTER>
__global__ void __launch_bounds__(kGsThreads)
move_rows_kernel(const float *__restrict__ src, int64_t lds, const int64_t *__restrict__ index, int64_t S, int F,
                 float *__restrict__ dst, int64_t ldd)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = (int64_t)gridDim.x * (kGsThreads / 32);
    for (int64_t r = (int64_t)blockIdx.x * (kGsThreads / 32) + (threadIdx.x >> 5); r < S; r += warps_total) {
        const int64_t i = __ldg(index + r);
        const float *s = src + (SCATTER ? r : i) * lds;
        float *d = dst + (SCATTER ? i : r) * ldd;
        if constexpr (VEC4) {
            for (int k = lane * 4; k < F; k += 128) {
                if constexpr (SCATTER) {
                    red_add_v4(d + k, ld_stream(reinterpret_cast<const float4 *>(s + k)));
                } else {
                    __stcs(reinterpret_cast<float4 *>(d + k), __ldg(reinterpret_cast<const float4 *>(s + k)));
                }
            }
        } else {
            for (int k = lane; k < F; k += 32) {
                if constexpr (SCATTER) red_add(d + k, s[k]);
                else d[k] = __ldg(s + k);
            }
        }
    }
}

template <bool SCATTER>
static int launch_move(const float *src, int64_t lds, const int64_t *index, int64_t S, int64_t F, float *dst,
                       int64_t ldd, cudaStream_t s, const char *who)
{
    SGNN_REQUIRE(S >= 0 && F >= 0, SGNN_ERR_INVALID_ARGUMENT, "%s: negative size", who);
    SGNN_REQUIRE(F <= (1 << 24), SGNN_ERR_TOO_LARGE, "%s: F <= 2^24", who);
    SGNN_REQUIRE(lds >= F && ldd >= F, SGNN_ERR_INVALID_ARGUMENT, "%s: leading dimension < F", who);
    if (S == 0 || F == 0) return SGNN_OK;
    SGNN_REQUIRE(src && index && dst, SGNN_ERR_INVALID_ARGUMENT, "%s: null pointer", who);
    int64_t blocks = ceil_div(S, kGsThreads / 32);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    const bool vec = (F % 4 == 0) && (lds % 4 == 0) && (ldd % 4 == 0) && aligned16(src) && aligned16(dst);
    if (vec)
        move_rows_kernel<true, SCATTER><<<(unsigned)blocks, kGsThreads, 0, s>>>(src, lds, index, S, (int)F, dst, ldd);
    else
        move_rows_kernel<false, SCATTER><<<(unsigned)blocks, kGsThreads, 0, s>>>(src, lds, index, S, (int)F, dst, ldd);
    SGNN_LAUNCH_OK("move_rows_kernel");
    return SGNN_OK;
}

}  // namespace sgnn

extern "C" SGNN_API int sgnn_gather_rows(const float *d_X, int64_t ldx, const int64_t *d_index, int64_t S, int64_t F,
                                float *d_out, int64_t ldo, void *stream)
{
    return sgnn::launch_move<false>(d_X, ldx, d_index, S, F, d_out, ldo, (cudaStream_t)stream, "gather_rows");
}

extern "C" SGNN_API int sgnn_scatter_add_rows(const float *d_src, int64_t lds, const int64_t *d_index, int64_t S, int64_t F,
                                     float *d_out, int64_t ldo, void *stream)
{
    return sgnn::launch_move<true>(d_src, lds, d_index, S, F, d_out, ldo, (cudaStream_t)stream, "scatter_add_rows");
}
