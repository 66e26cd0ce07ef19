// Fused epilogue of a hidden GraphSAGE layer (sm_100a):  y = relu(LayerNorm(dropout(h + bias)))
// and its backward, one pass over the activations each way.
//
// The reference runs these as separate framework ops between two aggregations
// (examples/graphsage/sage.py:189-196: conv bias add, F.dropout, LayerNorm, F.relu), i.e. eight
// to nine full passes over an [n, hidden] matrix forward and about twelve backward.  Here a warp
// owns a row, keeps it in registers, and the forward reads h once and writes y plus two numbers per
// row (mean, reciprocal standard deviation); the backward reads grad_y and h, RECOMPUTES x_hat and
// the sign of the output from them (same operations, same roundings as the forward), and writes
// grad_h, with the column sums for the bias / gamma / beta gradients accumulated per block and
// reduced in a fixed order.  Pure HBM streaming: 2 passes forward, 3 backward, of
// n * hidden * 4 bytes each; neither x_hat nor the dropout mask is ever stored.
#include "common.cuh"

namespace sgnn {

constexpr int kEpiThreads = 256;

// Counter-based dropout bits: one 64-bit mix per (row, group of 4 columns) gives four 16-bit
// uniform numbers; element kept iff its number >= p * 65536.  Same function forward and backward,
// so the mask is never stored.
__device__ __forceinline__ uint64_t mix64(uint64_t seed, uint64_t idx)
{
    uint64_t z = seed + 0x9E3779B97F4A7C15ULL * (idx + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

// mask * 1/(1-p) for the four columns starting at c (c % 4 == 0) of row r
__device__ __forceinline__ float4 dropout_scale4(uint64_t seed, int64_t r, int c, int H, unsigned thresh, float inv_keep)
{
    const uint64_t z = mix64(seed, (uint64_t)r * (uint64_t)(H / 4) + (uint64_t)(c >> 2));
    float4 m;
    m.x = ((unsigned)(z & 0xffffu) >= thresh) ? inv_keep : 0.f;
    m.y = ((unsigned)((z >> 16) & 0xffffu) >= thresh) ? inv_keep : 0.f;
    m.z = ((unsigned)((z >> 32) & 0xffffu) >= thresh) ? inv_keep : 0.f;
    m.w = ((unsigned)((z >> 48) & 0xffffu) >= thresh) ? inv_keep : 0.f;
    return m;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
    return v;
}

// The normalised value of one element, computed the same way (same roundings, nothing contracted into an FMA
// by the compiler) in the forward and in the backward, which recomputes it instead of reading it back:
//     v = (h + bias) * mask;  x_hat = (v - mean) * rstd
__device__ __forceinline__ float pre_norm(float h, float b, float m) { return __fmul_rn(__fadd_rn(h, b), m); }
__device__ __forceinline__ float normalised(float v, float mean, float rstd) { return __fmul_rn(__fsub_rn(v, mean), rstd); }

template <int MODE>
__device__ __forceinline__ float4 mask_of(const float *__restrict__ mask, int64_t ldm, uint64_t seed, int64_t r, int c, int H,
                                          unsigned thresh, float inv_keep)
{
    if (MODE == 1) return dropout_scale4(seed, r, c, H, thresh, inv_keep);
    if (MODE == 2) return ld_stream(reinterpret_cast<const float4 *>(mask + r * ldm + c));
    return make_float4(1.f, 1.f, 1.f, 1.f);
}

// MODE: 0 = no dropout (inference or p == 0), 1 = counter-based mask, 2 = caller-supplied mask (already scaled)
template <int NV, int MODE>
__global__ void __launch_bounds__(kEpiThreads)
sage_epilogue_fwd_kernel(const float *__restrict__ h, int64_t ldh, const float *__restrict__ bias,
                         const float *__restrict__ gamma, const float *__restrict__ beta,
                         const float *__restrict__ mask, int64_t ldm, uint64_t seed, unsigned thresh, float inv_keep,
                         float eps, float *__restrict__ y, int64_t ldy, float2 *__restrict__ stats, int64_t n, int H)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = (int64_t)gridDim.x * (kEpiThreads / 32);
    float4 b[NV], g[NV], be[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane * 4 + i * 128;
        if (c < H) {
            b[i] = bias ? __ldg(reinterpret_cast<const float4 *>(bias + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
            g[i] = __ldg(reinterpret_cast<const float4 *>(gamma + c));
            be[i] = __ldg(reinterpret_cast<const float4 *>(beta + c));
        }
    }
    const float invH = 1.0f / (float)H;
    // R rows per warp and iteration.  Two rows (both rows' loads issued before the first reduction) were slower
    // than one: 1.27 against 1.11 ms per 2.4 M x 256 layer, the extra registers cost a resident block per SM.
    constexpr int R = 1;
    for (int64_t r0 = (int64_t)blockIdx.x * (kEpiThreads / 32) + (threadIdx.x >> 5); r0 < n; r0 += R * warps_total) {
        float4 d[R][NV];
        float s[R];
#pragma unroll
        for (int k = 0; k < R; ++k) {
            const int64_t r = r0 + k * warps_total;
            s[k] = 0.f;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int c = lane * 4 + i * 128;
                if (c < H && r < n) {
                    const float4 v = ld_stream(reinterpret_cast<const float4 *>(h + r * ldh + c));
                    const float4 m = mask_of<MODE>(mask, ldm, seed, r, c, H, thresh, inv_keep);
                    d[k][i].x = pre_norm(v.x, b[i].x, m.x); d[k][i].y = pre_norm(v.y, b[i].y, m.y);
                    d[k][i].z = pre_norm(v.z, b[i].z, m.z); d[k][i].w = pre_norm(v.w, b[i].w, m.w);
                    s[k] += (d[k][i].x + d[k][i].y) + (d[k][i].z + d[k][i].w);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < R; ++k) {
            const int64_t r = r0 + k * warps_total;
            if (r >= n) break;  // uniform over the warp
            const float mean = warp_sum(s[k]) * invH;
            float q = 0.f;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                if (lane * 4 + i * 128 < H) {
                    const float dx = __fsub_rn(d[k][i].x, mean), dy = __fsub_rn(d[k][i].y, mean);
                    const float dz = __fsub_rn(d[k][i].z, mean), dw = __fsub_rn(d[k][i].w, mean);
                    q += (dx * dx + dy * dy) + (dz * dz + dw * dw);
                }
            }
            const float rstd = __frsqrt_rn(warp_sum(q) * invH + eps);
            if (lane == 0) stats[r] = make_float2(mean, rstd);
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int c = lane * 4 + i * 128;
                if (c < H) {
                    float4 o;
                    o.x = fmaxf(__fmaf_rn(normalised(d[k][i].x, mean, rstd), g[i].x, be[i].x), 0.f);
                    o.y = fmaxf(__fmaf_rn(normalised(d[k][i].y, mean, rstd), g[i].y, be[i].y), 0.f);
                    o.z = fmaxf(__fmaf_rn(normalised(d[k][i].z, mean, rstd), g[i].z, be[i].z), 0.f);
                    o.w = fmaxf(__fmaf_rn(normalised(d[k][i].w, mean, rstd), g[i].w, be[i].w), 0.f);
                    __stcs(reinterpret_cast<float4 *>(y + r * ldy + c), o);
                }
            }
        }
    }
}

// partials: [gridDim.x, 3, H] = per-block column sums of (grad_z, grad_gamma, grad_beta)
template <int NV, int MODE>
__global__ void __launch_bounds__(kEpiThreads, (NV <= 2 ? 4 : 2))
sage_epilogue_bwd_kernel(const float *__restrict__ gy, int64_t ldgy, const float *__restrict__ h, int64_t ldh,
                         const float2 *__restrict__ stats, const float *__restrict__ bias,
                         const float *__restrict__ gamma, const float *__restrict__ beta,
                         const float *__restrict__ mask, int64_t ldm, uint64_t seed, unsigned thresh, float inv_keep,
                         float *__restrict__ gh, int64_t ldgh, float *__restrict__ partials, int64_t n, int H)
{
    extern __shared__ float sred[];  // [warps, 3, H] column sums, then [2, H] bias and beta
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t warps_total = (int64_t)gridDim.x * (kEpiThreads / 32);
    // Column sums (grad_z, grad_gamma, grad_beta) live in this warp's slice of shared memory, not in registers:
    // every lane only ever touches its own columns, and the registers saved double the resident warps.  Bias and
    // beta, needed once per element to recompute x_hat and the sign of the output, sit in shared memory too.
    float *mine = sred + (size_t)warp * 3 * H;
    float *sb = sred + (size_t)(kEpiThreads / 32) * 3 * H;
    float *sbe = sb + H;
    for (int k = threadIdx.x; k < H; k += kEpiThreads) {
        sb[k] = bias ? __ldg(bias + k) : 0.f;
        sbe[k] = __ldg(beta + k);
    }
    float4 g[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = lane * 4 + i * 128;
        g[i] = (c < H) ? __ldg(reinterpret_cast<const float4 *>(gamma + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < H) {
            const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4 *>(mine + c) = z;
            *reinterpret_cast<float4 *>(mine + H + c) = z;
            *reinterpret_cast<float4 *>(mine + 2 * H + c) = z;
        }
    }
    __syncthreads();
    const float invH = 1.0f / (float)H;
    for (int64_t r = (int64_t)blockIdx.x * (kEpiThreads / 32) + warp; r < n; r += warps_total) {
        float4 gx[NV], xh[NV];
        float s1 = 0.f, s2 = 0.f;
        const float2 st = __ldg(stats + r);  // (mean, rstd) of the row
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = lane * 4 + i * 128;
            if (c < H) {
                const float4 go = ld_stream(reinterpret_cast<const float4 *>(gy + r * ldgy + c));
                const float4 hv = ld_stream(reinterpret_cast<const float4 *>(h + r * ldh + c));
                const float4 b = *reinterpret_cast<const float4 *>(sb + c);
                const float4 be = *reinterpret_cast<const float4 *>(sbe + c);
                const float4 mk = mask_of<MODE>(mask, ldm, seed, r, c, H, thresh, inv_keep);
                xh[i].x = normalised(pre_norm(hv.x, b.x, mk.x), st.x, st.y);
                xh[i].y = normalised(pre_norm(hv.y, b.y, mk.y), st.x, st.y);
                xh[i].z = normalised(pre_norm(hv.z, b.z, mk.z), st.x, st.y);
                xh[i].w = normalised(pre_norm(hv.w, b.w, mk.w), st.x, st.y);
                float4 g1;  // through the relu: the output was positive iff gamma * x_hat + beta is
                g1.x = __fmaf_rn(xh[i].x, g[i].x, be.x) > 0.f ? go.x : 0.f;
                g1.y = __fmaf_rn(xh[i].y, g[i].y, be.y) > 0.f ? go.y : 0.f;
                g1.z = __fmaf_rn(xh[i].z, g[i].z, be.z) > 0.f ? go.z : 0.f;
                g1.w = __fmaf_rn(xh[i].w, g[i].w, be.w) > 0.f ? go.w : 0.f;
                float4 a = *reinterpret_cast<float4 *>(mine + H + c);
                a.x += g1.x * xh[i].x; a.y += g1.y * xh[i].y; a.z += g1.z * xh[i].z; a.w += g1.w * xh[i].w;
                *reinterpret_cast<float4 *>(mine + H + c) = a;
                float4 b2 = *reinterpret_cast<float4 *>(mine + 2 * H + c);
                b2.x += g1.x; b2.y += g1.y; b2.z += g1.z; b2.w += g1.w;
                *reinterpret_cast<float4 *>(mine + 2 * H + c) = b2;
                gx[i].x = g1.x * g[i].x; gx[i].y = g1.y * g[i].y; gx[i].z = g1.z * g[i].z; gx[i].w = g1.w * g[i].w;
                s1 += (gx[i].x + gx[i].y) + (gx[i].z + gx[i].w);
                s2 += (gx[i].x * xh[i].x + gx[i].y * xh[i].y) + (gx[i].z * xh[i].z + gx[i].w * xh[i].w);
            }
        }
        const float m1 = warp_sum(s1) * invH, m2 = warp_sum(s2) * invH;
        const float rs = st.y;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = lane * 4 + i * 128;
            if (c < H) {
                float4 gd;
                gd.x = rs * (gx[i].x - m1 - xh[i].x * m2); gd.y = rs * (gx[i].y - m1 - xh[i].y * m2);
                gd.z = rs * (gx[i].z - m1 - xh[i].z * m2); gd.w = rs * (gx[i].w - m1 - xh[i].w * m2);
                if (MODE != 0) {  // the mask again (regenerated or re-read: cheaper than eight registers held across the row)
                    const float4 mk = mask_of<MODE>(mask, ldm, seed, r, c, H, thresh, inv_keep);
                    gd.x *= mk.x; gd.y *= mk.y; gd.z *= mk.z; gd.w *= mk.w;
                }
                float4 a = *reinterpret_cast<float4 *>(mine + c);
                a.x += gd.x; a.y += gd.y; a.z += gd.z; a.w += gd.w;
                *reinterpret_cast<float4 *>(mine + c) = a;
                __stcs(reinterpret_cast<float4 *>(gh + r * ldgh + c), gd);
            }
        }
    }
    // block-level column sums in a fixed order: one pass over the warps' slices
    __syncthreads();
    for (int k = threadIdx.x; k < 3 * H; k += kEpiThreads) {
        float acc = 0.f;
        for (int w = 0; w < kEpiThreads / 32; ++w) acc += sred[(size_t)w * 3 * H + k];
        partials[(size_t)blockIdx.x * 3 * H + k] = acc;
    }
}

// out[3,H] = sum over blocks of partials[blocks,3,H], fixed order
__global__ void sage_epilogue_reduce_kernel(const float *__restrict__ partials, int blocks, int H3, float *__restrict__ out)
{
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= H3) return;
    float acc = 0.f;
    for (int b = 0; b < blocks; ++b) acc += partials[(size_t)b * H3 + k];
    out[k] = acc;
}

// the scaled keep mask the counter-based dropout applies, materialised (tests and debugging)
__global__ void dropout_mask_kernel(uint64_t seed, unsigned thresh, float inv_keep, int64_t n, int H, float *__restrict__ out)
{
    const int64_t groups = n * (int64_t)(H / 4);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < groups; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / (H / 4);
        const int c = (int)(i % (H / 4)) * 4;
        *reinterpret_cast<float4 *>(out + r * H + c) = dropout_scale4(seed, r, c, H, thresh, inv_keep);
    }
}

static int epi_grid()
{
    return sm_count() * 4;  // whole waves of resident blocks; rows are strided over the warps
}

static int check_common(int64_t n, int64_t H, float p, int mode, const void *mask, const char *who)
{
    SGNN_REQUIRE(n >= 0 && H > 0, SGNN_ERR_INVALID_ARGUMENT, "%s: bad size", who);
    SGNN_REQUIRE(H % 4 == 0 && H <= 512, SGNN_ERR_UNSUPPORTED, "%s: hidden width must be a multiple of 4 and <= 512 (got %lld)",
                 who, (long long)H);
    SGNN_REQUIRE(n <= (1LL << 40), SGNN_ERR_TOO_LARGE, "%s: too many rows", who);
    SGNN_REQUIRE(mode >= 0 && mode <= 2, SGNN_ERR_INVALID_ARGUMENT, "%s: dropout mode must be 0, 1 or 2", who);
    SGNN_REQUIRE(mode != 2 || mask != nullptr, SGNN_ERR_INVALID_ARGUMENT, "%s: mode 2 needs a mask", who);
    SGNN_REQUIRE(mode != 1 || (p >= 0.f && p < 1.f), SGNN_ERR_INVALID_ARGUMENT, "%s: dropout p must be in [0, 1)", who);
    return SGNN_OK;
}

}  // namespace sgnn

using namespace sgnn;

extern "C" SGNN_API int sgnn_epilogue_blocks(void) { return epi_grid(); }

extern "C" SGNN_API int sgnn_sage_epilogue_forward(const float *d_h, int64_t ldh, const float *d_bias, const float *d_gamma,
                                                   const float *d_beta, const float *d_mask, int64_t ldm,
                                                   int dropout_mode, uint64_t seed, float p, float eps, float *d_y,
                                                   int64_t ldy, float *d_stats, int64_t n, int64_t H, void *stream)
{
    int rc = check_common(n, H, p, dropout_mode, d_mask, "sage_epilogue_forward");
    if (rc) return rc;
    if (n == 0) return SGNN_OK;
    SGNN_REQUIRE(d_h && d_gamma && d_beta && d_y && d_stats, SGNN_ERR_INVALID_ARGUMENT, "sage_epilogue_forward: null pointer");
    SGNN_REQUIRE(ldh >= H && ldy >= H && ldh % 4 == 0 && ldy % 4 == 0 && (d_mask == nullptr || (ldm >= H && ldm % 4 == 0)),
                 SGNN_ERR_INVALID_ARGUMENT, "sage_epilogue_forward: leading dimensions must be >= H and multiples of 4");
    SGNN_REQUIRE(aligned16(d_h) && aligned16(d_y) && aligned16(d_gamma) && aligned16(d_beta) &&
                     (reinterpret_cast<uintptr_t>(d_stats) & 7u) == 0 && (d_bias == nullptr || aligned16(d_bias)) &&
                     (d_mask == nullptr || aligned16(d_mask)),
                 SGNN_ERR_INVALID_ARGUMENT, "sage_epilogue_forward: pointers must be 16-byte aligned (stats: 8)");
    const unsigned thresh = (unsigned)(p * 65536.0f);
    const float inv_keep = 1.0f / (1.0f - p);
    cudaStream_t s = (cudaStream_t)stream;
    float2 *stats = reinterpret_cast<float2 *>(d_stats);
    // one wave of resident blocks (the register count differs between the instantiations)
#define SGNN_EF(NVv, MODEv)                                                                                              \
    do {                                                                                                                 \
        int per_sm = 0;                                                                                                  \
        SGNN_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, sage_epilogue_fwd_kernel<NVv, MODEv>,        \
                                                                   kEpiThreads, 0));                                     \
        const int grid = sm_count() * (per_sm > 0 ? per_sm : 1);                                                         \
        sage_epilogue_fwd_kernel<NVv, MODEv><<<grid, kEpiThreads, 0, s>>>(d_h, ldh, d_bias, d_gamma, d_beta, d_mask,     \
                                                                          ldm, seed, thresh, inv_keep, eps, d_y, ldy,    \
                                                                          stats, n, (int)H);                             \
    } while (0)
#define SGNN_EF_MODE(NVv)                                                                                                \
    do {                                                                                                                 \
        if (dropout_mode == 0) SGNN_EF(NVv, 0); else if (dropout_mode == 1) SGNN_EF(NVv, 1); else SGNN_EF(NVv, 2);       \
    } while (0)
    if (H <= 128) SGNN_EF_MODE(1); else if (H <= 256) SGNN_EF_MODE(2); else SGNN_EF_MODE(4);
#undef SGNN_EF_MODE
#undef SGNN_EF
    SGNN_LAUNCH_OK("sage_epilogue_fwd_kernel");
    return SGNN_OK;
}

extern "C" SGNN_API int sgnn_sage_epilogue_backward(const float *d_gy, int64_t ldgy, const float *d_h, int64_t ldh,
                                                    const float *d_stats, const float *d_bias, const float *d_gamma,
                                                    const float *d_beta, const float *d_mask, int64_t ldm,
                                                    int dropout_mode, uint64_t seed, float p, float *d_gh, int64_t ldgh,
                                                    float *d_partials, float *d_grads3, int64_t n, int64_t H,
                                                    void *stream)
{
    int rc = check_common(n, H, p, dropout_mode, d_mask, "sage_epilogue_backward");
    if (rc) return rc;
    SGNN_REQUIRE(d_grads3 != nullptr, SGNN_ERR_INVALID_ARGUMENT, "sage_epilogue_backward: grads pointer is null");
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0) {
        SGNN_CUDA_OK(cudaMemsetAsync(d_grads3, 0, (size_t)3 * H * sizeof(float), s));
        return SGNN_OK;
    }
    SGNN_REQUIRE(d_gy && d_h && d_stats && d_gamma && d_beta && d_gh && d_partials, SGNN_ERR_INVALID_ARGUMENT,
                 "sage_epilogue_backward: null pointer");
    SGNN_REQUIRE(ldgy >= H && ldh >= H && ldgh >= H && ldgy % 4 == 0 && ldh % 4 == 0 && ldgh % 4 == 0 &&
                     (d_mask == nullptr || (ldm >= H && ldm % 4 == 0)),
                 SGNN_ERR_INVALID_ARGUMENT, "sage_epilogue_backward: leading dimensions must be >= H and multiples of 4");
    SGNN_REQUIRE(aligned16(d_gy) && aligned16(d_h) && aligned16(d_gh) && aligned16(d_gamma) && aligned16(d_beta) &&
                     aligned16(d_partials) && (reinterpret_cast<uintptr_t>(d_stats) & 7u) == 0 &&
                     (d_bias == nullptr || aligned16(d_bias)) && (d_mask == nullptr || aligned16(d_mask)),
                 SGNN_ERR_INVALID_ARGUMENT, "sage_epilogue_backward: pointers must be 16-byte aligned (stats: 8)");
    const unsigned thresh = (unsigned)(p * 65536.0f);
    const float inv_keep = 1.0f / (1.0f - p);
    const int g = epi_grid();
    const size_t smem = ((size_t)(kEpiThreads / 32) * 3 + 2) * H * sizeof(float);  // 52 KB at H = 512
    const float2 *stats = reinterpret_cast<const float2 *>(d_stats);
#define SGNN_EB(NVv, MODEv)                                                                                              \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            SGNN_CUDA_OK(cudaFuncSetAttribute(sage_epilogue_bwd_kernel<NVv, MODEv>,                                      \
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                  \
        sage_epilogue_bwd_kernel<NVv, MODEv><<<g, kEpiThreads, smem, s>>>(d_gy, ldgy, d_h, ldh, stats, d_bias, d_gamma,  \
                                                                          d_beta, d_mask, ldm, seed, thresh, inv_keep,  \
                                                                          d_gh, ldgh, d_partials, n, (int)H);           \
    } while (0)
#define SGNN_EB_MODE(NVv)                                                                                                \
    do {                                                                                                                 \
        if (dropout_mode == 0) SGNN_EB(NVv, 0); else if (dropout_mode == 1) SGNN_EB(NVv, 1); else SGNN_EB(NVv, 2);       \
    } while (0)
    if (H <= 128) SGNN_EB_MODE(1); else if (H <= 256) SGNN_EB_MODE(2); else SGNN_EB_MODE(4);
#undef SGNN_EB_MODE
#undef SGNN_EB
    SGNN_LAUNCH_OK("sage_epilogue_bwd_kernel");
    const int H3 = 3 * (int)H;
    sage_epilogue_reduce_kernel<<<(H3 + 127) / 128, 128, 0, s>>>(d_partials, g, H3, d_grads3);
    SGNN_LAUNCH_OK("sage_epilogue_reduce_kernel");
    return SGNN_OK;
}

extern "C" SGNN_API int sgnn_dropout_mask(uint64_t seed, float p, int64_t n, int64_t H, float *d_out, void *stream)
{
    int rc = check_common(n, H, p, 1, nullptr, "dropout_mask");
    if (rc) return rc;
    if (n == 0) return SGNN_OK;
    SGNN_REQUIRE(d_out != nullptr && aligned16(d_out), SGNN_ERR_INVALID_ARGUMENT, "dropout_mask: bad output pointer");
    const unsigned thresh = (unsigned)(p * 65536.0f);
    dropout_mask_kernel<<<sm_count() * 8, 256, 0, (cudaStream_t)stream>>>(seed, thresh, 1.0f / (1.0f - p), n, (int)H, d_out);
    SGNN_LAUNCH_OK("dropout_mask_kernel");
    return SGNN_OK;
}
