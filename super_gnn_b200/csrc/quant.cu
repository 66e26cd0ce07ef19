// Per-row min-max quantize + pack and unpack + dequantize of boundary-node features (sm_100a).
//
// Wire format ("row-group packing"): peer p owns rows [wr[p], wr[p+1]); inside a peer EPB = 8/bits
// consecutive rows share one packed row of F bytes; byte k of that packed row holds the codes of the
// EPB rows at feature k, the first row of the group in the most significant bits.  Codes are
// rne((x - min) / scale) with IEEE fp32 subtract and divide.
//
// All kernels are streaming and HBM bound.  The fast quantiser keeps the EPB (<= 4) rows of a
// group in registers between the min/max reduction and the encode, so each input byte is read
// from HBM exactly once, and writes 32-bit words of packed bytes, coalesced across the warp.
#include "common.cuh"

namespace sgnn {

constexpr int kQuantThreads = 256;

// Shared-memory tables: wr[0..P] and the packed-row offset of each peer off[0..P].
__device__ __forceinline__ void build_peer_tables(int *smem, const int32_t *__restrict__ work_range, int P, int epb,
                                                  int64_t single_S)
{
    int *swr = smem, *soff = smem + (P + 1);
    if (work_range) {
        for (int i = threadIdx.x; i <= P; i += blockDim.x) swr[i] = work_range[i];
    } else if (threadIdx.x == 0) {
        swr[0] = 0;
        swr[1] = (int)single_S;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int p = 0; p < P; ++p) {
            soff[p] = acc;
            acc += (swr[p + 1] - swr[p] + epb - 1) / epb;
        }
        soff[P] = acc;
    }
    __syncthreads();
}

// Packed row q -> first input row and number of valid rows in the group.
__device__ __forceinline__ void locate_group(const int *smem, int P, int epb, int q, int &r0, int &nr)
{
    const int *swr = smem, *soff = smem + (P + 1);
    int lo = 0, hi = P;  // largest p with off[p] <= q (skips peers without rows)
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (soff[mid] <= q) lo = mid; else hi = mid;
    }
    r0 = swr[lo] + (q - soff[lo]) * epb;
    const int left = swr[lo + 1] - r0;
    nr = left < epb ? left : epb;
}

__device__ __forceinline__ float warp_min(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(FULL, v, o));
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, o));
    return v;
}

__device__ __forceinline__ int code_of(float x, float zp, float sc)
{
    return __float2int_rn(__fdiv_rn(__fsub_rn(x, zp), sc));
}

__device__ __forceinline__ void store_params(float *params, uint16_t *params_bf16, int64_t r, float zp, float sc)
{
    if (params) reinterpret_cast<float2 *>(params)[r] = make_float2(zp, sc);
    if (params_bf16)
        reinterpret_cast<uint32_t *>(params_bf16)[r] =
            (uint32_t)float_to_bf16_bits(zp) | ((uint32_t)float_to_bf16_bits(sc) << 16);
}

// ---------------------------------------------------------------------------
// Fast path: F % 4 == 0, F <= 128*NV, 16-byte aligned rows.  One warp handles
// U = 4/EPB packed rows (= up to 4 input rows) per step, all loads first.
// ---------------------------------------------------------------------------
template <int BITS, int NV>
__global__ void __launch_bounds__(kQuantThreads)
quant_pack_vec_kernel(const float *__restrict__ X, int64_t ldx, const int64_t *__restrict__ row_index, int F,
                      const int32_t *__restrict__ work_range, int P, uint8_t *__restrict__ packed,
                      float *__restrict__ params, uint16_t *__restrict__ params_bf16)
{
    constexpr int EPB = 8 / BITS;
    constexpr int U = 4 / EPB;
    constexpr float LEVELS = (float)((1 << BITS) - 1);
    extern __shared__ int smem[];
    build_peer_tables(smem, work_range, P, EPB, 0);
    const int total = smem[2 * P + 1];  // off[P]
    const int lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (kQuantThreads / 32);
    const int steps = (total + U - 1) / U;
    for (int step = blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5); step < steps; step += warps_total) {
        int r0[U], nr[U];
        float4 x[U][EPB][NV];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int q = step * U + u;
            r0[u] = 0; nr[u] = 0;
            if (q < total) locate_group(smem, P, EPB, q, r0[u], nr[u]);
#pragma unroll
            for (int j = 0; j < EPB; ++j) {
                const bool rv = j < nr[u];
                int64_t src = r0[u] + j;
                if (rv && row_index) src = __ldg(row_index + src);
                const float *xr = X + src * ldx;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    const int n = lane * 4 + i * 128;
                    if (rv && n < F) x[u][j][i] = ld_stream(reinterpret_cast<const float4 *>(xr + n));
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int q = step * U + u;
            if (q >= total) continue;
            uint32_t word[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) word[i] = 0;
#pragma unroll
            for (int j = 0; j < EPB; ++j) {
                if (j >= nr[u]) continue;
                float mn = INFINITY, mx = -INFINITY;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    if (lane * 4 + i * 128 < F) {
                        const float4 t = x[u][j][i];
                        mn = fminf(fminf(mn, t.x), fminf(t.y, fminf(t.z, t.w)));
                        mx = fmaxf(fmaxf(mx, t.x), fmaxf(t.y, fmaxf(t.z, t.w)));
                    }
                }
                mn = warp_min(mn);
                mx = warp_max(mx);
                float sc = __fdiv_rn(__fsub_rn(mx, mn), LEVELS);
                if (sc == 0.f) sc = 1.f;
                if (lane == 0) store_params(params, params_bf16, (int64_t)r0[u] + j, mn, sc);
                const int sh = (EPB - 1 - j) * BITS;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    if (lane * 4 + i * 128 < F) {
                        const float4 t = x[u][j][i];
                        // int32 shift/or, truncated to a byte at the end, like the reference
                        const uint32_t c0 = ((uint32_t)code_of(t.x, mn, sc) << sh) & 0xffu;
                        const uint32_t c1 = ((uint32_t)code_of(t.y, mn, sc) << sh) & 0xffu;
                        const uint32_t c2 = ((uint32_t)code_of(t.z, mn, sc) << sh) & 0xffu;
                        const uint32_t c3 = ((uint32_t)code_of(t.w, mn, sc) << sh) & 0xffu;
                        word[i] |= c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
                    }
                }
            }
            uint8_t *prow = packed + (int64_t)q * F;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int n = lane * 4 + i * 128;
                if (n < F) __stcs(reinterpret_cast<uint32_t *>(prow + n), word[i]);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// General path: any F / alignment, optional caller-supplied (min, scale).
// A warp per packed row, rows re-read from cache for the encode.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kQuantThreads)
quant_pack_generic_kernel(const float *__restrict__ X, int64_t ldx, const int64_t *__restrict__ row_index, int F,
                          const int32_t *__restrict__ work_range, int P, int64_t single_S, int bits,
                          uint8_t *__restrict__ packed, float *__restrict__ params, uint16_t *__restrict__ params_bf16,
                          const float *__restrict__ given_min, const float *__restrict__ given_scale)
{
    const int epb = 8 / bits;
    extern __shared__ int smem[];
    build_peer_tables(smem, work_range, P, epb, single_S);
    const int total = smem[2 * P + 1];
    const int lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (kQuantThreads / 32);
    const float levels = (float)((1 << bits) - 1);
    for (int q = blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5); q < total; q += warps_total) {
        int r0, nr;
        locate_group(smem, P, epb, q, r0, nr);
        float zp[4], sc[4];
        const float *xr[4];
        for (int j = 0; j < 4; ++j) {
            zp[j] = 0.f; sc[j] = 1.f; xr[j] = X;
            if (j < nr) {
                int64_t src = r0 + j;
                if (row_index) src = __ldg(row_index + src);
                xr[j] = X + src * ldx;
                if (given_min) {
                    zp[j] = __ldg(given_min + r0 + j);
                    sc[j] = __ldg(given_scale + r0 + j);
                } else {
                    float mn = INFINITY, mx = -INFINITY;
                    for (int k = lane; k < F; k += 32) {
                        const float v = __ldg(xr[j] + k);
                        mn = fminf(mn, v);
                        mx = fmaxf(mx, v);
                    }
                    mn = warp_min(mn);
                    mx = warp_max(mx);
                    float s = __fdiv_rn(__fsub_rn(mx, mn), levels);
                    if (s == 0.f) s = 1.f;
                    zp[j] = mn; sc[j] = s;
                    if (lane == 0) store_params(params, params_bf16, (int64_t)r0 + j, mn, s);
                }
            }
        }
        uint8_t *prow = packed + (int64_t)q * F;
        for (int k = lane; k < F; k += 32) {
            uint32_t acc = 0;
            for (int j = 0; j < 4; ++j)
                if (j < nr) acc |= (uint32_t)code_of(__ldg(xr[j] + k), zp[j], sc[j]) << ((epb - 1 - j) * bits);
            prow[k] = (uint8_t)acc;
        }
    }
}

// ---------------------------------------------------------------------------
// Unpack + dequantize: out = fma(code, scale, zero_point).  A warp per packed row.
// VEC4: F % 4 == 0 and 16-byte aligned output rows / 4-byte aligned packed rows.
// row_index != null: rows are atomically added to out[row_index[r]] instead of stored.
// ---------------------------------------------------------------------------
template <bool VEC4>
__global__ void __launch_bounds__(kQuantThreads)
unpack_dequant_kernel(const uint8_t *__restrict__ packed, const float *__restrict__ params,
                      const uint16_t *__restrict__ params_bf16, const float *__restrict__ given_min,
                      const float *__restrict__ given_scale, int F, const int32_t *__restrict__ work_range, int P,
                      int64_t single_S, int bits, float *__restrict__ out, int64_t ldo,
                      const int64_t *__restrict__ row_index)
{
    const int epb = 8 / bits;
    const unsigned m = (1u << bits) - 1u;
    extern __shared__ int smem[];
    build_peer_tables(smem, work_range, P, epb, single_S);
    const int total = smem[2 * P + 1];
    const int lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (kQuantThreads / 32);
    for (int q = blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5); q < total; q += warps_total) {
        int r0, nr;
        locate_group(smem, P, epb, q, r0, nr);
        float zp[4], sc[4];
        float *orow[4];
        for (int j = 0; j < 4; ++j) {
            zp[j] = 0.f; sc[j] = 0.f; orow[j] = out;
            if (j < nr) {
                const int64_t r = (int64_t)r0 + j;
                if (given_min) {
                    zp[j] = __ldg(given_min + r);
                    sc[j] = __ldg(given_scale + r);
                } else if (params) {
                    const float2 t = __ldg(reinterpret_cast<const float2 *>(params) + r);
                    zp[j] = t.x; sc[j] = t.y;
                } else {
                    const uint32_t t = __ldg(reinterpret_cast<const uint32_t *>(params_bf16) + r);
                    zp[j] = bf16_bits_to_float((uint16_t)(t & 0xffffu));
                    sc[j] = bf16_bits_to_float((uint16_t)(t >> 16));
                }
                orow[j] = out + (row_index ? __ldg(row_index + r) : r) * ldo;
            }
        }
        const uint8_t *prow = packed + (int64_t)q * F;
        if constexpr (VEC4) {
            for (int k = lane * 4; k < F; k += 128) {
                const uint32_t w = ld_stream(reinterpret_cast<const int *>(prow + k));
                for (int j = 0; j < 4; ++j) {
                    if (j < nr) {
                        const int sh = (epb - 1 - j) * bits;
                        float4 v;
                        v.x = __fmaf_rn((float)((w >> sh) & m), sc[j], zp[j]);
                        v.y = __fmaf_rn((float)((w >> (8 + sh)) & m), sc[j], zp[j]);
                        v.z = __fmaf_rn((float)((w >> (16 + sh)) & m), sc[j], zp[j]);
                        v.w = __fmaf_rn((float)((w >> (24 + sh)) & m), sc[j], zp[j]);
                        if (row_index) red_add_v4(orow[j] + k, v);
                        else __stcs(reinterpret_cast<float4 *>(orow[j] + k), v);
                    }
                }
            }
        } else {
            for (int k = lane; k < F; k += 32) {
                const unsigned w = prow[k];
                for (int j = 0; j < 4; ++j) {
                    if (j < nr) {
                        const float v = __fmaf_rn((float)((w >> ((epb - 1 - j) * bits)) & m), sc[j], zp[j]);
                        if (row_index) red_add(orow[j] + k, v);
                        else orow[j][k] = v;
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// v1: per-row bit width, packed along the feature axis.  A warp per row.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kQuantThreads)
quantize_v1_kernel(const float *__restrict__ X, int64_t S, int F, const int64_t *__restrict__ range,
                   float *__restrict__ params, uint8_t *__restrict__ out)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = (int64_t)gridDim.x * (kQuantThreads / 32);
    for (int64_t r = (int64_t)blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5); r < S; r += warps_total) {
        const int bits = (int)params[3 * r];
        if (bits != 8 && bits != 4 && bits != 2) continue;
        const float *xr = X + r * (int64_t)F;
        float mn = INFINITY, mx = -INFINITY;
        for (int k = lane; k < F; k += 32) {
            const float v = __ldg(xr + k);
            mn = fminf(mn, v);
            mx = fmaxf(mx, v);
        }
        mn = warp_min(mn);
        mx = warp_max(mx);
        float sc = __fdiv_rn(__fsub_rn(mx, mn), (float)((1 << bits) - 1));
        if (sc == 0.f) sc = 1.f;
        __syncwarp();  // every lane has read params[3r] before lane 0 rewrites the row
        if (lane == 0) {
            params[3 * r + 1] = mn;
            params[3 * r + 2] = sc;
        }
        const int epb = 8 / bits;
        const int nbytes = (F + epb - 1) / epb;
        uint8_t *o = out + range[r];
        for (int b = lane; b < nbytes; b += 32) {
            uint32_t acc = 0;
            for (int j = 0; j < epb; ++j) {
                const int k = b * epb + j;
                if (k < F) acc |= (uint32_t)code_of(__ldg(xr + k), mn, sc) << ((epb - 1 - j) * bits);
            }
            o[b] = (uint8_t)acc;
        }
    }
}

__global__ void __launch_bounds__(kQuantThreads)
dequantize_v1_kernel(const uint8_t *__restrict__ in, int64_t S, int F, const int64_t *__restrict__ range,
                     const float *__restrict__ params, float *__restrict__ out)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps_total = (int64_t)gridDim.x * (kQuantThreads / 32);
    for (int64_t r = (int64_t)blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5); r < S; r += warps_total) {
        const int bits = (int)params[3 * r];
        if (bits != 8 && bits != 4 && bits != 2) continue;
        const float zp = params[3 * r + 1], sc = params[3 * r + 2];
        const int epb = 8 / bits;
        const unsigned m = (1u << bits) - 1u;
        const int64_t b0 = range[r];
        const int nbytes = (int)(range[r + 1] - b0);
        float *o = out + r * (int64_t)F;
        for (int b = lane; b < nbytes; b += 32) {
            const unsigned w = in[b0 + b];
            for (int j = 0; j < epb; ++j) {
                const int k = b * epb + j;
                if (k < F) o[k] = __fmaf_rn((float)((w >> ((epb - 1 - j) * bits)) & m), sc, zp);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int grid_for(int64_t warp_items)
{
    int64_t blocks = ceil_div(warp_items > 0 ? warp_items : 1, kQuantThreads / 32);
    const int64_t cap = (int64_t)sm_count() * 8;  // whole waves of resident blocks
    if (blocks > cap) blocks = cap;
    return (int)blocks;
}

static int check_bits(int bits, const char *who)
{
    SGNN_REQUIRE(bits == 2 || bits == 4 || bits == 8, SGNN_ERR_INVALID_ARGUMENT, "%s: bits must be 2, 4 or 8 (got %d)",
                 who, bits);
    return SGNN_OK;
}

}  // namespace sgnn

using namespace sgnn;

extern "C" SGNN_API int sgnn_quant_pack_rows(const float *d_X, int64_t ldx, const int64_t *d_row_index, int64_t S, int64_t F,
                                    const int32_t *d_work_range, int P, int bits, uint8_t *d_packed, float *d_params,
                                    uint16_t *d_params_bf16, void *stream)
{
    int rc = check_bits(bits, "quant_pack_rows");
    if (rc) return rc;
    SGNN_REQUIRE(S >= 0 && F >= 0, SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rows: negative size");
    SGNN_REQUIRE(S <= 2147483647LL && F <= (1 << 24), SGNN_ERR_TOO_LARGE, "quant_pack_rows: S must fit int32, F <= 2^24");
    SGNN_REQUIRE(P >= 1 && P <= SGNN_MAX_PEERS, SGNN_ERR_TOO_LARGE, "quant_pack_rows: P=%d outside [1, %d]", P,
                 SGNN_MAX_PEERS);
    SGNN_REQUIRE(d_work_range != nullptr, SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rows: work_range is null");
    SGNN_REQUIRE(ldx >= F, SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rows: ldx < F");
    if (S == 0 || F == 0) return SGNN_OK;
    SGNN_REQUIRE(d_X && d_packed, SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rows: null data pointer");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(2 * (P + 1)) * sizeof(int);
    const int epb = 8 / bits;
    // upper bound of packed rows (exact count lives on the device): S/epb + P
    const int64_t groups_ub = S / epb + P;
    const bool vec = (F % 4 == 0) && (F <= 512) && (ldx % 4 == 0) && aligned16(d_X) &&
                     ((reinterpret_cast<uintptr_t>(d_packed) & 3u) == 0) &&
                     (d_params == nullptr || (reinterpret_cast<uintptr_t>(d_params) & 7u) == 0) &&
                     (d_params_bf16 == nullptr || (reinterpret_cast<uintptr_t>(d_params_bf16) & 3u) == 0);
    if (vec) {
        const int u = 4 / epb;
        const int g = grid_for(ceil_div(groups_ub, u));
#define SGNN_QP(B, NVv)                                                                                            \
    quant_pack_vec_kernel<B, NVv><<<g, kQuantThreads, smem, s>>>(d_X, ldx, d_row_index, (int)F, d_work_range, P, \
                                                                 d_packed, d_params, d_params_bf16)
        const int nv = F <= 128 ? 1 : (F <= 256 ? 2 : 4);
        if (bits == 8) { if (nv == 1) SGNN_QP(8, 1); else if (nv == 2) SGNN_QP(8, 2); else SGNN_QP(8, 4); }
        else if (bits == 4) { if (nv == 1) SGNN_QP(4, 1); else if (nv == 2) SGNN_QP(4, 2); else SGNN_QP(4, 4); }
        else { if (nv == 1) SGNN_QP(2, 1); else if (nv == 2) SGNN_QP(2, 2); else SGNN_QP(2, 4); }
#undef SGNN_QP
        SGNN_LAUNCH_OK("quant_pack_vec_kernel");
        return SGNN_OK;
    }
    SGNN_REQUIRE(d_params == nullptr || (reinterpret_cast<uintptr_t>(d_params) & 7u) == 0, SGNN_ERR_INVALID_ARGUMENT,
                 "quant_pack_rows: params must be 8-byte aligned");
    SGNN_REQUIRE(d_params_bf16 == nullptr || (reinterpret_cast<uintptr_t>(d_params_bf16) & 3u) == 0,
                 SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rows: params_bf16 must be 4-byte aligned");
    quant_pack_generic_kernel<<<grid_for(groups_ub), kQuantThreads, smem, s>>>(
        d_X, ldx, d_row_index, (int)F, d_work_range, P, 0, bits, d_packed, d_params, d_params_bf16, nullptr, nullptr);
    SGNN_LAUNCH_OK("quant_pack_generic_kernel");
    return SGNN_OK;
}

extern "C" SGNN_API int sgnn_quantize_tensor(const float *d_X, int64_t S, int64_t F, const float *d_min, const float *d_scale,
                                    int bits, uint8_t *d_packed, void *stream)
{
    int rc = check_bits(bits, "quantize_tensor");
    if (rc) return rc;
    SGNN_REQUIRE(S >= 0 && F >= 0, SGNN_ERR_INVALID_ARGUMENT, "quantize_tensor: negative size");
    SGNN_REQUIRE(S <= 2147483647LL && F <= (1 << 24), SGNN_ERR_TOO_LARGE, "quantize_tensor: S must fit int32, F <= 2^24");
    if (S == 0 || F == 0) return SGNN_OK;
    SGNN_REQUIRE(d_X && d_min && d_scale && d_packed, SGNN_ERR_INVALID_ARGUMENT, "quantize_tensor: null pointer");
    const int epb = 8 / bits;
    quant_pack_generic_kernel<<<grid_for(ceil_div(S, epb)), kQuantThreads, 4 * sizeof(int), (cudaStream_t)stream>>>(
        d_X, F, nullptr, (int)F, nullptr, 1, S, bits, d_packed, nullptr, nullptr, d_min, d_scale);
    SGNN_LAUNCH_OK("quant_pack_generic_kernel");
    return SGNN_OK;
}

static int launch_unpack(const uint8_t *d_packed, const float *d_params, const uint16_t *d_params_bf16,
                         const float *d_min, const float *d_scale, int64_t S, int64_t F, const int32_t *d_work_range,
                         int P, int bits, float *d_out, int64_t ldo, const int64_t *d_row_index, cudaStream_t s)
{
    const size_t smem = (size_t)(2 * (P + 1)) * sizeof(int);
    const int epb = 8 / bits;
    const int g = grid_for(S / epb + P);
    const bool vec = (F % 4 == 0) && (ldo % 4 == 0) && aligned16(d_out) &&
                     ((reinterpret_cast<uintptr_t>(d_packed) & 3u) == 0);
    if (vec)
        unpack_dequant_kernel<true><<<g, kQuantThreads, smem, s>>>(d_packed, d_params, d_params_bf16, d_min, d_scale,
                                                                   (int)F, d_work_range, P, S, bits, d_out, ldo,
                                                                   d_row_index);
    else
        unpack_dequant_kernel<false><<<g, kQuantThreads, smem, s>>>(d_packed, d_params, d_params_bf16, d_min, d_scale,
                                                                    (int)F, d_work_range, P, S, bits, d_out, ldo,
                                                                    d_row_index);
    SGNN_LAUNCH_OK("unpack_dequant_kernel");
    return SGNN_OK;
}

extern "C" SGNN_API int sgnn_unpack_dequant_rows(const uint8_t *d_packed, const float *d_params, const uint16_t *d_params_bf16,
                                        int64_t S, int64_t F, const int32_t *d_work_range, int P, int bits,
                                        float *d_out, int64_t ldo, const int64_t *d_row_index, void *stream)
{
    int rc = check_bits(bits, "unpack_dequant_rows");
    if (rc) return rc;
    SGNN_REQUIRE(S >= 0 && F >= 0, SGNN_ERR_INVALID_ARGUMENT, "unpack_dequant_rows: negative size");
    SGNN_REQUIRE(S <= 2147483647LL && F <= (1 << 24), SGNN_ERR_TOO_LARGE, "unpack_dequant_rows: S must fit int32, F <= 2^24");
    SGNN_REQUIRE(P >= 1 && P <= SGNN_MAX_PEERS, SGNN_ERR_TOO_LARGE, "unpack_dequant_rows: P=%d outside [1, %d]", P,
                 SGNN_MAX_PEERS);
    SGNN_REQUIRE(d_work_range != nullptr, SGNN_ERR_INVALID_ARGUMENT, "unpack_dequant_rows: work_range is null");
    SGNN_REQUIRE((d_params != nullptr) != (d_params_bf16 != nullptr), SGNN_ERR_INVALID_ARGUMENT,
                 "unpack_dequant_rows: give exactly one of params (fp32) and params_bf16");
    SGNN_REQUIRE(ldo >= F, SGNN_ERR_INVALID_ARGUMENT, "unpack_dequant_rows: ldo < F");
    SGNN_REQUIRE(d_params == nullptr || (reinterpret_cast<uintptr_t>(d_params) & 7u) == 0, SGNN_ERR_INVALID_ARGUMENT,
                 "unpack_dequant_rows: params must be 8-byte aligned");
    SGNN_REQUIRE(d_params_bf16 == nullptr || (reinterpret_cast<uintptr_t>(d_params_bf16) & 3u) == 0,
                 SGNN_ERR_INVALID_ARGUMENT, "unpack_dequant_rows: params_bf16 must be 4-byte aligned");
    if (S == 0 || F == 0) return SGNN_OK;
    SGNN_REQUIRE(d_packed && d_out, SGNN_ERR_INVALID_ARGUMENT, "unpack_dequant_rows: null data pointer");
    return launch_unpack(d_packed, d_params, d_params_bf16, nullptr, nullptr, S, F, d_work_range, P, bits, d_out, ldo,
                         d_row_index, (cudaStream_t)stream);
}

extern "C" SGNN_API int sgnn_dequantize_tensor(const uint8_t *d_packed, int64_t S, int64_t F, const float *d_min,
                                      const float *d_scale, int bits, float *d_out, void *stream)
{
    int rc = check_bits(bits, "dequantize_tensor");
    if (rc) return rc;
    SGNN_REQUIRE(S >= 0 && F >= 0, SGNN_ERR_INVALID_ARGUMENT, "dequantize_tensor: negative size");
    SGNN_REQUIRE(S <= 2147483647LL && F <= (1 << 24), SGNN_ERR_TOO_LARGE, "dequantize_tensor: S must fit int32, F <= 2^24");
    if (S == 0 || F == 0) return SGNN_OK;
    SGNN_REQUIRE(d_packed && d_min && d_scale && d_out, SGNN_ERR_INVALID_ARGUMENT, "dequantize_tensor: null pointer");
    return launch_unpack(d_packed, nullptr, nullptr, d_min, d_scale, S, F, nullptr, 1, bits, d_out, F, nullptr,
                         (cudaStream_t)stream);
}

extern "C" SGNN_API int sgnn_quantize_rows_v1(const float *d_X, int64_t S, int64_t F, const int64_t *d_range, float *d_params,
                                     uint8_t *d_out, void *stream)
{
    SGNN_REQUIRE(S >= 0 && F >= 0, SGNN_ERR_INVALID_ARGUMENT, "quantize_rows_v1: negative size");
    SGNN_REQUIRE(F <= (1 << 24), SGNN_ERR_TOO_LARGE, "quantize_rows_v1: F <= 2^24");
    if (S == 0 || F == 0) return SGNN_OK;
    SGNN_REQUIRE(d_X && d_range && d_params && d_out, SGNN_ERR_INVALID_ARGUMENT, "quantize_rows_v1: null pointer");
    quantize_v1_kernel<<<grid_for(S), kQuantThreads, 0, (cudaStream_t)stream>>>(d_X, S, (int)F, d_range, d_params, d_out);
    SGNN_LAUNCH_OK("quantize_v1_kernel");
    return SGNN_OK;
}

extern "C" SGNN_API int sgnn_dequantize_rows_v1(const uint8_t *d_in, int64_t S, int64_t F, const int64_t *d_range,
                                       const float *d_params, float *d_out, void *stream)
{
    SGNN_REQUIRE(S >= 0 && F >= 0, SGNN_ERR_INVALID_ARGUMENT, "dequantize_rows_v1: negative size");
    SGNN_REQUIRE(F <= (1 << 24), SGNN_ERR_TOO_LARGE, "dequantize_rows_v1: F <= 2^24");
    if (S == 0 || F == 0) return SGNN_OK;
    SGNN_REQUIRE(d_in && d_range && d_params && d_out, SGNN_ERR_INVALID_ARGUMENT, "dequantize_rows_v1: null pointer");
    dequantize_v1_kernel<<<grid_for(S), kQuantThreads, 0, (cudaStream_t)stream>>>(d_in, S, (int)F, d_range, d_params,
                                                                                  d_out);
    SGNN_LAUNCH_OK("dequantize_v1_kernel");
    return SGNN_OK;
}
