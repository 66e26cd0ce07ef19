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
#include "quant_core.cuh"

namespace sgnn {

// P2P == true: packed rows and bf16 parameters are stored straight into the destination peers' receive
// buffers (plain 32-bit stores to peer memory over NVLink, coalesced 128 B per warp), so quantisation and
// the boundary exchange are one kernel; `packed` / `params_bf16` are then unused.
template <int BITS, int NV, bool P2P>
__global__ void __launch_bounds__(kQuantThreads, (NV <= 2 ? 4 : 2))
quant_pack_vec_kernel(const float *__restrict__ X, int64_t ldx, const int64_t *__restrict__ row_index, int F,
                      const int32_t *__restrict__ work_range, int P, uint8_t *__restrict__ packed,
                      float *__restrict__ params, uint16_t *__restrict__ params_bf16, PeerDst dst)
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
        int r0[U], nr[U], peer[U];
        float4 x[U][EPB][NV];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int q = step * U + u;
            r0[u] = 0; nr[u] = 0; peer[u] = 0;
            if (q < total) locate_group_peer(smem, P, EPB, q, r0[u], nr[u], peer[u]);
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
                        mn = min3(min3(mn, t.x, t.y), t.z, t.w);
                        mx = max3(max3(mx, t.x, t.y), t.z, t.w);
                    }
                }
                RowQ rq;
                rq.mn = redux_min(mn);
                mx = redux_max(mx);
                rq.sc = __fdiv_rn(__fsub_rn(mx, rq.mn), LEVELS);
                if (rq.sc == 0.f) rq.sc = 1.f;
                rq.rinv = __fdiv_rn(1.0f, rq.sc);
                rq.thr = rq.sc * (0.5f * (1.0f - 1.0f / 4096.0f));
                if (lane == 0) {
                    if constexpr (P2P) {
                        const int64_t r = (int64_t)r0[u] + j;
                        if (params) reinterpret_cast<float2 *>(params)[r] = make_float2(rq.mn, rq.sc);
                        uint32_t *pp = reinterpret_cast<uint32_t *>(dst.params_base[peer[u]]);
                        pp[dst.params_row0[peer[u]] + (r - smem[peer[u]])] =
                            (uint32_t)float_to_bf16_bits(rq.mn) | ((uint32_t)float_to_bf16_bits(rq.sc) << 16);
                    } else {
                        store_params(params, params_bf16, (int64_t)r0[u] + j, rq.mn, rq.sc);
                    }
                }
                const int sh = (EPB - 1 - j) * BITS;
#pragma unroll
                for (int i = 0; i < NV; ++i)
                    if (lane * 4 + i * 128 < F)  // per-byte mask: what the reference's truncation to uint8 keeps
                        word[i] |= (encode4(x[u][j][i], rq) & (0x01010101u * (0xffu >> sh))) << sh;
            }
            uint8_t *prow;
            if constexpr (P2P) {
                const int g = q - smem[(P + 1) + peer[u]];  // packed row inside this peer's segment
                prow = reinterpret_cast<uint8_t *>(dst.packed_base[peer[u]]) + (dst.packed_row0[peer[u]] + g) * (int64_t)F;
            } else {
                prow = packed + (int64_t)q * F;
            }
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int n = lane * 4 + i * 128;
                if (n < F) {
                    if constexpr (P2P) *reinterpret_cast<uint32_t *>(prow + n) = word[i];
                    else __stcs(reinterpret_cast<uint32_t *>(prow + n), word[i]);
                }
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
template <bool VEC4, int BITS>
__global__ void __launch_bounds__(kQuantThreads, 3)
unpack_dequant_kernel(const uint8_t *__restrict__ packed, const float *__restrict__ params,
                      const uint16_t *__restrict__ params_bf16, const float *__restrict__ given_min,
                      const float *__restrict__ given_scale, int F, const int32_t *__restrict__ work_range, int P,
                      int64_t single_S, float *__restrict__ out, int64_t ldo, const int64_t *__restrict__ row_index)
{
    constexpr int EPB = 8 / BITS;
    constexpr unsigned MASK = (1u << BITS) - 1u;
    constexpr int U = 4;  // packed rows per warp step: four independent loads in flight per lane
    extern __shared__ int smem[];
    build_peer_tables(smem, work_range, P, EPB, single_S);
    const int total = smem[2 * P + 1];
    const int lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (kQuantThreads / 32);
    const int steps = (total + U - 1) / U;
    for (int step = blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5); step < steps; step += warps_total) {
        int r0[U], nr[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            r0[u] = 0; nr[u] = 0;
            if (step * U + u < total) locate_group(smem, P, EPB, step * U + u, r0[u], nr[u]);
        }
        const int kstep = VEC4 ? 128 : 32;
        for (int k = VEC4 ? lane * 4 : lane; k < F; k += kstep) {
            uint32_t w[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                w[u] = 0;
                if (nr[u] > 0) {
                    const uint8_t *p = packed + (int64_t)(step * U + u) * F + k;
                    if constexpr (VEC4) w[u] = (uint32_t)ld_stream(reinterpret_cast<const int *>(p));
                    else w[u] = *p;
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
#pragma unroll
                for (int j = 0; j < EPB; ++j) {
                    if (j < nr[u]) {
                        const int64_t r = (int64_t)r0[u] + j;
                        float zp, sc;
                        if (given_min) {
                            zp = __ldg(given_min + r);
                            sc = __ldg(given_scale + r);
                        } else if (params) {
                            const float2 t = __ldg(reinterpret_cast<const float2 *>(params) + r);
                            zp = t.x; sc = t.y;
                        } else {
                            const uint32_t t = __ldg(reinterpret_cast<const uint32_t *>(params_bf16) + r);
                            zp = bf16_bits_to_float((uint16_t)(t & 0xffffu));
                            sc = bf16_bits_to_float((uint16_t)(t >> 16));
                        }
                        float *o = out + (row_index ? __ldg(row_index + r) : r) * ldo + k;
                        const int sh = (EPB - 1 - j) * BITS;
                        if constexpr (VEC4) {
                            float4 v;
                            v.x = __fmaf_rn((float)((w[u] >> sh) & MASK), sc, zp);
                            v.y = __fmaf_rn((float)((w[u] >> (8 + sh)) & MASK), sc, zp);
                            v.z = __fmaf_rn((float)((w[u] >> (16 + sh)) & MASK), sc, zp);
                            v.w = __fmaf_rn((float)((w[u] >> (24 + sh)) & MASK), sc, zp);
                            if (row_index) red_add_v4(o, v);
                            else __stcs(reinterpret_cast<float4 *>(o), v);
                        } else {
                            const float v = __fmaf_rn((float)((w[u] >> sh) & MASK), sc, zp);
                            if (row_index) red_add(o, v);
                            else *o = v;
                        }
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
// v2: torch.quantize_per_channel-compatible codes, rne(x * (1/scale) + zero_point) with one fused multiply-add,
// packed along the feature axis with the first element in the LOW bits; decode (code - zero_point) * scale.
// A warp per row.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kQuantThreads)
quantize_v2_kernel(const float *__restrict__ X, int64_t S, int F, const int64_t *__restrict__ range,
                   const float *__restrict__ zero_points, const float *__restrict__ scales, int bits,
                   uint8_t *__restrict__ out)
{
    const int lane = threadIdx.x & 31;
    const int epb = 8 / bits;
    const int64_t warps_total = (int64_t)gridDim.x * (kQuantThreads / 32);
    for (int64_t r = (int64_t)blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5); r < S; r += warps_total) {
        const float zp = __ldg(zero_points + r), sc = __ldg(scales + r);
        const float inv = sc == 0.0f ? 1.0f : __fdiv_rn(1.0f, sc);
        const float *xr = X + r * (int64_t)F;
        const int nbytes = (F + epb - 1) / epb;
        uint8_t *o = out + range[r];
        for (int b = lane; b < nbytes; b += 32) {
            uint32_t acc = 0;
            for (int j = 0; j < epb; ++j) {
                const int k = b * epb + j;
                if (k < F) acc |= ((uint32_t)__float2int_rn(__fmaf_rn(__ldg(xr + k), inv, zp)) & 0xffu) << (j * bits);
            }
            o[b] = (uint8_t)acc;
        }
    }
}

__global__ void __launch_bounds__(kQuantThreads)
dequantize_v2_kernel(const uint8_t *__restrict__ in, int64_t S, int F, const int64_t *__restrict__ range,
                     const float *__restrict__ zero_points, const float *__restrict__ scales, int bits,
                     float *__restrict__ out)
{
    const int lane = threadIdx.x & 31;
    const int epb = 8 / bits;
    const unsigned m = (1u << bits) - 1u;
    const int64_t warps_total = (int64_t)gridDim.x * (kQuantThreads / 32);
    for (int64_t r = (int64_t)blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5); r < S; r += warps_total) {
        const float zp = __ldg(zero_points + r), sc = __ldg(scales + r);
        const int64_t b0 = range[r];
        const int nbytes = (int)(range[r + 1] - b0);
        float *o = out + r * (int64_t)F;
        for (int b = lane; b < nbytes; b += 32) {
            const unsigned w = in[b0 + b];
            for (int j = 0; j < epb; ++j) {
                const int k = b * epb + j;
                if (k < F) o[k] = __fmul_rn(__fsub_rn((float)((w >> (j * bits)) & m), zp), sc);
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
        const int64_t steps_ub = ceil_div(groups_ub, u);
        // one resident wave: blocks per SM from the occupancy calculator, times the SM count
#define SGNN_QP(B, NVv)                                                                                              \
    do {                                                                                                             \
        int per_sm = 1;                                                                                              \
        SGNN_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quant_pack_vec_kernel<B, NVv, false>,    \
                                                                   kQuantThreads, smem));                            \
        int64_t g = (int64_t)sm_count() * (per_sm > 0 ? per_sm : 1);                                                 \
        const int64_t need = ceil_div(steps_ub, kQuantThreads / 32);                                                 \
        if (need < g) g = need;                                                                                      \
        quant_pack_vec_kernel<B, NVv, false><<<(unsigned)g, kQuantThreads, smem, s>>>(                               \
            d_X, ldx, d_row_index, (int)F, d_work_range, P, d_packed, d_params, d_params_bf16, PeerDst{});           \
    } while (0)
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
    const int g = grid_for(ceil_div(S / epb + P, 4));
    const bool vec = (F % 4 == 0) && (ldo % 4 == 0) && aligned16(d_out) &&
                     ((reinterpret_cast<uintptr_t>(d_packed) & 3u) == 0);
#define SGNN_UD(V, B)                                                                                                  \
    unpack_dequant_kernel<V, B><<<g, kQuantThreads, smem, s>>>(d_packed, d_params, d_params_bf16, d_min, d_scale, (int)F, \
                                                               d_work_range, P, S, d_out, ldo, d_row_index)
    if (vec) {
        if (bits == 8) SGNN_UD(true, 8); else if (bits == 4) SGNN_UD(true, 4); else SGNN_UD(true, 2);
    } else {
        if (bits == 8) SGNN_UD(false, 8); else if (bits == 4) SGNN_UD(false, 4); else SGNN_UD(false, 2);
    }
#undef SGNN_UD
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

extern "C" SGNN_API int sgnn_quantize_rows_v2(const float *d_X, int64_t S, int64_t F, const int64_t *d_range,
                                              const float *d_zero_points, const float *d_scales, int bits,
                                              uint8_t *d_out, void *stream)
{
    int rc = check_bits(bits, "quantize_rows_v2");
    if (rc) return rc;
    SGNN_REQUIRE(S >= 0 && F >= 0, SGNN_ERR_INVALID_ARGUMENT, "quantize_rows_v2: negative size");
    SGNN_REQUIRE(F <= (1 << 24), SGNN_ERR_TOO_LARGE, "quantize_rows_v2: F <= 2^24");
    if (S == 0 || F == 0) return SGNN_OK;
    SGNN_REQUIRE(d_X && d_range && d_zero_points && d_scales && d_out, SGNN_ERR_INVALID_ARGUMENT,
                 "quantize_rows_v2: null pointer");
    quantize_v2_kernel<<<grid_for(S), kQuantThreads, 0, (cudaStream_t)stream>>>(d_X, S, (int)F, d_range, d_zero_points,
                                                                                d_scales, bits, d_out);
    SGNN_LAUNCH_OK("quantize_v2_kernel");
    return SGNN_OK;
}

extern "C" SGNN_API int sgnn_dequantize_rows_v2(const uint8_t *d_in, int64_t S, int64_t F, const int64_t *d_range,
                                                const float *d_zero_points, const float *d_scales, int bits,
                                                float *d_out, void *stream)
{
    int rc = check_bits(bits, "dequantize_rows_v2");
    if (rc) return rc;
    SGNN_REQUIRE(S >= 0 && F >= 0, SGNN_ERR_INVALID_ARGUMENT, "dequantize_rows_v2: negative size");
    SGNN_REQUIRE(F <= (1 << 24), SGNN_ERR_TOO_LARGE, "dequantize_rows_v2: F <= 2^24");
    if (S == 0 || F == 0) return SGNN_OK;
    SGNN_REQUIRE(d_in && d_range && d_zero_points && d_scales && d_out, SGNN_ERR_INVALID_ARGUMENT,
                 "dequantize_rows_v2: null pointer");
    dequantize_v2_kernel<<<grid_for(S), kQuantThreads, 0, (cudaStream_t)stream>>>(d_in, S, (int)F, d_range,
                                                                                  d_zero_points, d_scales, bits, d_out);
    SGNN_LAUNCH_OK("dequantize_v2_kernel");
    return SGNN_OK;
}

// One-sided exchange: quantise + pack + store into the peers' receive buffers.
extern "C" SGNN_API int sgnn_quant_pack_rows_p2p(const float *d_X, int64_t ldx, const int64_t *d_row_index, int64_t S,
                                                 int64_t F, const int32_t *d_work_range, int P, int bits,
                                                 const uint64_t *d_peer_packed, const int64_t *d_peer_packed_row0,
                                                 const uint64_t *d_peer_params, const int64_t *d_peer_params_row0,
                                                 float *d_params_fp32, void *stream)
{
    int rc = check_bits(bits, "quant_pack_rows_p2p");
    if (rc) return rc;
    SGNN_REQUIRE(S >= 0 && F >= 0, SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rows_p2p: negative size");
    SGNN_REQUIRE(S <= 2147483647LL, SGNN_ERR_TOO_LARGE, "quant_pack_rows_p2p: S must fit int32");
    SGNN_REQUIRE(P >= 1 && P <= SGNN_MAX_PEERS, SGNN_ERR_TOO_LARGE, "quant_pack_rows_p2p: P=%d outside [1, %d]", P,
                 SGNN_MAX_PEERS);
    SGNN_REQUIRE(d_work_range && d_peer_packed && d_peer_packed_row0 && d_peer_params && d_peer_params_row0,
                 SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rows_p2p: null table pointer");
    SGNN_REQUIRE(ldx >= F, SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rows_p2p: ldx < F");
    if (S == 0 || F == 0) return SGNN_OK;
    SGNN_REQUIRE(d_X != nullptr, SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rows_p2p: X is null");
    SGNN_REQUIRE((F % 4 == 0) && (F <= 512) && (ldx % 4 == 0) && aligned16(d_X), SGNN_ERR_UNSUPPORTED,
                 "quant_pack_rows_p2p: needs F %% 4 == 0, F <= 512 and 16-byte aligned rows (F=%lld)", (long long)F);
    SGNN_REQUIRE(d_params_fp32 == nullptr || (reinterpret_cast<uintptr_t>(d_params_fp32) & 7u) == 0,
                 SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rows_p2p: params must be 8-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(2 * (P + 1)) * sizeof(int);
    const int epb = 8 / bits;
    const int64_t steps_ub = ceil_div(S / epb + P, 4 / epb);
    PeerDst dst{reinterpret_cast<const unsigned long long *>(d_peer_packed),
                reinterpret_cast<const long long *>(d_peer_packed_row0),
                reinterpret_cast<const unsigned long long *>(d_peer_params),
                reinterpret_cast<const long long *>(d_peer_params_row0)};
#define SGNN_QP2(B, NVv)                                                                                            \
    do {                                                                                                            \
        int per_sm = 1;                                                                                             \
        SGNN_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quant_pack_vec_kernel<B, NVv, true>,    \
                                                                   kQuantThreads, smem));                           \
        int64_t g = (int64_t)sm_count() * (per_sm > 0 ? per_sm : 1);                                                \
        const int64_t need = ceil_div(steps_ub, kQuantThreads / 32);                                                \
        if (need < g) g = need;                                                                                     \
        quant_pack_vec_kernel<B, NVv, true><<<(unsigned)g, kQuantThreads, smem, s>>>(                               \
            d_X, ldx, d_row_index, (int)F, d_work_range, P, nullptr, d_params_fp32, nullptr, dst);                  \
    } while (0)
    const int nv = F <= 128 ? 1 : (F <= 256 ? 2 : 4);
    if (bits == 8) { if (nv == 1) SGNN_QP2(8, 1); else if (nv == 2) SGNN_QP2(8, 2); else SGNN_QP2(8, 4); }
    else if (bits == 4) { if (nv == 1) SGNN_QP2(4, 1); else if (nv == 2) SGNN_QP2(4, 2); else SGNN_QP2(4, 4); }
    else { if (nv == 1) SGNN_QP2(2, 1); else if (nv == 2) SGNN_QP2(2, 2); else SGNN_QP2(2, 4); }
#undef SGNN_QP2
    SGNN_LAUNCH_OK("quant_pack_vec_kernel (p2p)");
    return SGNN_OK;
}
