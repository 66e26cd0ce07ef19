// Quantise / dequantise of boundary rows in the "row codes" layout (see rowcodes.cuh): the same per-row
// min-max codes as the reference's quantiser, one contiguous run of F*bits/8 bytes per row.
//
// All three kernels are streaming and HBM bound: the quantiser reads every fp32 row once (rows held in
// registers between the min/max and the encode) and writes bits/32 of it; the one-sided variant stores the
// codes and the bf16 parameters straight into the destination peers' receive buffers (plain stores over
// NVLink), so quantisation and exchange are one kernel.
#include "quant_core.cuh"
#include "rowcodes.cuh"

namespace sgnn {

constexpr int kRowsPerStep = 4;  // rows a warp holds in registers at once

// Shared memory of the one-sided kernel: P + 1 ints of the work range, padded so that the 64-bit peer tables
// behind them start on an 8-byte boundary.  Returns the tables' offset in ints.
__host__ __device__ constexpr int rowcodes_p2p_table_offset(int P) { return (P + 2) & ~1; }

// lane value = the lane's NV quad fields side by side (NV * 4 * BITS bits), stored with one access
template <int BITS, int NV>
__device__ __forceinline__ void rowcodes_store_lane(uint8_t *rowp, int lane, const uint32_t (&q)[NV], bool stream_store)
{
    constexpr int QB = BITS / 2;  // bytes per quad
    uint8_t *p = rowp + lane * (NV * QB);
    if constexpr (NV * QB == 1) {
        *p = (uint8_t)q[0];
    } else if constexpr (NV * QB == 2) {
        const uint32_t v = (NV == 1) ? q[0] : (q[0] | (q[NV - 1] << 8));
        *reinterpret_cast<unsigned short *>(p) = (unsigned short)v;
    } else if constexpr (NV * QB == 4) {
        uint32_t v;
        if constexpr (NV == 1) v = q[0];
        else if constexpr (NV == 2) v = q[0] | (q[1] << 16);
        else v = q[0] | (q[1] << 8) | (q[2] << 16) | (q[3] << 24);
        if (stream_store) __stcs(reinterpret_cast<uint32_t *>(p), v);
        else *reinterpret_cast<uint32_t *>(p) = v;
    } else if constexpr (NV * QB == 8) {
        uint2 v;
        if constexpr (NV == 2) v = make_uint2(q[0], q[1]);
        else v = make_uint2(q[0] | (q[1] << 16), q[2] | (q[3] << 16));
        if (stream_store) __stcs(reinterpret_cast<uint2 *>(p), v);
        else *reinterpret_cast<uint2 *>(p) = v;
    } else {
        static_assert(NV == 4 && QB == 4, "unexpected lane width");
        const uint4 v = make_uint4(q[0], q[1], q[2], q[3]);
        if (stream_store) __stcs(reinterpret_cast<uint4 *>(p), v);
        else *reinterpret_cast<uint4 *>(p) = v;
    }
}

// P2P: codes and bf16 parameters go to the receive buffers of the peer that owns the row's segment
// (work_range[p] <= r < work_range[p+1]), at row  dst.params_row0[p] + r - work_range[p]  of that peer.
template <int BITS, int NV, bool P2P>
__global__ void __launch_bounds__(kQuantThreads, (NV <= 2 ? 4 : 2))
quant_pack_rowcodes_kernel(const float *__restrict__ X, int64_t ldx, const int64_t *__restrict__ row_index, int S, int F,
                           const int32_t *__restrict__ work_range, int P, uint8_t *__restrict__ codes,
                           float *__restrict__ params, uint16_t *__restrict__ params_bf16, PeerDst dst)
{
    constexpr float LEVELS = (float)((1 << BITS) - 1);
    constexpr uint32_t CODE_MASK = 0x01010101u * ((1u << BITS) - 1u);
    // P2P: work_range[0..P], then the three peer tables (codes base, params base, first row), so that the per-row
    // lookup of the destination costs shared-memory reads instead of three dependent global loads
    extern __shared__ int smem[];
    long long *tab = reinterpret_cast<long long *>(smem + rowcodes_p2p_table_offset(P));
    if constexpr (P2P) {
        for (int i = threadIdx.x; i <= P; i += blockDim.x) smem[i] = work_range[i];
        for (int i = threadIdx.x; i < P; i += blockDim.x) {
            tab[i] = (long long)dst.packed_base[i];
            tab[P + i] = (long long)dst.params_base[i];
            tab[2 * P + i] = dst.params_row0[i];
        }
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    const int64_t pitch = (int64_t)F * BITS / 8;
    const int warps_total = gridDim.x * (kQuantThreads / 32);
    const int steps = (S + kRowsPerStep - 1) / kRowsPerStep;
    for (int step = blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5); step < steps; step += warps_total) {
        float4 x[kRowsPerStep][NV];
#pragma unroll
        for (int j = 0; j < kRowsPerStep; ++j) {
            const int r = step * kRowsPerStep + j;
            const bool rv = r < S;
            int64_t src = r;
            if (rv && row_index) src = __ldg(row_index + r);
            const float *xr = X + src * ldx;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int n = lane * 4 + i * 128;
                if (rv && n < F) x[j][i] = ld_stream(reinterpret_cast<const float4 *>(xr + n));
            }
        }
        // destination peer of the step's first row, looked up while the loads above are in flight:
        // largest p with work_range[p] <= r (which skips peers without rows)
        int peer = 0, next_begin = 0x7fffffff;  // first row of the next peer's segment
        long long codes_base = 0, params_base = 0, row_shift = 0;  // destination row = row_shift + r
        if constexpr (P2P) {
            const int r0 = step * kRowsPerStep;
            int hi = P;
            while (hi - peer > 1) {
                const int mid = (peer + hi) >> 1;
                if (smem[mid] <= r0) peer = mid; else hi = mid;
            }
            next_begin = peer + 1 < P ? smem[peer + 1] : 0x7fffffff;
            codes_base = tab[peer], params_base = tab[P + peer], row_shift = tab[2 * P + peer] - smem[peer];
        }
#pragma unroll
        for (int j = 0; j < kRowsPerStep; ++j) {
            const int r = step * kRowsPerStep + j;
            if (r >= S) continue;
            float mn = INFINITY, mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                if (lane * 4 + i * 128 < F) {
                    const float4 t = x[j][i];
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
            uint8_t *rowp;
            if constexpr (P2P) {
                if (r >= next_begin) {  // a segment boundary inside the step (rare)
                    while (peer + 1 < P && smem[peer + 1] <= r) ++peer;
                    next_begin = peer + 1 < P ? smem[peer + 1] : 0x7fffffff;
                    codes_base = tab[peer], params_base = tab[P + peer], row_shift = tab[2 * P + peer] - smem[peer];
                }
                const int64_t drow = row_shift + r;
                if (lane == 0) {
                    if (params) reinterpret_cast<float2 *>(params)[r] = make_float2(rq.mn, rq.sc);
                    reinterpret_cast<uint32_t *>(params_base)[drow] =
                        (uint32_t)float_to_bf16_bits(rq.mn) | ((uint32_t)float_to_bf16_bits(rq.sc) << 16);
                }
                rowp = reinterpret_cast<uint8_t *>(codes_base) + drow * pitch;
            } else {
                if (lane == 0) store_params(params, params_bf16, r, rq.mn, rq.sc);
                rowp = codes + (int64_t)r * pitch;
            }
            uint32_t q[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                q[i] = 0;
                if (lane * 4 + i * 128 < F) q[i] = rowcodes_compress<BITS>(encode4(x[j][i], rq) & CODE_MASK);
            }
            if (lane * 4 < F) rowcodes_store_lane<BITS, NV>(rowp, lane, q, !P2P);
        }
    }
}

// out[r] (or out[row_index[r]] +=) = zero_point + code * scale.  A warp takes four rows at a time.
template <int BITS>
__global__ void __launch_bounds__(kQuantThreads, 3)
unpack_rowcodes_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ params,
                       const uint16_t *__restrict__ params_bf16, int S, int F, float *__restrict__ out, int64_t ldo,
                       const int64_t *__restrict__ row_index)
{
    const int lane = threadIdx.x & 31;
    const int64_t pitch = (int64_t)F * BITS / 8;
    const int nv = F <= 128 ? 1 : F / 128;
    const int lognv = nv == 4 ? 2 : (nv == 2 ? 1 : 0);
    const int warps_total = gridDim.x * (kQuantThreads / 32);
    const int steps = (S + kRowsPerStep - 1) / kRowsPerStep;
    for (int step = blockIdx.x * (kQuantThreads / 32) + (threadIdx.x >> 5); step < steps; step += warps_total) {
        float zp[kRowsPerStep], sc[kRowsPerStep];
        int64_t orow[kRowsPerStep];
#pragma unroll
        for (int j = 0; j < kRowsPerStep; ++j) {
            const int r = step * kRowsPerStep + j;
            zp[j] = 0.f; sc[j] = 0.f; orow[j] = 0;
            if (r < S) {
                if (params) {
                    const float2 t = __ldg(reinterpret_cast<const float2 *>(params) + r);
                    zp[j] = t.x; sc[j] = t.y;
                } else {
                    const uint32_t t = __ldg(reinterpret_cast<const uint32_t *>(params_bf16) + r);
                    zp[j] = bf16_bits_to_float((uint16_t)(t & 0xffffu));
                    sc[j] = bf16_bits_to_float((uint16_t)(t >> 16));
                }
                orow[j] = row_index ? __ldg(row_index + r) : (int64_t)r;
            }
        }
        for (int i = 0; i < nv; ++i) {
            const int n = lane * 4 + i * 128;
            if (n >= F) break;
            const int off = rowcodes_quad_offset<BITS>(n >> 2, lognv);
            uint32_t q[kRowsPerStep];
#pragma unroll
            for (int j = 0; j < kRowsPerStep; ++j) {
                const int r = step * kRowsPerStep + j;
                q[j] = 0;
                if (r < S) q[j] = rowcodes_load_quad<BITS>(codes + (int64_t)r * pitch + off);
            }
#pragma unroll
            for (int j = 0; j < kRowsPerStep; ++j) {
                const int r = step * kRowsPerStep + j;
                if (r >= S) continue;
                float v[4];
                rowcodes_expand<BITS>(q[j], sc[j], zp[j], v);
                float *o = out + orow[j] * ldo + n;
                const float4 f = make_float4(v[0], v[1], v[2], v[3]);
                if (row_index) red_add_v4(o, f);
                else __stcs(reinterpret_cast<float4 *>(o), f);
            }
        }
    }
}

static int rowcodes_check(const char *who, int64_t S, int64_t F, int bits)
{
    SGNN_REQUIRE(bits == 2 || bits == 4 || bits == 8, SGNN_ERR_INVALID_ARGUMENT, "%s: bits must be 2, 4 or 8 (got %d)",
                 who, bits);
    SGNN_REQUIRE(S >= 0 && F >= 0, SGNN_ERR_INVALID_ARGUMENT, "%s: negative size", who);
    SGNN_REQUIRE(S <= 2147483647LL, SGNN_ERR_TOO_LARGE, "%s: S must fit int32", who);
    SGNN_REQUIRE(S == 0 || F == 0 || rowcodes_width_ok(F), SGNN_ERR_UNSUPPORTED,
                 "%s: the row-codes layout needs F %% 4 == 0 and F <= 128, F == 256 or F == 512 (F=%lld)", who,
                 (long long)F);
    return SGNN_OK;
}

template <bool P2P>
static int launch_quant_rowcodes(const float *d_X, int64_t ldx, const int64_t *d_row_index, int64_t S, int64_t F,
                                 const int32_t *d_work_range, int P, int bits, uint8_t *d_codes, float *d_params,
                                 uint16_t *d_params_bf16, PeerDst dst, cudaStream_t s)
{
    const size_t smem = P2P ? (size_t)rowcodes_p2p_table_offset(P) * sizeof(int) + (size_t)3 * P * sizeof(long long) : 0;
    const int64_t steps = ceil_div(S, kRowsPerStep);
#define SGNN_RC(B, NVv)                                                                                              \
    do {                                                                                                             \
        int per_sm = 1;                                                                                              \
        SGNN_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quant_pack_rowcodes_kernel<B, NVv, P2P>, \
                                                                   kQuantThreads, smem));                            \
        int64_t g = (int64_t)sm_count() * (per_sm > 0 ? per_sm : 1); /* one resident wave */                         \
        const int64_t need = ceil_div(steps, kQuantThreads / 32);                                                    \
        if (need < g) g = need;                                                                                      \
        quant_pack_rowcodes_kernel<B, NVv, P2P><<<(unsigned)g, kQuantThreads, smem, s>>>(                            \
            d_X, ldx, d_row_index, (int)S, (int)F, d_work_range, P, d_codes, d_params, d_params_bf16, dst);          \
    } while (0)
    const int nv = rowcodes_nv(F);
    if (bits == 8) { if (nv == 1) SGNN_RC(8, 1); else if (nv == 2) SGNN_RC(8, 2); else SGNN_RC(8, 4); }
    else if (bits == 4) { if (nv == 1) SGNN_RC(4, 1); else if (nv == 2) SGNN_RC(4, 2); else SGNN_RC(4, 4); }
    else { if (nv == 1) SGNN_RC(2, 1); else if (nv == 2) SGNN_RC(2, 2); else SGNN_RC(2, 4); }
#undef SGNN_RC
    SGNN_LAUNCH_OK("quant_pack_rowcodes_kernel");
    return SGNN_OK;
}

}  // namespace sgnn

using namespace sgnn;

extern "C" SGNN_API int sgnn_rowcodes_width_supported(int64_t F) { return rowcodes_width_ok(F) ? 1 : 0; }

extern "C" SGNN_API int sgnn_quant_pack_rowcodes(const float *d_X, int64_t ldx, const int64_t *d_row_index, int64_t S,
                                                 int64_t F, int bits, uint8_t *d_codes, float *d_params,
                                                 uint16_t *d_params_bf16, void *stream)
{
    int rc = rowcodes_check("quant_pack_rowcodes", S, F, bits);
    if (rc) return rc;
    SGNN_REQUIRE(ldx >= F, SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rowcodes: ldx < F");
    if (S == 0 || F == 0) return SGNN_OK;
    SGNN_REQUIRE(d_X && d_codes, SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rowcodes: null data pointer");
    SGNN_REQUIRE((ldx % 4 == 0) && aligned16(d_X), SGNN_ERR_INVALID_ARGUMENT,
                 "quant_pack_rowcodes: rows of X must be 16-byte aligned");
    // a lane stores its NV quads with one access of NV * bits/2 bytes: the buffer must be aligned to that
    SGNN_REQUIRE(reinterpret_cast<uintptr_t>(d_codes) % (size_t)(rowcodes_nv(F) * bits / 2) == 0, SGNN_ERR_INVALID_ARGUMENT,
                 "quant_pack_rowcodes: the code buffer must be aligned to %d bytes", rowcodes_nv(F) * bits / 2);
    SGNN_REQUIRE(d_params == nullptr || (reinterpret_cast<uintptr_t>(d_params) & 7u) == 0, SGNN_ERR_INVALID_ARGUMENT,
                 "quant_pack_rowcodes: params must be 8-byte aligned");
    SGNN_REQUIRE(d_params_bf16 == nullptr || (reinterpret_cast<uintptr_t>(d_params_bf16) & 3u) == 0,
                 SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rowcodes: params_bf16 must be 4-byte aligned");
    return launch_quant_rowcodes<false>(d_X, ldx, d_row_index, S, F, nullptr, 1, bits, d_codes, d_params, d_params_bf16,
                                        PeerDst{}, (cudaStream_t)stream);
}

extern "C" SGNN_API int sgnn_quant_pack_rowcodes_p2p(const float *d_X, int64_t ldx, const int64_t *d_row_index, int64_t S,
                                                     int64_t F, const int32_t *d_work_range, int P, int bits,
                                                     const uint64_t *d_peer_codes, const uint64_t *d_peer_params,
                                                     const int64_t *d_peer_row0, float *d_params_fp32, void *stream)
{
    int rc = rowcodes_check("quant_pack_rowcodes_p2p", S, F, bits);
    if (rc) return rc;
    SGNN_REQUIRE(P >= 1 && P <= SGNN_MAX_PEERS, SGNN_ERR_TOO_LARGE, "quant_pack_rowcodes_p2p: P=%d outside [1, %d]", P,
                 SGNN_MAX_PEERS);
    SGNN_REQUIRE(d_work_range && d_peer_codes && d_peer_params && d_peer_row0, SGNN_ERR_INVALID_ARGUMENT,
                 "quant_pack_rowcodes_p2p: null table pointer");
    SGNN_REQUIRE(ldx >= F, SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rowcodes_p2p: ldx < F");
    if (S == 0 || F == 0) return SGNN_OK;
    SGNN_REQUIRE(d_X != nullptr, SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rowcodes_p2p: X is null");
    SGNN_REQUIRE((ldx % 4 == 0) && aligned16(d_X), SGNN_ERR_INVALID_ARGUMENT,
                 "quant_pack_rowcodes_p2p: rows of X must be 16-byte aligned");
    SGNN_REQUIRE(d_params_fp32 == nullptr || (reinterpret_cast<uintptr_t>(d_params_fp32) & 7u) == 0,
                 SGNN_ERR_INVALID_ARGUMENT, "quant_pack_rowcodes_p2p: params must be 8-byte aligned");
    PeerDst dst{reinterpret_cast<const unsigned long long *>(d_peer_codes), nullptr,
                reinterpret_cast<const unsigned long long *>(d_peer_params),
                reinterpret_cast<const long long *>(d_peer_row0)};
    return launch_quant_rowcodes<true>(d_X, ldx, d_row_index, S, F, d_work_range, P, bits, nullptr, d_params_fp32, nullptr,
                                       dst, (cudaStream_t)stream);
}

extern "C" SGNN_API int sgnn_unpack_dequant_rowcodes(const uint8_t *d_codes, const float *d_params,
                                                     const uint16_t *d_params_bf16, int64_t S, int64_t F, int bits,
                                                     float *d_out, int64_t ldo, const int64_t *d_row_index, void *stream)
{
    int rc = rowcodes_check("unpack_dequant_rowcodes", S, F, bits);
    if (rc) return rc;
    SGNN_REQUIRE((d_params != nullptr) != (d_params_bf16 != nullptr), SGNN_ERR_INVALID_ARGUMENT,
                 "unpack_dequant_rowcodes: give exactly one of params (fp32) and params_bf16");
    SGNN_REQUIRE(ldo >= F, SGNN_ERR_INVALID_ARGUMENT, "unpack_dequant_rowcodes: ldo < F");
    if (S == 0 || F == 0) return SGNN_OK;
    SGNN_REQUIRE(d_codes && d_out, SGNN_ERR_INVALID_ARGUMENT, "unpack_dequant_rowcodes: null data pointer");
    SGNN_REQUIRE((ldo % 4 == 0) && aligned16(d_out), SGNN_ERR_INVALID_ARGUMENT,
                 "unpack_dequant_rowcodes: output rows must be 16-byte aligned");
    SGNN_REQUIRE(reinterpret_cast<uintptr_t>(d_codes) % (size_t)(bits / 2) == 0, SGNN_ERR_INVALID_ARGUMENT,
                 "unpack_dequant_rowcodes: the code buffer must be aligned to %d bytes", bits / 2);
    SGNN_REQUIRE(d_params == nullptr || (reinterpret_cast<uintptr_t>(d_params) & 7u) == 0, SGNN_ERR_INVALID_ARGUMENT,
                 "unpack_dequant_rowcodes: params must be 8-byte aligned");
    SGNN_REQUIRE(d_params_bf16 == nullptr || (reinterpret_cast<uintptr_t>(d_params_bf16) & 3u) == 0,
                 SGNN_ERR_INVALID_ARGUMENT, "unpack_dequant_rowcodes: params_bf16 must be 4-byte aligned");
    int64_t blocks = ceil_div(ceil_div(S, kRowsPerStep), kQuantThreads / 32);
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    cudaStream_t s = (cudaStream_t)stream;
    if (bits == 8)
        unpack_rowcodes_kernel<8><<<(unsigned)blocks, kQuantThreads, 0, s>>>(d_codes, d_params, d_params_bf16, (int)S, (int)F, d_out, ldo, d_row_index);
    else if (bits == 4)
        unpack_rowcodes_kernel<4><<<(unsigned)blocks, kQuantThreads, 0, s>>>(d_codes, d_params, d_params_bf16, (int)S, (int)F, d_out, ldo, d_row_index);
    else
        unpack_rowcodes_kernel<2><<<(unsigned)blocks, kQuantThreads, 0, s>>>(d_codes, d_params, d_params_bf16, (int)S, (int)F, d_out, ldo, d_row_index);
    SGNN_LAUNCH_OK("unpack_rowcodes_kernel");
    return SGNN_OK;
}
