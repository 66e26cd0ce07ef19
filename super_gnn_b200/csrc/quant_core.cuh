// Device helpers shared by the quantise / pack kernels: per-peer segment tables, warp min/max, the
// verified-reciprocal encoder and the parameter stores.
#pragma once
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

// Same, plus the peer that owns the group (for the one-sided exchange).
__device__ __forceinline__ void locate_group_peer(const int *smem, int P, int epb, int q, int &r0, int &nr, int &peer)
{
    const int *swr = smem, *soff = smem + (P + 1);
    int lo = 0, hi = P;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (soff[mid] <= q) lo = mid; else hi = mid;
    }
    r0 = swr[lo] + (q - soff[lo]) * epb;
    const int left = swr[lo + 1] - r0;
    nr = left < epb ? left : epb;
    peer = lo;
}

// Destination of the one-sided exchange: for every peer, the address of its receive buffers (peer
// memory, mapped through NVLink) and the row at which this rank's segment starts inside them.
struct PeerDst {
    const unsigned long long *packed_base;   // [P] uint8* of the peer's packed receive buffer
    const long long *packed_row0;            // [P] first packed row of this rank's segment there
    const unsigned long long *params_base;   // [P] bf16 (zero_point, scale) pairs of the peer
    const long long *params_row0;            // [P] first row of this rank's segment there
};

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
//
// The encode must equal rne(RN((x - min) / scale)) bit for bit, but an IEEE divide per element
// would make the kernel issue bound.  Each code is therefore first computed with one multiply
// by the reciprocal and the add-magic-number rounding trick, and then PROVED right with one
// FMA: if |(x - min) - c * scale| <= scale/2 * (1 - 2^-12) the exact quotient lies strictly
// inside (c - 1/2, c + 1/2) by more than the 2^-16 by which the IEEE quotient of a value
// <= 256 can differ from it, so rne of the IEEE quotient is c.  The rare elements that fail
// the test (about 2^-12 of them, those near a rounding boundary, and any non-finite value)
// take the IEEE divide.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float redux_min(float v)
{
    float r;
    asm volatile("redux.sync.min.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ float redux_max(float v)
{
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}

struct RowQ {
    float mn, sc, rinv, thr;
};

// sm_100 packed fp32x2 arithmetic (two IEEE fp32 operations per instruction) and three-input min / max
__device__ __forceinline__ unsigned long long pk2(float lo, float hi)
{
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpk2(unsigned long long v, float &lo, float &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long sub2(unsigned long long a, unsigned long long b)
{
    unsigned long long r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c)
{
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ float min3(float a, float b, float c)
{
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c)
{
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// four codes of one float4 -> one word with a code per byte (each < 256)
__device__ __forceinline__ uint32_t encode4(const float4 t, const RowQ q)
{
    constexpr float MAGIC = 12582912.0f;  // 1.5 * 2^23: adding it rounds to an integer, to nearest even
    const unsigned long long mn2 = pk2(q.mn, q.mn), rinv2 = pk2(q.rinv, q.rinv), magic2 = pk2(MAGIC, MAGIC);
    const unsigned long long nsc2 = pk2(-q.sc, -q.sc);
    // candidate: u = (x - mn) * rinv + MAGIC (any candidate is acceptable: the residual test below decides)
    const unsigned long long d01 = sub2(pk2(t.x, t.y), mn2), d23 = sub2(pk2(t.z, t.w), mn2);
    const unsigned long long u01 = fma2(d01, rinv2, magic2), u23 = fma2(d23, rinv2, magic2);
    // residual (x - mn) - c * scale, exact product, one rounding
    const unsigned long long r01 = fma2(sub2(u01, magic2), nsc2, d01), r23 = fma2(sub2(u23, magic2), nsc2, d23);
    float r0, r1, r2, r3, u0, u1, u2, u3;
    unpk2(r01, r0, r1);
    unpk2(r23, r2, r3);
    unpk2(u01, u0, u1);
    unpk2(u23, u2, u3);
    const float worst = fmaxf(max3(fabsf(r0), fabsf(r1), fabsf(r2)), fabsf(r3));
    uint32_t b0 = __float_as_uint(u0), b1 = __float_as_uint(u1), b2 = __float_as_uint(u2), b3 = __float_as_uint(u3);
    if (!(worst <= q.thr)) {  // also taken for NaN / infinities
        b0 = (uint32_t)code_of(t.x, q.mn, q.sc);
        b1 = (uint32_t)code_of(t.y, q.mn, q.sc);
        b2 = (uint32_t)code_of(t.z, q.mn, q.sc);
        b3 = (uint32_t)code_of(t.w, q.mn, q.sc);
    }
    // low byte of each: {b0, b1, b2, b3} -> bytes 0..3
    const uint32_t lo = __byte_perm(b0, b1, 0x0040);  // byte0 = b0.0, byte1 = b1.0
    const uint32_t hi = __byte_perm(b2, b3, 0x0040);
    return __byte_perm(lo, hi, 0x5410);
}

}  // namespace sgnn
