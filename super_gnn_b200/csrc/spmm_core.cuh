// CSR SpMM core for sm_100a: Y[m,:] (+)= sum_e w[e] * row(col[e]).
//
// The work is an irregular gather of dense rows — HBM/L2 bound, CUDA cores only.
// Two kernels share one inner loop:
//   * row split : a group of G lanes (G = 8/16/32, a sub-warp or a warp) owns a row;
//                 deterministic, best when degrees are near uniform;
//   * nnz split : every warp owns an equal chunk of nonzeros (merge-path style);
//                 rows cut by a chunk boundary are finished with fp32 reductions
//                 into global memory, so a power-law degree distribution cannot
//                 create a straggler.
// Column indices and edge weights are staged 32 (or G) at a time with one
// coalesced streaming load and handed round with warp shuffles; each lane then
// issues up to four independent 128-bit row loads before the first FMA.
//
// `Src` abstracts where a dense row comes from: fp32 rows in memory (DenseSrc) or
// rows still in the packed 2/4/8-bit wire format, dequantised in flight (PackedSrcT).
#pragma once
#include "common.cuh"
#include "rowcodes.cuh"

namespace sgnn {

constexpr int kSpmmThreads = 256;
constexpr int kWarpChunk = 128;  // nonzeros per warp work item in the nnz-split kernel

// ---------------------------------------------------------------------------
// Row sources
// ---------------------------------------------------------------------------
// HAS_VAL == false: all-ones matrix and no column scale (sum aggregation) — no weight is staged or
// handed round.  With HAS_VAL the weight of a nonzero is val[e] (1 if val is null) times
// col_scale[col[e]] (if given): the column scale folds "divide the operand rows by the in-degree"
// of a mean aggregation's backward pass into the gather.
template <bool HAS_VAL, bool COL_SCALE = false>
struct DenseSrcT {
    const float *__restrict__ X;
    int ldx;  // row pitch in elements; 32 bits so that the row address is one 32x32->64 multiply-add
    const float *__restrict__ col_scale;

    struct Edge {
        int c;
        float w;
    };
    static constexpr int kSmemInts = 0;
    static constexpr bool kDense = true, kHasVal = HAS_VAL, kColScale = COL_SCALE;
    static constexpr int kBatch = 4;  // nonzeros whose row loads are issued together
    template <int VEC>
    struct Raw {
        float v[VEC];
    };
    __device__ __forceinline__ void init_block(int *) const {}
    static size_t smem_bytes(int) { return 0; }

    __device__ __forceinline__ Edge stage(const int *__restrict__ col, const float *__restrict__ val, int64_t e,
                                          bool valid, const int *) const
    {
        Edge s;
        s.c = valid ? ld_stream(col + e) : 0;
        s.w = 1.0f;
        if (HAS_VAL) {
            s.w = 0.0f;
            if (valid) {
                if constexpr (COL_SCALE) {
                    s.w = (val ? ld_stream(val + e) : 1.0f) * __ldg(col_scale + s.c);
                } else {
                    s.w = ld_stream(val + e);
                }
            }
        }
        return s;
    }
    __device__ __forceinline__ Edge bcast(const Edge &s, int j, unsigned mask, int width) const
    {
        Edge r;
        r.c = __shfl_sync(mask, s.c, j, width);
        r.w = 1.0f;
        if (HAS_VAL) r.w = __shfl_sync(mask, s.w, j, width);
        return r;
    }
    template <int VEC>
    __device__ __forceinline__ void load(const Edge &s, int n, Raw<VEC> &r) const
    {
        const float *p = X + ((int64_t)s.c * ldx + n);
        if constexpr (VEC == 4) {
            const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
            r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
        } else {
            r.v[0] = __ldg(p);
        }
    }
    template <int VEC>
    __device__ __forceinline__ void expand(const Edge &, const Raw<VEC> &r, float (&x)[VEC]) const
    {
#pragma unroll
        for (int k = 0; k < VEC; ++k) x[k] = r.v[k];
    }
};

// Rows in wire format: peer p owns received rows [wr[p], wr[p+1]); inside a peer EPB = 8/bits
// rows share a packed row of F bytes, row i%EPB == 0 in the high bits.
template <bool HAS_VAL>
struct PackedSrcT {
    const uint8_t *__restrict__ packed;
    int F;
    const float *__restrict__ params;          // [R,2] fp32 or null
    const uint16_t *__restrict__ params_bf16;  // [R,2] bf16 or null
    const int32_t *__restrict__ work_range;    // [P+1] device
    int P;
    int bits;

    struct Edge {
        int loc;  // packed row * 8 + shift (shift is 0, 2, 4 or 6)
        float zp, sc, w;
    };
    static constexpr bool kDense = false;
    static size_t smem_bytes(int P) { return (size_t)(2 * (P + 1)) * sizeof(int); }
    // a gathered row is only F bytes (4 or 1 per lane and slot), so twice as many nonzeros are kept in flight;
    // the packed words wait in registers and are dequantised when they are consumed
    static constexpr int kBatch = 8;
    template <int VEC>
    struct Raw {
        uint32_t w;
    };

    // smem: wr[0..P], off[0..P] (packed-row offset of each peer)
    __device__ __forceinline__ void init_block(int *smem) const
    {
        int *swr = smem, *soff = smem + (P + 1);
        for (int i = threadIdx.x; i <= P; i += blockDim.x) swr[i] = work_range[i];
        __syncthreads();
        if (threadIdx.x == 0) {
            const int epb = 8 / bits;
            int acc = 0;
            for (int p = 0; p < P; ++p) {
                soff[p] = acc;
                acc += (swr[p + 1] - swr[p] + epb - 1) / epb;
            }
            soff[P] = acc;
        }
        __syncthreads();
    }

    __device__ __forceinline__ Edge stage(const int *__restrict__ col, const float *__restrict__ val, int64_t e,
                                          bool valid, const int *smem) const
    {
        Edge s;
        s.loc = 0; s.zp = 0.f; s.sc = 0.f; s.w = HAS_VAL ? 0.f : 1.f;
        if (valid) {
            const int c = ld_stream(col + e);
            if (HAS_VAL) s.w = ld_stream(val + e);
            const int *swr = smem, *soff = smem + (P + 1);
            int lo = 0, hi = P;  // largest p with wr[p] <= c
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (swr[mid] <= c) lo = mid; else hi = mid;
            }
            const int epb = 8 / bits;
            const int i = c - swr[lo];
            s.loc = ((soff[lo] + i / epb) << 3) | ((epb - 1 - i % epb) * bits);
            if (params) {
                const float2 t = __ldg(reinterpret_cast<const float2 *>(params) + c);
                s.zp = t.x; s.sc = t.y;
            } else {
                const uint32_t t = __ldg(reinterpret_cast<const uint32_t *>(params_bf16) + c);
                s.zp = bf16_bits_to_float((uint16_t)(t & 0xffffu));
                s.sc = bf16_bits_to_float((uint16_t)(t >> 16));
            }
        }
        return s;
    }
    __device__ __forceinline__ Edge bcast(const Edge &s, int j, unsigned mask, int width) const
    {
        Edge r;
        r.loc = __shfl_sync(mask, s.loc, j, width);
        r.zp = __shfl_sync(mask, s.zp, j, width);
        r.sc = __shfl_sync(mask, s.sc, j, width);
        r.w = 1.0f;
        if (HAS_VAL) r.w = __shfl_sync(mask, s.w, j, width);
        return r;
    }
    template <int VEC>
    __device__ __forceinline__ void load(const Edge &s, int n, Raw<VEC> &r) const
    {
        const uint8_t *p = packed + ((int64_t)(s.loc >> 3) * F + n);
        if constexpr (VEC == 4) r.w = __ldg(reinterpret_cast<const uint32_t *>(p));
        else r.w = __ldg(p);
    }
    template <int VEC>
    __device__ __forceinline__ void expand(const Edge &s, const Raw<VEC> &r, float (&x)[VEC]) const
    {
        const int shift = s.loc & 7;
        const unsigned m = (1u << bits) - 1u;
        if constexpr (VEC == 4) {
            // four codes per word: one shift + one mask for the word, then a byte permute drops each code into
            // the mantissa of 2^23 (exact int -> float: a permute and a subtract instead of shift/and/convert)
            const uint32_t t = (r.w >> shift) & (0x01010101u * m);
            x[0] = __fmaf_rn(__uint_as_float(__byte_perm(t, 0x4B000000u, 0x7650)) - 8388608.0f, s.sc, s.zp);
            x[1] = __fmaf_rn(__uint_as_float(__byte_perm(t, 0x4B000000u, 0x7651)) - 8388608.0f, s.sc, s.zp);
            x[2] = __fmaf_rn(__uint_as_float(__byte_perm(t, 0x4B000000u, 0x7652)) - 8388608.0f, s.sc, s.zp);
            x[3] = __fmaf_rn(__uint_as_float(__byte_perm(t, 0x4B000000u, 0x7653)) - 8388608.0f, s.sc, s.zp);
        } else {
            const float c = (float)((r.w >> shift) & m);
            x[0] = __fmaf_rn(c, s.sc, s.zp);
        }
    }
};

// Rows in the row-codes layout (rowcodes.cuh): operand row c owns F*BITS/8 contiguous bytes, so a gathered
// row costs exactly its codes (64 bytes at 2 bits and F = 256 against 256 bytes in the wire format above), there
// is no per-peer offset table, and the quad of four codes a lane needs is one 1-, 2- or 4-byte load.
template <bool HAS_VAL, int BITS>
struct RowCodesSrcT {
    const uint8_t *__restrict__ codes;
    int pitch;   // bytes per row = F * BITS / 8
    int lognv;   // log2 of the quads per lane (F / 128 for F > 128, else 0)
    const float *__restrict__ params;          // [R,2] fp32 or null
    const uint16_t *__restrict__ params_bf16;  // [R,2] bf16 or null

    struct Edge {
        int c;
        float zp, sc, w;
    };
    static constexpr bool kDense = false;
    static size_t smem_bytes(int) { return 0; }
    static constexpr int kBatch = 8;
    template <int VEC>
    struct Raw {
        uint32_t w;
    };
    __device__ __forceinline__ void init_block(int *) const {}

    __device__ __forceinline__ Edge stage(const int *__restrict__ col, const float *__restrict__ val, int64_t e,
                                          bool valid, const int *) const
    {
        Edge s;
        s.c = 0; s.zp = 0.f; s.sc = 0.f; s.w = HAS_VAL ? 0.f : 1.f;
        if (valid) {
            s.c = ld_stream(col + e);
            if (HAS_VAL) s.w = ld_stream(val + e);
            if (params) {
                const float2 t = __ldg(reinterpret_cast<const float2 *>(params) + s.c);
                s.zp = t.x; s.sc = t.y;
            } else {
                const uint32_t t = __ldg(reinterpret_cast<const uint32_t *>(params_bf16) + s.c);
                s.zp = bf16_bits_to_float((uint16_t)(t & 0xffffu));
                s.sc = bf16_bits_to_float((uint16_t)(t >> 16));
            }
        }
        return s;
    }
    __device__ __forceinline__ Edge bcast(const Edge &s, int j, unsigned mask, int width) const
    {
        Edge r;
        r.c = __shfl_sync(mask, s.c, j, width);
        r.zp = __shfl_sync(mask, s.zp, j, width);
        r.sc = __shfl_sync(mask, s.sc, j, width);
        r.w = 1.0f;
        if (HAS_VAL) r.w = __shfl_sync(mask, s.w, j, width);
        return r;
    }
    template <int VEC>
    __device__ __forceinline__ void load(const Edge &s, int n, Raw<VEC> &r) const
    {
        const uint8_t *p = codes + ((int64_t)s.c * pitch + rowcodes_quad_offset<BITS>(n >> 2, lognv));
        r.w = rowcodes_load_quad<BITS>(p);
        if constexpr (VEC == 1) r.w = (r.w >> ((n & 3) * BITS)) & ((1u << BITS) - 1u);  // scalar path: one code
    }
    template <int VEC>
    __device__ __forceinline__ void expand(const Edge &s, const Raw<VEC> &r, float (&x)[VEC]) const
    {
        if constexpr (VEC == 4) rowcodes_expand<BITS>(r.w, s.sc, s.zp, x);
        else x[0] = __fmaf_rn((float)r.w, s.sc, s.zp);
    }
};

// ---------------------------------------------------------------------------
// Inner loop: consume staged edges [j0, j1) of the current stage into acc.
// `lane_n` = first column of this lane inside the tile, `stride` = columns
// between two vector slots of the same lane (G*VEC).
// ---------------------------------------------------------------------------
template <class Src, int VEC, int NV>
__device__ __forceinline__ void consume(const Src &src, const typename Src::Edge &st, int j0, int j1, unsigned mask,
                                        int width, int lane_n, int stride, int N, float (&acc)[NV][VEC])
{
    constexpr int B = Src::kBatch;
    using Raw = typename Src::template Raw<VEC>;
    int j = j0;
    for (; j + B <= j1; j += B) {
        typename Src::Edge e[B];
        Raw r[B][NV];
#pragma unroll
        for (int b = 0; b < B; ++b) e[b] = src.bcast(st, j + b, mask, width);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int n = lane_n + i * stride;
            if (n < N) {
#pragma unroll
                for (int b = 0; b < B; ++b) src.template load<VEC>(e[b], n, r[b][i]);
            }
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int n = lane_n + i * stride;
            if (n < N) {
#pragma unroll
                for (int b = 0; b < B; ++b) {
                    float x[VEC];
                    src.template expand<VEC>(e[b], r[b][i], x);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) acc[i][k] = __fmaf_rn(e[b].w, x[k], acc[i][k]);
                }
            }
        }
    }
    for (; j < j1; ++j) {
        typename Src::Edge e0 = src.bcast(st, j, mask, width);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int n = lane_n + i * stride;
            if (n < N) {
                Raw r0;
                float x0[VEC];
                src.template load<VEC>(e0, n, r0);
                src.template expand<VEC>(e0, r0, x0);
#pragma unroll
                for (int k = 0; k < VEC; ++k) acc[i][k] = __fmaf_rn(e0.w, x0[k], acc[i][k]);
            }
        }
    }
}

// Narrow rows (N <= G*VEC*NV with G < 32): the warp's 32/G lane groups take alternate nonzeros of
// the staged range, so that 32/G times as many row loads are in flight per warp; every group
// accumulates a partial sum of the SAME output row, combined by the caller with warp shuffles.
template <class Src, int VEC, int NV, int G>
__device__ __forceinline__ void consume_grouped(const Src &src, const typename Src::Edge &st, int j0, int j1, int sg,
                                                int lane_n, int stride, int N, float (&acc)[NV][VEC])
{
    constexpr int B = Src::kBatch;
    constexpr int NG = 32 / G;
    using Raw = typename Src::template Raw<VEC>;
    for (int j = j0; j < j1; j += NG * B) {  // uniform over the warp
        typename Src::Edge e[B];
        bool ok[B];
        Raw r[B][NV];
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const int idx = j + b * NG + sg;
            ok[b] = idx < j1;
            e[b] = src.bcast(st, idx & 31, FULL, 32);
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int n = lane_n + i * stride;
            if (n < N) {
#pragma unroll
                for (int b = 0; b < B; ++b)
                    if (ok[b]) src.template load<VEC>(e[b], n, r[b][i]);
            }
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int n = lane_n + i * stride;
            if (n < N) {
#pragma unroll
                for (int b = 0; b < B; ++b) {
                    if (ok[b]) {
                        float x[VEC];
                        src.template expand<VEC>(e[b], r[b][i], x);
#pragma unroll
                        for (int k = 0; k < VEC; ++k) acc[i][k] = __fmaf_rn(e[b].w, x[k], acc[i][k]);
                    }
                }
            }
        }
    }
}

template <int VEC, int NV>
__device__ __forceinline__ void scale_acc(float (&acc)[NV][VEC], float s)
{
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[i][k] *= s;
}

enum class Out { Store, AddPlain, AddAtomic };

template <int VEC, int NV>
__device__ __forceinline__ void write_row(float *__restrict__ yrow, int lane_n, int stride, int N, float (&acc)[NV][VEC],
                                          Out mode)
{
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int n = lane_n + i * stride;
        if (n < N) {
            float *p = yrow + n;
            if constexpr (VEC == 4) {
                float4 a = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
                if (mode == Out::AddAtomic) {
                    red_add_v4(p, a);
                } else {
                    if (mode == Out::AddPlain) {
                        const float4 y = *reinterpret_cast<const float4 *>(p);
                        a.x += y.x; a.y += y.y; a.z += y.z; a.w += y.w;
                    }
                    *reinterpret_cast<float4 *>(p) = a;
                }
            } else {
                if (mode == Out::AddAtomic) red_add(p, acc[i][0]);
                else if (mode == Out::AddPlain) *p = *p + acc[i][0];
                else *p = acc[i][0];
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Row-split kernel: G lanes per row.
// ---------------------------------------------------------------------------
template <class Src, int VEC, int NV, int G, bool ROW_SCALE>
__global__ void __launch_bounds__(kSpmmThreads)
spmm_row_split_kernel(Src src, const int64_t *__restrict__ rowptr, const int *__restrict__ col,
                      const float *__restrict__ val, float *__restrict__ Y, int64_t ldy, int64_t M, int N,
                      int accumulate, const float *__restrict__ row_scale)
{
    extern __shared__ int smem[];
    src.init_block(smem);
    const int lane = threadIdx.x & 31;
    const int gl = lane & (G - 1);                   // lane inside the group
    const unsigned mask = (G == 32) ? FULL : (((1u << G) - 1u) << (lane & ~(G - 1)));
    const int n_base = blockIdx.y * (G * VEC * NV);
    const int lane_n = n_base + gl * VEC;
    constexpr int stride = G * VEC;
    const int64_t groups_per_block = kSpmmThreads / G;
    const int64_t row = (int64_t)blockIdx.x * groups_per_block + threadIdx.x / G;
    if (row >= M) return;

    float acc[NV][VEC];
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int k = 0; k < VEC; ++k) acc[i][k] = 0.f;

    const int64_t rs = __ldg(rowptr + row), re = __ldg(rowptr + row + 1);
    for (int64_t eb = rs; eb < re; eb += G) {
        const int64_t e = eb + gl;
        const typename Src::Edge st = src.stage(col, val, e, e < re, smem);
        const int cnt = (int)((re - eb) < G ? (re - eb) : G);
        consume<Src, VEC, NV>(src, st, 0, cnt, mask, G, lane_n, stride, N, acc);
    }
    if constexpr (ROW_SCALE) scale_acc<VEC, NV>(acc, __ldg(row_scale + row));
    write_row<VEC, NV>(Y + row * ldy, lane_n, stride, N, acc, accumulate ? Out::AddPlain : Out::Store);
}

// ---------------------------------------------------------------------------
// nnz-split kernel: a warp per chunk of kWarpChunk nonzeros.  Y must already hold
// the values to accumulate into (zeros for an overwrite).
// ---------------------------------------------------------------------------
// G = lanes that span one output row tile (G*VEC*NV columns): 32, or 16 / 8 for narrow rows, where the
// two / four lane groups of a warp share the nonzeros of a row (consume_grouped).
template <class Src, int VEC, int NV, bool ROW_SCALE, int G = 32>
__global__ void __launch_bounds__(kSpmmThreads)
spmm_nnz_split_kernel(Src src, const int64_t *__restrict__ rowptr, const int *__restrict__ col,
                      const float *__restrict__ val, int64_t nnz, float *__restrict__ Y, int64_t ldy, int64_t M, int N,
                      int y_is_zero, const float *__restrict__ row_scale, int64_t e0)
{
    // e0 = rowptr[0]: 0 for a whole matrix; for a range of rows of a larger matrix (rowptr points at the first
    // row of the range, col / val at the whole arrays) the position of the range's first nonzero
    extern __shared__ int smem[];
    src.init_block(smem);
    const int lane = threadIdx.x & 31;
    const int n_base = blockIdx.y * (G * VEC * NV);
    const int lane_n = n_base + (lane & (G - 1)) * VEC;
    constexpr int stride = G * VEC;
    const int64_t nchunks = (nnz + kWarpChunk - 1) / kWarpChunk;
    const int64_t warps_total = (int64_t)gridDim.x * (kSpmmThreads / 32);
    for (int64_t ch = (int64_t)blockIdx.x * (kSpmmThreads / 32) + (threadIdx.x >> 5); ch < nchunks; ch += warps_total) {
        const int64_t wB = e0 + ch * kWarpChunk;
        const int64_t wE = (wB + kWarpChunk < e0 + nnz) ? (wB + kWarpChunk) : (e0 + nnz);
        // row that contains nonzero wB (never an empty row)
        int64_t r = warp_upper_row(rowptr, M, wB, lane);
        bool starts_row = (__ldg(rowptr + r) == wB);
        int64_t e = wB, eb = wB;
        typename Src::Edge st = src.stage(col, val, eb + lane, eb + lane < wE, smem);
        while (e < wE) {
            // first row r' >= r whose end lies beyond e (skips empty rows 32 at a time)
            int64_t re;
            for (;;) {
                const int64_t idx = r + 1 + lane;
                const int64_t v = (idx <= M) ? __ldg(rowptr + idx) : INT64_MAX;
                const unsigned m = __ballot_sync(FULL, v > e);
                if (m) {
                    const int k = __ffs(m) - 1;
                    r += k;
                    re = __shfl_sync(FULL, v, k);
                    break;
                }
                r += 32;
            }
            if (r >= M) break;  // only with a malformed matrix (nnz beyond rowptr[M]): never write past Y
            const int64_t se = re < wE ? re : wE;
            const bool complete = starts_row && (se == re);
            float acc[NV][VEC];
#pragma unroll
            for (int i = 0; i < NV; ++i)
#pragma unroll
                for (int k = 0; k < VEC; ++k) acc[i][k] = 0.f;
            while (e < se) {
                if (e - eb == 32) {
                    eb += 32;
                    st = src.stage(col, val, eb + lane, eb + lane < wE, smem);
                }
                const int j0 = (int)(e - eb);
                const int j1 = (int)((se - eb) < 32 ? (se - eb) : 32);
                if constexpr (G == 32) {
                    consume<Src, VEC, NV>(src, st, j0, j1, FULL, 32, lane_n, stride, N, acc);
                } else {
                    consume_grouped<Src, VEC, NV, G>(src, st, j0, j1, lane / G, lane_n, stride, N, acc);
                }
                e = eb + j1;
            }
            if constexpr (G < 32) {  // sum the lane groups' partial rows (fixed order: deterministic)
#pragma unroll
                for (int o = G; o < 32; o <<= 1)
#pragma unroll
                    for (int i = 0; i < NV; ++i)
#pragma unroll
                        for (int k = 0; k < VEC; ++k) acc[i][k] += __shfl_xor_sync(FULL, acc[i][k], o);
            }
            if constexpr (ROW_SCALE) scale_acc<VEC, NV>(acc, __ldg(row_scale + r));  // partial rows too: it distributes
            if (G == 32 || lane < G)
                write_row<VEC, NV>(Y + r * ldy, lane_n, stride, N, acc,
                                   complete ? (y_is_zero ? Out::Store : Out::AddPlain) : Out::AddAtomic);
            starts_row = true;
            r += 1;
        }
    }
}

// ---------------------------------------------------------------------------
// nnz-split kernel with the gathered rows staged through shared memory.
//
// The kernels above land every gathered row in registers, so the bytes a warp can have in flight are bounded
// by its register budget (four rows per lane group) and the SM's by the occupancy those registers allow; the
// gather is latency bound well before HBM or L2 is busy.  Here every lane copies its 16-byte pieces of the
// rows with cp.async into a ring in shared memory that only it reads back (D groups of B rows in flight per
// warp, no landing registers, no cross-lane synchronisation: a lane waits for its own copies with
// cp.async.wait_group, a hardware wait), so the bytes in flight scale with shared memory instead.
// fp32 operand rows, 128-bit path (N % 4 == 0), one output row tile of 128 * NV columns per lane set.
//
// Measured on the 2.4 M-node / 116 M-edge R-MAT benchmark graph (B200): 10.2 ms at N = 256 against 9.5 ms for
// the register kernel, 6.7 against 4.4 ms at N = 128: more bytes in flight do not help, because the register
// kernel already moves 12.5-13.7 TB/s of gathered rows out of L2 (that rate, not latency, is what it sits on,
// next to 84 % of the HBM copy rate for the misses), and the shared-memory ring shrinks the L1 that serves the
// hub rows.  It is kept selectable (SGNN_SPMM_NNZ_SPLIT_STAGED) and tested, but nothing selects it by default.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src)
{
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_PENDING>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N_PENDING) : "memory");
}

template <int NV, int D, int B>
constexpr size_t staged_smem_per_warp()
{
    return (size_t)D * B * NV * 32 * 16 + kWarpChunk * 8;  // row ring + the chunk's columns and weights
}

template <bool HAS_VAL, bool COL_SCALE, int NV, bool ROW_SCALE, int D, int B>
__global__ void __launch_bounds__(kSpmmThreads)
spmm_nnz_split_staged_kernel(DenseSrcT<HAS_VAL, COL_SCALE> src, const int64_t *__restrict__ rowptr,
                             const int *__restrict__ col, const float *__restrict__ val, int64_t nnz,
                             float *__restrict__ Y, int64_t ldy, int64_t M, int N, int y_is_zero,
                             const float *__restrict__ row_scale, int64_t e0)
{
    using Src = DenseSrcT<HAS_VAL, COL_SCALE>;
    extern __shared__ __align__(16) unsigned char staged_smem[];
    const int lane = threadIdx.x & 31;
    unsigned char *mine = staged_smem + (threadIdx.x >> 5) * staged_smem_per_warp<NV, D, B>();
    float4 *ring = reinterpret_cast<float4 *>(mine);  // [D][B][NV][32 lanes]
    int *scol = reinterpret_cast<int *>(mine + (size_t)D * B * NV * 32 * 16);
    float *sw = reinterpret_cast<float *>(scol + kWarpChunk);
    const int n_base = blockIdx.y * (128 * NV);
    const int lane_n = n_base + lane * 4;
    const int64_t nchunks = (nnz + kWarpChunk - 1) / kWarpChunk;
    const int64_t warps_total = (int64_t)gridDim.x * (kSpmmThreads / 32);
    for (int64_t ch = (int64_t)blockIdx.x * (kSpmmThreads / 32) + (threadIdx.x >> 5); ch < nchunks; ch += warps_total) {
        const int64_t wB = e0 + ch * kWarpChunk;
        const int64_t wE = (wB + kWarpChunk < e0 + nnz) ? (wB + kWarpChunk) : (e0 + nnz);
        const int cnt = (int)(wE - wB);
        __syncwarp();  // every lane has finished with the previous chunk's columns
#pragma unroll
        for (int k = lane; k < kWarpChunk; k += 32) {
            const typename Src::Edge s = src.stage(col, val, wB + k, k < cnt, nullptr);
            scol[k] = s.c;
            if (HAS_VAL) sw[k] = s.w;
        }
        __syncwarp();
        const int nb = (cnt + B - 1) / B;
        auto issue = [&](int b) {  // start the copies of batch b (nothing for b >= nb) and close the group
            if (b < nb) {
#pragma unroll
                for (int j = 0; j < B; ++j) {
                    const int k = b * B + j;
                    if (k < cnt) {
                        const float *p = src.X + ((int64_t)scol[k] * src.ldx + lane_n);
#pragma unroll
                        for (int i = 0; i < NV; ++i)
                            if (lane_n + i * 128 < N) cp_async16(&ring[(((b % D) * B + j) * NV + i) * 32 + lane], p + i * 128);
                    }
                }
            }
            cp_async_commit();
        };
#pragma unroll
        for (int b = 0; b < D - 1; ++b) issue(b);

        int64_t r = warp_upper_row(rowptr, M, wB, lane);
        bool starts_row = (__ldg(rowptr + r) == wB);
        int64_t re = wB;  // end of the current row: found below for the first nonzero
        bool have_row = false, bad = false;
        float acc[NV][4];
        for (int b = 0; b < nb && !bad; ++b) {
            issue(b + D - 1);
            cp_async_wait<D - 1>();  // this lane's copies of batch b have landed
#pragma unroll
            for (int j = 0; j < B; ++j) {
                const int k = b * B + j;
                if (k >= cnt || bad) break;
                const int64_t e = wB + k;
                if (!have_row || e == re) {
                    if (have_row) {  // row r ends here: write it and move on
                        if constexpr (ROW_SCALE) scale_acc<4, NV>(acc, __ldg(row_scale + r));
                        write_row<4, NV>(Y + r * ldy, lane_n, 128, N, acc,
                                         starts_row ? (y_is_zero ? Out::Store : Out::AddPlain) : Out::AddAtomic);
                        starts_row = true;
                        r += 1;
                    }
                    for (;;) {  // first row r' >= r whose end lies beyond e (skips empty rows 32 at a time)
                        const int64_t idx = r + 1 + lane;
                        const int64_t v = (idx <= M) ? __ldg(rowptr + idx) : INT64_MAX;
                        const unsigned m = __ballot_sync(FULL, v > e);
                        if (m) {
                            const int q = __ffs(m) - 1;
                            r += q;
                            re = __shfl_sync(FULL, v, q);
                            break;
                        }
                        r += 32;
                    }
                    if (r >= M) {  // only with a malformed matrix (nonzeros beyond rowptr[M]): never write past Y
                        bad = true;
                        have_row = false;
                        break;
                    }
                    have_row = true;
#pragma unroll
                    for (int i = 0; i < NV; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
                }
                const float w = HAS_VAL ? sw[k] : 1.0f;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    if (lane_n + i * 128 < N) {
                        const float4 x = ring[(((b % D) * B + j) * NV + i) * 32 + lane];
                        acc[i][0] = __fmaf_rn(w, x.x, acc[i][0]);
                        acc[i][1] = __fmaf_rn(w, x.y, acc[i][1]);
                        acc[i][2] = __fmaf_rn(w, x.z, acc[i][2]);
                        acc[i][3] = __fmaf_rn(w, x.w, acc[i][3]);
                    }
                }
            }
        }
        cp_async_wait<0>();  // nothing of this chunk is still landing when the ring is reused
        if (have_row) {
            if constexpr (ROW_SCALE) scale_acc<4, NV>(acc, __ldg(row_scale + r));
            const bool complete = starts_row && (wE == re);
            write_row<4, NV>(Y + r * ldy, lane_n, 128, N, acc,
                             complete ? (y_is_zero ? Out::Store : Out::AddPlain) : Out::AddAtomic);
        }
    }
}

// Zero-fill of a pitched [M, N] block whose rows are 16-byte aligned (a column slice of a wider buffer).
static __global__ void zero_rows_vec4_kernel(float *__restrict__ Y, int64_t ldy, int64_t M, int n4)
{
    const int64_t total = M * n4;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / n4;
        const int c = (int)(i - r * n4) * 4;
        *reinterpret_cast<float4 *>(Y + r * ldy + c) = z;
    }
}

// ---------------------------------------------------------------------------
// Host-side dispatch shared by the fp32 and the packed-operand entry points.
// ---------------------------------------------------------------------------
template <class Src, int VEC, int NV, int G = 32>
int launch_nnz_split(const Src &src, size_t smem, const int64_t *rowptr, const int *col, const float *val, int64_t nnz,
                     float *Y, int64_t ldy, int64_t M, int N, int y_is_zero, const float *row_scale, cudaStream_t s,
                     int64_t e0)
{
    const int64_t nchunks = ceil_div(nnz, kWarpChunk);
    const int64_t blocks_needed = ceil_div(nchunks, kSpmmThreads / 32);
    // one chunk per warp while the grid stays small enough for the hardware block scheduler to
    // balance it; beyond that (a multiple of the SM count) the warps stride over the chunks
    int64_t gx = (int64_t)sm_count() * 2048;
    if (blocks_needed < gx) gx = blocks_needed;
    const int tile = G * VEC * NV;
    dim3 grid((unsigned)gx, (unsigned)ceil_div(N, tile));
    if (row_scale)
        spmm_nnz_split_kernel<Src, VEC, NV, true, G><<<grid, kSpmmThreads, smem, s>>>(src, rowptr, col, val, nnz, Y, ldy,
                                                                                      M, N, y_is_zero, row_scale, e0);
    else
        spmm_nnz_split_kernel<Src, VEC, NV, false, G><<<grid, kSpmmThreads, smem, s>>>(src, rowptr, col, val, nnz, Y,
                                                                                       ldy, M, N, y_is_zero, row_scale, e0);
    SGNN_LAUNCH_OK("spmm_nnz_split_kernel");
    return SGNN_OK;
}

// Rows staged through shared memory: D groups of B rows in flight per warp.
template <class Src, int NV, int D, int B>
int launch_nnz_split_staged(const Src &src, const int64_t *rowptr, const int *col, const float *val, int64_t nnz,
                            float *Y, int64_t ldy, int64_t M, int N, int y_is_zero, const float *row_scale,
                            cudaStream_t s, int64_t e0)
{
    if constexpr (Src::kDense) {
        constexpr size_t smem = staged_smem_per_warp<NV, D, B>() * (kSpmmThreads / 32);
        const int64_t nchunks = ceil_div(nnz, kWarpChunk);
        const int64_t blocks_needed = ceil_div(nchunks, kSpmmThreads / 32);
        int64_t gx = (int64_t)sm_count() * 2048;
        if (blocks_needed < gx) gx = blocks_needed;
        dim3 grid((unsigned)gx, (unsigned)ceil_div(N, 128 * NV));
        auto go = [&](auto kernel) -> int {
            SGNN_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            kernel<<<grid, kSpmmThreads, smem, s>>>(src, rowptr, col, val, nnz, Y, ldy, M, N, y_is_zero, row_scale, e0);
            SGNN_LAUNCH_OK("spmm_nnz_split_staged_kernel");
            return SGNN_OK;
        };
        if (row_scale) return go(spmm_nnz_split_staged_kernel<Src::kHasVal, Src::kColScale, NV, true, D, B>);
        return go(spmm_nnz_split_staged_kernel<Src::kHasVal, Src::kColScale, NV, false, D, B>);
    } else {
        set_error("spmm: the staged kernel takes fp32 operand rows only");
        return SGNN_ERR_UNSUPPORTED;
    }
}

template <class Src, int VEC, int NV, int G>
int launch_row_split(const Src &src, size_t smem, const int64_t *rowptr, const int *col, const float *val, float *Y,
                     int64_t ldy, int64_t M, int N, int accumulate, const float *row_scale, cudaStream_t s)
{
    const int64_t rows_per_block = kSpmmThreads / G;
    const int64_t gx = ceil_div(M, rows_per_block);
    SGNN_REQUIRE(gx <= 2147483647LL, SGNN_ERR_TOO_LARGE, "spmm: too many rows for one launch");
    const int tile = G * VEC * NV;
    dim3 grid((unsigned)gx, (unsigned)ceil_div(N, tile));
    if (row_scale)
        spmm_row_split_kernel<Src, VEC, NV, G, true><<<grid, kSpmmThreads, smem, s>>>(src, rowptr, col, val, Y, ldy, M,
                                                                                      N, accumulate, row_scale);
    else
        spmm_row_split_kernel<Src, VEC, NV, G, false><<<grid, kSpmmThreads, smem, s>>>(src, rowptr, col, val, Y, ldy, M,
                                                                                       N, accumulate, row_scale);
    SGNN_LAUNCH_OK("spmm_row_split_kernel");
    return SGNN_OK;
}

// vec4 == true requires N % 4 == 0 and 16-byte aligned rows on both operands.
template <class Src>
int spmm_dispatch(const Src &src, size_t smem, const int64_t *rowptr, const int *col, const float *val, int64_t nnz,
                  float *Y, int64_t ldy, int64_t M, int64_t N64, int accumulate, int algo, bool vec4,
                  const float *row_scale, cudaStream_t s, int64_t e0 = 0)
{
    const int N = (int)N64;
    if (M == 0 || N == 0) return SGNN_OK;
    if (algo == SGNN_SPMM_AUTO) algo = SGNN_SPMM_NNZ_SPLIT;
    // staged variant: fp32 operand, 128-bit path, more than 64 columns; anything else takes the register kernel
    bool staged = false;
    if (algo == SGNN_SPMM_NNZ_SPLIT_STAGED) {
        staged = Src::kDense && vec4 && N > 64 && N <= 512;
        algo = SGNN_SPMM_NNZ_SPLIT;
    }
    if (algo == SGNN_SPMM_NNZ_SPLIT) {
        if (!accumulate) {
            if (ldy == N) {
                SGNN_CUDA_OK(cudaMemsetAsync(Y, 0, (size_t)M * N * sizeof(float), s));
            } else if (vec4) {
                zero_rows_vec4_kernel<<<sm_count() * 8, 256, 0, s>>>(Y, ldy, M, N / 4);
                SGNN_LAUNCH_OK("zero_rows_vec4_kernel");
            } else {
                SGNN_CUDA_OK(cudaMemset2DAsync(Y, (size_t)ldy * sizeof(float), 0, (size_t)N * sizeof(float), (size_t)M, s));
            }
        }
        if (nnz == 0) return SGNN_OK;
        const int zero = accumulate ? 0 : 1;
        if (staged) {
            // ring of 4 groups of 2 rows per warp: the shape that kept three blocks resident per SM and came closest
            // to the register kernel (deeper or wider rings left one block per SM and were 1.6-1.9x slower)
            if (N <= 128) return launch_nnz_split_staged<Src, 1, 4, 2>(src, rowptr, col, val, nnz, Y, ldy, M, N, zero, row_scale, s, e0);
            if (N <= 256) return launch_nnz_split_staged<Src, 2, 4, 2>(src, rowptr, col, val, nnz, Y, ldy, M, N, zero, row_scale, s, e0);
            return launch_nnz_split_staged<Src, 4, 2, 2>(src, rowptr, col, val, nnz, Y, ldy, M, N, zero, row_scale, s, e0);
        }
        if (vec4) {
            if (N <= 32) return launch_nnz_split<Src, 4, 1, 8>(src, smem, rowptr, col, val, nnz, Y, ldy, M, N, zero, row_scale, s, e0);
            // 33..64 columns: two groups of 16 lanes with one slot each beat four groups of 8 lanes with two slots
            // (4.7 against 5.2 ms at N = 48 on the 116 M-edge benchmark graph; batches of 2 or 8 rows were no better)
            if (N <= 64) return launch_nnz_split<Src, 4, 1, 16>(src, smem, rowptr, col, val, nnz, Y, ldy, M, N, zero, row_scale, s, e0);
            if (N <= 128) return launch_nnz_split<Src, 4, 1>(src, smem, rowptr, col, val, nnz, Y, ldy, M, N, zero, row_scale, s, e0);
            if (N <= 256) return launch_nnz_split<Src, 4, 2>(src, smem, rowptr, col, val, nnz, Y, ldy, M, N, zero, row_scale, s, e0);
            return launch_nnz_split<Src, 4, 4>(src, smem, rowptr, col, val, nnz, Y, ldy, M, N, zero, row_scale, s, e0);
        }
        if (N <= 32) return launch_nnz_split<Src, 1, 1>(src, smem, rowptr, col, val, nnz, Y, ldy, M, N, zero, row_scale, s, e0);
        if (N <= 64) return launch_nnz_split<Src, 1, 2>(src, smem, rowptr, col, val, nnz, Y, ldy, M, N, zero, row_scale, s, e0);
        return launch_nnz_split<Src, 1, 4>(src, smem, rowptr, col, val, nnz, Y, ldy, M, N, zero, row_scale, s, e0);
    }
    if (algo == SGNN_SPMM_ROW_SPLIT) {
        if (vec4) {
            if (N <= 32) return launch_row_split<Src, 4, 1, 8>(src, smem, rowptr, col, val, Y, ldy, M, N, accumulate, row_scale, s);
            if (N <= 64) return launch_row_split<Src, 4, 1, 16>(src, smem, rowptr, col, val, Y, ldy, M, N, accumulate, row_scale, s);
            if (N <= 128) return launch_row_split<Src, 4, 1, 32>(src, smem, rowptr, col, val, Y, ldy, M, N, accumulate, row_scale, s);
            if (N <= 256) return launch_row_split<Src, 4, 2, 32>(src, smem, rowptr, col, val, Y, ldy, M, N, accumulate, row_scale, s);
            return launch_row_split<Src, 4, 4, 32>(src, smem, rowptr, col, val, Y, ldy, M, N, accumulate, row_scale, s);
        }
        if (N <= 8) return launch_row_split<Src, 1, 1, 8>(src, smem, rowptr, col, val, Y, ldy, M, N, accumulate, row_scale, s);
        if (N <= 16) return launch_row_split<Src, 1, 1, 16>(src, smem, rowptr, col, val, Y, ldy, M, N, accumulate, row_scale, s);
        if (N <= 32) return launch_row_split<Src, 1, 1, 32>(src, smem, rowptr, col, val, Y, ldy, M, N, accumulate, row_scale, s);
        if (N <= 64) return launch_row_split<Src, 1, 2, 32>(src, smem, rowptr, col, val, Y, ldy, M, N, accumulate, row_scale, s);
        return launch_row_split<Src, 1, 4, 32>(src, smem, rowptr, col, val, Y, ldy, M, N, accumulate, row_scale, s);
    }
    set_error("spmm: unknown algo %d", algo);
    return SGNN_ERR_INVALID_ARGUMENT;
}

}  // namespace sgnn
