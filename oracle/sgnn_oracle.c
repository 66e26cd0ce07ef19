/*
 * CPU restatement of the reference's GraphSAGE hot-path arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY: this file is the checker the CUDA path is compared
 * against (tests, the smoke check and the timed CPU baseline).  Nothing in the
 * product package links, loads or calls it.
 *
 * Parity status: PINNED.  Every function here is checked bit-for-bit against
 * the reference's own x86 ops compiled from their sources (oracle/build_ref.py)
 * and against the byte-exact vectors in the reference's tests/test_quantizer.py
 * (see tests/test_oracle_pins.py and tests/golden/).  The only function with no
 * compilable counterpart on x86 is the per-peer ("for_all_procs") packing,
 * which exists in the SVE build only; it is pinned segment by segment against
 * the x86 quantize_tensor exactly as the reference's own
 * tests/test_quantization_ops.py:214-228 does.
 *
 * Citations are file:line inside the reference project.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -mfma -shared -fPIC sgnn_oracle.c -lm
 * (contraction is off so that a fused multiply-add appears exactly where fmaf is
 * written and nowhere else).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

/* ------------------------------------------------------------------------- */
/* SpMM: out[m,:] += sum_e value[e] * mat[col[e],:]                           */
/* super_gnn/ops/csrc/spmm.cpp:87-162 (kernel_1xN: accumulators are loaded     */
/* from `out`, one fused multiply-add per nonzero in CSR order, then stored)   */
/* and :483-511 (row loop).  `value == NULL` means all ones.                   */
/* ------------------------------------------------------------------------- */
API int oracle_spmm_csr_f32(const int64_t *rowptr, const int64_t *col, const float *value,
                            const float *mat, float *out, int64_t M, int64_t N)
{
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t m = 0; m < M; ++m) {
        float *o = out + m * N;
        for (int64_t e = rowptr[m]; e < rowptr[m + 1]; ++e) {
            const float v = value ? value[e] : 1.0f;
            const float *x = mat + col[e] * N;
            for (int64_t n = 0; n < N; ++n) o[n] = fmaf(v, x[n], o[n]);
        }
    }
    return 0;
}

/* Greedy nnz-balanced split of the rows over T workers.                       */
/* super_gnn/ops/spmm_kernel.py:8-29 (value sums per row are the "flops").     */
API void oracle_distribute_work_for_row(const int64_t *rowptr, const float *value, int64_t M, int T,
                                        int32_t *row_splits)
{
    /* the reference sums per row in fp32 (segment_csr) and then over rows */
    float totalf = 0.0f;
    for (int64_t m = 0; m < M; ++m) {
        float s = 0.0f;
        for (int64_t e = rowptr[m]; e < rowptr[m + 1]; ++e) s += value[e];
        totalf += s;
    }
    const float target = floorf(totalf / (float)T);
    for (int t = 0; t <= T; ++t) row_splits[t] = (int32_t)M;
    row_splits[0] = 0;
    float cur = 0.0f;
    int tid = 0;
    for (int64_t m = 0; m < M; ++m) {
        float s = 0.0f;
        for (int64_t e = rowptr[m]; e < rowptr[m + 1]; ++e) s += value[e];
        cur += s;
        if (cur > target && tid < T) {
            row_splits[tid + 1] = (int32_t)m;
            ++tid;
            cur = s;
        }
    }
    row_splits[T] = (int32_t)M;
}

/* ------------------------------------------------------------------------- */
/* Per-row min-max parameters.                                                 */
/* super_gnn/ops/csrc/quantization_arm.cpp:93-113: zero_point = row minimum,   */
/* scale = (max - min) / (2^bits - 1), a zero scale becomes 1.  Comparisons    */
/* are plain `>` / `<`, so the first of equal values wins.                     */
/* ------------------------------------------------------------------------- */
static inline void row_params(const float *x, int64_t F, int bits, float *zp, float *scale)
{
    float mx = x[0], mn = x[0];
    for (int64_t k = 1; k < F; ++k) {
        const float v = x[k];
        if (v > mx) mx = v;
        if (v < mn) mn = v;
    }
    float s = (mx - mn) / (float)((1 << bits) - 1);
    if (s == 0.0f) s = 1.0f;
    *zp = mn;
    *scale = s;
}

API void oracle_row_params(const float *x, int64_t S, int64_t F, int bits, float *params)
{
#pragma omp parallel for
    for (int64_t r = 0; r < S; ++r) row_params(x + r * F, F, bits, params + 2 * r, params + 2 * r + 1);
}

/* Code of one element: IEEE fp32 subtract, IEEE fp32 divide, round half to    */
/* even.  quantization_x86.cpp:73 (_mm512_div_ps + _MM_FROUND_TO_NEAREST_INT), */
/* :93 (std::nearbyint), quantization_arm.cpp:293 (svdiv + svrintn remainder   */
/* path).  The SVE main loop's reciprocal *estimate* (:157-165) is ISA-defined  */
/* and is deliberately not the parity target.                                  */
static inline int32_t code_of(float x, float zp, float scale)
{
    return (int32_t)nearbyintf((x - zp) / scale);
}

/* ------------------------------------------------------------------------- */
/* x86 row-group packing with caller-supplied min/scale.                       */
/* super_gnn/ops/csrc/quantization_x86.cpp:17-102.  EPB = 8/bits consecutive   */
/* rows share one packed row; row i of a group sits at shift (EPB-1-i)*bits;   */
/* the int32 OR of the shifted codes is truncated to its low byte (:81).       */
/* ------------------------------------------------------------------------- */
API int oracle_quantize_tensor(const float *x, int64_t S, int64_t F, const float *mn, const float *scale,
                               int bits, uint8_t *out)
{
    if (bits <= 0 || 8 % bits != 0) return 1;
    const int epb = 8 / bits;
    const int64_t groups = ceil_div64(S, epb);
#pragma omp parallel for
    for (int64_t g = 0; g < groups; ++g) {
        const int64_t r0 = g * epb;
        const int nr = (int)((S - r0) < epb ? (S - r0) : epb);
        for (int64_t k = 0; k < F; ++k) {
            int32_t acc = 0;
            for (int j = 0; j < nr; ++j) {
                const int32_t c = code_of(x[(r0 + j) * F + k], mn[r0 + j], scale[r0 + j]);
                acc |= (int32_t)((uint32_t)c << ((epb - 1 - j) * bits));
            }
            out[g * F + k] = (uint8_t)acc;
        }
    }
    return 0;
}

/* super_gnn/ops/csrc/quantization_x86.cpp:104-168; `val * scale + min` is      */
/* compiled as one fused multiply-add in the reference's -O3 AVX-512 build (and */
/* is an explicit svmla in quantization_arm.cpp:349-352).                      */
API int oracle_dequantize_tensor(const uint8_t *in, int64_t S, int64_t F, const float *mn,
                                 const float *scale, int bits, float *out)
{
    if (bits <= 0 || 8 % bits != 0) return 1;
    const int epb = 8 / bits;
    const int mask = (1 << bits) - 1;
#pragma omp parallel for
    for (int64_t r = 0; r < S; ++r) {
        const int64_t g = r / epb;
        const int sh = (epb - 1 - (int)(r % epb)) * bits;
        for (int64_t k = 0; k < F; ++k) {
            const float c = (float)((in[g * F + k] >> sh) & mask);
            out[r * F + k] = fmaf(c, scale[r], mn[r]);
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* Per-peer packing ("for_all_procs"): the wire format of the boundary         */
/* exchange.  super_gnn/ops/csrc/quantization_arm.cpp:496-578 (entry),         */
/* :21-77 (per-peer packed offsets: off_p = sum_{q<p} ceil(n_q / EPB)),        */
/* :79-301 (encode), buffers from super_gnn/data_manager/CommBuffer.py:28-48.  */
/* Peer p owns input rows [wr[p], wr[p+1]); inside a peer the rows are packed  */
/* EPB at a time, the last group zero-padded.  params[r] = (zero_point, scale). */
/* ------------------------------------------------------------------------- */
API int64_t oracle_packed_rows(const int32_t *wr, int P, int bits)
{
    const int epb = 8 / bits;
    int64_t tot = 0;
    for (int p = 0; p < P; ++p) tot += ceil_div64((int64_t)wr[p + 1] - wr[p], epb);
    return tot;
}

API int oracle_quantize_for_all_procs(const float *x, int64_t F, const int32_t *wr, int P, int bits,
                                      uint8_t *out, float *params)
{
    if (bits <= 0 || 8 % bits != 0) return 1;
    const int epb = 8 / bits;
    int64_t off = 0;
    for (int p = 0; p < P; ++p) {
        const int64_t b = wr[p], n = (int64_t)wr[p + 1] - wr[p];
        const int64_t groups = ceil_div64(n, epb);
#pragma omp parallel for
        for (int64_t g = 0; g < groups; ++g) {
            const int64_t r0 = b + g * epb;
            const int nr = (int)((b + n - r0) < epb ? (b + n - r0) : epb);
            for (int j = 0; j < nr; ++j)
                row_params(x + (r0 + j) * F, F, bits, params + 2 * (r0 + j), params + 2 * (r0 + j) + 1);
            for (int64_t k = 0; k < F; ++k) {
                int32_t acc = 0;
                for (int j = 0; j < nr; ++j) {
                    const int32_t c = code_of(x[(r0 + j) * F + k], params[2 * (r0 + j)], params[2 * (r0 + j) + 1]);
                    acc |= (int32_t)((uint32_t)c << ((epb - 1 - j) * bits));
                }
                out[(off + g) * F + k] = (uint8_t)acc;
            }
        }
        off += groups;
    }
    return 0;
}

/* super_gnn/ops/csrc/quantization_arm.cpp:580-633, 303-431:                   */
/* x = zero_point + code * scale as one fused multiply-add (svmla, :349-352).  */
API int oracle_dequantize_for_all_procs(const uint8_t *in, const float *params, int64_t F, const int32_t *wr,
                                        int P, int bits, float *out)
{
    if (bits <= 0 || 8 % bits != 0) return 1;
    const int epb = 8 / bits;
    const int mask = (1 << bits) - 1;
    int64_t off = 0;
    for (int p = 0; p < P; ++p) {
        const int64_t b = wr[p], n = (int64_t)wr[p + 1] - wr[p];
#pragma omp parallel for
        for (int64_t i = 0; i < n; ++i) {
            const int64_t r = b + i, g = off + i / epb;
            const int sh = (epb - 1 - (int)(i % epb)) * bits;
            const float zp = params[2 * r], sc = params[2 * r + 1];
            for (int64_t k = 0; k < F; ++k)
                out[r * F + k] = fmaf((float)((in[g * F + k] >> sh) & mask), sc, zp);
        }
        off += ceil_div64(n, epb);
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* v1: per-row bit width, packing along the feature axis.                      */
/* super_gnn/ops/csrc/quantization_x86.cpp:170-253 and :255-312;               */
/* params[r] = (bits, zero_point, scale); range[r] = first output byte of row r */
/* (super_gnn/quantizer.py:66-73).  First element of a byte in the high bits.  */
/* The decode is `val*scale+zp` (8-bit: quantization_kernel_x86.h:42-75 as a   */
/* multiply and an add intrinsic); g++ -O3 contracts both forms into one fused */
/* multiply-add, which is what the compiled reference returns.                 */
/* ------------------------------------------------------------------------- */
API int oracle_quantize_v1(const float *x, int64_t S, int64_t F, const int64_t *range, float *params,
                           uint8_t *out)
{
    int bad = 0;
    for (int64_t r = 0; r < S; ++r) {
        const int bits = (int)params[3 * r];
        if (bits != 8 && bits != 4 && bits != 2) { bad = 1; continue; }
        float zp, sc;
        row_params(x + r * F, F, bits, &zp, &sc);
        params[3 * r + 1] = zp;
        params[3 * r + 2] = sc;
        const int epb = 8 / bits;
        for (int64_t k0 = 0; k0 < F; k0 += epb) {
            const int nk = (int)((F - k0) < epb ? (F - k0) : epb);
            int32_t acc = 0;
            for (int j = 0; j < nk; ++j)
                acc |= (int32_t)((uint32_t)code_of(x[r * F + k0 + j], zp, sc) << ((epb - 1 - j) * bits));
            out[range[r] + k0 / epb] = (uint8_t)acc;
        }
    }
    return bad;
}

API int oracle_dequantize_v1(const uint8_t *in, int64_t S, int64_t F, const int64_t *range,
                             const float *params, float *out)
{
    int bad = 0;
    for (int64_t r = 0; r < S; ++r) {
        const int bits = (int)params[3 * r];
        if (bits != 8 && bits != 4 && bits != 2) { bad = 1; continue; }
        const float zp = params[3 * r + 1], sc = params[3 * r + 2];
        const int epb = 8 / bits, mask = (1 << bits) - 1;
        const int64_t nbytes = range[r + 1] - range[r];
        for (int64_t b = 0; b < nbytes; ++b) {
            const uint8_t pv = in[range[r] + b];
            for (int j = 0; j < epb && b * epb + j < F; ++j) {
                const float c = (float)((pv >> ((epb - 1 - j) * bits)) & mask);
                const float v = fmaf(c, sc, zp);
                out[r * F + b * epb + j] = v;
            }
        }
    }
    return bad;
}

/* ------------------------------------------------------------------------- */
/* v2: torch.quantize_per_channel-compatible layout.                           */
/* super_gnn/ops/csrc/quantization_x86.cpp:314-388 (encode: lrintf(x*(1/scale) */
/* + zero_point), first element in the LOW bits) and :390-459 (decode:         */
/* (code - zero_point) * scale).                                               */
/* ------------------------------------------------------------------------- */
API int oracle_quantize_v2_torch(const float *x, int64_t S, int64_t F, const int64_t *range,
                                 const float *zero_points, const float *scales, int bits, uint8_t *out)
{
    if (bits <= 0 || 8 % bits != 0) return 1;
    const int epb = 8 / bits;
    for (int64_t r = 0; r < S; ++r) {
        const float zp = zero_points[r], sc = scales[r];
        const float inv = sc == 0.0f ? 1.0f : 1.0f / sc;
        for (int64_t k0 = 0; k0 < F; k0 += epb) {
            const int nk = (int)((F - k0) < epb ? (F - k0) : epb);
            uint8_t acc = 0;
            for (int j = 0; j < nk; ++j) {
                const int32_t c = (int32_t)lrintf(fmaf(x[r * F + k0 + j], inv, zp));
                acc |= (uint8_t)((uint8_t)c << (j * bits));
            }
            out[range[r] + k0 / epb] = acc;
        }
    }
    return 0;
}

API int oracle_dequantize_v2_torch(const uint8_t *in, int64_t S, int64_t F, const int64_t *range,
                                   const float *zero_points, const float *scales, int bits, float *out)
{
    if (bits <= 0 || 8 % bits != 0) return 1;
    const int epb = 8 / bits, mask = (1 << bits) - 1;
    for (int64_t r = 0; r < S; ++r) {
        const float zp = zero_points[r], sc = scales[r];
        const int64_t nbytes = range[r + 1] - range[r];
        for (int64_t b = 0; b < nbytes; ++b) {
            const uint8_t pv = in[range[r] + b];
            for (int j = 0; j < epb && b * epb + j < F; ++j) {
                const float c = (float)((pv >> (j * bits)) & mask);
                out[r * F + b * epb + j] = (c - zp) * sc;
            }
        }
    }
    return 0;
}

/* Round-to-nearest-even fp32 -> bf16 -> fp32, the trip the (zero_point, scale) */
/* pairs make on the wire (super_gnn/communicator.py:283-294).                  */
API void oracle_round_bf16(const float *in, int64_t n, float *out)
{
    for (int64_t i = 0; i < n; ++i) {
        uint32_t u;
        memcpy(&u, in + i, 4);
        if ((u & 0x7fffffffu) > 0x7f800000u) {
            u |= 0x00400000u; /* quiet NaN */
            u &= 0xffff0000u;
        } else {
            u += 0x7fffu + ((u >> 16) & 1u);
            u &= 0xffff0000u;
        }
        memcpy(out + i, &u, 4);
    }
}
