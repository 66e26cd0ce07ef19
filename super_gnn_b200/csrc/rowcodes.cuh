// "Row codes": the layout in which quantised boundary rows are kept on the GPU when both ends of the
// exchange are this library.
//
// The reference's wire format interleaves EPB = 8/bits rows in every byte (row-group packing), so a
// consumer that needs ONE row — the gather of a fused dequantise-SpMM — still moves F bytes per row at
// every bit width.  Here every row owns F*bits/8 contiguous bytes, so a gathered row costs exactly its
// codes.  The codes themselves are the reference's (same min / scale / rounding); only their position
// differs, and the permutation back to the reference bytes is exact (tests check it against the oracle).
//
//   quad q = features 4q .. 4q+3, stored as one little-endian field of 4*bits bits (feature j of the quad
//   at bit j*bits); a row has Q = F/4 quads;
//   position of quad q inside the row: q for F <= 128, else (q % 32) * NV + q / 32 with NV = F / 128:
//   the NV quads a lane of a warp owns (columns lane*4 + i*128) are adjacent, so the lane reads or
//   writes them with one access and a warp covers the row with one contiguous access;
//   row r starts at byte r * F*bits/8; there is no per-peer padding, rows are indexed as the fp32 rows are.
//
// Supported widths: F % 4 == 0 and (F <= 128 or F == 256 or F == 512).
#pragma once
#include "common.cuh"

namespace sgnn {

inline bool rowcodes_width_ok(int64_t F) { return F > 0 && F % 4 == 0 && (F <= 128 || F == 256 || F == 512); }
inline int rowcodes_nv(int64_t F) { return F <= 128 ? 1 : (int)(F / 128); }

#ifdef __CUDACC__

// four codes, one per byte (each < 2^BITS)  ->  one field of 4*BITS bits
template <int BITS>
__device__ __forceinline__ uint32_t rowcodes_compress(uint32_t w)
{
    if constexpr (BITS == 8) return w;
    else if constexpr (BITS == 4) return (w & 0xFu) | ((w >> 4) & 0xF0u) | ((w >> 8) & 0xF00u) | ((w >> 12) & 0xF000u);
    else return (w & 0x3u) | ((w >> 6) & 0xCu) | ((w >> 12) & 0x30u) | ((w >> 18) & 0xC0u);
}

// one quad field -> four dequantised values fma(code, scale, zero_point).  The int -> float conversion is a
// mask-and-or that drops the code into the mantissa of 2^(23-s) where it sits (s = its bit offset), and one
// exact subtraction; no shift, no convert instruction.
template <int BITS>
__device__ __forceinline__ void rowcodes_expand(uint32_t q, float sc, float zp, float (&x)[4])
{
    if constexpr (BITS == 8) {
        x[0] = __fmaf_rn(__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7650)) - 8388608.0f, sc, zp);
        x[1] = __fmaf_rn(__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7651)) - 8388608.0f, sc, zp);
        x[2] = __fmaf_rn(__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7652)) - 8388608.0f, sc, zp);
        x[3] = __fmaf_rn(__uint_as_float(__byte_perm(q, 0x4B000000u, 0x7653)) - 8388608.0f, sc, zp);
    } else {
        constexpr uint32_t M = (1u << BITS) - 1u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int s = j * BITS;
            const float f = __uint_as_float((q & (M << s)) | (0x4B000000u - ((uint32_t)s << 23)));
            x[j] = __fmaf_rn(f - (float)(1u << (23 - s)), sc, zp);
        }
    }
}

// byte offset of quad `q` (0-based) inside a row; lognv = log2(NV)
template <int BITS>
__device__ __forceinline__ int rowcodes_quad_offset(int q, int lognv)
{
    const int pos = lognv ? (((q & 31) << lognv) + (q >> 5)) : q;
    return pos * (BITS / 2);
}

template <int BITS>
__device__ __forceinline__ uint32_t rowcodes_load_quad(const uint8_t *p)
{
    if constexpr (BITS == 8) return __ldg(reinterpret_cast<const uint32_t *>(p));
    else if constexpr (BITS == 4) return (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(p));
    else return (uint32_t)__ldg(p);
}

#endif  // __CUDACC__
}  // namespace sgnn
