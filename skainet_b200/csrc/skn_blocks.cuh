// Device-side decoders for the GGUF block types.
//
// Every type splits into "groups" of 32 weights that are contiguous in the row and share
// their scale arithmetic:
//   Q4_0 / Q8_0 : group = block (18 / 34 bytes)
//   Q4_K        : group = sub-block j of a 144-byte super-block (8 per block)
//   Q6_K        : group = (half h, quarter g) of a 210-byte super-block (8 per block)
//   Q4_1 / Q5_0 / Q5_1 : group = block (20 / 22 / 24 bytes); Q5_K: sub-block of a 176-byte super-block
// decode_group<T>() returns the 32 fp32 weights of one group, evaluated in the order that
// makes them bit-identical to gguf-py: (d*sc)*q - dmin*m for Q4_K, (d*sc)*(q-32) for Q6_K,
// q*d for Q8_0, (q-8)*d for Q4_0.  __fmul_rn / __fsub_rn keep the compiler from fusing or
// reassociating.  Byte-granular loads only: a group may start at any address.
#pragma once
#include "skn_internal.cuh"

template <int TYPE> struct BlockTraits;
template <> struct BlockTraits<SKN_TYPE_Q4_0> { static constexpr int ELEMS = 32,  BYTES = 18;  };
template <> struct BlockTraits<SKN_TYPE_Q8_0> { static constexpr int ELEMS = 32,  BYTES = 34;  };
template <> struct BlockTraits<SKN_TYPE_Q4_K> { static constexpr int ELEMS = 256, BYTES = 144; };
template <> struct BlockTraits<SKN_TYPE_Q6_K> { static constexpr int ELEMS = 256, BYTES = 210; };
template <> struct BlockTraits<SKN_TYPE_Q4_1> { static constexpr int ELEMS = 32,  BYTES = 20;  };
template <> struct BlockTraits<SKN_TYPE_Q5_0> { static constexpr int ELEMS = 32,  BYTES = 22;  };
template <> struct BlockTraits<SKN_TYPE_Q5_1> { static constexpr int ELEMS = 32,  BYTES = 24;  };
template <> struct BlockTraits<SKN_TYPE_Q5_K> { static constexpr int ELEMS = 256, BYTES = 176; };

__device__ __forceinline__ float skn_half_bits_to_float(uint32_t h) {
    return __half2float(__ushort_as_half((unsigned short)h));
}

__device__ __forceinline__ uint32_t skn_ld16(const uint8_t *p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8);
}

// 6-bit scale / min of sub-block j of a Q4_K block from its 12 packed bytes
__device__ __forceinline__ void skn_q4k_scale_min(const uint8_t *s, int j, int &sc, int &mn) {
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

// `row` points at the first block of a row, `g` is the group index within the row.
template <int TYPE>
__device__ __forceinline__ void decode_group(const uint8_t *row, int64_t g, float (&w)[32]);

template <>
__device__ __forceinline__ void decode_group<SKN_TYPE_Q4_0>(const uint8_t *row, int64_t g, float (&w)[32]) {
    const uint8_t *b = row + g * 18;
    const float d = skn_half_bits_to_float(skn_ld16(b));
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const int v = b[2 + e];
        w[e]      = __fmul_rn((float)((v & 15) - 8), d);
        w[e + 16] = __fmul_rn((float)((v >> 4) - 8), d);
    }
}

template <>
__device__ __forceinline__ void decode_group<SKN_TYPE_Q8_0>(const uint8_t *row, int64_t g, float (&w)[32]) {
    const uint8_t *b = row + g * 34;
    const float d = skn_half_bits_to_float(skn_ld16(b));
#pragma unroll
    for (int e = 0; e < 32; ++e) w[e] = __fmul_rn((float)(int8_t)b[2 + e], d);
}

template <>
__device__ __forceinline__ void decode_group<SKN_TYPE_Q4_K>(const uint8_t *row, int64_t g, float (&w)[32]) {
    const uint8_t *b = row + (g >> 3) * 144;
    const int j = (int)(g & 7);
    const float d = skn_half_bits_to_float(skn_ld16(b));
    const float dmin = skn_half_bits_to_float(skn_ld16(b + 2));
    int sc, mn;
    skn_q4k_scale_min(b + 4, j, sc, mn);
    const float dl = __fmul_rn(d, (float)sc);
    const float ml = __fmul_rn(dmin, (float)mn);
    const uint8_t *q = b + 16 + 32 * (j >> 1);
    const int sh = (j & 1) * 4;
#pragma unroll
    for (int l = 0; l < 32; ++l) {
        const int nib = (q[l] >> sh) & 15;
        w[l] = __fsub_rn(__fmul_rn(dl, (float)nib), ml);
    }
}

template <>
__device__ __forceinline__ void decode_group<SKN_TYPE_Q6_K>(const uint8_t *row, int64_t g, float (&w)[32]) {
    const uint8_t *b = row + (g >> 3) * 210;
    const int h = (int)((g >> 2) & 1), gq = (int)(g & 3);
    const uint8_t *ql = b + 64 * h + 32 * (gq & 1);
    const uint8_t *qh = b + 128 + 32 * h;
    const int8_t *sc = (const int8_t *)(b + 192 + 8 * h + 2 * gq);
    const float d = skn_half_bits_to_float(skn_ld16(b + 208));
    const float dl0 = __fmul_rn(d, (float)sc[0]);
    const float dl1 = __fmul_rn(d, (float)sc[1]);
    const int shl = (gq >> 1) * 4;
    const int shh = 2 * gq;
#pragma unroll
    for (int l = 0; l < 32; ++l) {
        const int nib = (ql[l] >> shl) & 15;
        const int q = (nib | (((qh[l] >> shh) & 3) << 4)) - 32;
        w[l] = __fmul_rn(l < 16 ? dl0 : dl1, (float)q);
    }
}

// q * d + m with the two roundings of gguf-py's `(d * qs) + m`
template <>
__device__ __forceinline__ void decode_group<SKN_TYPE_Q4_1>(const uint8_t *row, int64_t g, float (&w)[32]) {
    const uint8_t *b = row + g * 20;
    const float d = skn_half_bits_to_float(skn_ld16(b)), m = skn_half_bits_to_float(skn_ld16(b + 2));
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const int v = b[4 + e];
        w[e]      = __fadd_rn(__fmul_rn(d, (float)(v & 15)), m);
        w[e + 16] = __fadd_rn(__fmul_rn(d, (float)(v >> 4)), m);
    }
}

// fifth bit of weight i = bit i of the little-endian 32-bit word after d
template <>
__device__ __forceinline__ void decode_group<SKN_TYPE_Q5_0>(const uint8_t *row, int64_t g, float (&w)[32]) {
    const uint8_t *b = row + g * 22;
    const float d = skn_half_bits_to_float(skn_ld16(b));
    const uint32_t qh = skn_ld16(b + 2) | (skn_ld16(b + 4) << 16);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const int v = b[6 + e];
        const int lo = (v & 15) | (int)(((qh >> e) & 1u) << 4);
        const int hi = (v >> 4) | (int)(((qh >> (e + 16)) & 1u) << 4);
        w[e]      = __fmul_rn(d, (float)(lo - 16));
        w[e + 16] = __fmul_rn(d, (float)(hi - 16));
    }
}

template <>
__device__ __forceinline__ void decode_group<SKN_TYPE_Q5_1>(const uint8_t *row, int64_t g, float (&w)[32]) {
    const uint8_t *b = row + g * 24;
    const float d = skn_half_bits_to_float(skn_ld16(b)), m = skn_half_bits_to_float(skn_ld16(b + 2));
    const uint32_t qh = skn_ld16(b + 4) | (skn_ld16(b + 6) << 16);
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const int v = b[8 + e];
        const int lo = (v & 15) | (int)(((qh >> e) & 1u) << 4);
        const int hi = (v >> 4) | (int)(((qh >> (e + 16)) & 1u) << 4);
        w[e]      = __fadd_rn(__fmul_rn(d, (float)lo), m);
        w[e + 16] = __fadd_rn(__fmul_rn(d, (float)hi), m);
    }
}

// Q4_K's layout with a fifth bit per weight: bit j of byte qh[l] belongs to weight l of sub-block j
template <>
__device__ __forceinline__ void decode_group<SKN_TYPE_Q5_K>(const uint8_t *row, int64_t g, float (&w)[32]) {
    const uint8_t *b = row + (g >> 3) * 176;
    const int j = (int)(g & 7);
    const float d = skn_half_bits_to_float(skn_ld16(b));
    const float dmin = skn_half_bits_to_float(skn_ld16(b + 2));
    int sc, mn;
    skn_q4k_scale_min(b + 4, j, sc, mn);
    const float dl = __fmul_rn(d, (float)sc);
    const float ml = __fmul_rn(dmin, (float)mn);
    const uint8_t *qh = b + 16;
    const uint8_t *q = b + 48 + 32 * (j >> 1);
    const int sh = (j & 1) * 4;
#pragma unroll
    for (int l = 0; l < 32; ++l) {
        const int v = ((q[l] >> sh) & 15) | (((qh[l] >> j) & 1) << 4);
        w[l] = __fsub_rn(__fmul_rn(dl, (float)v), ml);
    }
}
