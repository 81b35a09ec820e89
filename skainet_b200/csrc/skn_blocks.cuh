// Device-side decoders for the GGUF block types.
//
// Every type splits into "groups" of 32 weights that are contiguous in the row and share
// their scale arithmetic:
//   Q4_0 / Q8_0 : group = block (18 / 34 bytes)
//   Q4_K        : group = sub-block j of a 144-byte super-block (8 per block)
//   Q6_K        : group = (half h, quarter g) of a 210-byte super-block (8 per block)
//   Q4_1 / Q5_0 / Q5_1 : group = block (20 / 22 / 24 bytes); Q5_K: sub-block of a 176-byte super-block
//   Q2_K / Q3_K : group = (half h, bit pair s) of an 84- / 110-byte super-block (two 16-weight scale groups)
//   IQ4_NL : group = block (18 bytes); IQ4_XS : sub-block of a 136-byte super-block
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
template <> struct BlockTraits<SKN_TYPE_Q2_K> { static constexpr int ELEMS = 256, BYTES = 84;  };
template <> struct BlockTraits<SKN_TYPE_Q3_K> { static constexpr int ELEMS = 256, BYTES = 110; };
template <> struct BlockTraits<SKN_TYPE_IQ4_NL> { static constexpr int ELEMS = 32,  BYTES = 18;  };
template <> struct BlockTraits<SKN_TYPE_IQ4_XS> { static constexpr int ELEMS = 256, BYTES = 136; };

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

// Q2_K: weight 128h + 32s + l is bits 2s..2s+1 of byte qs[32h + l]; scale byte (128h + 32s + l) / 16 holds
// the 4-bit scale (low nibble) and the 4-bit min (high nibble): (d*sc)*q - dmin*m
template <>
__device__ __forceinline__ void decode_group<SKN_TYPE_Q2_K>(const uint8_t *row, int64_t g, float (&w)[32]) {
    const uint8_t *b = row + (g >> 3) * 84;
    const int j = (int)(g & 7), h = j >> 2, sh = 2 * (j & 3);
    const float d = skn_half_bits_to_float(skn_ld16(b + 80));
    const float dmin = skn_half_bits_to_float(skn_ld16(b + 82));
    const int s0 = b[2 * j], s1 = b[2 * j + 1];
    const float dl0 = __fmul_rn(d, (float)(s0 & 15)), ml0 = __fmul_rn(dmin, (float)(s0 >> 4));
    const float dl1 = __fmul_rn(d, (float)(s1 & 15)), ml1 = __fmul_rn(dmin, (float)(s1 >> 4));
    const uint8_t *q = b + 16 + 32 * h;
#pragma unroll
    for (int l = 0; l < 32; ++l) {
        const int v = (q[l] >> sh) & 3;
        w[l] = __fsub_rn(__fmul_rn(l < 16 ? dl0 : dl1, (float)v), l < 16 ? ml0 : ml1);
    }
}

// sixteen 6-bit scales (offset 32) of a Q3_K block from its 12 packed bytes
__device__ __forceinline__ int skn_q3k_scale(const uint8_t *s, int i) {
    const int lo = (i < 8) ? (s[i] & 15) : (s[i - 8] >> 4);
    const int hi = (s[8 + (i & 3)] >> (2 * (i >> 2))) & 3;
    return (lo | (hi << 4)) - 32;
}

// Q3_K: Q2_K's 2-bit layout; bit j of hmask[l] belongs to weight 32j + l and a CLEAR bit subtracts 4
template <>
__device__ __forceinline__ void decode_group<SKN_TYPE_Q3_K>(const uint8_t *row, int64_t g, float (&w)[32]) {
    const uint8_t *b = row + (g >> 3) * 110;
    const int j = (int)(g & 7), h = j >> 2, sh = 2 * (j & 3);
    const float d = skn_half_bits_to_float(skn_ld16(b + 108));
    const float dl0 = __fmul_rn(d, (float)skn_q3k_scale(b + 96, 2 * j));
    const float dl1 = __fmul_rn(d, (float)skn_q3k_scale(b + 96, 2 * j + 1));
    const uint8_t *hm = b, *q = b + 32 + 32 * h;
#pragma unroll
    for (int l = 0; l < 32; ++l) {
        const int v = ((q[l] >> sh) & 3) - ((((hm[l] >> j) & 1) ^ 1) << 2);
        w[l] = __fmul_rn(l < 16 ? dl0 : dl1, (float)v);
    }
}

// entry i of the 16-entry non-linear IQ4 codebook (part of the published format), as two packed words
__device__ __forceinline__ int skn_iq4_value(int i) {
    const unsigned long long lo = 0xF6EADDCFBFAD9881ull;   // -127 -104 -83 -65 -49 -35 -22 -10
    const unsigned long long hi = 0x7159453526190D01ull;   //    1   13  25  38  53  69  89 113
    return (int)(signed char)(((i & 8) ? hi : lo) >> (8 * (i & 7)));
}

template <>
__device__ __forceinline__ void decode_group<SKN_TYPE_IQ4_NL>(const uint8_t *row, int64_t g, float (&w)[32]) {
    const uint8_t *b = row + g * 18;
    const float d = skn_half_bits_to_float(skn_ld16(b));
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const int v = b[2 + e];
        w[e]      = __fmul_rn(d, (float)skn_iq4_value(v & 15));
        w[e + 16] = __fmul_rn(d, (float)skn_iq4_value(v >> 4));
    }
}

// IQ4_XS: sub-block j = bytes qs[16j .. 16j+15] (low nibbles first); 6-bit scale (offset 32) from
// scales_l (nibble j) and scales_h (bits 2j, 2j+1)
template <>
__device__ __forceinline__ void decode_group<SKN_TYPE_IQ4_XS>(const uint8_t *row, int64_t g, float (&w)[32]) {
    const uint8_t *b = row + (g >> 3) * 136;
    const int j = (int)(g & 7);
    const float d = skn_half_bits_to_float(skn_ld16(b));
    const int lo = (b[4 + (j >> 1)] >> (4 * (j & 1))) & 15;
    const int hi = (int)((skn_ld16(b + 2) >> (2 * j)) & 3u);
    const float dl = __fmul_rn(d, (float)((lo | (hi << 4)) - 32));
    const uint8_t *q = b + 8 + 16 * j;
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const int v = q[e];
        w[e]      = __fmul_rn(dl, (float)skn_iq4_value(v & 15));
        w[e + 16] = __fmul_rn(dl, (float)skn_iq4_value(v >> 4));
    }
}
