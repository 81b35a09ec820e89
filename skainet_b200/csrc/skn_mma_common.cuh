// Pieces shared by the integer tensor-core matvec kernels (skn_matvec_mma.cu: one to four activation rows,
// x prepared inside the kernel; skn_matvec_rows.cu: up to sixteen rows, x prepared by a kernel of its own):
// block formats, mma.sync wrappers, shared-memory load helpers, the digit planes of the activations and the
// scalar dequantiser used for outlier activations.
#pragma once
#include "skn_mv_common.cuh"

#include <math.h>

// Block formats of this kernel.  A "super-block" is 256 weights: one Q4_K block, or eight of the
// 32-weight blocks of Q8_0 / Q4_0 (each with its own fp16 scale).  KS super-blocks (one bulk copy
// per row) make a K super-chunk; rows are padded by 32 bytes in shared memory, which puts the
// eight row groups of a fragment load on disjoint banks (row stride = 8 words mod 32).
// Q6_K: one 210-byte block per super-block; eight of them are 1680 bytes = a multiple of 16 (a bulk
// copy's granularity) and 420 words = 4 mod 32: its fragments are read with 32-bit loads (lane (g, t) reads
// word t of row g), which that stride spreads over all 32 banks without padding (a stride of 8 words mod 32,
// right for the 64-bit loads of the other formats, made rows g and g + 4 collide: 2.5 M bank conflicts per
// 32000 x 4096 launch).  Its scale groups are 16 weights, so the group sums of x are kept per 16
// activations (XS per super-block).
constexpr int MM_FMT_Q4K = 0, MM_FMT_Q80 = 1, MM_FMT_Q40 = 2, MM_FMT_Q6K = 3;
template <int FMT> struct MmFmt;
template <> struct MmFmt<MM_FMT_Q4K> { static constexpr int KS = 16, SB_BYTES = 144, PAD = 32, XS = 8; };
template <> struct MmFmt<MM_FMT_Q80> { static constexpr int KS = 8, SB_BYTES = 272, PAD = 32, XS = 8; };
template <> struct MmFmt<MM_FMT_Q40> { static constexpr int KS = 16, SB_BYTES = 144, PAD = 16, XS = 8; };   // 32-bit fragment loads: 4 words mod 32
template <> struct MmFmt<MM_FMT_Q6K> { static constexpr int KS = 8, SB_BYTES = 210, PAD = 0, XS = 16; };
static constexpr int mm_ks(int fmt) { return (fmt == MM_FMT_Q80 || fmt == MM_FMT_Q6K) ? 8 : 16; }
static constexpr int mm_sb_bytes(int fmt) { return fmt == MM_FMT_Q80 ? 272 : (fmt == MM_FMT_Q6K ? 210 : 144); }
static constexpr int mm_xs(int fmt) { return fmt == MM_FMT_Q6K ? 16 : 8; }
static constexpr int mm_stage_bytes(int fmt) { return 16 * (mm_ks(fmt) * mm_sb_bytes(fmt) + (fmt == MM_FMT_Q6K ? 0 : (fmt == MM_FMT_Q40 ? 16 : 32))); }

__device__ __forceinline__ void skn_mma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void skn_mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}


// byte i (0..3) of w as a float without the conversion pipe: (2^23 + b) - 2^23
__device__ __forceinline__ float mm_byte_f(uint32_t w, uint32_t i) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440u + i)) - 8388608.f;
}
__device__ __forceinline__ int mm_byte_i(uint32_t w, uint32_t i) { return (int)__byte_perm(w, 0u, 0x4440u + i); }
// signed byte i of w, sign-extended (selector values 8..15 replicate a byte's sign bit)
// (the __byte_perm intrinsic only honours three bits per selector, so the instruction is spelled out)
__device__ __forceinline__ int mm_sbyte_i(uint32_t w, uint32_t i) {
    int r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0u), "r"(0x8880u + 0x1111u * i));
    return r;
}
// signed byte i of w as a float, w given with its bytes' sign bits flipped: (2^23 + 128 + b) - (2^23 + 128)
__device__ __forceinline__ float mm_sbyte_f(uint32_t w_flipped, uint32_t i) {
    return __uint_as_float(__byte_perm(w_flipped, 0x4B000000u, 0x7440u + i)) - 8388736.f;
}

// loads from a 32-bit shared-memory address (explicit state space: no generic addressing, no
// 64-bit address arithmetic in the inner loops)
__device__ __forceinline__ uint2 mm_lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 mm_lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t mm_lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
// fp16 at a 2-byte aligned shared address, widened
__device__ __forceinline__ float mm_lds_half(uint32_t a) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ float mm_lds32f(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float4 mm_lds128f(uint32_t a) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
    return v;
}

__device__ __forceinline__ void mm_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Digit planes of the activations.  A super-block of 256 activations becomes a 32-bit fixed-point number per
// activation with one power-of-two scale for the block, X = rint(x * 2^(29-e)) with e the exponent of the
// block's largest |x|, split into four balanced signed byte digits X = d0 + 2^8 d1 + 2^16 d2 + 2^24 d3 (the
// bytes of (X + 0x80808080) ^ 0x80808080); plane n holds digit n of every activation.  Activations within 2^6
// of the block's largest are represented exactly, the others to 2^-30 of the largest.
//
// Outliers: when at most four activations tower over the rest of their block -- everything below 2^-6 of the
// largest lies at least 2^10 below it -- those few are taken out of the planes (their digits are zero) and kept
// as fp32 values with their positions; the planes then describe the others relative to THEIR largest, so an
// outlier does not cost its neighbours their precision.  The dot product adds weight x outlier in fp32.
// Guaranteed: every activation enters the product exactly (fp32), or within 2^-21 of the largest activation
// that shares its planes.
constexpr int MM_ND = 4;                        // digit planes
constexpr int MM_MAX_OUT = 4;                   // outliers kept per (activation row, super-block)
constexpr int MM_OUT_GAP = 10;                  // exponent gap between the block's largest and the largest of the small ones
constexpr int MM_OUT_BAND = 6;                  // activations within 2^6 of the largest count as large

// D[i] = the four digit bytes of element i: a 4 x 4 byte transpose per four elements gives the plane words (digit n
// of elements 0..3 and of 4..7); two permute stages, eight instructions per four elements
__device__ __forceinline__ void mm_store_planes(const uint32_t (&D)[8], uint8_t *base, int plane_stride, int word) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t t0 = __byte_perm(D[4 * h], D[4 * h + 1], 0x5140u), t1 = __byte_perm(D[4 * h], D[4 * h + 1], 0x7362u);
        const uint32_t t2 = __byte_perm(D[4 * h + 2], D[4 * h + 3], 0x5140u), t3 = __byte_perm(D[4 * h + 2], D[4 * h + 3], 0x7362u);
        const uint32_t P[4] = {__byte_perm(t0, t2, 0x5410u), __byte_perm(t0, t2, 0x7632u), __byte_perm(t1, t3, 0x5410u),
                               __byte_perm(t1, t3, 0x7632u)};
#pragma unroll
        for (int n = 0; n < MM_ND; ++n) *reinterpret_cast<uint32_t *>(base + (size_t)n * plane_stride + 4 * (word + 32 * h)) = P[n];
    }
}

// Group sums of one super-block (lane: elements 4*lane.. and 128 + 4*lane..) into xsum, their total returned in every
// lane.  XS16: sixteen 16-element sums instead of the eight 32-element ones.
template <bool XS16>
static __device__ __forceinline__ float mm_group_sums(const float (&in)[8], int sbi, int lane, float *xsum) {
    float s0 = (in[0] + in[1]) + (in[2] + in[3]), s1 = (in[4] + in[5]) + (in[6] + in[7]);
    if constexpr (XS16) {
#pragma unroll
        for (int o = 2; o > 0; o >>= 1) {
            s0 += __shfl_xor_sync(0xffffffffu, s0, o);
            s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        }
        if ((lane & 3) == 0) {
            xsum[sbi * 16 + (lane >> 2)] = s0;
            xsum[sbi * 16 + 8 + (lane >> 2)] = s1;
        }
        s0 += __shfl_xor_sync(0xffffffffu, s0, 4);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 4);
    } else {
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
            s0 += __shfl_xor_sync(0xffffffffu, s0, o);
            s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        }
        if ((lane & 7) == 0) {
            xsum[sbi * 8 + (lane >> 3)] = s0;
            xsum[sbi * 8 + 4 + (lane >> 3)] = s1;
        }
    }
    float tot = s0 + s1;
    tot += __shfl_xor_sync(0xffffffffu, tot, 8);
    tot += __shfl_xor_sync(0xffffffffu, tot, 16);
    return tot;
}

// The rare half of mm_digitize, kept out of line (the preparation is unrolled four super-blocks deep, and a launch
// runs it once from a cold instruction cache: its size is paid in instruction fetches).  Called when at most four
// lanes hold anything within 2^-MM_OUT_BAND of the block's largest: the exact test on the elements; if it passes,
// the outliers go to the block's record, leave `in`, and the group sums are formed again without them.
struct mm_outlier_result {
    float in[8];
    float tot;
    int n_out, ES;
};
template <bool XS16>
static __device__ __noinline__ mm_outlier_result mm_take_outliers(float i0, float i1, float i2, float i3, float i4, float i5, float i6,
                                                                  float i7, float tot, int E, int sbi, int lane, float *xsum,
                                                                  float *oval, uint32_t *oidx, int *any_out) {
    mm_outlier_result r;
    r.in[0] = i0; r.in[1] = i1; r.in[2] = i2; r.in[3] = i3; r.in[4] = i4; r.in[5] = i5; r.in[6] = i6; r.in[7] = i7;
    r.tot = tot; r.n_out = 0; r.ES = E;
    const uint32_t thr = (uint32_t)(E - MM_OUT_BAND) << 23;
    uint32_t big[8], mb = 0;
    int total = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t a = __float_as_uint(r.in[i]) & 0x7FFFFFFFu;
        big[i] = __ballot_sync(0xffffffffu, a >= thr);
        total += __popc(big[i]);
        mb = max(mb, a < thr ? a : 0u);
    }
    mb = __reduce_max_sync(0xffffffffu, mb);    // the largest of the small ones
    int EB = (int)(mb >> 23);
    EB = EB < 30 ? 30 : EB;
    if (total <= MM_MAX_OUT && mb != 0u && E - EB >= MM_OUT_GAP) {      // warp-uniform
        int before = 0;                     // large ones in lower (element, lane) order
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if ((big[i] >> lane) & 1u) {
                const int pos = before + __popc(big[i] & ((1u << lane) - 1u));
                oval[4 * sbi + pos] = r.in[i];
                reinterpret_cast<uint8_t *>(oidx + sbi)[pos] = (uint8_t)(i < 4 ? 4 * lane + i : 128 + 4 * lane + (i - 4));
                r.in[i] = 0.f;              // out of the planes and of the sums
            }
            before += __popc(big[i]);
        }
        r.n_out = total;
        r.ES = EB;
        if (any_out && lane == 0) *any_out = 1;
        r.tot = mm_group_sums<XS16>(r.in, sbi, lane, xsum);
    }
    return r;
}

// One super-block (256 activations, two float4 per lane: elements 4*lane.. and 128 + 4*lane..)
// -> four digit planes (byte k of a plane = that digit of activation k), the scale 2^(e-29)
// (NaN when the block holds a NaN or an infinity), the eight 32-element sums (outliers excluded: their whole
// product, offset terms included, is formed in fp32) and the block's outlier record:
// ocnt[sbi] = how many (0..4), oval[4 * sbi + i] their values, oidx[sbi] their positions (one byte each).
// XS16: sixteen 16-element sums instead of the eight 32-element ones.  any_out (may be NULL): set to 1 when the
// block has outliers.
template <bool XS16>
static __device__ __forceinline__ void mm_digitize(const float4 v0, const float4 v1, int sbi, int lane, uint8_t *dig, int PL,
                                                   float *sgrp, float *xsum, float *oval, uint32_t *oidx, uint8_t *ocnt,
                                                   int *any_out = nullptr) {
    float in[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    const float mx = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                           fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
    // the group sums first, so that their shuffles overlap the maximum's reduction
    float tot = mm_group_sums<XS16>(in, sbi, lane, xsum);
    // mx >= 0 (or NaN-free by fmaxf): its bit pattern orders like the value, one integer reduction
    const uint32_t mxb = __reduce_max_sync(0xffffffffu, __float_as_uint(mx));
    int E = (int)(mxb >> 23);
    E = E < 30 ? 30 : (E > 254 ? 254 : E);
    int ES = E;                                 // exponent the planes are scaled by
    int n_out = 0;
    // Outliers?  Only when at most four lanes hold anything within 2^-6 of the block's largest (ordinary data
    // fails this at once: one comparison and a vote).
    const uint32_t thr = (uint32_t)(E - MM_OUT_BAND) << 23;
    if (__popc(__ballot_sync(0xffffffffu, __float_as_uint(mx) >= thr)) <= MM_MAX_OUT && mxb < 0x7F800000u) {
        const mm_outlier_result r = mm_take_outliers<XS16>(in[0], in[1], in[2], in[3], in[4], in[5], in[6], in[7], tot, E, sbi, lane,
                                                           xsum, oval, oidx, any_out);
#pragma unroll
        for (int i = 0; i < 8; ++i) in[i] = r.in[i];
        tot = r.tot; n_out = r.n_out; ES = r.ES;
    }
    const float mul = __int_as_float((283 - ES) << 23);           // 2^(29-e)
    uint32_t D[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) D[i] = ((uint32_t)__float2int_rn(in[i] * mul) + 0x80808080u) ^ 0x80808080u;
    mm_store_planes(D, dig, PL, sbi * 64 + lane);
    if (lane == 0) {
        ocnt[sbi] = (uint8_t)n_out;
        sgrp[sbi] = (fabsf(tot) <= 3.4028234e38f && mxb < 0x7F800000u) ? __int_as_float((ES - 29) << 23) : __int_as_float(0x7FC00000);
    }
}

// The weight at column k (0..255) of the super-block at shared address `blk`, dequantised as the format defines
// it (offset terms included): what an outlier activation is multiplied by.
template <int FMT>
__device__ __forceinline__ float mm_weight_at(uint32_t blk, int k);
__device__ __forceinline__ uint32_t mm_lds8(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
template <>
__device__ __forceinline__ float mm_weight_at<0>(uint32_t blk, int k) {       // Q4_K: (d * sc) * q - dmin * m
    const int j = k >> 5;
    const uint32_t qb = mm_lds8(blk + 16 + 32 * (j >> 1) + (k & 31));
    const int q = (j & 1) ? (int)(qb >> 4) : (int)(qb & 15u);
    int sc, mn;
    if (j < 4) {
        sc = (int)(mm_lds8(blk + 4 + j) & 63u);
        mn = (int)(mm_lds8(blk + 8 + j) & 63u);
    } else {
        const uint32_t hi = mm_lds8(blk + 8 + j);
        sc = (int)((hi & 15u) | ((mm_lds8(blk + j) >> 6) << 4));
        mn = (int)((hi >> 4) | ((mm_lds8(blk + 4 + j) >> 6) << 4));
    }
    return __fsub_rn(__fmul_rn(mm_lds_half(blk) * (float)sc, (float)q), mm_lds_half(blk + 2) * (float)mn);
}
template <>
__device__ __forceinline__ float mm_weight_at<1>(uint32_t blk, int k) {       // Q8_0 (eight 34-byte blocks): d * q
    const uint32_t b = blk + 34 * (k >> 5);
    return mm_lds_half(b) * (float)(int)(int8_t)mm_lds8(b + 2 + (k & 31));
}
template <>
__device__ __forceinline__ float mm_weight_at<2>(uint32_t blk, int k) {       // Q4_0 (eight 18-byte blocks): d * (q - 8)
    const uint32_t b = blk + 18 * (k >> 5);
    const int e = k & 31;
    const uint32_t qb = mm_lds8(b + 2 + (e & 15));
    return mm_lds_half(b) * (float)((int)(e < 16 ? (qb & 15u) : (qb >> 4)) - 8);
}
template <>
__device__ __forceinline__ float mm_weight_at<3>(uint32_t blk, int k) {       // Q6_K: (d * sc) * (q - 32)
    const int h = k >> 7, l = k & 127, gq = l >> 5, li = l & 31;
    const uint32_t lb = mm_lds8(blk + 64 * h + 32 * (gq & 1) + li);
    const uint32_t hb = mm_lds8(blk + 128 + 32 * h + li);
    const int q = (int)((gq < 2 ? (lb & 15u) : (lb >> 4)) | (((hb >> (2 * gq)) & 3u) << 4));
    const int sc = (int)(int8_t)mm_lds8(blk + 192 + 8 * h + 2 * gq + (li >> 4));
    return (mm_lds_half(blk + 208) * (float)sc) * (float)(q - 32);
}

// Outlier number t of block e times the weights of rows g (block at `ba`) and g + 8 (`bb`), scaled by inv_dw; out of
// line: rare, and the tile loop is better off without its code.
template <int FMT>
static __device__ __noinline__ float2 mm_outlier_products(uint32_t ba, uint32_t bb, uint32_t oidx_s, uint32_t oval_s, uint32_t e, int t,
                                                          float inv_dw) {
    const int k = (int)mm_lds8(oidx_s + 4u * e + (uint32_t)t);
    const float xv = mm_lds32f(oval_s + 4u * (MM_MAX_OUT * e + (uint32_t)t)) * inv_dw;
    return make_float2(mm_weight_at<FMT>(ba, k) * xv, mm_weight_at<FMT>(bb, k) * xv);
}
