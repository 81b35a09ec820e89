// K3 / K4: prefill matmul on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   Y[M,N] = A[M,K] . W_q[N,K]^T      A = bf16 copy of the activations, W_q = raw GGUF blocks
//
// One CTA computes a 128 (tokens) x 128 (features) tile over the whole K in steps of 64:
//   warps 0-3  dequantise the weight tile: thread t owns weight row t and turns 64 weights of
//              raw blocks into one 128-byte bf16 row of the K-major, 128B-swizzled operand
//              tile in shared memory (DUAL: a second tile from a second weight, same rows)
//   warps 4-7  copy the activation tile (128 rows x 64 bf16) into the same layout
//   warp  8    allocates tensor memory; its lane 0 issues tcgen05.mma (M=128, N=128, K=16,
//              kind::f16, bf16 operands, fp32 accumulation in TMEM) four times per stage and
//              commits each stage to the mbarrier that frees it
//   warps 0-3  epilogue: tcgen05.ld the accumulator (lane = token row) and store fp32 rows,
//              or, DUAL, silu(gate) * up as bf16 for the next matmul
// A 4-stage ring of (A tile, B tile[, B2 tile]) with full/empty mbarriers decouples the three
// roles.  Operand tiles are written by ordinary stores, so every producer thread issues
// fence.proxy.async before its warp arrives on the full barrier.  All waits are bounded.
#include "skn_blocks.cuh"
#include "skn_ptx.cuh"

#include <cuda.h>
#include <cuda_bf16.h>

constexpr int TC_BM = 128, TC_BN = 128, TC_BK = 64;
constexpr int TC_TILE_BYTES = TC_BM * TC_BK * 2;   // 16 KB, one operand tile
constexpr int TC_THREADS = 10 * 32;   // 8 dequant warps, 1 MMA warp, 1 TMA warp

// ---- tcgen05 wrappers ---------------------------------------------------------------------
__device__ __forceinline__ void tc_alloc(uint32_t *slot_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(skn_smem_u32(slot_smem)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(skn_smem_u32(bar))
                 : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, 128 x N x 16, bf16 in, fp32 out
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 32 columns of 32-bit accumulators -> 32 registers per thread
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 2-D tiled TMA load (no multicast) of a box at element coordinates (x = column, y = row); the
// tensor map's 128-byte swizzle lays the box out exactly as tc_store_chunk does
__device__ __forceinline__ void tc_tma_load_2d(void *dst_smem, const CUtensorMap *tmap, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(skn_smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(skn_smem_u32(bar))
        : "memory");
}

// Shared-memory matrix descriptor: K-major operand, rows of 64 bf16 (128 bytes) in 8-row
// groups of 1024 bytes, 128-byte swizzle (16-byte chunk c of row r sits at chunk c ^ (r & 7)).
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset: 8 rows * 128 bytes
    d |= (uint64_t)1 << 46;                          // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                          // swizzle mode: 128 bytes
    return d;
}
// Instruction descriptor: fp32 accumulator, bf16 A and B, both K-major, M x N tile
__device__ __forceinline__ uint32_t tc_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// store 8 consecutive bf16 (one 16-byte chunk `c` of row `r`) into a swizzled tile
__device__ __forceinline__ void tc_store_chunk(uint8_t *tile, int r, int c, uint4 v) {
    *reinterpret_cast<uint4 *>(tile + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)) = v;
}

__device__ __forceinline__ uint32_t tc_pack_bf16(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// ---- 64 weights of one row -> one 128-byte bf16 row of the operand tile ------------------------
// Generic form (any type): two 32-weight groups through the byte-granular decoder.
template <int TYPE>
__device__ __forceinline__ void tc_dequant_row(const uint8_t *rp, int k0, uint8_t *tile, int r, bool valid) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        float w[32];
        if (valid) {
            decode_group<TYPE>(rp, (int64_t)(k0 >> 5) + half, w);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) w[i] = 0.f;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint4 v;
            v.x = tc_pack_bf16(w[8 * c + 0], w[8 * c + 1]);
            v.y = tc_pack_bf16(w[8 * c + 2], w[8 * c + 3]);
            v.z = tc_pack_bf16(w[8 * c + 4], w[8 * c + 5]);
            v.w = tc_pack_bf16(w[8 * c + 6], w[8 * c + 7]);
            tc_store_chunk(tile, r, half * 4 + c, v);
        }
    }
}

// (2^23 + k * 2^pos) read as a float, minus 2^23, times scale * 2^-pos, minus off: the value
// scale * k - off of a quant field left in place at bit `pos` (no shift, no int->float unit).
// Products and the subtraction round exactly as (scale * k) - off does in fp32.
__device__ __forceinline__ float tc_field(uint32_t masked_or_magic, float scale_shifted, float off) {
    return fmaf(__uint_as_float(masked_or_magic) - 8388608.f, scale_shifted, -off);
}

// Q4_K: 64 weights at k0 = one 32-byte run of quants (low nibbles: sub-block 2p, high nibbles:
// sub-block 2p+1) plus the block header; three 16-byte loads.
template <int TYPE> struct TcRaw { };                       // generic types: nothing is prefetched
template <> struct TcRaw<SKN_TYPE_Q4_K> { uint4 hdr, qa, qb; };
template <> struct TcRaw<SKN_TYPE_Q4_0> { uint32_t w[9]; };
template <> struct TcRaw<SKN_TYPE_Q8_0> { uint32_t w[17]; };
template <> struct TcRaw<SKN_TYPE_Q6_K> { uint32_t rq[17], rh[9], s_lo, s_hi, dword; };

// raw bytes of the 64 weights at k0 into registers (issued one stage ahead of their decode)
template <int TYPE>
__device__ __forceinline__ void tc_load_row(const uint8_t *, int, bool, TcRaw<TYPE> &) {}
template <>
__device__ __forceinline__ void tc_load_row<SKN_TYPE_Q4_K>(const uint8_t *rp, int k0, bool valid, TcRaw<SKN_TYPE_Q4_K> &raw) {
    if (!valid) return;
    const int p = (k0 >> 6) & 3;
    const uint8_t *bp = rp + (size_t)(k0 >> 8) * 144;
    raw.hdr = __ldg(reinterpret_cast<const uint4 *>(bp));
    raw.qa = __ldg(reinterpret_cast<const uint4 *>(bp + 16 + 32 * p));
    raw.qb = __ldg(reinterpret_cast<const uint4 *>(bp + 32 + 32 * p));
}

template <int TYPE>
__device__ __forceinline__ void tc_decode_row(const TcRaw<TYPE> &, const uint8_t *rp, int k0, uint8_t *tile, int r, bool valid) {
    tc_dequant_row<TYPE>(rp, k0, tile, r, valid);
}

template <>
__device__ __forceinline__ void tc_decode_row<SKN_TYPE_Q4_K>(const TcRaw<SKN_TYPE_Q4_K> &raw, const uint8_t *, int k0,
                                                             uint8_t *tile, int r, bool valid) {
    if (!valid) {
#pragma unroll
        for (int c = 0; c < 8; ++c) tc_store_chunk(tile, r, c, make_uint4(0u, 0u, 0u, 0u));
        return;
    }
    const int p = (k0 >> 6) & 3;
    const uint4 hdr = raw.hdr, qa = raw.qa, qb = raw.qb;
    // scales / mins of sub-blocks 2p, 2p+1 (p is the same for every thread of the CTA)
    const int sh = (p & 1) * 16;
    const uint32_t a2 = (hdr.y >> sh) & 0xFFFFu, b2 = (hdr.z >> sh) & 0xFFFFu, c2 = (hdr.w >> sh) & 0xFFFFu;
    const uint32_t sc2 = (p < 2) ? (a2 & 0x3F3Fu) : ((c2 & 0x0F0Fu) | ((a2 >> 2) & 0x3030u));
    const uint32_t mn2 = (p < 2) ? (b2 & 0x3F3Fu) : (((c2 >> 4) & 0x0F0Fu) | ((b2 >> 2) & 0x3030u));
    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
    const float dl0 = __fmul_rn(dd.x, (float)(sc2 & 0xFFu)), dl1 = __fmul_rn(dd.x, (float)(sc2 >> 8));
    const float ml0 = __fmul_rn(dd.y, (float)(mn2 & 0xFFu)), ml1 = __fmul_rn(dd.y, (float)(mn2 >> 8));
    const float l0 = dl0, l8 = dl0 * (1.f / 256.f), l16 = dl0 * (1.f / 65536.f);
    const float h4 = dl1 * (1.f / 16.f), h12 = dl1 * (1.f / 4096.f), h8 = dl1 * (1.f / 256.f), h16 = dl1 * (1.f / 65536.f);
    const uint32_t M = 0x4B000000u;
    const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    uint32_t lo[16], hi[16];   // bf16 pairs: lo = sub-block 2p (weights 0..31), hi = sub-block 2p+1
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t w = qw[i], w8 = w >> 8, w12 = w >> 12;
        const float a0 = tc_field((w & 0x0000000Fu) | M, l0, ml0), a1 = tc_field((w & 0x00000F00u) | M, l8, ml0);
        const float a2f = tc_field((w & 0x000F0000u) | M, l16, ml0), a3 = tc_field((w8 & 0x000F0000u) | M, l16, ml0);
        const float b0 = tc_field((w & 0x000000F0u) | M, h4, ml1), b1 = tc_field((w & 0x0000F000u) | M, h12, ml1);
        const float b2f = tc_field((w12 & 0x00000F00u) | M, h8, ml1), b3 = tc_field((w12 & 0x000F0000u) | M, h16, ml1);
        lo[2 * i] = tc_pack_bf16(a0, a1);
        lo[2 * i + 1] = tc_pack_bf16(a2f, a3);
        hi[2 * i] = tc_pack_bf16(b0, b1);
        hi[2 * i + 1] = tc_pack_bf16(b2f, b3);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        tc_store_chunk(tile, r, c, make_uint4(lo[4 * c], lo[4 * c + 1], lo[4 * c + 2], lo[4 * c + 3]));
        tc_store_chunk(tile, r, 4 + c, make_uint4(hi[4 * c], hi[4 * c + 1], hi[4 * c + 2], hi[4 * c + 3]));
    }
}

// Q4_0: 64 weights at k0 = two 18-byte blocks = nine aligned words; block A's quants straddle
// the words by two bytes.  Byte e of a block: low nibble = weight e, high nibble = weight e+16.
template <>
__device__ __forceinline__ void tc_load_row<SKN_TYPE_Q4_0>(const uint8_t *rp, int k0, bool valid, TcRaw<SKN_TYPE_Q4_0> &raw) {
    if (!valid) return;
    const uint32_t *p = reinterpret_cast<const uint32_t *>(rp + (size_t)(k0 >> 6) * 36);
#pragma unroll
    for (int i = 0; i < 9; ++i) raw.w[i] = __ldg(p + i);
}

// four quant words of one Q4_0 block -> 32 bf16 (16 packed pairs) at out[0..15]
__device__ __forceinline__ void tc_q40_block(const uint32_t (&q)[4], float d, uint32_t *out) {
    const float off = 8.f * d;
    const float l0 = d, l8 = d * (1.f / 256.f), l16 = d * (1.f / 65536.f);
    const float h4 = d * (1.f / 16.f), h12 = d * (1.f / 4096.f);
    const uint32_t M = 0x4B000000u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t w = q[i], w8 = w >> 8, w12 = w >> 12;
        out[2 * i] = tc_pack_bf16(tc_field((w & 0x0000000Fu) | M, l0, off), tc_field((w & 0x00000F00u) | M, l8, off));
        out[2 * i + 1] = tc_pack_bf16(tc_field((w & 0x000F0000u) | M, l16, off), tc_field((w8 & 0x000F0000u) | M, l16, off));
        out[8 + 2 * i] = tc_pack_bf16(tc_field((w & 0x000000F0u) | M, h4, off), tc_field((w & 0x0000F000u) | M, h12, off));
        out[8 + 2 * i + 1] = tc_pack_bf16(tc_field((w12 & 0x00000F00u) | M, l8, off), tc_field((w12 & 0x000F0000u) | M, l16, off));
    }
}

template <>
__device__ __forceinline__ void tc_decode_row<SKN_TYPE_Q4_0>(const TcRaw<SKN_TYPE_Q4_0> &raw, const uint8_t *, int,
                                                             uint8_t *tile, int r, bool valid) {
    if (!valid) {
#pragma unroll
        for (int c = 0; c < 8; ++c) tc_store_chunk(tile, r, c, make_uint4(0u, 0u, 0u, 0u));
        return;
    }
    const uint32_t qa[4] = {__funnelshift_r(raw.w[0], raw.w[1], 16), __funnelshift_r(raw.w[1], raw.w[2], 16),
                            __funnelshift_r(raw.w[2], raw.w[3], 16), __funnelshift_r(raw.w[3], raw.w[4], 16)};
    const uint32_t qb[4] = {raw.w[5], raw.w[6], raw.w[7], raw.w[8]};
    uint32_t out[32];
    tc_q40_block(qa, skn_half_bits_to_float(raw.w[0] & 0xFFFFu), out);
    tc_q40_block(qb, skn_half_bits_to_float(raw.w[4] >> 16), out + 16);
#pragma unroll
    for (int c = 0; c < 8; ++c) tc_store_chunk(tile, r, c, make_uint4(out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]));
}

// Q8_0: 64 weights at k0 = two 34-byte blocks = seventeen aligned words.  A signed byte b is
// widened as (2^23 + (b ^ 0x80)) - (2^23 + 128) = b, then multiplied by d.
template <>
__device__ __forceinline__ void tc_load_row<SKN_TYPE_Q8_0>(const uint8_t *rp, int k0, bool valid, TcRaw<SKN_TYPE_Q8_0> &raw) {
    if (!valid) return;
    const uint32_t *p = reinterpret_cast<const uint32_t *>(rp + (size_t)(k0 >> 6) * 68);
#pragma unroll
    for (int i = 0; i < 17; ++i) raw.w[i] = __ldg(p + i);
}

__device__ __forceinline__ void tc_q80_word(uint32_t w, float d, uint32_t *out) {
    const uint32_t u = w ^ 0x80808080u;
    const float f0 = __fmul_rn(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7440)) - 8388736.f, d);
    const float f1 = __fmul_rn(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7441)) - 8388736.f, d);
    const float f2 = __fmul_rn(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7442)) - 8388736.f, d);
    const float f3 = __fmul_rn(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7443)) - 8388736.f, d);
    out[0] = tc_pack_bf16(f0, f1);
    out[1] = tc_pack_bf16(f2, f3);
}

template <>
__device__ __forceinline__ void tc_decode_row<SKN_TYPE_Q8_0>(const TcRaw<SKN_TYPE_Q8_0> &raw, const uint8_t *, int,
                                                             uint8_t *tile, int r, bool valid) {
    if (!valid) {
#pragma unroll
        for (int c = 0; c < 8; ++c) tc_store_chunk(tile, r, c, make_uint4(0u, 0u, 0u, 0u));
        return;
    }
    const float da = skn_half_bits_to_float(raw.w[0] & 0xFFFFu), db = skn_half_bits_to_float(raw.w[8] >> 16);
    uint32_t out[32];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        tc_q80_word(__funnelshift_r(raw.w[i], raw.w[i + 1], 16), da, out + 2 * i);
        tc_q80_word(raw.w[9 + i], db, out + 16 + 2 * i);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) tc_store_chunk(tile, r, c, make_uint4(out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]));
}

// Q6_K: 64 weights at k0 = quarter u of a 210-byte super-block: half h = u/2, groups g0 = 2*(u&1)
// and g0+1.  Blocks start on 2-byte boundaries, so the 64 ql bytes, 32 qh bytes, 4 scales and d
// are read as aligned words and re-aligned with funnel shifts (the shift is the same for all
// threads: every thread of the CTA works on the same k0).
template <>
__device__ __forceinline__ void tc_load_row<SKN_TYPE_Q6_K>(const uint8_t *rp, int k0, bool valid, TcRaw<SKN_TYPE_Q6_K> &raw) {
    if (!valid) return;
    const int b = k0 >> 8, u = (k0 >> 6) & 3, h = u >> 1, g0 = 2 * (u & 1);
    const uint8_t *bp = rp + (size_t)b * 210;
    const uint32_t *wq = reinterpret_cast<const uint32_t *>(reinterpret_cast<uintptr_t>(bp + 64 * h) & ~(uintptr_t)3);
    const uint32_t *wh = reinterpret_cast<const uint32_t *>(reinterpret_cast<uintptr_t>(bp + 128 + 32 * h) & ~(uintptr_t)3);
    const uint32_t *ws = reinterpret_cast<const uint32_t *>(reinterpret_cast<uintptr_t>(bp + 192 + 8 * h + 2 * g0) & ~(uintptr_t)3);
    const uint32_t *wd = reinterpret_cast<const uint32_t *>(reinterpret_cast<uintptr_t>(bp + 208) & ~(uintptr_t)3);
#pragma unroll
    for (int i = 0; i < 17; ++i) raw.rq[i] = __ldg(wq + i);
#pragma unroll
    for (int i = 0; i < 9; ++i) raw.rh[i] = __ldg(wh + i);
    raw.s_lo = __ldg(ws);
    raw.s_hi = __ldg(ws + 1);
    raw.dword = __ldg(wd);
}

template <>
__device__ __forceinline__ void tc_decode_row<SKN_TYPE_Q6_K>(const TcRaw<SKN_TYPE_Q6_K> &raw, const uint8_t *rp, int k0,
                                                             uint8_t *tile, int r, bool valid) {
    if (!valid) {
#pragma unroll
        for (int c = 0; c < 8; ++c) tc_store_chunk(tile, r, c, make_uint4(0u, 0u, 0u, 0u));
        return;
    }
    const int b = k0 >> 8, u = (k0 >> 6) & 3, g0 = 2 * (u & 1);
    const uint32_t sh = (uint32_t)((reinterpret_cast<uintptr_t>(rp + (size_t)b * 210) & 2) * 8);     // 0 or 16
    const uint32_t *rq = raw.rq, *rh = raw.rh;
    const uint32_t s_lo = raw.s_lo, s_hi = raw.s_hi, dword = raw.dword;
    const uint32_t sc4 = __funnelshift_rc(s_lo, s_hi, sh);                        // four int8 scales
    const float d = skn_half_bits_to_float((dword >> sh) & 0xFFFFu);
    float dl[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) dl[i] = __fmul_rn(d, (float)(int8_t)((sc4 >> (8 * i)) & 0xFFu));
    const int sn = (g0 == 2) ? 4 : 0;           // low nibbles for groups 0/1, high nibbles for 2/3
    const int sq = 2 * g0;
    uint32_t out[32];                           // bf16 pairs, weights 0..63
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t qh = __funnelshift_rc(rh[i], rh[i + 1], sh);
        const uint32_t qa = __funnelshift_rc(rq[i], rq[i + 1], sh);            // ql[4i..4i+3]      -> group g0
        const uint32_t qb = __funnelshift_rc(rq[8 + i], rq[9 + i], sh);        // ql[32+4i..]       -> group g0+1
        const uint32_t a4 = ((qa >> sn) & 0x0F0F0F0Fu) | (((qh >> sq) & 0x03030303u) << 4);
        const uint32_t b4 = ((qb >> sn) & 0x0F0F0F0Fu) | (((qh >> (sq + 2)) & 0x03030303u) << 4);
        const float da = dl[i >> 2], db = dl[2 + (i >> 2)];                    // l/16 = i/4
        float fa[4], fb[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            fa[k] = __fmul_rn(__uint_as_float(__byte_perm(a4, 0x4B000000u, 0x7440 + k)) - 8388640.f, da);
            fb[k] = __fmul_rn(__uint_as_float(__byte_perm(b4, 0x4B000000u, 0x7440 + k)) - 8388640.f, db);
        }
        out[2 * i] = tc_pack_bf16(fa[0], fa[1]);
        out[2 * i + 1] = tc_pack_bf16(fa[2], fa[3]);
        out[16 + 2 * i] = tc_pack_bf16(fb[0], fb[1]);
        out[16 + 2 * i + 1] = tc_pack_bf16(fb[2], fb[3]);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) tc_store_chunk(tile, r, c, make_uint4(out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]));
}

__global__ void skn_f32_to_bf16_kernel(const float *__restrict__ in, __nv_bfloat16 *__restrict__ out, int64_t n4) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(in) + i);
        uint2 o;
        o.x = tc_pack_bf16(v.x, v.y);
        o.y = tc_pack_bf16(v.z, v.w);
        reinterpret_cast<uint2 *>(out)[i] = o;
    }
}

// TYPE: block type of W (and W2).  DUAL: out_bf16[m][n] = silu(A.W^T) * (A.W2^T), else
// out_f32[m][n] = A.W^T (+ bias[n]).
// A CTA owns 256 token rows (two 128-row accumulators that share every dequantised weight
// tile) x 128 features.  TMEM columns: [0,128) rows 0-127, [128,256) rows 128-255 and, DUAL,
// [256,512) the same for W2.
template <int TYPE, bool DUAL>
__global__ void __launch_bounds__(TC_THREADS, 1)
skn_matmul_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, int M, int K, const uint8_t *__restrict__ W,
                     const uint8_t *__restrict__ W2, int64_t pitch, int N, const float *__restrict__ bias,
                     float *__restrict__ out_f32, __nv_bfloat16 *__restrict__ out_bf16, int64_t ld_out,
                     int32_t *__restrict__ status, int halves) {
    extern __shared__ uint8_t smem_raw[];
    // operand tiles need 1024-byte alignment for the 128-byte swizzle
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int NB = DUAL ? 2 : 1;
    constexpr int STAGES = DUAL ? 3 : 4;
    constexpr int STAGE_BYTES = (2 + NB) * TC_TILE_BYTES;     // A0 | A1 | B [| B2]
    __shared__ uint64_t full_bar[4], empty_bar[4], accum_bar;
    __shared__ uint32_t tmem_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * (halves * TC_BM), n0 = blockIdx.y * TC_BN;
    const int ksteps = K / TC_BK;
    const bool two = halves == 2 && M - m0 > TC_BM;            // second 128-row half in use
    constexpr uint32_t TMEM_COLS = DUAL ? 512 : 256;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            skn_mbar_init(&full_bar[s], DUAL ? 9 : 5);   // dequant warps of the stage + the TMA thread
            skn_mbar_init(&empty_bar[s], 1);     // one tcgen05.commit
        }
        skn_mbar_init(&accum_bar, 1);
        skn_fence_mbar_init();
    }
    if (warp == 8) tc_alloc(&tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp < 8) {
        // ---------------- weight producers ----------------
        // DUAL: warps 0-3 dequantise W, warps 4-7 W2, every stage.  Otherwise the two groups
        // of four warps take the stages in turn.  Thread t fills tile row t & 127.
        const int grp = warp >> 2;
        const int r = threadIdx.x & 127;
        const bool b_valid = n0 + r < N;
        const uint8_t *wrow = ((DUAL && grp == 1) ? W2 : W) + (int64_t)(b_valid ? n0 + r : 0) * pitch;
        const int tile_off = (DUAL && grp == 1) ? 3 * TC_TILE_BYTES : 2 * TC_TILE_BYTES;
        const int step = DUAL ? 1 : 2, first = DUAL ? 0 : grp;
        bool failed = false;
        TcRaw<TYPE> raw, nraw;                   // this turn's raw weights and the next turn's
        if (first < ksteps) tc_load_row<TYPE>(wrow, first * TC_BK, b_valid, raw);
        for (int it = first; it < ksteps; it += step) {
            const int s = it % STAGES;
            const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
            const int k0 = it * TC_BK;
            if (it + step < ksteps) tc_load_row<TYPE>(wrow, k0 + step * TC_BK, b_valid, nraw);   // flies during this decode
            if (!failed && !skn_mbar_wait(&empty_bar[s], ph ^ 1u)) {
                failed = true;
                atomicExch(status, SKN_ERR_TIMEOUT);
            }
            tc_decode_row<TYPE>(raw, wrow, k0, smem + (size_t)s * STAGE_BYTES + tile_off, r, b_valid);
            raw = nraw;
            skn_fence_proxy_async();     // generic-proxy stores -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) skn_mbar_arrive(&full_bar[s]);
        }
    } else if (warp == 9) {
        // ---------------- activation producer: one thread, TMA ----------------
        if (lane == 0) {
            bool failed = false;
            const uint32_t bytes = (two ? 2u : 1u) * TC_TILE_BYTES;
            for (int it = 0; it < ksteps; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                if (!failed && !skn_mbar_wait(&empty_bar[s], ph ^ 1u)) {
                    failed = true;
                    atomicExch(status, SKN_ERR_TIMEOUT);
                }
                uint8_t *stage = smem + (size_t)s * STAGE_BYTES;
                skn_mbar_expect_tx(&full_bar[s], bytes);
                // rows beyond M are filled with zeros by the tensor map
                tc_tma_load_2d(stage, &tmap_a, it * TC_BK, m0, &full_bar[s]);
                if (two) tc_tma_load_2d(stage + TC_TILE_BYTES, &tmap_a, it * TC_BK, m0 + TC_BM, &full_bar[s]);
            }
        }
    } else if (lane == 0) {
        // ---------------- MMA issuer (warp 8) ----------------
        const uint32_t idesc = tc_idesc(TC_BM, TC_BN);
        bool failed = false;
        for (int it = 0; it < ksteps; ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
            if (!failed && !skn_mbar_wait(&full_bar[s], ph)) {
                failed = true;
                atomicExch(status, SKN_ERR_TIMEOUT);
            }
            tc_fence_after();
            const uint32_t base = skn_smem_u32(smem + (size_t)s * STAGE_BYTES);
            const uint64_t a0desc = tc_smem_desc(base), a1desc = tc_smem_desc(base + TC_TILE_BYTES);
            const uint64_t bdesc = tc_smem_desc(base + 2 * TC_TILE_BYTES);
            const uint64_t b2desc = tc_smem_desc(base + 3 * TC_TILE_BYTES);
#pragma unroll
            for (int k = 0; k < TC_BK / 16; ++k) {
                const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
                // advancing 16 bf16 (32 bytes) along K inside the swizzle atom = +2 in the address field
                tc_mma_bf16(tmem_base, a0desc + 2 * k, bdesc + 2 * k, idesc, acc);
                if (two) tc_mma_bf16(tmem_base + 128, a1desc + 2 * k, bdesc + 2 * k, idesc, acc);
                if (DUAL) {
                    tc_mma_bf16(tmem_base + 256, a0desc + 2 * k, b2desc + 2 * k, idesc, acc);
                    if (two) tc_mma_bf16(tmem_base + 384, a1desc + 2 * k, b2desc + 2 * k, idesc, acc);
                }
            }
            tc_commit(&empty_bar[s]);    // frees the stage once these MMAs have read it
        }
        tc_commit(&accum_bar);           // all MMAs done: the accumulators are complete
    }

    // ---------------- epilogue: warps 0-3, TMEM lane = token row ----------------
    if (warp < 4) {
        const bool ok = skn_mbar_wait(&accum_bar, 0u);
        if (!ok) atomicExch(status, SKN_ERR_TIMEOUT);
        tc_fence_after();
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
        for (int half = 0; half < (two ? 2 : 1) && ok; ++half) {
            const int m = m0 + half * TC_BM + warp * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < TC_BN; c0 += 32) {
                uint32_t acc[32];
                tc_ld32(lane_addr + half * 128 + c0, acc);
                if (DUAL) {
                    uint32_t up[32];
                    tc_ld32(lane_addr + 256 + half * 128 + c0, up);
                    if (m < M) {
                        __nv_bfloat16 *dst = out_bf16 + (int64_t)m * ld_out + n0 + c0;
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            if (n0 + c0 + i < N) {      // N is a multiple of 8 on this path
                                uint32_t hv[4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const float g0 = __uint_as_float(acc[i + 2 * j]), g1 = __uint_as_float(acc[i + 2 * j + 1]);
                                    const float h0 = g0 / (1.f + __expf(-g0)) * __uint_as_float(up[i + 2 * j]);
                                    const float h1 = g1 / (1.f + __expf(-g1)) * __uint_as_float(up[i + 2 * j + 1]);
                                    hv[j] = tc_pack_bf16(h0, h1);
                                }
                                *reinterpret_cast<uint4 *>(dst + i) = make_uint4(hv[0], hv[1], hv[2], hv[3]);
                            }
                        }
                    }
                } else if (m < M) {
                    float *dst = out_f32 + (int64_t)m * ld_out + n0 + c0;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        if (n0 + c0 + i < N) {          // N is a multiple of 4
                            float4 v = make_float4(__uint_as_float(acc[i]), __uint_as_float(acc[i + 1]),
                                                   __uint_as_float(acc[i + 2]), __uint_as_float(acc[i + 3]));
                            if (bias) {
                                const float4 bv = __ldg(reinterpret_cast<const float4 *>(bias + n0 + c0 + i));
                                v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
                            }
                            *reinterpret_cast<float4 *>(dst + i) = v;
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        __syncwarp();
        tc_fence_after();
        tc_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------
typedef CUresult (*skn_encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                        const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                        CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map of the bf16 activations [M][K]: boxes of 64 columns x 128 rows, 128-byte swizzle,
// rows past M read as zeros.
static cudaError_t make_a_tmap(const __nv_bfloat16 *A, int M, int K, CUtensorMap *out) {
    static skn_encode_tiled_fn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess) return e;
        if (!fn || q != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
        encode = (skn_encode_tiled_fn)fn;
    }
    const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t gstride[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)TC_BM};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16 *>(A), gdim, gstride, box,
                              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <int TYPE, bool DUAL>
static cudaError_t launch_tc(const __nv_bfloat16 *A, int M, int K, const skn_tensor *w, const skn_tensor *w2,
                             const float *bias, float *out_f32, __nv_bfloat16 *out_bf16, int64_t ld_out,
                             int32_t *status, cudaStream_t stream) {
    auto kern = skn_matmul_tc_kernel<TYPE, DUAL>;
    const size_t smem = (size_t)(DUAL ? 3 * 4 : 4 * 3) * TC_TILE_BYTES + 1024;
    static bool attr_done[64] = {false};   // per device
    int dev = 0;
    cudaError_t e0 = cudaGetDevice(&dev);
    if (e0 != cudaSuccess) return e0;
    if (!attr_done[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_done[dev & 63] = true;
    }
    CUtensorMap tmap;
    e0 = make_a_tmap(A, M, K, &tmap);
    if (e0 != cudaSuccess) return e0;
    // 256-row CTAs share each dequantised weight tile between two accumulators; when that leaves
    // SMs idle (few feature tiles), 128-row CTAs double the CTA count instead
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t ntiles = (w->n_rows + TC_BN - 1) / TC_BN;
    int halves = (M > TC_BM && ntiles * ((M + 2 * TC_BM - 1) / (2 * TC_BM)) >= sms) ? 2 : 1;
    const dim3 grid((unsigned)((M + halves * TC_BM - 1) / (halves * TC_BM)), (unsigned)ntiles);
    kern<<<grid, TC_THREADS, smem, stream>>>(tmap, M, K, w->d_blocks, w2 ? w2->d_blocks : nullptr, w->pitch, (int)w->n_rows,
                                             bias, out_f32, out_bf16, ld_out, status, halves);
    return cudaGetLastError();
}

template <bool DUAL>
static cudaError_t dispatch_tc(const __nv_bfloat16 *A, int M, int K, const skn_tensor *w, const skn_tensor *w2,
                               const float *bias, float *out_f32, __nv_bfloat16 *out_bf16, int64_t ld_out,
                               int32_t *status, cudaStream_t stream) {
    switch (w->type) {
    case SKN_TYPE_Q4_0: return launch_tc<SKN_TYPE_Q4_0, DUAL>(A, M, K, w, w2, bias, out_f32, out_bf16, ld_out, status, stream);
    case SKN_TYPE_Q8_0: return launch_tc<SKN_TYPE_Q8_0, DUAL>(A, M, K, w, w2, bias, out_f32, out_bf16, ld_out, status, stream);
    case SKN_TYPE_Q4_K: return launch_tc<SKN_TYPE_Q4_K, DUAL>(A, M, K, w, w2, bias, out_f32, out_bf16, ld_out, status, stream);
    case SKN_TYPE_Q6_K: return launch_tc<SKN_TYPE_Q6_K, DUAL>(A, M, K, w, w2, bias, out_f32, out_bf16, ld_out, status, stream);
    default: return cudaErrorInvalidValue;
    }
}

bool skn_tc_supported(const skn_tensor *w, int32_t M) {
    const bool type_ok = w->type == SKN_TYPE_Q4_0 || w->type == SKN_TYPE_Q8_0 || w->type == SKN_TYPE_Q4_K || w->type == SKN_TYPE_Q6_K;
    return type_ok && M >= 1 && (w->n_cols % TC_BK) == 0 && w->n_cols >= TC_BK && (w->n_rows % 8) == 0 && (w->pitch % 16) == 0 &&
           (reinterpret_cast<uintptr_t>(w->d_blocks) & 1) == 0;
}

cudaError_t skn_launch_f32_to_bf16(const float *in, void *out_bf16, int64_t n, int sm_count, cudaStream_t stream) {
    const int64_t n4 = n / 4;
    if (n4 == 0) return cudaSuccess;
    int64_t blocks = (n4 + 255) / 256;
    if (blocks > (int64_t)sm_count * 8) blocks = (int64_t)sm_count * 8;
    skn_f32_to_bf16_kernel<<<(unsigned)blocks, 256, 0, stream>>>(in, (__nv_bfloat16 *)out_bf16, n4);
    return cudaGetLastError();
}

// Y = A_bf16 . W^T (+bias), fp32 out
cudaError_t skn_launch_matmul_tc(skn_ctx *ctx, const skn_tensor *w, const void *a_bf16, int32_t M, const float *bias,
                                 float *y, cudaStream_t stream) {
    return dispatch_tc<false>((const __nv_bfloat16 *)a_bf16, M, (int)w->n_cols, w, nullptr, bias, y, nullptr, w->n_rows,
                              ctx->d_status, stream);
}

// H_bf16 = silu(A . Wg^T) * (A . Wu^T)
cudaError_t skn_launch_gate_up_tc(skn_ctx *ctx, const skn_tensor *wg, const skn_tensor *wu, const void *a_bf16,
                                  int32_t M, void *h_bf16, cudaStream_t stream) {
    return dispatch_tc<true>((const __nv_bfloat16 *)a_bf16, M, (int)wg->n_cols, wg, wu, nullptr, nullptr,
                             (__nv_bfloat16 *)h_bf16, wg->n_rows, ctx->d_status, stream);
}
