// K2: fused dequant-dot  Y[M,N] = X[M,K] . W_q[N,K]^T  for small M (decode).
//
// HBM-bound, CUDA cores only.  Raw GGUF blocks stay unchanged in HBM; nothing is
// dequantised to memory.  Two families:
//
//  * skn_matvec_stream_<type> (M = 1): each warp owns one K-chunk of the row (a run of
//    blocks whose byte length is a multiple of 16) for a strided set of rows.  Its slice of x
//    lives in registers for the whole kernel.  Row-chunks arrive through a warp-private ring
//    of 1-D bulk async copies (TMA) signalled on mbarriers, so HBM requests stay in flight
//    without occupying registers; the weight prefetch is issued before the programmatic
//    dependent-launch wait, x is read after it.  Quant nibbles / bytes are used as fp32
//    operands without an int->float conversion: for an integer k < 2^24 the bit pattern k,
//    read as a float, is exactly k * 2^-149, so `word & mask` is already the operand and x
//    is pre-scaled by a power of two per nibble position (all exact).  Products are fp32
//    FMAs issued as packed f32x2.  Per-row partial sums of the K-chunks meet in shared
//    memory and are added in chunk order (deterministic).
//
//  * skn_matvec_generic<type, MT> (any M, any K multiple of the block, any pitch): one warp
//    per output row, byte-granular decode, MT activation rows per pass.
#include "skn_blocks.cuh"
#include "skn_ptx.cuh"
#include "skn_mv_common.cuh"

// ----------------------------------------------------------------------------------------
// generic kernel
// ----------------------------------------------------------------------------------------
template <int TYPE, int MT>
__global__ void __launch_bounds__(256)
skn_matvec_generic(const uint8_t *__restrict__ W, int64_t pitch, int64_t N, int64_t gpr,
                   const float *__restrict__ x, int M, int64_t K, const float *__restrict__ bias,
                   float *__restrict__ y) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t row = warp; row < N; row += nwarps) {
        const uint8_t *rp = W + row * pitch;
        for (int m0 = 0; m0 < M; m0 += MT) {
            float acc[MT];
#pragma unroll
            for (int mi = 0; mi < MT; ++mi) acc[mi] = 0.f;
            for (int64_t g = lane; g < gpr; g += 32) {
                float w[32];
                decode_group<TYPE>(rp, g, w);
#pragma unroll
                for (int mi = 0; mi < MT; ++mi) {
                    if (m0 + mi < M) {
                        const float4 *xp = reinterpret_cast<const float4 *>(x + (int64_t)(m0 + mi) * K + g * 32);
                        float a = acc[mi];
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const float4 v = __ldg(xp + q);
                            a = fmaf(w[4 * q], v.x, a);
                            a = fmaf(w[4 * q + 1], v.y, a);
                            a = fmaf(w[4 * q + 2], v.z, a);
                            a = fmaf(w[4 * q + 3], v.w, a);
                        }
                        acc[mi] = a;
                    }
                }
            }
#pragma unroll
            for (int mi = 0; mi < MT; ++mi) {
                float a = acc[mi];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                if (lane == 0 && m0 + mi < M) y[(int64_t)(m0 + mi) * N + row] = a + (bias ? bias[row] : 0.f);
            }
        }
    }
}

template <int TYPE>
static cudaError_t launch_generic(const skn_tensor *w, const float *x, int M, const float *bias, float *y,
                                  int sm_count, cudaStream_t stream) {
    const int64_t gpr = w->n_cols / 32;
    int64_t blocks = (w->n_rows + 7) / 8;  // 8 warps per CTA, one row per warp per pass
    const int64_t cap = (int64_t)sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (M == 1)
        skn_matvec_generic<TYPE, 1><<<(unsigned)blocks, 256, 0, stream>>>(w->d_blocks, w->pitch, w->n_rows, gpr, x, M,
                                                                         w->n_cols, bias, y);
    else if (M == 2)
        skn_matvec_generic<TYPE, 2><<<(unsigned)blocks, 256, 0, stream>>>(w->d_blocks, w->pitch, w->n_rows, gpr, x, M,
                                                                         w->n_cols, bias, y);
    else
        skn_matvec_generic<TYPE, 4><<<(unsigned)blocks, 256, 0, stream>>>(w->d_blocks, w->pitch, w->n_rows, gpr, x, M,
                                                                         w->n_cols, bias, y);
    return cudaGetLastError();
}

// ----------------------------------------------------------------------------------------
// streaming M = 1 kernels
// ----------------------------------------------------------------------------------------
constexpr int MV_NST = 8;          // ring stages per warp == rows per reduction group

// Sum 8 per-lane values across the warp in 9 shuffles.  On return the lanes whose
// (lane >> 2) == r hold the total of v[r].
__device__ __forceinline__ float skn_warp_reduce8(const float (&v)[8], int lane) {
    float a[4], b[2];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float send = (lane & 16) ? v[k] : v[k + 4];
        const float keep = (lane & 16) ? v[k + 4] : v[k];
        a[k] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const float send = (lane & 8) ? a[k] : a[k + 2];
        const float keep = (lane & 8) ? a[k + 2] : a[k];
        b[k] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    const float send = (lane & 4) ? b[0] : b[1];
    const float keep = (lane & 4) ? b[1] : b[0];
    float c = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    return c;
}

// CTA-cooperative preparation of x for the 4-bit decoders: K activations from global memory ->
// per group of 64: 32 packed pairs (pre-scaled by 2^(S - nibble position)), the two 32-element
// sums and the factor 2^(149 - S).  kpad (a multiple of 2048) is the padded length; columns
// >= K are written as zeros.  A float4 of x is always the four bytes k = 0..3 of one quant
// word, low-nibble (h = 0) or high-nibble (h = 1) half:
//   Q4_K  (Q40 = false): group = sub-block pair; float4 f -> h = (f>>3)&1, word = f&7
//   Q4_0  (Q40 = true) : group = two blocks;     float4 f -> block = (f>>3)&1, h = (f>>2)&1, word = f&3
// The pair of word-pair j, nibble position n = 2k+h is {x[word 2j], x[word 2j+1]} and sits in
// 16-byte slot j*4 + k (rotated by the group index, see load_x), float 2h + (word & 1).
template <bool Q40>
static __device__ __forceinline__ void skn_prep_nibble_groups(const float *__restrict__ x, int K, int kpad, uint8_t *xs,
                                                              const skn_xform &xf) {
    float *gsum = reinterpret_cast<float *>(xs + (size_t)kpad * 4);
    float *gun = gsum + kpad / 32;
    const int nf = kpad / 4;
    const int lane = threadIdx.x & 31;
    constexpr int B = 4;   // float4 loads in flight per thread
    for (int f0 = 0; f0 < nf; f0 += B * blockDim.x) {
        float4 v[B];
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const int f = f0 + b * blockDim.x + threadIdx.x;
            v[b] = (f < nf && 4 * f < K) ? skn_load_x4(x, f, xf) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const int f = f0 + b * blockDim.x + threadIdx.x;   // 16 consecutive f = one group
            float mx = fmaxf(fmaxf(fabsf(v[b].x), fabsf(v[b].y)), fmaxf(fabsf(v[b].z), fabsf(v[b].w)));
            float sm = (v[b].x + v[b].y) + (v[b].z + v[b].w);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
            int S = 217 - (int)(__float_as_uint(mx) >> 23);
            S = S > 120 ? 120 : (S < 23 ? 23 : S);
            if (f < nf) {
                const int G = f >> 4;
                const int half8 = (f >> 3) & 1;         // which 32-element sum this float4 belongs to
                int h, j, comp;
                if (Q40) {
                    const int q = f & 3;
                    h = (f >> 2) & 1;
                    j = 2 * half8 + (q >> 1);
                    comp = q & 1;
                } else {
                    const int wi = f & 7;
                    h = half8;
                    j = wi >> 1;
                    comp = wi & 1;
                }
                const int ph = 4 * h;
                float *g32 = reinterpret_cast<float *>(xs + (size_t)G * 256);
                g32[((j * 4 + 0 + G) & 15) * 4 + 2 * h + comp] = v[b].x * skn_pow2f(S - ph);
                g32[((j * 4 + 1 + G) & 15) * 4 + 2 * h + comp] = v[b].y * skn_pow2f(S - 8 - ph);
                g32[((j * 4 + 2 + G) & 15) * 4 + 2 * h + comp] = v[b].z * skn_pow2f(S - 16 - ph);
                g32[((j * 4 + 3 + G) & 15) * 4 + 2 * h + comp] = v[b].w * skn_pow2f(S - 16 - ph);
                if ((lane & 7) == 0) gsum[2 * G + half8] = sm;
                if ((lane & 15) == 0) gun[G] = skn_pow2f(149 - S);
            }
        }
    }
}

// eight packed FMAs of one 64-bit pair of quant words against the eight nibble positions
#define SKN_NIBBLE_PAIR_FMA(P, X, A0, A1, A2, A3)                                         \
    do {                                                                                  \
        const uint64_t P8__ = (P) >> 8;                                                    \
        A0 = skn_fma2((P) & 0x0000000F0000000Full, (X)[0], A0);                            \
        A1 = skn_fma2((P) & 0x000000F0000000F0ull, (X)[1], A1);                            \
        A2 = skn_fma2((P) & 0x00000F0000000F00ull, (X)[2], A2);                            \
        A3 = skn_fma2((P) & 0x0000F0000000F000ull, (X)[3], A3);                            \
        A0 = skn_fma2((P) & 0x000F0000000F0000ull, (X)[4], A0);                            \
        A1 = skn_fma2((P) & 0x00F0000000F00000ull, (X)[5], A1);                            \
        A2 = skn_fma2(P8__ & 0x000F0000000F0000ull, (X)[6], A2);                           \
        A3 = skn_fma2(P8__ & 0x00F0000000F00000ull, (X)[7], A3);                           \
    } while (0)

// ---- Q4_K ------------------------------------------------------------------------------
// chunk = 8 super-blocks (2048 weights, 1152 bytes); lane = (block cb = lane/4, pair p =
// lane%4): the 32 quant bytes whose low nibbles are sub-block 2p and high nibbles
// sub-block 2p+1, i.e. the 64 consecutive weights ("group") starting at 256*cb + 64*p.
//
// The 32 quant bytes are read as four 64-bit values (two 32-bit words each).  The two
// halves of a packed f32x2 operand are the SAME nibble position of the two words, so
// `pair & mask64` is already the packed operand (no register shuffling).  Nibble position
// n = 2k+h of byte k (h = 0 low nibble, 1 high nibble) sits at bit 4n; byte 3 is taken
// from (pair >> 8), i.e. at bits 16 / 20, to stay inside the 24 bits that read as k*2^-149.
//
// Shared x layout produced by prep_x, per group G of 64 activations:
//   xp[G]  : 32 packed pairs; pair j*8+n = {x[32h + 8j + k], x[32h + 8j + 4 + k]} * 2^(S-pos(n));
//            the sixteen 16-byte slots of a group are rotated by G so that the lanes of a warp
//            (consecutive groups) read conflict-free
//   gsum[2G], gsum[2G+1] : plain sums of the low / high 32 activations (for the -dmin*m term)
//   gun[G] : 2^(149-S), which undoes the 2^(S-149) carried by the dot
// S (23..120) is chosen per group so that its largest |x| lands near 2^90 (for |x| up to
// 2^67; larger activations simply keep S = 23): the pre-scaled activations do not overflow
// and their products with k * 2^-149 stay normal numbers.
struct Q4KStream {
    static constexpr int CHUNK_BLOCKS = 8;
    static constexpr int BLOCK_BYTES = 144;
    static constexpr int BLOCK_WEIGHTS = 256;
    static constexpr int CHUNK_BYTES = CHUNK_BLOCKS * BLOCK_BYTES;
    static constexpr int CHUNK_WEIGHTS = CHUNK_BLOCKS * BLOCK_WEIGHTS;
    // bytes of prepared x per weight column: 4 (pairs) + 2/32*4 (sums) + 1/64*4 (unscale)
    static __host__ __device__ size_t xprep_bytes(int64_t kpad) { return (size_t)kpad * 4 + (size_t)kpad / 8 + (size_t)kpad / 16; }

    struct Raw { ulonglong2 q0, q1; uint4 hdr; };   // one lane's share of a staged row-chunk

    uint64_t x2[32];
    float sum_lo, sum_hi, unscale;
    int off;          // byte offset of this lane's block inside a staged chunk
    int p;
    uint32_t sel, m_low, m_top, m_nib;   // per-lane constants of the scale decode
    bool active;

    static __device__ __forceinline__ void prep_x(const float *__restrict__ x, int K, int kpad, uint8_t *xs, const skn_xform &xf) {
        skn_prep_nibble_groups<false>(x, K, kpad, xs, xf);
    }

    __device__ __forceinline__ void load_x(const uint8_t *xs, int kpad, int chunk, int lane, int nblocks_in_chunk) {
        const int cb = lane >> 2;
        p = lane & 3;
        off = cb * BLOCK_BYTES;
        active = cb < nblocks_in_chunk;
        sel = (p & 1) ? 0x4432u : 0x4410u;            // bytes (2,3) or (0,1), upper half zero
        m_low = (p < 2) ? 0x3F3Fu : 0u;
        m_top = (p < 2) ? 0u : 0x3030u;
        m_nib = (p < 2) ? 0u : 0x0F0Fu;
        const int G = (chunk * CHUNK_BLOCKS + cb) * 4 + p;
        const ulonglong2 *g = reinterpret_cast<const ulonglong2 *>(xs + (size_t)G * 256);
        const float *gsum = reinterpret_cast<const float *>(xs + (size_t)kpad * 4);
        const float *gun = gsum + kpad / 32;
#pragma unroll
        for (int s = 0; s < 16; ++s) {
            const ulonglong2 v = g[(s + G) & 15];
            x2[2 * s] = v.x;
            x2[2 * s + 1] = v.y;
        }
        sum_lo = gsum[2 * G];
        sum_hi = gsum[2 * G + 1];
        unscale = gun[G];
    }

    __device__ __forceinline__ Raw fetch(const uint8_t *sb) const {
        Raw r;
        r.hdr = *reinterpret_cast<const uint4 *>(sb + off);
        r.q0 = *reinterpret_cast<const ulonglong2 *>(sb + off + 16 + 32 * p);
        r.q1 = *reinterpret_cast<const ulonglong2 *>(sb + off + 32 + 32 * p);
        return r;
    }

    // scale / min decode and final combination shared by dot() and dot2()
    __device__ __forceinline__ float finish(const uint4 hdr, float dlo, float dhi) const {
        // 6-bit scales / mins of sub-blocks 2p and 2p+1: two adjacent bytes of each of the three
        // 4-byte groups; sel picks them with one byte-permute each, the three masks make the
        // two packing rules (sub-blocks 0-3 / 4-7) one branch-free expression
        const uint32_t a2 = __byte_perm(hdr.y, 0u, sel), b2 = __byte_perm(hdr.z, 0u, sel), c2 = __byte_perm(hdr.w, 0u, sel);
        const uint32_t sc2 = (a2 & m_low) | ((a2 >> 2) & m_top) | (c2 & m_nib);
        const uint32_t mn2 = (b2 & m_low) | ((b2 >> 2) & m_top) | ((c2 >> 4) & m_nib);
        // small ints -> float without the conversion pipe: (2^23 + k) - 2^23
        const float sc_lo = __uint_as_float(__byte_perm(sc2, 0x4B000000u, 0x7440)) - 8388608.f;
        const float sc_hi = __uint_as_float(__byte_perm(sc2, 0x4B000000u, 0x7441)) - 8388608.f;
        const float mn_lo = __uint_as_float(__byte_perm(mn2, 0x4B000000u, 0x7440)) - 8388608.f;
        const float mn_hi = __uint_as_float(__byte_perm(mn2, 0x4B000000u, 0x7441)) - 8388608.f;
        const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));   // {d, dmin}
        const float t1 = fmaf(sc_hi, dhi, sc_lo * dlo) * unscale;
        const float t2 = fmaf(mn_hi, sum_hi, mn_lo * sum_lo);
        const float res = fmaf(dd.x, t1, -dd.y * t2);
        return active ? res : 0.f;
    }

    // partial dot of this lane's 64 weights
    __device__ __forceinline__ float dot(const Raw &r) const {
        const uint64_t qp[4] = {r.q0.x, r.q0.y, r.q1.x, r.q1.y};
        uint64_t lo0 = 0ull, lo1 = 0ull, hi0 = 0ull, hi1 = 0ull;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint64_t P = qp[j];
            const uint64_t P8 = P >> 8;
            lo0 = skn_fma2(P & 0x0000000F0000000Full, x2[8 * j + 0], lo0);
            hi0 = skn_fma2(P & 0x000000F0000000F0ull, x2[8 * j + 1], hi0);
            lo1 = skn_fma2(P & 0x00000F0000000F00ull, x2[8 * j + 2], lo1);
            hi1 = skn_fma2(P & 0x0000F0000000F000ull, x2[8 * j + 3], hi1);
            lo0 = skn_fma2(P & 0x000F0000000F0000ull, x2[8 * j + 4], lo0);
            hi0 = skn_fma2(P & 0x00F0000000F00000ull, x2[8 * j + 5], hi0);
            lo1 = skn_fma2(P8 & 0x000F0000000F0000ull, x2[8 * j + 6], lo1);
            hi1 = skn_fma2(P8 & 0x00F0000000F00000ull, x2[8 * j + 7], hi1);
        }
        float la, lb, ha, hb;
        skn_unpack2(skn_add2(lo0, lo1), la, lb);
        skn_unpack2(skn_add2(hi0, hi1), ha, hb);
        const float dlo = la + lb, dhi = ha + hb;

        return finish(r.hdr, dlo, dhi);
    }
};

// ---- Q4_0 ------------------------------------------------------------------------------
// chunk = 64 blocks (2048 weights, 1152 bytes); lane = two adjacent 18-byte blocks = nine
// aligned words [dA|q0 q1][q2..5][q6..9][q10..13][q14 q15|dB][B: q0..3] ... [B: q12..15].
// Byte e of a block: low nibble = weight e, high nibble = weight e+16; value (n - 8) * d, so
// a block contributes d * (sum n*x - 8 * sum x).
struct Q40Stream {
    static constexpr int CHUNK_BLOCKS = 64;
    static constexpr int BLOCK_BYTES = 18;
    static constexpr int BLOCK_WEIGHTS = 32;
    static constexpr int CHUNK_BYTES = CHUNK_BLOCKS * BLOCK_BYTES;
    static constexpr int CHUNK_WEIGHTS = CHUNK_BLOCKS * BLOCK_WEIGHTS;
    static __host__ __device__ size_t xprep_bytes(int64_t kpad) { return (size_t)kpad * 4 + (size_t)kpad / 8 + (size_t)kpad / 16; }

    struct Raw { uint32_t w[9]; };

    uint64_t x2[32];
    float sum_a, sum_b, unscale;
    int off;
    bool act_a, act_b;

    static __device__ __forceinline__ void prep_x(const float *__restrict__ x, int K, int kpad, uint8_t *xs, const skn_xform &xf) {
        skn_prep_nibble_groups<true>(x, K, kpad, xs, xf);
    }

    __device__ __forceinline__ void load_x(const uint8_t *xs, int kpad, int chunk, int lane, int nblocks_in_chunk) {
        off = lane * 2 * BLOCK_BYTES;
        act_a = 2 * lane < nblocks_in_chunk;
        act_b = 2 * lane + 1 < nblocks_in_chunk;
        const int G = chunk * (CHUNK_BLOCKS / 2) + lane;
        const ulonglong2 *g = reinterpret_cast<const ulonglong2 *>(xs + (size_t)G * 256);
        const float *gsum = reinterpret_cast<const float *>(xs + (size_t)kpad * 4);
        const float *gun = gsum + kpad / 32;
#pragma unroll
        for (int s = 0; s < 16; ++s) {
            const ulonglong2 v = g[(s + G) & 15];
            x2[2 * s] = v.x;
            x2[2 * s + 1] = v.y;
        }
        sum_a = gsum[2 * G];
        sum_b = gsum[2 * G + 1];
        unscale = gun[G];
    }

    __device__ __forceinline__ Raw fetch(const uint8_t *sb) const {
        Raw r;
        const uint32_t *p = reinterpret_cast<const uint32_t *>(sb + off);
#pragma unroll
        for (int i = 0; i < 9; ++i) r.w[i] = p[i];
        return r;
    }

    __device__ __forceinline__ float dot(const Raw &r) const {
        // block A's quant words straddle the aligned words by two bytes
        const uint32_t a0 = __funnelshift_r(r.w[0], r.w[1], 16), a1 = __funnelshift_r(r.w[1], r.w[2], 16);
        const uint32_t a2 = __funnelshift_r(r.w[2], r.w[3], 16), a3 = __funnelshift_r(r.w[3], r.w[4], 16);
        const uint64_t pa0 = ((uint64_t)a1 << 32) | a0, pa1 = ((uint64_t)a3 << 32) | a2;
        const uint64_t pb0 = ((uint64_t)r.w[6] << 32) | r.w[5], pb1 = ((uint64_t)r.w[8] << 32) | r.w[7];
        uint64_t a_0 = 0ull, a_1 = 0ull, a_2 = 0ull, a_3 = 0ull, b_0 = 0ull, b_1 = 0ull, b_2 = 0ull, b_3 = 0ull;
        SKN_NIBBLE_PAIR_FMA(pa0, x2 + 0, a_0, a_1, a_2, a_3);
        SKN_NIBBLE_PAIR_FMA(pb0, x2 + 16, b_0, b_1, b_2, b_3);
        SKN_NIBBLE_PAIR_FMA(pa1, x2 + 8, a_0, a_1, a_2, a_3);
        SKN_NIBBLE_PAIR_FMA(pb1, x2 + 24, b_0, b_1, b_2, b_3);
        float a_lo, a_hi, b_lo, b_hi;
        skn_unpack2(skn_add2(skn_add2(a_0, a_1), skn_add2(a_2, a_3)), a_lo, a_hi);
        skn_unpack2(skn_add2(skn_add2(b_0, b_1), skn_add2(b_2, b_3)), b_lo, b_hi);
        const float da = skn_half_bits_to_float(r.w[0] & 0xFFFFu);
        const float db = skn_half_bits_to_float(r.w[4] >> 16);
        const float ra = da * fmaf(a_lo + a_hi, unscale, -8.f * sum_a);
        const float rb = db * fmaf(b_lo + b_hi, unscale, -8.f * sum_b);
        return (act_a ? ra : 0.f) + (act_b ? rb : 0.f);
    }
};

// ---- Q8_0 ------------------------------------------------------------------------------
// chunk = 32 blocks (1024 weights, 1088 bytes); lane = one 34-byte block, read as nine aligned
// words and re-aligned with funnel shifts (blocks start on 2-byte boundaries).  A signed
// byte b is used as the unsigned u = b ^ 0x80 = b + 128, so a block contributes
// d * (sum u*x - 128 * sum x).  The two halves of a packed operand are the same byte position
// of two adjacent quant words; byte 3 is taken from (pair >> 8).
//
// Shared x layout per group of 32 activations (one block): 16 packed pairs, pair j*4+k =
// {x[8j + k], x[8j + 4 + k]} * 2^(S - pos(k)), pos = 0, 8, 16, 16; eight 16-byte slots rotated
// by the group index; gsum[G] = plain sum, gun[G] = 2^(149 - S).
struct Q80Stream {
    static constexpr int CHUNK_BLOCKS = 32;
    static constexpr int BLOCK_BYTES = 34;
    static constexpr int BLOCK_WEIGHTS = 32;
    static constexpr int CHUNK_BYTES = CHUNK_BLOCKS * BLOCK_BYTES;
    static constexpr int CHUNK_WEIGHTS = CHUNK_BLOCKS * BLOCK_WEIGHTS;
    static __host__ __device__ size_t xprep_bytes(int64_t kpad) { return (size_t)kpad * 4 + (size_t)kpad / 8 + (size_t)kpad / 8; }

    struct Raw { uint32_t w[9]; };

    uint64_t x2[16];
    float sum, unscale;
    int woff;       // byte offset of the aligned 36-byte window inside a staged chunk
    int sh;         // 0 or 16: bit offset of the block inside the window
    bool active;

    static __device__ __forceinline__ void prep_x(const float *__restrict__ x, int K, int kpad, uint8_t *xs, const skn_xform &xf) {
        float *gsum = reinterpret_cast<float *>(xs + (size_t)kpad * 4);
        float *gun = gsum + kpad / 32;
        const int nf = kpad / 4;
        const int lane = threadIdx.x & 31;
        constexpr int B = 4;
        for (int f0 = 0; f0 < nf; f0 += B * blockDim.x) {
            float4 v[B];
#pragma unroll
            for (int b = 0; b < B; ++b) {
                const int f = f0 + b * blockDim.x + threadIdx.x;
                v[b] = (f < nf && 4 * f < K) ? skn_load_x4(x, f, xf) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int b = 0; b < B; ++b) {
                const int f = f0 + b * blockDim.x + threadIdx.x;   // 8 consecutive f = one group
                float mx = fmaxf(fmaxf(fabsf(v[b].x), fabsf(v[b].y)), fmaxf(fabsf(v[b].z), fabsf(v[b].w)));
                float sm = (v[b].x + v[b].y) + (v[b].z + v[b].w);
#pragma unroll
                for (int o = 4; o > 0; o >>= 1) {
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                    sm += __shfl_xor_sync(0xffffffffu, sm, o);
                }
                int S = 217 - (int)(__float_as_uint(mx) >> 23);
                S = S > 120 ? 120 : (S < 23 ? 23 : S);
                if (f < nf) {
                    const int G = f >> 3;
                    const int q = f & 7, j = q >> 1, comp = q & 1;
                    float *g32 = reinterpret_cast<float *>(xs + (size_t)G * 128);
                    // byte k -> pair j*4 + k -> 16-byte slot 2j + (k>>1), float 2*(k&1) + comp
                    g32[((2 * j + 0 + G) & 7) * 4 + 0 + comp] = v[b].x * skn_pow2f(S);
                    g32[((2 * j + 0 + G) & 7) * 4 + 2 + comp] = v[b].y * skn_pow2f(S - 8);
                    g32[((2 * j + 1 + G) & 7) * 4 + 0 + comp] = v[b].z * skn_pow2f(S - 16);
                    g32[((2 * j + 1 + G) & 7) * 4 + 2 + comp] = v[b].w * skn_pow2f(S - 16);
                    if ((lane & 7) == 0) {
                        gsum[G] = sm;
                        gun[G] = skn_pow2f(149 - S);
                    }
                }
            }
        }
    }

    __device__ __forceinline__ void load_x(const uint8_t *xs, int kpad, int chunk, int lane, int nblocks_in_chunk) {
        const int boff = lane * BLOCK_BYTES;
        woff = boff & ~3;
        sh = (boff & 2) * 8;
        active = lane < nblocks_in_chunk;
        const int G = chunk * CHUNK_BLOCKS + lane;
        const ulonglong2 *g = reinterpret_cast<const ulonglong2 *>(xs + (size_t)G * 128);
        const float *gsum = reinterpret_cast<const float *>(xs + (size_t)kpad * 4);
        const float *gun = gsum + kpad / 32;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const ulonglong2 v = g[(s + G) & 7];
            x2[2 * s] = v.x;
            x2[2 * s + 1] = v.y;
        }
        sum = gsum[G];
        unscale = gun[G];
    }

    __device__ __forceinline__ Raw fetch(const uint8_t *sb) const {
        Raw r;
        const uint32_t *p = reinterpret_cast<const uint32_t *>(sb + woff);
#pragma unroll
        for (int i = 0; i < 9; ++i) r.w[i] = p[i];
        return r;
    }

    __device__ __forceinline__ float dot(const Raw &r) const {
        uint32_t q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = __funnelshift_rc(r.w[i], r.w[i + 1], sh + 16);
        uint64_t a0 = 0ull, a1 = 0ull, a2 = 0ull, a3 = 0ull;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint64_t P = (((uint64_t)q[2 * j + 1] << 32) | q[2 * j]) ^ 0x8080808080808080ull;
            const uint64_t P8 = P >> 8;
            a0 = skn_fma2(P & 0x000000FF000000FFull, x2[4 * j + 0], a0);
            a1 = skn_fma2(P & 0x0000FF000000FF00ull, x2[4 * j + 1], a1);
            a2 = skn_fma2(P & 0x00FF000000FF0000ull, x2[4 * j + 2], a2);
            a3 = skn_fma2(P8 & 0x00FF000000FF0000ull, x2[4 * j + 3], a3);
        }
        float lo, hi;
        skn_unpack2(skn_add2(skn_add2(a0, a1), skn_add2(a2, a3)), lo, hi);
        const float d = skn_half_bits_to_float((r.w[0] >> sh) & 0xFFFFu);
        const float res = d * fmaf(lo + hi, unscale, -128.f * sum);
        return active ? res : 0.f;
    }
};

// ---- Q6_K ------------------------------------------------------------------------------
// chunk = 8 super-blocks (2048 weights, 1680 bytes); lane = (block cb = lane/4, quarter u =
// lane%4): half h = u/2, groups g0 = 2*(u&1) and g0+1, i.e. the 64 consecutive weights starting
// at 256*cb + 64*u.  They use 64 ql bytes (low nibbles for groups 0/1, high for 2/3), 32 qh
// bytes (two bits per group), four int8 scales and d.  Blocks start on 2-byte boundaries:
// everything is read as aligned words and re-aligned with a per-lane funnel shift.
// The 6-bit quant q = nibble | (two bits << 4) is assembled four at a time with integer
// ops; each byte of the result, masked in place, is the fp32 operand q * 2^(8k) * 2^-149.
// A 16-weight sub-group with scale sc contributes d * sc * (sum q*x - 32 * sum x).
//
// Shared x layout per group of 64 activations: 32 packed pairs, pair grp*16 + j*4 + k =
// {x[32grp + 8j + k], x[32grp + 8j + 4 + k]} * 2^(S - pos(k)), pos = 0, 8, 16, 16 (sixteen
// 16-byte slots rotated by the group index); gsum[4G + i] = sum of activations 16i..16i+15;
// gun[G] = 2^(149 - S).
struct Q6KStream {
    static constexpr int CHUNK_BLOCKS = 8;
    static constexpr int BLOCK_BYTES = 210;
    static constexpr int BLOCK_WEIGHTS = 256;
    static constexpr int CHUNK_BYTES = CHUNK_BLOCKS * BLOCK_BYTES;
    static constexpr int CHUNK_WEIGHTS = CHUNK_BLOCKS * BLOCK_WEIGHTS;
    static __host__ __device__ size_t xprep_bytes(int64_t kpad) { return (size_t)kpad * 4 + (size_t)kpad / 4 + (size_t)kpad / 16; }

    struct Raw { uint32_t ql[17], qh[9], sc[2], dw; };

    uint64_t x2[32];
    float sums[4], unscale;
    int o_ql, o_qh, o_sc, o_d;    // aligned byte offsets inside a staged chunk
    uint32_t sh;                  // 0 or 16: the block's misalignment in bits
    int sn, sq;                   // nibble shift (0 / 4) and qh shift (0 / 4) of group g0
    bool active;

    static __device__ __forceinline__ void prep_x(const float *__restrict__ x, int K, int kpad, uint8_t *xs, const skn_xform &xf) {
        float *gsum = reinterpret_cast<float *>(xs + (size_t)kpad * 4);
        float *gun = gsum + kpad / 16;
        const int nf = kpad / 4;
        const int lane = threadIdx.x & 31;
        constexpr int B = 4;
        for (int f0 = 0; f0 < nf; f0 += B * blockDim.x) {
            float4 v[B];
#pragma unroll
            for (int b = 0; b < B; ++b) {
                const int f = f0 + b * blockDim.x + threadIdx.x;
                v[b] = (f < nf && 4 * f < K) ? skn_load_x4(x, f, xf) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int b = 0; b < B; ++b) {
                const int f = f0 + b * blockDim.x + threadIdx.x;   // 16 consecutive f = one group
                float mx = fmaxf(fmaxf(fabsf(v[b].x), fabsf(v[b].y)), fmaxf(fabsf(v[b].z), fabsf(v[b].w)));
                float sm = (v[b].x + v[b].y) + (v[b].z + v[b].w);
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
#pragma unroll
                for (int o = 2; o > 0; o >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, o);
                int S = 217 - (int)(__float_as_uint(mx) >> 23);
                S = S > 120 ? 120 : (S < 23 ? 23 : S);
                if (f < nf) {
                    const int G = f >> 4, idx = f & 15;
                    const int grp = idx >> 3, word = idx & 7, j = word >> 1, comp = word & 1;
                    float *g32 = reinterpret_cast<float *>(xs + (size_t)G * 256);
                    // byte k -> pair grp*16 + j*4 + k -> slot grp*8 + j*2 + (k>>1), float 2*(k&1) + comp
                    const int sl = grp * 8 + j * 2;
                    g32[((sl + 0 + G) & 15) * 4 + 0 + comp] = v[b].x * skn_pow2f(S);
                    g32[((sl + 0 + G) & 15) * 4 + 2 + comp] = v[b].y * skn_pow2f(S - 8);
                    g32[((sl + 1 + G) & 15) * 4 + 0 + comp] = v[b].z * skn_pow2f(S - 16);
                    g32[((sl + 1 + G) & 15) * 4 + 2 + comp] = v[b].w * skn_pow2f(S - 16);
                    if ((lane & 3) == 0) gsum[4 * G + (idx >> 2)] = sm;
                    if ((lane & 15) == 0) gun[G] = skn_pow2f(149 - S);
                }
            }
        }
    }

    __device__ __forceinline__ void load_x(const uint8_t *xs, int kpad, int chunk, int lane, int nblocks_in_chunk) {
        const int cb = lane >> 2, u = lane & 3, h = u >> 1, g0 = 2 * (u & 1);
        active = cb < nblocks_in_chunk;
        const int base = cb * BLOCK_BYTES;            // chunk starts are 16-byte aligned
        sh = (uint32_t)(base & 2) * 8;
        o_ql = (base + 64 * h) & ~3;
        o_qh = (base + 128 + 32 * h) & ~3;
        o_sc = (base + 192 + 8 * h + 2 * g0) & ~3;
        o_d = (base + 208) & ~3;
        sn = (g0 == 2) ? 4 : 0;
        sq = 2 * g0;
        const int G = (chunk * CHUNK_BLOCKS + cb) * 4 + u;
        const ulonglong2 *g = reinterpret_cast<const ulonglong2 *>(xs + (size_t)G * 256);
        const float *gsum = reinterpret_cast<const float *>(xs + (size_t)kpad * 4);
        const float *gun = gsum + kpad / 16;
#pragma unroll
        for (int s = 0; s < 16; ++s) {
            const ulonglong2 v = g[(s + G) & 15];
            x2[2 * s] = v.x;
            x2[2 * s + 1] = v.y;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) sums[i] = gsum[4 * G + i];
        unscale = gun[G];
    }

    __device__ __forceinline__ Raw fetch(const uint8_t *sb) const {
        Raw r;
        const uint32_t *pq = reinterpret_cast<const uint32_t *>(sb + o_ql);
        const uint32_t *ph = reinterpret_cast<const uint32_t *>(sb + o_qh);
        const uint32_t *ps = reinterpret_cast<const uint32_t *>(sb + o_sc);
#pragma unroll
        for (int i = 0; i < 17; ++i) r.ql[i] = pq[i];
#pragma unroll
        for (int i = 0; i < 9; ++i) r.qh[i] = ph[i];
        r.sc[0] = ps[0];
        r.sc[1] = ps[1];
        r.dw = *reinterpret_cast<const uint32_t *>(sb + o_d);
        return r;
    }

    __device__ __forceinline__ float dot(const Raw &r) const {
        uint64_t acc[4] = {0ull, 0ull, 0ull, 0ull};        // (group, 16-weight half)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t h0 = __funnelshift_rc(r.qh[2 * j], r.qh[2 * j + 1], sh);
            const uint32_t h1 = __funnelshift_rc(r.qh[2 * j + 1], r.qh[2 * j + 2], sh);
            const uint64_t H = (((uint64_t)h1 << 32) | h0) >> sq;
#pragma unroll
            for (int grp = 0; grp < 2; ++grp) {
                const uint32_t a0 = __funnelshift_rc(r.ql[8 * grp + 2 * j], r.ql[8 * grp + 2 * j + 1], sh);
                const uint32_t a1 = __funnelshift_rc(r.ql[8 * grp + 2 * j + 1], r.ql[8 * grp + 2 * j + 2], sh);
                const uint64_t P = (((uint64_t)a1 << 32) | a0) >> sn;
                // bits 4-5 of every byte from qh (group g0: bits 0-1 after the shift, g0+1: bits 2-3)
                const uint64_t hb = grp ? ((H << 2) & 0x3030303030303030ull) : ((H << 4) & 0x3030303030303030ull);
                const uint64_t Q = (P & 0x0F0F0F0F0F0F0F0Full) | hb;
                const uint64_t Q8 = Q >> 8;
                uint64_t a = acc[2 * grp + (j >> 1)];
                a = skn_fma2(Q & 0x000000FF000000FFull, x2[grp * 16 + j * 4 + 0], a);
                a = skn_fma2(Q & 0x0000FF000000FF00ull, x2[grp * 16 + j * 4 + 1], a);
                a = skn_fma2(Q & 0x00FF000000FF0000ull, x2[grp * 16 + j * 4 + 2], a);
                a = skn_fma2(Q8 & 0x00FF000000FF0000ull, x2[grp * 16 + j * 4 + 3], a);
                acc[2 * grp + (j >> 1)] = a;
            }
        }
        const uint32_t sc4 = __funnelshift_rc(r.sc[0], r.sc[1], sh);
        const float d = skn_half_bits_to_float((r.dw >> sh) & 0xFFFFu);
        float res = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float lo, hi;
            skn_unpack2(acc[i], lo, hi);
            // signed 8-bit scale -> float without the conversion pipe: (2^23 + 128 + s) - (2^23 + 128)
            const uint32_t sb8 = ((sc4 >> (8 * i)) & 0xFFu) ^ 0x80u;
            const float scf = __uint_as_float(0x4B000000u | sb8) - 8388736.f;
            res = fmaf(scf, fmaf(lo + hi, unscale, -32.f * sums[i]), res);
        }
        res *= d;
        return active ? res : 0.f;
    }
};

// One kernel for every streaming decoder S.
//   grid  : CTA b owns rows [b*N/grid, (b+1)*N/grid)
//   block : nch * wg warps; warp w -> chunk c = w % nch, row slot g = w / nch
//   smem  : [warps][MV_NST][CHUNK_BYTES] ring | prepared x | [warps][MV_NST] mbarriers | [rows][nch] partials
// Each warp walks its rows two at a time; stage s of its ring holds row i with i % MV_NST == s.
//
template <class S>
__global__ void __launch_bounds__(512, 1)
skn_matvec_stream(const skn_mv_group grp, int64_t pitch, int K, int nch, int wg, const float *__restrict__ x,
                  int32_t *__restrict__ status, int relaxed) {
    const int64_t N = grp.n_end[grp.count - 1];
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const int c = warp % nch;
    const int g = warp / nch;
    const int kpad = nch * S::CHUNK_WEIGHTS;
    const int nb = K / S::BLOCK_WEIGHTS;

    const size_t ring_bytes = (size_t)nwarps * MV_NST * S::CHUNK_BYTES;
    uint8_t *ring = smem + (size_t)warp * MV_NST * S::CHUNK_BYTES;
    uint8_t *xs = smem + ring_bytes;
    const size_t xs_bytes = (S::xprep_bytes(kpad) + 127) / 128 * 128;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + ring_bytes + xs_bytes) + warp * MV_NST;
    float *part = reinterpret_cast<float *>(smem + ring_bytes + xs_bytes + (size_t)nwarps * MV_NST * sizeof(uint64_t));

    const int64_t row_begin = (int64_t)blockIdx.x * N / gridDim.x;
    const int64_t row_end = (int64_t)(blockIdx.x + 1) * N / gridDim.x;
    const int rows = (int)(row_end - row_begin);
    const int cnt = (rows > g) ? (rows - g + wg - 1) / wg : 0;   // rows this warp visits

    int nbc = nb - c * S::CHUNK_BLOCKS;
    if (nbc > S::CHUNK_BLOCKS) nbc = S::CHUNK_BLOCKS;
    // a short last chunk may end off a 16-byte boundary: the copy runs a few bytes into the
    // next row (or the slack after the last one); those bytes are never decoded
    const uint32_t bytes = ((uint32_t)nbc * S::BLOCK_BYTES + 15u) & ~15u;
    // global address of the chunk this warp reads from its i-th row
    auto row_src = [&](int i) -> const uint8_t * {
        int64_t local;
        const int t = skn_group_find(grp, row_begin + g + (int64_t)i * wg, local);
        return grp.W[t] + local * pitch + (size_t)c * S::CHUNK_BYTES;
    };

    MV_TRACE_VARS;
    MV_STAMP(0);
    // weights never depend on the previous kernel: start streaming them right away, one
    // stage per lane
    if (lane < MV_NST) {
        skn_mbar_init(&bars[lane], 1);
        skn_fence_mbar_init();
        skn_fence_proxy_async();
        if (lane < cnt) {
            skn_mbar_expect_tx(&bars[lane], bytes);
            skn_bulk_g2s(ring + lane * S::CHUNK_BYTES, row_src(lane), bytes, &bars[lane]);
        }
    }
    __syncwarp();
    MV_STAMP(1);
    skn_pdl_launch_dependents();
    // x (and y) may belong to the previous kernel in the stream, unless the caller has
    // declared its launches independent
    if (!relaxed) skn_pdl_wait();
    MV_STAMP(2);

    skn_xform xf{grp.norm_gain, grp.silu_u, 1.f};
    if (grp.norm_gain) {
        // RMSNorm scale of the whole vector: every CTA reads all of x anyway
        __shared__ float red[16];
        float ss = 0.f;
        for (int f = threadIdx.x; f < K / 4; f += blockDim.x) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(x) + f);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w2 = 0; w2 < nwarps; ++w2) tot += red[w2];
        xf.scale = rsqrtf(tot / (float)K + grp.norm_eps);
    }
    S::prep_x(x, K, kpad, xs, xf);
    __syncthreads();
    MV_STAMP(3);
    S dec;
    dec.load_x(xs, kpad, c, lane, nbc);
    MV_STAMP(4);

    // Two rows per iteration.  The warp-level sum of an iteration's two partial dots is a
    // five-step butterfly; its steps are spread over the NEXT iteration so that the shuffle
    // latency overlaps barrier polling, shared-memory reads and arithmetic.
    // A wait that runs out records SKN_ERR_TIMEOUT and lets the thread go on (the result is
    // then garbage, the status word says so); no thread ever leaves the warp's sync points.
    bool failed = false;
    float pend = 0.f;          // previous iteration: lanes 0-15 row i-2, lanes 16-31 row i-1
    int pend_i = -1;
    for (int i = 0; i < cnt; i += 2) {
        const int s0 = i & (MV_NST - 1), s1 = (i + 1) & (MV_NST - 1);
        const uint32_t parity = (uint32_t)(i / MV_NST) & 1u;    // i even: i and i+1 share the ring pass
        const bool two = i + 1 < cnt;
        pend += __shfl_xor_sync(0xffffffffu, pend, 8);
        if (!failed && !(skn_mbar_wait(&bars[s0], parity) && (!two || skn_mbar_wait(&bars[s1], parity)))) {
            failed = true;
            atomicExch(status, SKN_ERR_TIMEOUT);
        }
        pend += __shfl_xor_sync(0xffffffffu, pend, 4);
        const typename S::Raw r0 = dec.fetch(ring + s0 * S::CHUNK_BYTES);
        const typename S::Raw r1 = dec.fetch(ring + (two ? s1 : s0) * S::CHUNK_BYTES);
        __syncwarp();   // every lane holds its share in registers: the stages may be refilled
        if (lane < 2 && i + lane + MV_NST < cnt) {
            const int st = lane ? s1 : s0;
            skn_fence_proxy_async();
            skn_mbar_expect_tx(&bars[st], bytes);
            skn_bulk_g2s(ring + st * S::CHUNK_BYTES, row_src(i + lane + MV_NST), bytes, &bars[st]);
        }
        pend += __shfl_xor_sync(0xffffffffu, pend, 2);
        const float v0 = dec.dot(r0);
        const float v1 = two ? dec.dot(r1) : 0.f;
        pend += __shfl_xor_sync(0xffffffffu, pend, 1);
        if ((lane & 15) == 0 && pend_i >= 0) {
            const int ir = pend_i + (lane >> 4);
            if (ir < cnt) part[(size_t)(g + ir * wg) * nch + c] = pend;
        }
        // first butterfly step: the upper half-warp takes over row i+1, the lower row i
        pend = ((lane & 16) ? v1 : v0) + __shfl_xor_sync(0xffffffffu, (lane & 16) ? v0 : v1, 16);
        pend_i = i;
    }
    if (pend_i >= 0) {
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) pend += __shfl_xor_sync(0xffffffffu, pend, o);
        if ((lane & 15) == 0) {
            const int ir = pend_i + (lane >> 4);
            if (ir < cnt) part[(size_t)(g + ir * wg) * nch + c] = pend;
        }
    }
    MV_STAMP(5);
    __syncthreads();
    MV_STAMP(6);
    for (int lr = threadIdx.x; lr < rows; lr += blockDim.x) {
        float s = 0.f;
        for (int cc = 0; cc < nch; ++cc) s += part[(size_t)lr * nch + cc];
        int64_t local;
        const int t = skn_group_find(grp, row_begin + lr, local);
        if (grp.add[t]) s += grp.add[t][local];
        grp.y[t][local] = s;
    }
    MV_STAMP(7);
}

// Launch geometry of the streaming kernel for one weight tensor; computed on first use and
// cached in the tensor (it depends only on the tensor's shape and the device).
//   - one CTA per SM (a second CTA slot is left free so that, under programmatic dependent
//     launch, the next matvec's CTA can become resident and prefetch its weights while this
//     one computes);
//   - warps = nch * wg with wg chosen for about 8 warps.
template <class S>
static cudaError_t plan_stream(skn_ctx *ctx, int64_t n_rows, int64_t n_cols, skn_mv_plan &pl, bool relaxed) {
    auto kern = skn_matvec_stream<S>;
    pl.state = -1;  // "no streaming plan" unless everything below works out
    if (n_cols % S::BLOCK_WEIGHTS || n_cols > (1 << 20)) return cudaSuccess;
    const int64_t nb = n_cols / S::BLOCK_WEIGHTS;
    const int nch = (int)((nb + S::CHUNK_BLOCKS - 1) / S::CHUNK_BLOCKS);
    if (nch < 1 || nch > 16 || n_rows < 1) return cudaSuccess;
    static const int wg_env = env_int("SKN_MV_WG", 0);
    // Stream order: 8 warps per CTA (one launch computes while the next one only prefetches).
    // Relaxed order: 4 warps per CTA, so that CTAs of up to four consecutive launches share an
    // SM and their phases (prefetch, x preparation, arithmetic, epilogue) overlap.
    static const int warps_env_cfg = env_int("SKN_MV_WARPS", 0);
    const int warps_env = warps_env_cfg > 0 ? warps_env_cfg : (relaxed ? 4 : 8);
    // about `warps_env` warps per CTA; long rows (nch > 4) get two row slots when they fit
    int wg = wg_env > 0 ? wg_env : (nch <= warps_env ? warps_env / nch : 1);
    if (wg_env <= 0 && nch > 4 && nch <= 8) wg = 2;
    if (wg < 1) wg = 1;
    while (nch * wg > 16) --wg;
    if (wg < 1) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return e;
    static const int ctas_env = env_int("SKN_MV_CTAS_PER_SM", 1);
    int64_t grid = (int64_t)ctx->sm_count * (ctas_env > 0 ? ctas_env : 1);
    if (grid > n_rows) grid = n_rows;
    const int64_t rows_max = (n_rows + grid - 1) / grid;
    const int kpad = nch * S::CHUNK_WEIGHTS;
    int threads = 0;
    size_t smem = 0;
    for (;; --wg) {       // fewer row slots until the ring, the prepared x and the partials fit
        if (wg < 1) return cudaSuccess;
        const int warps = nch * wg;
        threads = warps * 32;
        smem = (size_t)warps * MV_NST * S::CHUNK_BYTES + (S::xprep_bytes(kpad) + 127) / 128 * 128 +
               (size_t)warps * MV_NST * sizeof(uint64_t) + (size_t)rows_max * nch * sizeof(float);
        if (smem <= 220 * 1024) break;
    }
    int occ = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, threads, smem);
    if (e != cudaSuccess) return e;
    if (occ < 1) return cudaSuccess;
    pl.nch = nch; pl.wg = wg; pl.grid = (int)grid; pl.threads = threads; pl.smem = smem;
    pl.state = 1;
    return cudaSuccess;
}

template <class S>
static cudaError_t launch_stream(skn_ctx *ctx, const skn_mv_group &grp, int64_t pitch, int K, const float *x,
                                 const skn_mv_plan &pl, cudaStream_t stream) {
    auto kern = skn_matvec_stream<S>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl.grid);
    cfg.blockDim = dim3((unsigned)pl.threads);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    static const int pdl = env_int("SKN_PDL", 1);
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, grp, pitch, K, pl.nch, pl.wg, x, ctx->d_status, ctx->relaxed_order);
}

template <class S>
static bool try_stream(skn_ctx *ctx, const skn_tensor *w, const float *x, const float *bias, float *y,
                       cudaStream_t stream, cudaError_t &err) {
    skn_mv_plan &pl = const_cast<skn_tensor *>(w)->mv_plan[ctx->relaxed_order ? 1 : 0];
    if (pl.state == 0) {
        err = plan_stream<S>(ctx, w->n_rows, w->n_cols, pl, ctx->relaxed_order != 0);
        if (err != cudaSuccess) { pl.state = 0; return true; }
    }
    if (pl.state != 1) return false;
    skn_mv_group grp = {};
    grp.W[0] = w->d_blocks; grp.y[0] = y; grp.add[0] = bias; grp.n_end[0] = w->n_rows; grp.count = 1;
    err = launch_stream<S>(ctx, grp, w->pitch, (int)w->n_cols, x, pl, stream);
    return true;
}

// Up to three tensors sharing x in one launch (M = 1).  Returns false when the shapes are not
// covered by the streaming kernel (the caller then issues separate products).
template <class S>
static bool try_stream_group(skn_ctx *ctx, int n, const skn_tensor *const *w, const float *x, float *const *y,
                             const float *const *add, const float *norm_gain, float norm_eps, const float *silu_u,
                             cudaStream_t stream, cudaError_t &err) {
    skn_mv_group grp = {};
    grp.norm_gain = norm_gain; grp.norm_eps = norm_eps; grp.silu_u = silu_u;
    int64_t tot = 0;
    for (int t = 0; t < n; ++t) {
        tot += w[t]->n_rows;
        grp.W[t] = w[t]->d_blocks; grp.y[t] = y[t]; grp.add[t] = add ? add[t] : nullptr; grp.n_end[t] = tot;
    }
    for (int t = n; t < 3; ++t) grp.n_end[t] = tot;
    grp.count = n;
    // plans of grouped launches live in the context (one host thread drives a context at a time)
    skn_mv_plan pl;
    pl.state = 0;
    for (int i = 0; i < ctx->n_group_plans; ++i) {
        const skn_group_plan &c = ctx->group_plans[i];
        if (c.type == w[0]->type && c.rows == tot && c.cols == w[0]->n_cols && c.relaxed == ctx->relaxed_order) { pl = c.pl; break; }
    }
    if (pl.state == 0) {
        err = plan_stream<S>(ctx, tot, w[0]->n_cols, pl, ctx->relaxed_order != 0);
        if (err != cudaSuccess) return true;
        if (ctx->n_group_plans < 32)
            ctx->group_plans[ctx->n_group_plans++] = skn_group_plan{w[0]->type, ctx->relaxed_order, tot, w[0]->n_cols, pl};
    }
    if (pl.state != 1) return false;
    err = launch_stream<S>(ctx, grp, w[0]->pitch, (int)w[0]->n_cols, x, pl, stream);
    return true;
}

// y[t] = W[t] . f(x) (+ add[t]) for n <= 3 tensors of one type, K and pitch in ONE launch of the
// streaming kernel; f is the identity, an RMSNorm (norm_gain) and / or x <- silu(x) * silu_u.
// Returns cudaErrorNotSupported when the shapes are not covered (nothing has been launched).
cudaError_t skn_launch_matvec_fused(skn_ctx *ctx, int n, const skn_tensor *const *w, const float *x, float *const *y,
                                    const float *const *add, const float *norm_gain, float norm_eps,
                                    const float *silu_u, cudaStream_t stream) {
    bool same = n >= 1 && n <= 3;
    for (int t = 1; t < n && same; ++t)
        same = w[t]->type == w[0]->type && w[t]->n_cols == w[0]->n_cols && w[t]->pitch == w[0]->pitch;
    if (!same || (w[0]->pitch % 16) != 0) return cudaErrorNotSupported;
    cudaError_t err = cudaSuccess;
    // a single activation row: the four formats of the tensor-core kernel run there (the same route
    // skn_launch_matvec takes, so grouped and separate launches give identical bits); the CUDA-core
    // streaming kernels remain for shapes that kernel does not cover
    if (skn_mma_try_group(ctx, n, w, x, y, add, norm_gain, norm_eps, silu_u, stream, err)) return err;
    bool took = false;
    switch (w[0]->type) {
    case SKN_TYPE_Q4_K: took = try_stream_group<Q4KStream>(ctx, n, w, x, y, add, norm_gain, norm_eps, silu_u, stream, err); break;
    case SKN_TYPE_Q4_0: took = try_stream_group<Q40Stream>(ctx, n, w, x, y, add, norm_gain, norm_eps, silu_u, stream, err); break;
    case SKN_TYPE_Q8_0: took = try_stream_group<Q80Stream>(ctx, n, w, x, y, add, norm_gain, norm_eps, silu_u, stream, err); break;
    case SKN_TYPE_Q6_K: took = try_stream_group<Q6KStream>(ctx, n, w, x, y, add, norm_gain, norm_eps, silu_u, stream, err); break;
    default: break;
    }
    return took ? err : cudaErrorNotSupported;
}

cudaError_t skn_launch_matvec_acts(skn_ctx *ctx, int n, const skn_tensor *const *w, const float *x, int M, float *const *y,
                                   const float *const *add, bool add_per_act, const float *norm_gain, float norm_eps,
                                   const float *silu_u, bool swiglu, cudaStream_t stream, const skn_mv_exchange *xc,
                                   const skn_mv_rope *rope) {
    if (n < 1 || n > 3 || M < 1) return cudaErrorNotSupported;
    int64_t tot = 0;
    for (int t = 0; t < n; ++t) {
        if (w[t]->type != w[0]->type || w[t]->n_cols != w[0]->n_cols || w[t]->pitch != w[0]->pitch) return cudaErrorNotSupported;
        tot += w[t]->n_rows;
    }
    if ((w[0]->pitch % 16) != 0) return cudaErrorNotSupported;
    const int64_t K = w[0]->n_cols;
    // three rows or more: the many-row kernel (x prepared once per launch by its own kernel, up to sixteen rows
    // per pass over the weights); it has no rotary epilogue and no exchange
    if (M >= 3 && !xc && !rope) {
        const int maxr = skn_rows_max_acts(ctx, n, w);
        if (maxr >= 4) {
            const int launches = (M + maxr - 1) / maxr;
            for (int i = 0, m0 = 0; i < launches; ++i) {
                int na = (M - m0 + (launches - i) - 1) / (launches - i);     // even shares, at least three rows each
                if (M - m0 - na > 0 && M - m0 - na < 3) na = M - m0;
                if (na > maxr || na < 3) break;                               // (cannot happen for M >= 3: kept as a guard)
                float *ys[3] = {nullptr, nullptr, nullptr};
                const float *as[3] = {nullptr, nullptr, nullptr};
                for (int t = 0; t < n; ++t) {
                    ys[t] = y[t] + (int64_t)m0 * w[swiglu ? 0 : t]->n_rows;
                    if (add && add[t]) as[t] = add[t] + (add_per_act ? (int64_t)m0 * w[t]->n_rows : 0);
                }
                cudaError_t err = cudaSuccess;
                if (!skn_rows_try_group(ctx, n, w, x + (int64_t)m0 * K, na, ys, add ? as : nullptr, add_per_act, norm_gain, norm_eps,
                                        silu_u ? silu_u + (int64_t)m0 * K : nullptr, swiglu, stream, err)) {
                    if (i == 0) break;                                        // not covered after all: the route below
                    return cudaErrorUnknown;
                }
                if (err != cudaSuccess) return err;
                m0 += na;
                if (m0 == M) return cudaSuccess;
            }
        }
    }
    const int maxa = skn_mma_max_acts(ctx, w[0]->type, tot, w[0]->n_cols);
    if (maxa < 1) return cudaErrorNotSupported;
    const int launches = (M + maxa - 1) / maxa;
    if (xc && launches != 1) return cudaErrorNotSupported;      // an exchange covers all rows of one launch
    for (int i = 0, m0 = 0; i < launches; ++i) {
        const int na = (M - m0 + (launches - i) - 1) / (launches - i);       // even shares
        float *ys[3] = {nullptr, nullptr, nullptr};
        const float *as[3] = {nullptr, nullptr, nullptr};
        for (int t = 0; t < n; ++t) {
            ys[t] = y[t] + (int64_t)m0 * w[swiglu ? 0 : t]->n_rows;
            if (add && add[t]) as[t] = add[t] + (add_per_act ? (int64_t)m0 * w[t]->n_rows : 0);
        }
        cudaError_t err = cudaSuccess;
        skn_mv_rope rp;
        if (rope) {
            rp = *rope;
            rp.seq0 = rope->seq0 + m0;
        }
        if (!skn_mma_try_group(ctx, n, w, x + (int64_t)m0 * K, ys, add ? as : nullptr, norm_gain, norm_eps,
                               silu_u ? silu_u + (int64_t)m0 * K : nullptr, stream, err, swiglu, na, add_per_act, xc, rope ? &rp : nullptr))
            return cudaErrorNotSupported;
        if (err != cudaSuccess) return err;
        m0 += na;
    }
    return cudaSuccess;
}

cudaError_t skn_launch_gate_up_swiglu(skn_ctx *ctx, const skn_tensor *wg, const skn_tensor *wu, const float *x, float *h,
                                      const float *norm_gain, float norm_eps, cudaStream_t stream) {
    if (wg->type != wu->type || wg->n_cols != wu->n_cols || wg->n_rows != wu->n_rows || wg->pitch != wu->pitch ||
        (wg->pitch % 16) != 0)
        return cudaErrorNotSupported;
    const skn_tensor *ws[2] = {wg, wu};
    float *ys[2] = {h, h};
    cudaError_t err = cudaSuccess;
    if (skn_mma_try_group(ctx, 2, ws, x, ys, nullptr, norm_gain, norm_eps, nullptr, stream, err, true)) return err;
    return cudaErrorNotSupported;
}

// y[t] = W[t] . x (+ add[t]): one launch when the streaming kernel covers the shapes, separate
// launches otherwise.
cudaError_t skn_launch_matvec_group(skn_ctx *ctx, int n, const skn_tensor *const *w, const float *x, float *const *y,
                                    const float *const *add, cudaStream_t stream) {
    if (n > 1) {
        const cudaError_t e = skn_launch_matvec_fused(ctx, n, w, x, y, add, nullptr, 0.f, nullptr, stream);
        if (e != cudaErrorNotSupported) return e;
    }
    for (int t = 0; t < n; ++t) {
        cudaError_t e = skn_launch_matvec(ctx, w[t], x, 1, add ? add[t] : nullptr, y[t], stream);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

cudaError_t skn_launch_matvec(skn_ctx *ctx, const skn_tensor *w, const float *x, int32_t M, const float *bias,
                              float *y, cudaStream_t stream) {
    static const int force_generic = env_int("SKN_MV_GENERIC", 0);
    if (M >= 1 && !force_generic) {
        const skn_tensor *w1[1] = {w};
        float *y1[1] = {y};
        const float *b1[1] = {bias};
        const cudaError_t e = skn_launch_matvec_acts(ctx, 1, w1, x, M, y1, b1, false, nullptr, 0.f, nullptr, false, stream);
        if (e != cudaErrorNotSupported) return e;
    }
    if (M >= 1 && !force_generic && (w->pitch % 16) == 0) {
        // small batches run the streaming matvec once per activation row (the weights of the
        // later rows come from L2); each launch is a complete fp32 fused dequant-dot
        cudaError_t err = cudaSuccess;
        bool done = false;
        for (int32_t m = 0; m < M; ++m) {
            const float *xm = x + (int64_t)m * w->n_cols;
            float *ym = y + (int64_t)m * w->n_rows;
            bool took = false;
            if (w->type == SKN_TYPE_Q4_K) took = try_stream<Q4KStream>(ctx, w, xm, bias, ym, stream, err);
            else if (w->type == SKN_TYPE_Q4_0) took = try_stream<Q40Stream>(ctx, w, xm, bias, ym, stream, err);
            else if (w->type == SKN_TYPE_Q8_0) took = try_stream<Q80Stream>(ctx, w, xm, bias, ym, stream, err);
            else if (w->type == SKN_TYPE_Q6_K) took = try_stream<Q6KStream>(ctx, w, xm, bias, ym, stream, err);
            if (!took) break;               // shape not covered: the generic kernel below does all rows
            if (err != cudaSuccess) return err;
            done = (m == M - 1);
        }
        if (done) return cudaSuccess;
    }
    switch (w->type) {
    case SKN_TYPE_Q4_0: return launch_generic<SKN_TYPE_Q4_0>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_Q8_0: return launch_generic<SKN_TYPE_Q8_0>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_Q4_K: return launch_generic<SKN_TYPE_Q4_K>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_Q6_K: return launch_generic<SKN_TYPE_Q6_K>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_Q4_1: return launch_generic<SKN_TYPE_Q4_1>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_Q5_0: return launch_generic<SKN_TYPE_Q5_0>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_Q5_1: return launch_generic<SKN_TYPE_Q5_1>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_Q5_K: return launch_generic<SKN_TYPE_Q5_K>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_Q2_K: return launch_generic<SKN_TYPE_Q2_K>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_Q3_K: return launch_generic<SKN_TYPE_Q3_K>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_IQ4_NL: return launch_generic<SKN_TYPE_IQ4_NL>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_IQ4_XS: return launch_generic<SKN_TYPE_IQ4_XS>(w, x, M, bias, y, ctx->sm_count, stream);
    default: return cudaErrorInvalidValue;
    }
}
