// K2 (decode matvec), integer tensor-core form:  y[N] = W_q[N,K] . x[K]  for Q4_K weights.
//
// The CUDA-core kernels of skn_matvec.cu spend one logic operation and half a packed FMA per
// weight and end up bound by instruction issue at about half of the HBM rate.  Here the dot
// product of a 32-weight sub-block with its 32 activations is an EXACT integer dot product
// on the tensor cores (mma.sync m16n8k32, u8 x s8 -> s32), and the 6-bit sub-block scales are
// applied in integers as well, so the per-weight work shrinks to a fraction of an instruction:
//
//   * x, per super-block of 256 activations, becomes a 23-bit fixed-point number with a
//     power-of-two scale: X = rint(x * 2^(21-e)), e = exponent of the super-block's largest |x|,
//     split into three balanced signed byte digits X = d0 + 256 d1 + 65536 d2 (the bytes of
//     (X + 0x808080) ^ 0x808080).  The digit planes are columns 0..2 of the B operand (columns
//     3..7 are zero), prepared once per CTA in shared memory.  The rounding error per
//     activation is at most 2^-23 of the super-block's largest one.
//   * the A operand is the quant bytes as they lie in the block.  For the byte pair p of a
//     super-block (sub-block 2p in the low nibbles, 2p+1 in the high ones) two MMAs run: one on
//     `word & 0x0F0F0F0F` (L = the low-nibble dot) and one on the raw bytes (L + 16 H).  With
//     the integer scales s0, s1 of the two sub-blocks, 16 (s0 L + s1 H) = (16 s0 - s1) L +
//     s1 (L + 16 H): two integer multiply-adds per result, accumulated over the super-block in
//     s32 (at most 2^29 in magnitude).
//   * once per (row, super-block) the digit columns are recombined in fp32 and scaled by
//     d * 2^(e-21) / 16; the -dmin * m * sum(x) term is added per row and super-block.
//
// Work split: CTA b owns rows [b*N/grid, (b+1)*N/grid).  A tile is 16 rows x one K super-chunk
// (up to 16 super-blocks, i.e. one bulk async copy of at most 2304 bytes per row: few, large
// copies).  The CTA walks its tiles through a ring of `nst` stages.  A producer warp issues the
// sixteen row copies of a tile (they signal the stage's "full" mbarrier) and refills a stage
// when the W compute warps have arrived on its "empty" mbarrier; issuing blocks while the copy
// queue is full, i.e. at the speed of HBM, which is why it has a warp of its own.  Compute warp
// w takes the super-blocks w, w + W, ... of every tile.  Rows are padded by 32 bytes in shared
// memory, which makes the 64-bit fragment loads of the eight row groups conflict-free.  Weights
// are prefetched before the programmatic dependent-launch wait, x is read after it.  Partial
// sums per (row, super-chunk, warp) meet in shared memory and are added in a fixed order.
#include "skn_mv_common.cuh"

constexpr int MM_KS = 16;                       // super-blocks per K super-chunk (one row copy)
constexpr int MM_BLOCK_BYTES = 144;
constexpr int MM_ROW_STRIDE = MM_KS * MM_BLOCK_BYTES + 32;   // 2336 B = 584 words = 8 mod 32
constexpr int MM_STAGE = 16 * MM_ROW_STRIDE;

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

__device__ __forceinline__ void mm_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// One super-block (256 activations, two float4 per lane: elements 4*lane.. and 128 + 4*lane..)
// -> three digit planes (byte k of a plane = that digit of activation k), the scale 2^(e-21)
// (NaN when the block holds a NaN or an infinity) and the eight 32-element sums.
static __device__ __forceinline__ void mm_digitize(const float4 v0, const float4 v1, int sbi, int lane, uint8_t *dig, int PL,
                                                   float *sgrp, float *xsum) {
    float mx = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                     fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
    float s0 = (v0.x + v0.y) + (v0.z + v0.w), s1 = (v1.x + v1.y) + (v1.z + v1.w);
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
        s0 += __shfl_xor_sync(0xffffffffu, s0, o);
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float tot = s0 + s1;
    tot += __shfl_xor_sync(0xffffffffu, tot, 8);
    tot += __shfl_xor_sync(0xffffffffu, tot, 16);
    int E = (int)(__float_as_uint(mx) >> 23);
    E = E < 22 ? 22 : (E > 254 ? 254 : E);
    const float mul = __int_as_float((275 - E) << 23);          // 2^(21-e)
    // rint(v * mul) sits in the mantissa of v * mul + 1.5 * 2^23; adding 0x808080 and flipping
    // the three sign bits leaves the three balanced digits in bytes 0..2
    constexpr int C = 0x808080 - 0x4B400000;
    const float in[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    uint32_t D[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) D[i] = (uint32_t)(__float_as_int(fmaf(in[i], mul, 12582912.f)) + C) ^ 0x808080u;
    const int f = sbi * 64 + lane;
#pragma unroll
    for (int n = 0; n < 3; ++n) {
        const uint32_t sel = 0x0040u + 0x11u * n;               // byte n of both operands
        const uint32_t a = __byte_perm(__byte_perm(D[0], D[1], sel), __byte_perm(D[2], D[3], sel), 0x5410u);
        const uint32_t b = __byte_perm(__byte_perm(D[4], D[5], sel), __byte_perm(D[6], D[7], sel), 0x5410u);
        *reinterpret_cast<uint32_t *>(dig + (size_t)n * PL + 4 * f) = a;
        *reinterpret_cast<uint32_t *>(dig + (size_t)n * PL + 4 * (f + 32)) = b;
    }
    if ((lane & 7) == 0) {
        xsum[sbi * 8 + (lane >> 3)] = s0;
        xsum[sbi * 8 + 4 + (lane >> 3)] = s1;
    }
    if (lane == 0) sgrp[sbi] = (fabsf(tot) <= 3.4028234e38f) ? __int_as_float((E - 21) << 23) : __int_as_float(0x7FC00000);
}

// Register caps: the register file is split over the SM's four schedulers (16K registers each), so
// two resident CTAs of 9 warps need five warps per scheduler, i.e. at most 102 registers per
// thread; three CTAs of 5 warps need four per scheduler (at most 128).
template <int SPW>                              // super-blocks of a tile per compute warp: W = 16 / SPW compute warps
__global__ void __launch_bounds__(SPW == 1 ? 544 : (SPW == 2 ? 320 : 256), SPW == 1 ? 1 : 2)
skn_matvec_q4k_mma(const skn_mv_group grp, int64_t pitch, int K, int nst, const float *__restrict__ x,
                   int32_t *__restrict__ status, int relaxed) {
    constexpr int W = 16 / SPW;
    const int64_t N = grp.n_end[grp.count - 1];
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;          // 0..W-1 compute, W = producer
    const int g = lane >> 2, t = lane & 3;
    const int nb = K / 256;
    const int nks = (nb + MM_KS - 1) / MM_KS;   // K super-chunks
    const int PL = nb * 256 + 32;               // plane stride: 8 words mod 32, planes 0..2 on disjoint banks

    // shared memory: ring | digit planes | block scales | group sums | barriers | partials
    uint8_t *ring = smem;
    uint8_t *dig = smem + (size_t)nst * MM_STAGE;
    float *sgrp = reinterpret_cast<float *>(dig + ((size_t)3 * PL + 127) / 128 * 128);
    float *xsum = sgrp + (nb + 3) / 4 * 4;
    uint64_t *full = reinterpret_cast<uint64_t *>(xsum + nb * 8);
    uint64_t *empty = full + nst;
    float *part = reinterpret_cast<float *>(empty + nst);

    // with interleaved gate / up rows every CTA owns whole (gate, up) pairs: even boundaries
    const int64_t even = grp.swiglu ? ~(int64_t)1 : ~(int64_t)0;
    const int64_t row_begin = ((int64_t)blockIdx.x * N / gridDim.x) & even;
    const int64_t row_end = (blockIdx.x + 1 == gridDim.x) ? N : (((int64_t)(blockIdx.x + 1) * N / gridDim.x) & even);
    const int rows = (int)(row_end - row_begin);
    const int nrt = (rows + 15) >> 4;           // row tiles
    const int ntiles = nrt * nks;               // tile i -> super-chunk i / nrt, row tile i % nrt
    const int pw = nks * W;                     // partial slots per row

    MV_STAMP(0);
    if (warp == W && lane < nst) {
        skn_mbar_init(&full[lane], 1);
        skn_mbar_init(&empty[lane], (uint32_t)W);
    }
    if (warp == W) skn_fence_mbar_init();
    __syncthreads();                            // barriers are initialised for everyone

    if (warp == W) {
        // ---- producer: one copy per valid row of a tile, all on the stage's full barrier ----
        int ks = 0, rt = 0, stg = 0;
        uint32_t par = 0;                       // parity of the stage's previous use
        bool failed = false;
        for (int i = 0; i < ntiles; ++i) {
            if (i >= nst && !failed && !skn_mbar_wait(&empty[stg], par ^ 1u)) {
                failed = true;
                atomicExch(status, SKN_ERR_TIMEOUT);
            }
            int nsb = nb - ks * MM_KS;
            nsb = nsb > MM_KS ? MM_KS : nsb;
            const uint32_t bytes = (uint32_t)nsb * MM_BLOCK_BYTES;
            int nvalid = rows - rt * 16;
            nvalid = nvalid > 16 ? 16 : nvalid;
            if (lane == 0) skn_mbar_expect_tx(&full[stg], bytes * (uint32_t)nvalid);
            __syncwarp();
            if (lane < nvalid) {
                int64_t local;
                const int tt = skn_group_row(grp, row_begin + rt * 16 + lane, local);
                skn_fence_proxy_async();
                skn_bulk_g2s(ring + (size_t)stg * MM_STAGE + lane * MM_ROW_STRIDE,
                             grp.W[tt] + local * pitch + (size_t)ks * MM_KS * MM_BLOCK_BYTES, bytes, &full[stg]);
            }
            if (i == nst - 1 || i == ntiles - 1) skn_pdl_launch_dependents();   // the first ring-full is on its way
            if (++rt == nrt) { rt = 0; ++ks; }
            if (++stg == nst) { stg = 0; par ^= 1u; }
        }
        return;
    }

    // ---- compute warps ----
    skn_pdl_launch_dependents();
    if (!relaxed) skn_pdl_wait();
    MV_STAMP(2);
    skn_xform xf{grp.norm_gain, grp.silu_u, 1.f};
    if (grp.norm_gain) {
        __shared__ float red[16];
        float ss = 0.f;
        for (int f = threadIdx.x; f < K / 4; f += W * 32) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(x) + f);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[warp] = ss;
        mm_bar_sync(1, W * 32);
        float tot = 0.f;
        for (int w2 = 0; w2 < W; ++w2) tot += red[w2];
        xf.scale = rsqrtf(tot / (float)K + grp.norm_eps);
    }
    // x -> digit planes: a warp takes whole super-blocks, two at a time (four loads in flight)
    for (int sbi = warp; sbi < nb; sbi += 2 * W) {
        const int sb2 = sbi + W;
        const float4 a0 = skn_load_x4(x, sbi * 64 + lane, xf), a1 = skn_load_x4(x, sbi * 64 + 32 + lane, xf);
        float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
        if (sb2 < nb) {
            b0 = skn_load_x4(x, sb2 * 64 + lane, xf);
            b1 = skn_load_x4(x, sb2 * 64 + 32 + lane, xf);
        }
        mm_digitize(a0, a1, sbi, lane, dig, PL, sgrp, xsum);
        if (sb2 < nb) mm_digitize(b0, b1, sb2, lane, dig, PL, sgrp, xsum);
    }
    mm_bar_sync(1, W * 32);
    MV_STAMP(3);

    bool failed = false;
    uint2 bq[SPW * 8];                          // B fragments of this warp's super-blocks in the current super-chunk
    int cur_ks = -1;
    int ks = 0, rt = 0, stg = 0;
    uint32_t par = 0;
    for (int i = 0; i < ntiles; ++i) {
        const uint8_t *st = ring + (size_t)stg * MM_STAGE;
        int nsb = nb - ks * MM_KS;
        nsb = nsb > MM_KS ? MM_KS : nsb;
        if (ks != cur_ks) {
            // column n = g of the B operand holds digit plane n (n < 3), zero otherwise
            cur_ks = ks;
#pragma unroll
            for (int hh = 0; hh < SPW; ++hh) {
                const int sb = warp + W * hh;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    uint2 v = make_uint2(0u, 0u);
                    if (g < 3 && sb < nsb) v = *reinterpret_cast<const uint2 *>(dig + (size_t)g * PL + ((size_t)(ks * MM_KS + sb) * 8 + j) * 32 + 8 * t);
                    bq[hh * 8 + j] = v;
                }
            }
        }
        if (!failed && !skn_mbar_wait(&full[stg], par)) {
            failed = true;
            atomicExch(status, SKN_ERR_TIMEOUT);
        }
        if (i == 0) MV_STAMP(4);
        float acc0 = 0.f, acc1 = 0.f;           // rows g, g + 8: this lane's digit columns, all own super-blocks
        float ms = 0.f;                         // min term of row g + 8 * (t & 1), sub-blocks 4 * (t >> 1) .. + 3
#pragma unroll
        for (int hh = 0; hh < SPW; ++hh) {
            const int sb = warp + W * hh;
            if (sb >= nsb) break;
            const uint8_t *ba = st + g * MM_ROW_STRIDE + sb * MM_BLOCK_BYTES;
            const uint8_t *bb = ba + 8 * MM_ROW_STRIDE;
            const uint4 ha = *reinterpret_cast<const uint4 *>(ba), hb = *reinterpret_cast<const uint4 *>(bb);
            const int sbi = ks * MM_KS + sb;
            // 6-bit scales as bytes: word 0 = sub-blocks 0..3, word 1 = sub-blocks 4..7
            const uint32_t sa[2] = {ha.y & 0x3F3F3F3Fu, (ha.w & 0x0F0F0F0Fu) | ((ha.y >> 2) & 0x30303030u)};
            const uint32_t sq[2] = {hb.y & 0x3F3F3F3Fu, (hb.w & 0x0F0F0F0Fu) | ((hb.y >> 2) & 0x30303030u)};
            int lo[4] = {0, 0, 0, 0}, hi[4] = {0, 0, 0, 0};       // [row g col 0, col 1, row g+8 col 0, col 1]
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const uint2 wa = *reinterpret_cast<const uint2 *>(ba + 16 + 32 * p + 8 * t);
                const uint2 wb = *reinterpret_cast<const uint2 *>(bb + 16 + 32 * p + 8 * t);
                const int s0a = mm_byte_i(sa[p >> 1], 2 * (p & 1)), s1a = mm_byte_i(sa[p >> 1], 2 * (p & 1) + 1);
                const int s0b = mm_byte_i(sq[p >> 1], 2 * (p & 1)), s1b = mm_byte_i(sq[p >> 1], 2 * (p & 1) + 1);
                int cl[4], ch[4];
                skn_mma_u8s8(cl, wa.x & 0x0F0F0F0Fu, wb.x & 0x0F0F0F0Fu, wa.y & 0x0F0F0F0Fu, wb.y & 0x0F0F0F0Fu, bq[hh * 8 + 2 * p].x,
                             bq[hh * 8 + 2 * p].y);
                skn_mma_u8s8(ch, wa.x & 0xF0F0F0F0u, wb.x & 0xF0F0F0F0u, wa.y & 0xF0F0F0F0u, wb.y & 0xF0F0F0F0u, bq[hh * 8 + 2 * p + 1].x,
                             bq[hh * 8 + 2 * p + 1].y);
                lo[0] += s0a * cl[0]; lo[1] += s0a * cl[1]; lo[2] += s0b * cl[2]; lo[3] += s0b * cl[3];
                hi[0] += s1a * ch[0]; hi[1] += s1a * ch[1]; hi[2] += s1b * ch[2]; hi[3] += s1b * ch[3];
            }
            // 16 * sum_j sc_j dot_j per digit column (high-nibble results carry a factor 16)
            const float sg = sgrp[sbi] * 0.0625f;
            const float2 da = __half22float2(*reinterpret_cast<const __half2 *>(&ha.x));   // {d, dmin} of row g
            const float2 db = __half22float2(*reinterpret_cast<const __half2 *>(&hb.x));   // ... of row g + 8
            const float va = fmaf((float)(lo[1] * 16 + hi[1]), 256.f, (float)(lo[0] * 16 + hi[0]));
            const float vb = fmaf((float)(lo[3] * 16 + hi[3]), 256.f, (float)(lo[2] * 16 + hi[2]));
            acc0 = fmaf(da.x * sg, va, acc0);
            acc1 = fmaf(db.x * sg, vb, acc1);
            // min term: this lane covers one row and four sub-blocks
            const uint4 hm = (t & 1) ? hb : ha;
            const uint32_t mw = (t & 2) ? (((hm.w >> 4) & 0x0F0F0F0Fu) | ((hm.z >> 2) & 0x30303030u)) : (hm.z & 0x3F3F3F3Fu);
            const float4 xs = *reinterpret_cast<const float4 *>(xsum + sbi * 8 + 4 * (t >> 1));
            float m = mm_byte_f(mw, 0) * xs.x;
            m = fmaf(mm_byte_f(mw, 1), xs.y, m);
            m = fmaf(mm_byte_f(mw, 2), xs.z, m);
            m = fmaf(mm_byte_f(mw, 3), xs.w, m);
            ms = fmaf((t & 1) ? db.y : da.y, m, ms);
        }
        __syncwarp();      // every lane has read its share of the stage
        if (lane == 0) skn_mbar_arrive(&empty[stg]);
        // ---- tile epilogue: digits 0-1 sit in lanes t = 0, digit 2 in lanes t = 1
        float a0 = (t == 0) ? acc0 : ((t == 1) ? acc0 * 65536.f : 0.f);
        float a1 = (t == 0) ? acc1 : ((t == 1) ? acc1 * 65536.f : 0.f);
        a0 += __shfl_xor_sync(0xffffffffu, a0, 1);
        a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
        ms += __shfl_xor_sync(0xffffffffu, ms, 2);          // both sub-block halves: lane t = 0 row g, t = 1 row g + 8
        const float m1 = __shfl_xor_sync(0xffffffffu, ms, 1);
        if (t == 0) {
            const int r0 = rt * 16 + g;
            if (r0 < rows) part[(size_t)r0 * pw + ks * W + warp] = a0 - ms;
            if (r0 + 8 < rows) part[(size_t)(r0 + 8) * pw + ks * W + warp] = a1 - m1;
        }
        if (++rt == nrt) { rt = 0; ++ks; }
        if (++stg == nst) { stg = 0; par ^= 1u; }
    }
    MV_STAMP(5);
    mm_bar_sync(1, W * 32);
    MV_STAMP(6);
    // L lanes per row (16, 4 or 1, the most that still covers the CTA's rows in about one pass):
    // each adds its share of the row's partials in index order, then a fixed butterfly, so the
    // summation tree depends on the shape only
    const int lsh = (rows * 16 <= W * 32) ? 4 : ((rows * 4 <= W * 32) ? 2 : 0);
    const int L = 1 << lsh;
    for (int lb = warp * (32 >> lsh); lb < rows; lb += W * (32 >> lsh)) {     // warp-uniform trip count
        const int lr = lb + (lane >> lsh);
        const int sub = lane & (L - 1);
        float s = 0.f;
        if (lr < rows)
            for (int cc = sub; cc < pw; cc += L) s += part[(size_t)lr * pw + cc];
        for (int o = L >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float up = __shfl_xor_sync(0xffffffffu, s, L);      // the next row: the `up` product of a gate row
        if (sub == 0 && lr < rows) {
            int64_t local;
            const int tt = skn_group_row(grp, row_begin + lr, local);
            if (grp.swiglu) {
                if (tt == 0) grp.y[0][local] = s / (1.f + expf(-s)) * up;
            } else {
                if (grp.add[tt]) s += grp.add[tt][local];
                grp.y[tt][local] = s;
            }
        }
    }
    MV_STAMP(7);
}

// Launch geometry: compute warps per CTA and ring depth that fit the shared-memory budget.  The
// budget is half of an SM's shared memory: the CTA of the next launch can then become resident
// (programmatic dependent launch) and prefetch its weights while this one computes.
static cudaError_t mm_plan(skn_ctx *ctx, int64_t n_rows, int64_t n_cols, skn_mv_plan &pl, bool relaxed) {
    pl = skn_mv_plan{-1, 0, 0, 0, 0, 0};
    if (n_cols % 256 || n_cols > (1 << 18) || n_rows < 1) return cudaSuccess;
    const int nb = (int)(n_cols / 256);
    const int nks = (nb + MM_KS - 1) / MM_KS;
    int64_t grid = ctx->sm_count;
    if (grid > n_rows) grid = n_rows;
    const int64_t rows_max = (n_rows + grid - 1) / grid + 2;      // + 2: interleaved launches round to even boundaries
    const int ntiles = (int)((rows_max + 15) / 16) * nks;
    static const int warps_env = env_int("SKN_MM_WARPS", 0);
    static const int nst_env = env_int("SKN_MM_NST", 0);
    static const int budget_env = env_int("SKN_MM_SMEM_KB", 0);
    int warps = warps_env > 0 ? warps_env : 8;
    warps = warps >= 16 ? 16 : (warps >= 8 ? 8 : 4);
    // few tiles: half an SM, so that the next launch's CTA is resident early; many tiles: a deeper
    // ring matters more than the neighbour
    const size_t budget = (size_t)(budget_env > 0 ? budget_env : (ntiles >= 6 ? 200 : 110)) * 1024;
    const size_t fixed = ((size_t)3 * (nb * 256 + 32) + 127) / 128 * 128 + (size_t)((nb + 3) / 4 * 4) * 4 + (size_t)nb * 8 * 4 +
                         (size_t)rows_max * nks * warps * 4 + 64;
    int nst = nst_env > 0 ? nst_env : (ntiles < 4 ? ntiles : 4);
    while (nst > 1 && fixed + (size_t)nst * (MM_STAGE + 16) > budget) --nst;
    if (nst < 2 && ntiles > 1 && budget_env <= 0) {
        // long rows: the digit planes leave no room for two stages in half an SM; take all of it
        nst = ntiles < 4 ? ntiles : 4;
        while (nst > 1 && fixed + (size_t)nst * (MM_STAGE + 16) > 200 * 1024) --nst;
    }
    const size_t smem = fixed + (size_t)nst * (MM_STAGE + 16);
    if (smem > 220 * 1024) return cudaSuccess;
    cudaError_t e = cudaSuccess;
    if (warps == 16) e = cudaFuncSetAttribute(skn_matvec_q4k_mma<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    else if (warps == 8) e = cudaFuncSetAttribute(skn_matvec_q4k_mma<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    else e = cudaFuncSetAttribute(skn_matvec_q4k_mma<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return e;
    // all of the SM's L1 / shared memory as shared memory, so that two CTAs (consecutive launches) fit
    if (warps == 16) e = cudaFuncSetAttribute(skn_matvec_q4k_mma<1>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    else if (warps == 8) e = cudaFuncSetAttribute(skn_matvec_q4k_mma<2>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    else e = cudaFuncSetAttribute(skn_matvec_q4k_mma<4>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    // wg carries the ring depth; threads = compute warps + the producer warp
    pl.nch = nks; pl.wg = nst; pl.grid = (int)grid; pl.threads = (warps + 1) * 32; pl.smem = smem;
    pl.state = 1;
    return cudaSuccess;
}

// y[t] = W[t] . f(x) (+ add[t]) for n <= 3 Q4_K tensors of one K and pitch.  Returns false when
// the shapes are not covered (nothing launched).
bool skn_mma_try_group(skn_ctx *ctx, int n, const skn_tensor *const *w, const float *x, float *const *y,
                       const float *const *add, const float *norm_gain, float norm_eps, const float *silu_u,
                       cudaStream_t stream, cudaError_t &err, bool swiglu) {
    static const int enabled = env_int("SKN_MM", 1);
    err = cudaSuccess;
    if (!enabled || w[0]->type != SKN_TYPE_Q4_K) return false;
    if (swiglu && (n != 2 || w[0]->n_rows != w[1]->n_rows)) return false;
    skn_mv_group grp = {};
    grp.norm_gain = norm_gain; grp.norm_eps = norm_eps; grp.silu_u = silu_u;
    grp.swiglu = swiglu ? 1 : 0;
    int64_t tot = 0;
    for (int t = 0; t < n; ++t) {
        tot += w[t]->n_rows;
        grp.W[t] = w[t]->d_blocks; grp.y[t] = y[t]; grp.add[t] = add ? add[t] : nullptr; grp.n_end[t] = tot;
    }
    for (int t = n; t < 3; ++t) grp.n_end[t] = tot;
    grp.count = n;
    skn_mv_plan pl = skn_mv_plan{0, 0, 0, 0, 0, 0};
    const int32_t key_type = 1000 + w[0]->type;       // distinct from the CUDA-core kernels' plans
    for (int i = 0; i < ctx->n_group_plans; ++i) {
        const skn_group_plan &c = ctx->group_plans[i];
        if (c.type == key_type && c.rows == tot && c.cols == w[0]->n_cols && c.relaxed == ctx->relaxed_order) { pl = c.pl; break; }
    }
    if (pl.state == 0) {
        err = mm_plan(ctx, tot, w[0]->n_cols, pl, ctx->relaxed_order != 0);
        if (err != cudaSuccess) return true;
        if (ctx->n_group_plans < 32)
            ctx->group_plans[ctx->n_group_plans++] = skn_group_plan{key_type, ctx->relaxed_order, tot, w[0]->n_cols, pl};
    }
    if (pl.state != 1) return false;
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
    auto kern = pl.threads == 17 * 32 ? skn_matvec_q4k_mma<1> : (pl.threads == 9 * 32 ? skn_matvec_q4k_mma<2> : skn_matvec_q4k_mma<4>);
    err = cudaLaunchKernelEx(&cfg, kern, grp, w[0]->pitch, (int)w[0]->n_cols, pl.wg, x, ctx->d_status, ctx->relaxed_order);
    return true;
}
