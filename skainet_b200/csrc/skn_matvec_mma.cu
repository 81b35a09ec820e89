// K2 (decode matvec), integer tensor-core form:  y[N] = W_q[N,K] . x[K]  for Q4_K weights.
//
// The CUDA-core kernels of skn_matvec.cu spend one logic operation and half a packed FMA per
// weight and end up bound by instruction issue at about half of the HBM rate.  Here the dot
// product of a 32-weight sub-block with its 32 activations is an EXACT integer dot product
// on the tensor cores (mma.sync m16n8k32, u8 x s8 -> s32), so the per-weight work shrinks to
// a fraction of an instruction and the kernel waits for HBM instead:
//
//   * x, per group of 32 activations, becomes a 23-bit fixed-point number with a power-of-two
//     group scale: X = rint(x * 2^(21-e)), e = exponent of the group's largest |x|, split into
//     three balanced signed byte digits X = d0 + 256 d1 + 65536 d2.  The digit planes are the
//     columns 0..2 of the B operand (columns 3..7 are zero), in shared memory, prepared once per
//     CTA.  The rounding error per activation is at most 2^-23 of the group's largest one.
//   * the A operand is the quant bytes as they lie in the block: `word & 0x0F0F0F0F` are four
//     low-nibble weights (sub-block 2p), `word & 0xF0F0F0F0` four high-nibble weights times 16
//     (sub-block 2p+1; the 1/16 goes into the scale).  One MMA = 16 rows x one sub-block.
//   * per (row, sub-block) the s32 results of the three digit columns are recombined
//     (c0 + 256 c1 in integers, the third digit through a factor 65536 applied once per tile)
//     and scaled by d * sc * 2^(e-21); the -dmin * m * sum(x) term is added per row and
//     super-block by the lane that decodes that block's header.
//
// Work split: CTA b owns rows [b*N/grid, (b+1)*N/grid).  A tile is 16 rows x one K super-chunk
// (up to 16 super-blocks, i.e. one bulk async copy of at most 2304 bytes per row: few, large
// copies).  The CTA walks its tiles through a ring of `nst` stages; the sixteen row copies of a
// tile are issued by sixteen lanes of warp 0 and signal the stage's "full" mbarrier, every warp
// takes the super-blocks warp, warp + W, ... of the tile and arrives on the stage's "empty"
// mbarrier when it has read its share.  Rows are padded by 32 bytes in shared memory, which
// makes the 64-bit fragment loads of the eight row groups conflict-free.  Weights are
// prefetched before the programmatic dependent-launch wait, x is read after it.  Partial sums
// per (row, super-chunk, warp) meet in shared memory and are added in a fixed order.
#include "skn_mv_common.cuh"

constexpr int MM_KS = 16;                       // super-blocks per K super-chunk (one row copy)
constexpr int MM_BLOCK_BYTES = 144;
constexpr int MM_ROW_STRIDE = MM_KS * MM_BLOCK_BYTES + 32;   // 2336 B = 584 words = 8 mod 32
constexpr int MM_STAGE = 16 * MM_ROW_STRIDE;
constexpr int MM_FROW = 12;                     // floats per row of the scale scratch (8 used): 48 B stride, no bank conflicts

__device__ __forceinline__ void skn_mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// |v| < 2^22 as a float without the conversion pipe: (1.5 * 2^23 + v) - 1.5 * 2^23
__device__ __forceinline__ float mm_int_f(int v) { return __int_as_float(0x4B400000 + v) - 12582912.f; }

// byte i (0..3) of w as a float without the conversion pipe: (2^23 + b) - 2^23
__device__ __forceinline__ float mm_byte_f(uint32_t w, int i) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440u + i)) - 8388608.f;
}

// CTA-cooperative preparation of x: digit planes, group scales and group sums.
//   dig  : 3 planes of PL bytes, byte k of a plane = that digit of activation k (the MMA's k index
//          is mapped so that thread-in-group t owns activations 8t..8t+7 of a group: one 64-bit load)
//   sgrp : 2^(e-21) per group (NaN when the group holds a NaN or an infinity)
//   xsum : plain fp32 sum of the group
// Columns >= K are zero.
template <int B>                                // float4 loads in flight per thread
static __device__ __forceinline__ void mm_prep_x(const float *__restrict__ x, int K, int kpad, uint8_t *dig, int PL,
                                                 float *sgrp, float *xsum, const skn_xform &xf) {
    const int nf = kpad / 4;
    for (int f0 = 0; f0 < nf; f0 += B * blockDim.x) {
        float4 v[B];
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const int f = f0 + b * blockDim.x + threadIdx.x;
            v[b] = (f < nf && 4 * f < K) ? skn_load_x4(x, f, xf) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const int f = f0 + b * blockDim.x + threadIdx.x;      // 8 consecutive f = one group
            float mx = fmaxf(fmaxf(fabsf(v[b].x), fabsf(v[b].y)), fmaxf(fabsf(v[b].z), fabsf(v[b].w)));
            float sm = (v[b].x + v[b].y) + (v[b].z + v[b].w);
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) {
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                sm += __shfl_xor_sync(0xffffffffu, sm, o);
            }
            int E = (int)(__float_as_uint(mx) >> 23);
            E = E < 22 ? 22 : (E > 254 ? 254 : E);
            const float mul = __int_as_float((275 - E) << 23);          // 2^(21-e)
            const int X[4] = {__float2int_rn(v[b].x * mul), __float2int_rn(v[b].y * mul), __float2int_rn(v[b].z * mul),
                              __float2int_rn(v[b].w * mul)};
            uint32_t p0 = 0, p1 = 0, p2 = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int d0 = (int)(int8_t)(X[i] & 0xFF);
                const int X1 = (X[i] - d0) >> 8;
                const int d1 = (int)(int8_t)(X1 & 0xFF);
                const int d2 = (X1 - d1) >> 8;
                p0 |= (uint32_t)(d0 & 0xFF) << (8 * i);
                p1 |= (uint32_t)(d1 & 0xFF) << (8 * i);
                p2 |= (uint32_t)(d2 & 0xFF) << (8 * i);
            }
            if (f < nf) {
                const int G = f >> 3, q = f & 7;
                const int off = 4 * f;
                *reinterpret_cast<uint32_t *>(dig + off) = p0;
                *reinterpret_cast<uint32_t *>(dig + PL + off) = p1;
                *reinterpret_cast<uint32_t *>(dig + 2 * PL + off) = p2;
                if (q == 0) {
                    const bool finite = fabsf(sm) <= 3.4028234e38f;       // false for NaN and infinities
                    sgrp[G] = finite ? __int_as_float((E - 21) << 23) : __int_as_float(0x7FC00000);
                    xsum[G] = sm;
                }
            }
        }
    }
}


template <int SPW>                              // super-blocks of a tile per warp: blockDim = 32 * ceil(16 / SPW)
__global__ void __launch_bounds__(512 / SPW, 1)
skn_matvec_q4k_mma(const skn_mv_group grp, int64_t pitch, int K, int nst, const float *__restrict__ x,
                   int32_t *__restrict__ status, int relaxed) {
    const int64_t N = grp.n_end[grp.count - 1];
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int W = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nb = K / 256;
    const int nks = (nb + MM_KS - 1) / MM_KS;   // K super-chunks
    constexpr int spw = SPW;
    const int kpad = nb * 256;
    const int PL = kpad + 32;                   // plane stride: 8 words mod 32, planes 0..2 on disjoint banks

    // shared memory: ring | digit planes | group scales | group sums | F scratch | barriers | partials
    uint8_t *ring = smem;
    uint8_t *dig = smem + (size_t)nst * MM_STAGE;
    float *sgrp = reinterpret_cast<float *>(dig + ((size_t)3 * PL + 127) / 128 * 128);
    float *xsum = sgrp + (kpad / 32 + 3) / 4 * 4;
    float *Fs_all = xsum + (kpad / 32 + 3) / 4 * 4;
    float *Fs = Fs_all + (size_t)warp * spw * MM_FROW * 16;               // [own super-block][row][MM_FROW]
    uint64_t *full = reinterpret_cast<uint64_t *>(Fs_all + (size_t)W * spw * MM_FROW * 16);
    uint64_t *empty = full + nst;
    float *part = reinterpret_cast<float *>(empty + nst);

    const int64_t row_begin = (int64_t)blockIdx.x * N / gridDim.x;
    const int64_t row_end = (int64_t)(blockIdx.x + 1) * N / gridDim.x;
    const int rows = (int)(row_end - row_begin);
    const int nrt = (rows + 15) >> 4;           // row tiles
    const int ntiles = nrt * nks;               // tile i -> super-chunk i / nrt, row tile i % nrt
    const int pw = nks * W;                     // partial slots per row

    // warp 0: stage i % nst <- tile i (one copy per valid row, all on the stage's full barrier)
    auto issue = [&](int ks, int rt, int stg) {
        int nsb = nb - ks * MM_KS;
        nsb = nsb > MM_KS ? MM_KS : nsb;
        const uint32_t bytes = (uint32_t)nsb * MM_BLOCK_BYTES;
        int nvalid = rows - rt * 16;
        nvalid = nvalid > 16 ? 16 : nvalid;
        if (lane == 0) skn_mbar_expect_tx(&full[stg], bytes * (uint32_t)nvalid);
        __syncwarp();
        if (lane < nvalid) {
            int64_t local;
            const int tt = skn_group_find(grp, row_begin + rt * 16 + lane, local);
            skn_fence_proxy_async();
            skn_bulk_g2s(ring + (size_t)stg * MM_STAGE + lane * MM_ROW_STRIDE,
                         grp.W[tt] + local * pitch + (size_t)ks * MM_KS * MM_BLOCK_BYTES, bytes, &full[stg]);
        }
    };

    MV_STAMP(0);
    int iks = 0, irt = 0;                       // warp 0: the next tile to issue
    if (warp == 0) {
        if (lane < nst) {
            skn_mbar_init(&full[lane], 1);
            skn_mbar_init(&empty[lane], (uint32_t)W);
        }
        skn_fence_mbar_init();
        skn_fence_proxy_async();
        __syncwarp();
#ifdef MM_FINE2
        MV_STAMP(5);
#endif
        for (int i = 0; i < nst && i < ntiles; ++i) {
#ifdef MM_FINE2
            if (i == 1) MV_STAMP(6);
#endif
            issue(iks, irt, i);
            if (++irt == nrt) { irt = 0; ++iks; }
        }
    }
    MV_STAMP(1);
    skn_pdl_launch_dependents();
    if (!relaxed) skn_pdl_wait();
    MV_STAMP(2);

    skn_xform xf{grp.norm_gain, grp.silu_u, 1.f};
    if (grp.norm_gain) {
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
        for (int w2 = 0; w2 < W; ++w2) tot += red[w2];
        xf.scale = rsqrtf(tot / (float)K + grp.norm_eps);
    }
    mm_prep_x<2 * SPW>(x, K, kpad, dig, PL, sgrp, xsum, xf);
    __syncthreads();     // also publishes the barrier initialisation to the other warps
    MV_STAMP(3);

    bool failed = false;
    uint2 bq[SPW * 8];                          // B fragments of this warp's super-blocks in the current super-chunk
    int cur_ks = -1;
    // tile i = (super-chunk ks, row tile rt) sits in stage stg with barrier parity par; the same
    // for the tile issued nst - 1 tiles ahead (n*) and for the stage of the previous tile (p*)
    int ks = 0, rt = 0, stg = 0;
    uint32_t par = 0;
    int pstg = 0;
    uint32_t ppar = 0;
    for (int i = 0; i < ntiles; ++i) {
        const uint8_t *st = ring + (size_t)stg * MM_STAGE;
        int nsb = nb - ks * MM_KS;
        nsb = nsb > MM_KS ? MM_KS : nsb;
        // refill the stage the previous tile used, once every warp has read its share of it
        if (warp == 0 && i > 0 && i - 1 + nst < ntiles) {
            if (!failed && !skn_mbar_wait(&empty[pstg], ppar)) {
                failed = true;
                atomicExch(status, SKN_ERR_TIMEOUT);
            }
            issue(iks, irt, pstg);
            if (++irt == nrt) { irt = 0; ++iks; }
        }
        if (!failed && !skn_mbar_wait(&full[stg], par)) {
            failed = true;
            atomicExch(status, SKN_ERR_TIMEOUT);
        }
        if (i == 0) MV_STAMP(4);
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
        // ---- block headers of this warp's super-blocks: lane -> row lane & 15, own block (lane >> 4) + 2h
        float ms = 0.f;
        {
            const int hr = lane & 15;
#pragma unroll
            for (int h2 = 0; h2 < (SPW + 1) / 2; ++h2) {
                const int hh = (lane >> 4) + 2 * h2;
                const int sb = warp + W * hh;
                if (hh < spw && sb < nsb) {
                    const uint4 hd = *reinterpret_cast<const uint4 *>(st + hr * MM_ROW_STRIDE + sb * MM_BLOCK_BYTES);
                    const int G0 = (ks * MM_KS + sb) * 8;
                    const float4 sg0 = *reinterpret_cast<const float4 *>(sgrp + G0), sg1 = *reinterpret_cast<const float4 *>(sgrp + G0 + 4);
                    const float4 xs0 = *reinterpret_cast<const float4 *>(xsum + G0), xs1 = *reinterpret_cast<const float4 *>(xsum + G0 + 4);
                    const uint32_t sc_lo = hd.y & 0x3F3F3F3Fu, mn_lo = hd.z & 0x3F3F3F3Fu;
                    const uint32_t sc_hi = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
                    const uint32_t mn_hi = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
                    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hd.x));   // {d, dmin}
                    const float d = dd.x, d16 = dd.x * 0.0625f;
                    float4 f0, f1;
                    f0.x = (d * mm_byte_f(sc_lo, 0)) * sg0.x;
                    f0.y = (d16 * mm_byte_f(sc_lo, 1)) * sg0.y;
                    f0.z = (d * mm_byte_f(sc_lo, 2)) * sg0.z;
                    f0.w = (d16 * mm_byte_f(sc_lo, 3)) * sg0.w;
                    f1.x = (d * mm_byte_f(sc_hi, 0)) * sg1.x;
                    f1.y = (d16 * mm_byte_f(sc_hi, 1)) * sg1.y;
                    f1.z = (d * mm_byte_f(sc_hi, 2)) * sg1.z;
                    f1.w = (d16 * mm_byte_f(sc_hi, 3)) * sg1.w;
                    float *fd = Fs + ((size_t)hh * 16 + hr) * MM_FROW;
                    *reinterpret_cast<float4 *>(fd) = f0;
                    *reinterpret_cast<float4 *>(fd + 4) = f1;
                    float m = mm_byte_f(mn_lo, 0) * xs0.x;
                    m = fmaf(mm_byte_f(mn_lo, 1), xs0.y, m);
                    m = fmaf(mm_byte_f(mn_lo, 2), xs0.z, m);
                    m = fmaf(mm_byte_f(mn_lo, 3), xs0.w, m);
                    m = fmaf(mm_byte_f(mn_hi, 0), xs1.x, m);
                    m = fmaf(mm_byte_f(mn_hi, 1), xs1.y, m);
                    m = fmaf(mm_byte_f(mn_hi, 2), xs1.z, m);
                    m = fmaf(mm_byte_f(mn_hi, 3), xs1.w, m);
                    ms = fmaf(dd.y, m, ms);
                }
            }
        }
        __syncwarp();
#ifdef MM_FINE
        if (i == 0) MV_STAMP(5);
#endif
        // ---- integer dot products: rows g and g + 8, one MMA per sub-block
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int hh = 0; hh < spw; ++hh) {
            const int sb = warp + W * hh;
            if (sb >= nsb) break;
            const float4 fa0 = *reinterpret_cast<const float4 *>(Fs + ((size_t)hh * 16 + g) * MM_FROW);
            const float4 fa1 = *reinterpret_cast<const float4 *>(Fs + ((size_t)hh * 16 + g) * MM_FROW + 4);
            const float4 fb0 = *reinterpret_cast<const float4 *>(Fs + ((size_t)hh * 16 + g + 8) * MM_FROW);
            const float4 fb1 = *reinterpret_cast<const float4 *>(Fs + ((size_t)hh * 16 + g + 8) * MM_FROW + 4);
            const float fa[8] = {fa0.x, fa0.y, fa0.z, fa0.w, fa1.x, fa1.y, fa1.z, fa1.w};
            const float fb[8] = {fb0.x, fb0.y, fb0.z, fb0.w, fb1.x, fb1.y, fb1.z, fb1.w};
            const uint8_t *q = st + sb * MM_BLOCK_BYTES + 16 + 8 * t;
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const uint2 wa = *reinterpret_cast<const uint2 *>(q + 32 * p + g * MM_ROW_STRIDE);
                const uint2 wb = *reinterpret_cast<const uint2 *>(q + 32 * p + (g + 8) * MM_ROW_STRIDE);
                const uint2 b0 = bq[hh * 8 + 2 * p], b1 = bq[hh * 8 + 2 * p + 1];
                int cc[4];
                skn_mma_u8s8(cc, wa.x & 0x0F0F0F0Fu, wb.x & 0x0F0F0F0Fu, wa.y & 0x0F0F0F0Fu, wb.y & 0x0F0F0F0Fu, b0.x, b0.y);
                acc0 = fmaf(fa[2 * p], fmaf(mm_int_f(cc[1]), 256.f, mm_int_f(cc[0])), acc0);
                acc1 = fmaf(fb[2 * p], fmaf(mm_int_f(cc[3]), 256.f, mm_int_f(cc[2])), acc1);
                skn_mma_u8s8(cc, wa.x & 0xF0F0F0F0u, wb.x & 0xF0F0F0F0u, wa.y & 0xF0F0F0F0u, wb.y & 0xF0F0F0F0u, b1.x, b1.y);
                acc0 = fmaf(fa[2 * p + 1], fmaf(mm_int_f(cc[1]), 256.f, mm_int_f(cc[0])), acc0);
                acc1 = fmaf(fb[2 * p + 1], fmaf(mm_int_f(cc[3]), 256.f, mm_int_f(cc[2])), acc1);
            }
        }
        __syncwarp();      // every lane has read its share of the stage and of Fs
#ifdef MM_FINE
        if (i == 0) MV_STAMP(6);
#endif
        if (lane == 0) skn_mbar_arrive(&empty[stg]);
        // ---- tile epilogue: digits 0-1 sit in lanes t = 0, digit 2 in lanes t = 1
        float a0 = (t == 0) ? acc0 : ((t == 1) ? acc0 * 65536.f : 0.f);
        float a1 = (t == 0) ? acc1 : ((t == 1) ? acc1 * 65536.f : 0.f);
        a0 += __shfl_xor_sync(0xffffffffu, a0, 1);
        a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
        ms += __shfl_xor_sync(0xffffffffu, ms, 16);
        const float m0 = __shfl_sync(0xffffffffu, ms, g), m1 = __shfl_sync(0xffffffffu, ms, g + 8);
        if (t == 0) {
            const int r0 = rt * 16 + g;
            if (r0 < rows) part[(size_t)r0 * pw + ks * W + warp] = a0 - m0;
            if (r0 + 8 < rows) part[(size_t)(r0 + 8) * pw + ks * W + warp] = a1 - m1;
        }
        pstg = stg;
        ppar = par;
        if (++rt == nrt) { rt = 0; ++ks; }
        if (++stg == nst) { stg = 0; par ^= 1u; }
    }
#if !defined(MM_FINE) && !defined(MM_FINE2)
    MV_STAMP(5);
#endif
    __syncthreads();
#if !defined(MM_FINE) && !defined(MM_FINE2)
    MV_STAMP(6);
#endif
    // sixteen lanes per row: each adds its share of the row's partials in index order, then a
    // fixed butterfly (the same summation tree on every run)
    for (int lb = warp * 2; lb < rows; lb += W * 2) {          // warp-uniform trip count
        const int lr = lb + (lane >> 4);
        const int sub = lane & 15;
        float s = 0.f;
        if (lr < rows)
            for (int cc = sub; cc < pw; cc += 16) s += part[(size_t)lr * pw + cc];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (sub == 0 && lr < rows) {
            int64_t local;
            const int tt = skn_group_find(grp, row_begin + lr, local);
            if (grp.add[tt]) s += grp.add[tt][local];
            grp.y[tt][local] = s;
        }
    }
    MV_STAMP(7);
}

// Launch geometry: warps per CTA and ring depth that fit the shared-memory budget.  The
// budget is half of an SM's shared memory: the CTA of the next launch can then become resident
// (programmatic dependent launch) and prefetch its weights while this one computes.
static cudaError_t mm_plan(skn_ctx *ctx, int64_t n_rows, int64_t n_cols, skn_mv_plan &pl, bool relaxed) {
    pl = skn_mv_plan{-1, 0, 0, 0, 0, 0};
    if (n_cols % 256 || n_cols > (1 << 18) || n_rows < 1) return cudaSuccess;
    const int nb = (int)(n_cols / 256);
    const int nks = (nb + MM_KS - 1) / MM_KS;
    int64_t grid = ctx->sm_count;
    if (grid > n_rows) grid = n_rows;
    const int64_t rows_max = (n_rows + grid - 1) / grid;
    const int ntiles = (int)((rows_max + 15) / 16) * nks;
    static const int warps_env = env_int("SKN_MM_WARPS", 0);
    static const int nst_env = env_int("SKN_MM_NST", 0);
    static const int budget_env = env_int("SKN_MM_SMEM_KB", 0);
    int warps = warps_env > 0 ? warps_env : (relaxed ? 8 : 16);
    warps = warps >= 16 ? 16 : (warps >= 8 ? 8 : 4);
    const int spw = (MM_KS + warps - 1) / warps;
    const int kpad = nb * 256;
    const size_t budget = (size_t)(budget_env > 0 ? budget_env : 110) * 1024;
    const size_t fixed = ((size_t)3 * (kpad + 32) + 127) / 128 * 128 + (size_t)2 * ((kpad / 32 + 3) / 4 * 4) * 4 +
                         (size_t)warps * spw * MM_FROW * 16 * 4 + (size_t)rows_max * nks * warps * 4 + 64;
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
    pl.nch = nks; pl.wg = nst; pl.grid = (int)grid; pl.threads = warps * 32; pl.smem = smem;
    pl.state = 1;
    return cudaSuccess;
}

// y[t] = W[t] . f(x) (+ add[t]) for n <= 3 Q4_K tensors of one K and pitch.  Returns false when
// the shapes are not covered (nothing launched).
bool skn_mma_try_group(skn_ctx *ctx, int n, const skn_tensor *const *w, const float *x, float *const *y,
                       const float *const *add, const float *norm_gain, float norm_eps, const float *silu_u,
                       cudaStream_t stream, cudaError_t &err) {
    static const int enabled = env_int("SKN_MM", 1);
    err = cudaSuccess;
    if (!enabled || w[0]->type != SKN_TYPE_Q4_K) return false;
    skn_mv_group grp = {};
    grp.norm_gain = norm_gain; grp.norm_eps = norm_eps; grp.silu_u = silu_u;
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
    auto kern = pl.threads == 512 ? skn_matvec_q4k_mma<1> : (pl.threads == 256 ? skn_matvec_q4k_mma<2> : skn_matvec_q4k_mma<4>);
    err = cudaLaunchKernelEx(&cfg, kern, grp, w[0]->pitch, (int)w[0]->n_cols, pl.wg, x, ctx->d_status, ctx->relaxed_order);
    return true;
}
