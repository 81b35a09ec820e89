// K2 (decode matvec), integer tensor-core form:  y[N] = W_q[N,K] . x[K]  for Q4_K (described here), Q6_K, Q8_0 and
// Q4_0 weights (further down).
//
// The CUDA-core kernels of skn_matvec.cu spend one logic operation and half a packed FMA per
// weight and end up bound by instruction issue at about half of the HBM rate.  Here the dot
// product of a 32-weight sub-block with its 32 activations is an EXACT integer dot product
// on the tensor cores (mma.sync m16n8k32, u8 x s8 -> s32), and the 6-bit sub-block scales are
// applied in integers as well, so the per-weight work shrinks to a fraction of an instruction:
//
//   * x, per super-block of 256 activations, becomes a 32-bit fixed-point number with a
//     power-of-two scale: X = rint(x * 2^(29-e)), e = exponent of the super-block's largest |x|,
//     split into four balanced signed byte digits X = d0 + 2^8 d1 + 2^16 d2 + 2^24 d3.  The digit
//     planes are B columns 0, 2, 4, 6 (a second activation row takes 1, 3, 5, 7), prepared once per
//     CTA in shared memory.  Activations within 2^6 of the block's largest are exact, the others
//     are rounded to 2^-30 of it; a few outliers that tower over their block are taken out of the
//     planes and multiplied in fp32 (see mm_digitize).
//   * the A operand is the quant bytes as they lie in the block.  For the byte pair p of a
//     super-block (sub-block 2p in the low nibbles, 2p+1 in the high ones) two MMAs run: one on
//     `word & 0x0F0F0F0F` against the digits of the activations of sub-block 2p, one on
//     `word & 0xF0F0F0F0` (the high nibbles times 16) against those of sub-block 2p+1.  The integer
//     scales of the two sub-blocks multiply the s32 results (two integer multiply-adds per result),
//     accumulated over the super-block as lo and hi sums (at most 2^29 in magnitude); lo * 16 + hi
//     is 16 times the scaled dot product.
//   * once per (row, super-block) the digit columns are recombined in fp32 and scaled by
//     d * 2^(e-29) / 16; the -dmin * m * sum(x) term is added per row and super-block.
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
#include "skn_mma_common.cuh"

// Register caps: the register file is split over the SM's four schedulers (16K registers each), so
// two resident CTAs of 9 warps need five warps per scheduler, i.e. at most 102 registers per
// thread.
//
// Several activation rows per launch: one MMA serves TWO rows (digit columns 0..2 and 3..5 of the
// B operand), NP such pairs share the A fragments, block headers and scale decoding.
//
// FEAT selects what is compiled in besides the product and the bias / residual add: 0 nothing, 1 the
// RMSNorm folded into the preparation of x and the SwiGLU epilogue, 2 the RMSNorm and the
// rotary-embedding / cache epilogue, 3 all of those, the silu(x) * u preparation and the tensor-parallel
// exchange.  Code size matters: the kernels of a decoder layer take turns, so every launch starts from a cold
// instruction cache and fetches its preparation code (run once) from L2; the rare paths (outliers) are out of
// line for the same reason.  Single-row Q4_K variants: 38 / 50 / 56 / 82 KB.
template <int FMT, int SPW, int NP, bool ODD, int FEAT>   // format; super-blocks of a tile per compute warp (W = KS / SPW warps); row pairs;
                                                // ODD: the last pair has one row only (its odd columns are skipped)
__global__ void __launch_bounds__(MmFmt<FMT>::KS / SPW == 16 ? 544 : (MmFmt<FMT>::KS / SPW == 8 ? 320 : 256),
                                  (MmFmt<FMT>::KS / SPW == 16 || NP > 1) ? 1 : 2)
skn_matvec_mma(const skn_mv_group grp, int64_t pitch, int K, int nst, const float *__restrict__ x,
               int32_t *__restrict__ status, int relaxed) {
    constexpr int MM_KS = MmFmt<FMT>::KS, MM_BLOCK_BYTES = MmFmt<FMT>::SB_BYTES;
    constexpr int MM_ROW_STRIDE = MM_KS * MM_BLOCK_BYTES + MmFmt<FMT>::PAD, MM_STAGE = 16 * MM_ROW_STRIDE;
    constexpr int XS = MmFmt<FMT>::XS;
    constexpr int W = MM_KS / SPW;
    constexpr int NAMAX = 2 * NP;
    constexpr bool F_PREP = FEAT >= 1, F_ROPE = FEAT >= 2, F_XC = FEAT == 3;
    const float *const f_gain = F_PREP ? grp.norm_gain : nullptr;
    const float *const f_silu = F_XC ? grp.silu_u : nullptr;       // (the rare silu(x) * u preparation rides with the largest variant)
    const bool f_swiglu = (FEAT == 1 || FEAT == 3) && grp.swiglu;
    const int f_rope_hd = F_ROPE ? grp.rope_hd : 0;
    const int64_t N = grp.n_end[grp.count - 1];
    const int NA = grp.n_act;                   // 1 .. NAMAX activation rows
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;          // 0..W-1 compute, W = producer
    const int g = lane >> 2, t = lane & 3;
    const int nb = K / 256;
    // launches of three or four rows keep the digit planes of ONE K super-chunk at a time (their
    // planes would not fit otherwise); one or two rows prepare all of x up front
    constexpr bool CHUNKED = NP > 1;
    const int nbp = ((CHUNKED ? MM_KS : nb) + 3) / 4 * 4;        // scale slots per activation row
    const int nxs = CHUNKED ? MM_KS : nb;       // super-blocks of group sums per activation row
    const int nks = (nb + MM_KS - 1) / MM_KS;   // K super-chunks
    const int ksb = CHUNKED ? (nb < MM_KS ? nb : MM_KS) : nb;    // super-blocks whose digit planes are resident
    const int PL = ksb * 256 + 32;              // plane stride: 8 words mod 32, the four planes on disjoint banks
    const int RS = MM_ND * PL + 64;             // activation-row stride: 16 words mod 32, the two rows of a pair apart

    // shared memory: ring | digit planes [row][4] | block scales [row] | group sums [row] | outlier values, positions,
    //                counts [row][block] | barriers | partials [row]
    uint8_t *ring = smem;
    uint8_t *dig = smem + (size_t)nst * MM_STAGE;
    float *sgrp = reinterpret_cast<float *>(dig + ((size_t)NA * RS + 127) / 128 * 128);
    float *xsum = sgrp + (size_t)NA * nbp;
    float *oval = xsum + (size_t)NA * nxs * XS;
    uint32_t *oidx = reinterpret_cast<uint32_t *>(oval + (size_t)NA * nbp * MM_MAX_OUT);
    uint8_t *ocnt = reinterpret_cast<uint8_t *>(oidx + (size_t)NA * nbp);
    uint64_t *full = reinterpret_cast<uint64_t *>(ocnt + ((size_t)NA * nbp + 15) / 16 * 16);
    uint64_t *empty = full + nst;
    float *part = reinterpret_cast<float *>(empty + nst);

    // with interleaved gate / up rows every CTA owns whole (gate, up) pairs: even boundaries
    const int64_t even = (f_swiglu || f_rope_hd) ? ~(int64_t)1 : ~(int64_t)0;
    const int64_t row_begin = ((int64_t)blockIdx.x * N / gridDim.x) & even;
    const int64_t row_end = (blockIdx.x + 1 == gridDim.x) ? N : (((int64_t)(blockIdx.x + 1) * N / gridDim.x) & even);
    const int rows = (int)(row_end - row_begin);
    const int nrt = (rows + 15) >> 4;           // row tiles
    const int ntiles = nrt * nks;               // tile i -> super-chunk i / nrt, row tile i % nrt
    const int pw = nks * W;                     // partial slots per (activation row, weight row)

    __shared__ int s_anyout;                    // some prepared block of x has outliers (rare): the tile loop looks only then
    if (threadIdx.x == 0) s_anyout = 0;
    MV_TRACE_VARS;
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
            // a short last chunk of 210-byte blocks ends off a 16-byte boundary: the copy runs on into the row's padding
            const uint32_t bytes = ((uint32_t)nsb * MM_BLOCK_BYTES + 15u) & ~15u;
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
    // the norm's gain is a parameter, not a product of the launch before: asked into L2 ahead of the wait (last used
    // a whole step ago, it comes from HBM, behind this launch's own weight stream if requested any later)
    if (F_PREP && f_gain)
        for (int i = (int)threadIdx.x * 32; i < K; i += W * 32 * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(f_gain + i));
    if (!relaxed) skn_pdl_wait();
    MV_STAMP(2);
    // rotary epilogue: positions and ring starts are requested now and used at the very end
    int rp_pos[NAMAX], rp_start[NAMAX];
#pragma unroll
    for (int a = 0; a < NAMAX; ++a) {
        rp_pos[a] = rp_start[a] = 0;
        if (f_rope_hd && a < NA) {
            rp_pos[a] = grp.rope_len[grp.rope_a0 + a];
            rp_start[a] = grp.rope_start[grp.rope_a0 + a];
        }
    }
    // Tensor-parallel consumer: the previous launch of every rank pushed its partial products into
    // this rank's inbox; wait for the peers' flags (bounded), then every load of x adds them up.
    const float *redp = nullptr;
    if (F_XC && grp.xc_reduce && grp.xc_world > 1) {
        const uint32_t q = *reinterpret_cast<volatile uint32_t *>(grp.xc_state) - 1u;    // the exchange this rank completed last
        const int buf = (int)(q % SKN_COMM_NBUF);
        if (warp == 0 && lane < grp.xc_world && lane != grp.xc_rank && *reinterpret_cast<volatile int32_t *>(status) == 0) {
            const uint32_t *flag = reinterpret_cast<const uint32_t *>(grp.xc_base[grp.xc_rank]) + buf * SKN_COMM_MAX_WORLD + lane;
            const uint64_t t0 = skn_globaltimer_ns(), limit = skn_wait_limit_ns(status);
            uint32_t spins = 0, v;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
                if (v == q + 1u) break;
                if ((++spins & 1023u) == 0 && skn_globaltimer_ns() - t0 > limit) {
                    atomicExch(status, SKN_ERR_TIMEOUT);
                    break;
                }
            }
        }
        mm_bar_sync(1, W * 32);
        redp = reinterpret_cast<const float *>(grp.xc_base[grp.xc_rank] + SKN_COMM_FLAG_BYTES) + (size_t)buf * grp.xc_world * grp.xc_cap;
    }
    // RMSNorm folded in without a pass of its own: the digits are taken of x * gain, the sum of
    // squares of x is collected on the way (per warp, in shared memory), and the scalar 1 / rms
    // multiplies the outputs at the end.
    __shared__ float red[NAMAX][16];
    if (lane < NAMAX) red[lane][warp] = 0.f;
    __syncwarp();
    // x -> digit planes of K super-chunk kc: a warp takes whole super-blocks, two per round (four loads in
    // flight, two independent digitisations for the scheduler to interleave; four per round made the code 11 KB
    // longer, and a launch runs this once from a cold instruction cache);
    // unit u = activation row u / nsb, super-block (of the chunk) u % nsb.  The planes of one chunk are
    // resident at a time, so shared memory does not grow with K.
    auto prep_chunk = [&](int kc) {
        int nsbc = nb - kc * MM_KS;
        nsbc = nsbc > MM_KS ? MM_KS : nsbc;
        const int units = NA * nsbc;
        constexpr int UR = 2;
        float sq[NAMAX];
#pragma unroll
        for (int a = 0; a < NAMAX; ++a) sq[a] = 0.f;
        for (int u0 = warp; u0 < units; u0 += UR * W) {
            float4 v[UR][2];
            int ua[UR], us[UR], ux[UR];
            // every load of the round is issued before anything waits for one (the norm's gain included: a load
            // behind a use of the previous one would cost a trip to L2 per unit)
#pragma unroll
            for (int h = 0; h < UR; ++h) {
                const int uu = u0 + h * W;
                ua[h] = -1;
                us[h] = ux[h] = 0;
                if (uu < units) {
                    const int a = uu / nsbc, sbl = uu - a * nsbc, sbx = kc * MM_KS + sbl;      // sbx: index in x
                    skn_xform xf{nullptr, f_silu ? f_silu + (size_t)a * K : nullptr, 1.f,
                                 redp ? redp + (size_t)a * K : nullptr, redp ? grp.xc_world : 0, grp.xc_cap,
                                 (redp && grp.xc_wb && blockIdx.x == 0) ? grp.xc_wb + (size_t)a * K : nullptr};
                    const float *xa = x + (size_t)a * K;
                    v[h][0] = skn_load_x4(xa, sbx * 64 + lane, xf);
                    v[h][1] = skn_load_x4(xa, sbx * 64 + 32 + lane, xf);
                    ua[h] = a;
                    us[h] = CHUNKED ? sbl : sbx;      // index among the resident planes
                    ux[h] = sbx;
                }
            }
            if (f_gain) {
                float4 gq[UR][2];
#pragma unroll
                for (int h = 0; h < UR; ++h) {
                    gq[h][0] = __ldg(reinterpret_cast<const float4 *>(f_gain) + ux[h] * 64 + lane);
                    gq[h][1] = __ldg(reinterpret_cast<const float4 *>(f_gain) + ux[h] * 64 + 32 + lane);
                }
#pragma unroll
                for (int h = 0; h < UR; ++h) {
                    if (ua[h] >= 0) {
                        float4 &r0 = v[h][0], &r1 = v[h][1];
                        const float e = (r0.x * r0.x + r0.y * r0.y) + (r0.z * r0.z + r0.w * r0.w) + (r1.x * r1.x + r1.y * r1.y) +
                                        (r1.z * r1.z + r1.w * r1.w);
#pragma unroll
                        for (int k = 0; k < NAMAX; ++k)
                            if (k == ua[h]) sq[k] += e;
                        const float4 g0 = gq[h][0], g1 = gq[h][1];
                        r0.x *= g0.x; r0.y *= g0.y; r0.z *= g0.z; r0.w *= g0.w;
                        r1.x *= g1.x; r1.y *= g1.y; r1.z *= g1.z; r1.w *= g1.w;
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < UR; ++h)
                if (ua[h] >= 0)
                    mm_digitize<XS == 16>(v[h][0], v[h][1], us[h], lane, dig + (size_t)ua[h] * RS, PL, sgrp + (size_t)ua[h] * nbp,
                                          xsum + (size_t)ua[h] * nxs * XS, oval + (size_t)ua[h] * nbp * MM_MAX_OUT,
                                          oidx + (size_t)ua[h] * nbp, ocnt + (size_t)ua[h] * nbp, &s_anyout);
        }
        if (f_gain) {
#pragma unroll
            for (int a = 0; a < NAMAX; ++a) {
                float ss = sq[a];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0) red[a][warp] += ss;
            }
        }
    };

    // B column c of a row pair = digit c / 2 of its row c & 1: a lane LOADS column g and READS BACK
    // columns 2t (first row of the pair) and 2t + 1 (second row), both of digit t
    const int bcol_row = g & 1, bcol_dig = g >> 1;
    const float inv_dw = (t == 0) ? 1.f : ((t == 1) ? (1.f / 256.f) : ((t == 2) ? (1.f / 65536.f) : (1.f / 16777216.f)));
    constexpr int rowA = 0, rowB = 1;
    bool failed = false;
    int ks = 0, rt = 0, stg = 0;
    uint32_t par = 0;
    const uint32_t ring_s = skn_smem_u32(ring), dig_s = skn_smem_u32(dig), sgrp_s = skn_smem_u32(sgrp), xsum_s = skn_smem_u32(xsum);
    const uint32_t oval_s = skn_smem_u32(oval), oidx_s = skn_smem_u32(oidx), ocnt_s = skn_smem_u32(ocnt);
    int cur_ks = -1;
    if (!CHUNKED) {
        for (int kc = 0; kc < nks; ++kc) prep_chunk(kc);
        mm_bar_sync(1, W * 32);
    }
    MV_STAMP(3);
    for (int i = 0; i < ntiles; ++i) {
        const uint32_t st = ring_s + (uint32_t)stg * MM_STAGE;
        int nsb = nb - ks * MM_KS;
        nsb = nsb > MM_KS ? MM_KS : nsb;
        if (CHUNKED && ks != cur_ks) {
            // every compute warp walks the same tile sequence, so all of them get here together:
            // nobody reads the old planes any more, then everybody sees the new ones
            if (cur_ks >= 0) mm_bar_sync(1, W * 32);
            prep_chunk(ks);
            mm_bar_sync(1, W * 32);
            cur_ks = ks;
        }
        const int sb0 = CHUNKED ? 0 : ks * MM_KS;   // resident index of the tile's first super-block
        if (!failed && !skn_mbar_wait(&full[stg], par)) {
            failed = true;
            atomicExch(status, SKN_ERR_TIMEOUT);
        }
        if (i == 0) MV_STAMP(4);
        const bool anyout = *reinterpret_cast<volatile int *>(&s_anyout) != 0;     // (after this tile's planes were prepared)
        float accA[NP][2], accB[NP][2];         // [pair][weight row g / g + 8]: columns 2t and 2t + 1, all own super-blocks
        float ms[NAMAX];                        // min term of weight row g + 8 * (t & 1), sub-blocks 4 * (t >> 1) .. + 3
#pragma unroll
        for (int ap = 0; ap < NP; ++ap) accA[ap][0] = accA[ap][1] = accB[ap][0] = accB[ap][1] = 0.f;
#pragma unroll
        for (int a = 0; a < NAMAX; ++a) ms[a] = 0.f;
#pragma unroll
        for (int hh = 0; hh < SPW; ++hh) {
            const int sb = warp + W * hh;
            if (sb >= nsb) break;
            const uint32_t ba = st + g * MM_ROW_STRIDE + sb * MM_BLOCK_BYTES;
            const uint32_t bb = ba + 8 * MM_ROW_STRIDE;
            // outlier counts of this block per activation row (almost always zero): loaded now, looked at after the MMAs
            int ocn[NAMAX];
#pragma unroll
            for (int a = 0; a < NAMAX; ++a) ocn[a] = (anyout && a < NA) ? (int)mm_lds8(ocnt_s + (uint32_t)(a * nbp + sb0 + sb)) : 0;
            if constexpr (FMT == MM_FMT_Q4K) {
            const uint4 ha = mm_lds128(ba), hb = mm_lds128(bb);
            // 6-bit scales as bytes: word 0 = sub-blocks 0..3, word 1 = sub-blocks 4..7
            const uint32_t sa[2] = {ha.y & 0x3F3F3F3Fu, (ha.w & 0x0F0F0F0Fu) | ((ha.y >> 2) & 0x30303030u)};
            const uint32_t sq[2] = {hb.y & 0x3F3F3F3Fu, (hb.w & 0x0F0F0F0Fu) | ((hb.y >> 2) & 0x30303030u)};
            int lo[NP][4], hi[NP][4];           // [pair][weight row g col 2t, col 2t+1, weight row g+8 col 2t, col 2t+1]
#pragma unroll
            for (int ap = 0; ap < NP; ++ap)
#pragma unroll
                for (int c = 0; c < 4; ++c) lo[ap][c] = hi[ap][c] = 0;
            uint32_t bsrc[NP];
            bool bon[NP];
#pragma unroll
            for (int ap = 0; ap < NP; ++ap) {
                const int arow = 2 * ap + bcol_row;
                bon[ap] = arow < NA;
                bsrc[ap] = dig_s + (uint32_t)((bon[ap] ? arow : 0) * RS + bcol_dig * PL + (sb0 + sb) * 256 + 8 * t);
            }
            // The MMAs of byte pair p + 1 are issued before the results of pair p are consumed, so
            // that their latency overlaps the integer multiply-adds.
            int cl[2][NP][4], ch[2][NP][4];
            auto issue_pair = [&](int p, int buf) {
                const uint2 wa = mm_lds64(ba + 16 + 32 * p + 8 * t);
                const uint2 wb = mm_lds64(bb + 16 + 32 * p + 8 * t);
                const uint32_t al0 = wa.x & 0x0F0F0F0Fu, al1 = wb.x & 0x0F0F0F0Fu, al2 = wa.y & 0x0F0F0F0Fu, al3 = wb.y & 0x0F0F0F0Fu;
                const uint32_t ah0 = wa.x & 0xF0F0F0F0u, ah1 = wb.x & 0xF0F0F0F0u, ah2 = wa.y & 0xF0F0F0F0u, ah3 = wb.y & 0xF0F0F0F0u;
#pragma unroll
                for (int ap = 0; ap < NP; ++ap) {
                    // (unconditional: lanes whose column has no activation row read row 0 again; those columns are never used)
                    const uint2 b0 = mm_lds64(bsrc[ap] + (2 * p) * 32);
                    const uint2 b1 = mm_lds64(bsrc[ap] + (2 * p + 1) * 32);
                    skn_mma_u8s8(cl[buf][ap], al0, al1, al2, al3, b0.x, b0.y);
                    skn_mma_u8s8(ch[buf][ap], ah0, ah1, ah2, ah3, b1.x, b1.y);
                }
            };
            issue_pair(0, 0);
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                if (p < 3) issue_pair(p + 1, (p + 1) & 1);
                const int s0a = mm_byte_i(sa[p >> 1], 2 * (p & 1)), s1a = mm_byte_i(sa[p >> 1], 2 * (p & 1) + 1);
                const int s0b = mm_byte_i(sq[p >> 1], 2 * (p & 1)), s1b = mm_byte_i(sq[p >> 1], 2 * (p & 1) + 1);
#pragma unroll
                for (int ap = 0; ap < NP; ++ap) {
                    const int *c = cl[p & 1][ap], *h = ch[p & 1][ap];
                    lo[ap][0] += s0a * c[0]; lo[ap][2] += s0b * c[2];
                    hi[ap][0] += s1a * h[0]; hi[ap][2] += s1b * h[2];
                    if (!(ODD && ap == NP - 1)) {
                        lo[ap][1] += s0a * c[1]; lo[ap][3] += s0b * c[3];
                        hi[ap][1] += s1a * h[1]; hi[ap][3] += s1b * h[3];
                    }
                }
            }
            // 16 * sum_j sc_j dot_j per digit column (high-nibble results carry a factor 16), scaled
            // by d of the weight row and the block scale of the column's activation row
            const float2 da = __half22float2(*reinterpret_cast<const __half2 *>(&ha.x));   // {d, dmin} of row g
            const float2 db = __half22float2(*reinterpret_cast<const __half2 *>(&hb.x));   // ... of row g + 8
#pragma unroll
            for (int ap = 0; ap < NP; ++ap) {
                const int ra = min(2 * ap + rowA, NA - 1), rb = min(2 * ap + rowB, NA - 1);
                const float sgA = mm_lds32f(sgrp_s + 4u * (uint32_t)(ra * nbp + sb0 + sb)) * 0.0625f;
                const float sgB = mm_lds32f(sgrp_s + 4u * (uint32_t)(rb * nbp + sb0 + sb)) * 0.0625f;
                accA[ap][0] = fmaf(da.x * sgA, (float)(lo[ap][0] * 16 + hi[ap][0]), accA[ap][0]);
                accA[ap][1] = fmaf(db.x * sgA, (float)(lo[ap][2] * 16 + hi[ap][2]), accA[ap][1]);
                if (!(ODD && ap == NP - 1)) {
                    accB[ap][0] = fmaf(da.x * sgB, (float)(lo[ap][1] * 16 + hi[ap][1]), accB[ap][0]);
                    accB[ap][1] = fmaf(db.x * sgB, (float)(lo[ap][3] * 16 + hi[ap][3]), accB[ap][1]);
                }
            }
            // min term: this lane covers one weight row and four sub-blocks, every activation row
            const uint4 hm = (t & 1) ? hb : ha;
            const uint32_t mw = (t & 2) ? (((hm.w >> 4) & 0x0F0F0F0Fu) | ((hm.z >> 2) & 0x30303030u)) : (hm.z & 0x3F3F3F3Fu);
            const float m0 = mm_byte_f(mw, 0), m1 = mm_byte_f(mw, 1), m2 = mm_byte_f(mw, 2), m3 = mm_byte_f(mw, 3);
            const float dmin = (t & 1) ? db.y : da.y;
#pragma unroll
            for (int a = 0; a < NAMAX; ++a) {
                if (a < NA) {
                    const float4 xs = mm_lds128f(xsum_s + 4u * (uint32_t)((a * nxs + sb0 + sb) * 8 + 4 * (t >> 1)));
                    float m = m0 * xs.x;
                    m = fmaf(m1, xs.y, m);
                    m = fmaf(m2, xs.z, m);
                    m = fmaf(m3, xs.w, m);
                    ms[a] = fmaf(dmin, m, ms[a]);
                }
            }
            } else if constexpr (FMT == MM_FMT_Q6K) {
            // A 210-byte block starts two bytes off a word boundary when its index in the row is odd:
            // every word is taken from two aligned words with a funnel shift (by 0 or 16 bits).
            const uint32_t sh = (ba & 2u) * 8u;
            const uint32_t wa = ba & ~3u, wb = bb & ~3u;
            auto ldw = [&](uint32_t base, int off) {
                return __funnelshift_r(mm_lds32(base + off), mm_lds32(base + off + 4), sh);
            };
            uint32_t bsrc[NP];
            bool bon[NP];
#pragma unroll
            for (int ap = 0; ap < NP; ++ap) {
                const int arow = 2 * ap + bcol_row;
                bon[ap] = arow < NA;
                bsrc[ap] = dig_s + (uint32_t)((bon[ap] ? arow : 0) * RS + bcol_dig * PL + (sb0 + sb) * 256) + 4 * t;
            }
            // sixteen int8 scales of each row: five aligned words -> four block words
            uint32_t sa[4], sq[4];
            {
                uint32_t ua[5], ub[5];
#pragma unroll
                for (int j = 0; j < 5; ++j) { ua[j] = mm_lds32(wa + 192 + 4 * j); ub[j] = mm_lds32(wb + 192 + 4 * j); }
#pragma unroll
                for (int j = 0; j < 4; ++j) { sa[j] = __funnelshift_r(ua[j], ua[j + 1], sh); sq[j] = __funnelshift_r(ub[j], ub[j + 1], sh); }
            }
            int acc[NP][4];                 // [pair][row g col 2t, col 2t+1, row g+8 col 2t, col 2t+1]: sum of scale * dot
#pragma unroll
            for (int ap = 0; ap < NP; ++ap)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[ap][c] = 0;
            // Weight 128h + 32q + l (quarter q, l = 0..31) has its low four bits in ql[64h + 32(q & 1) + l]
            // (low nibble for q < 2) and its top two in bits 2q, 2q+1 of qh[32h + l]; its scale is number
            // 8h + 2q + l / 16.  Lane t holds bytes l = 4t..4t+3 (part 0) and 16 + 4t.. (part 1) of every
            // 32-byte run; a 16-weight scale group is one MMA on the k slots 0..15 (slots 16..31 are zero).
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t Ha[2], Hb[2];
#pragma unroll
                for (int pt = 0; pt < 2; ++pt) {
                    Ha[pt] = ldw(wa, 128 + 32 * h + 16 * pt + 4 * t);
                    Hb[pt] = ldw(wb, 128 + 32 * h + 16 * pt + 4 * t);
                }
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    uint32_t La[2], Lb[2];
#pragma unroll
                    for (int pt = 0; pt < 2; ++pt) {
                        La[pt] = ldw(wa, 64 * h + 32 * r + 16 * pt + 4 * t);
                        Lb[pt] = ldw(wb, 64 * h + 32 * r + 16 * pt + 4 * t);
                    }
#pragma unroll
                    for (int hi = 0; hi < 2; ++hi) {
                        const int q = r + 2 * hi;               // quarter of the half
#pragma unroll
                        for (int pt = 0; pt < 2; ++pt) {
                            const uint32_t na = hi ? (La[pt] >> 4) : La[pt], nq = hi ? (Lb[pt] >> 4) : Lb[pt];
                            const uint32_t ta = (q < 2) ? (Ha[pt] << (4 - 2 * q)) : (Ha[pt] >> (2 * q - 4));
                            const uint32_t tq = (q < 2) ? (Hb[pt] << (4 - 2 * q)) : (Hb[pt] >> (2 * q - 4));
                            const uint32_t a0 = (na & 0x0F0F0F0Fu) | (ta & 0x30303030u);
                            const uint32_t a1 = (nq & 0x0F0F0F0Fu) | (tq & 0x30303030u);
                            const int si = 8 * h + 2 * q + pt;  // scale index
                            const int s_a = mm_sbyte_i(sa[si >> 2], si & 3), s_b = mm_sbyte_i(sq[si >> 2], si & 3);
#pragma unroll
                            for (int ap = 0; ap < NP; ++ap) {
                                const uint32_t b0 = mm_lds32(bsrc[ap] + (4 * h + q) * 32 + 16 * pt);
                                int c[4];
                                skn_mma_u8s8(c, a0, a1, 0u, 0u, b0, 0u);
                                acc[ap][0] += s_a * c[0]; acc[ap][2] += s_b * c[2];
                                if (!(ODD && ap == NP - 1)) { acc[ap][1] += s_a * c[1]; acc[ap][3] += s_b * c[3]; }
                            }
                        }
                    }
                }
            }
            const float d_a = mm_lds_half(ba + 208), d_b = mm_lds_half(bb + 208);
#pragma unroll
            for (int ap = 0; ap < NP; ++ap) {
                const int ra = min(2 * ap + rowA, NA - 1), rb = min(2 * ap + rowB, NA - 1);
                const float sgA = mm_lds32f(sgrp_s + 4u * (uint32_t)(ra * nbp + sb0 + sb));
                const float sgB = mm_lds32f(sgrp_s + 4u * (uint32_t)(rb * nbp + sb0 + sb));
                accA[ap][0] = fmaf(d_a * sgA, (float)acc[ap][0], accA[ap][0]);
                accA[ap][1] = fmaf(d_b * sgA, (float)acc[ap][2], accA[ap][1]);
                if (!(ODD && ap == NP - 1)) {
                    accB[ap][0] = fmaf(d_a * sgB, (float)acc[ap][1], accB[ap][0]);
                    accB[ap][1] = fmaf(d_b * sgB, (float)acc[ap][3], accB[ap][1]);
                }
            }
            // offset term 32 * d * sum_i scale_i * sum(x of group i): this lane covers one weight row and
            // eight of the sixteen scale groups, every activation row
            {
                const uint32_t r0 = (t & 1) ? ((t & 2) ? sq[2] : sq[0]) : ((t & 2) ? sa[2] : sa[0]);
                const uint32_t r1 = (t & 1) ? ((t & 2) ? sq[3] : sq[1]) : ((t & 2) ? sa[3] : sa[1]);
                const uint32_t f0 = r0 ^ 0x80808080u, f1 = r1 ^ 0x80808080u;
                const float dd = 32.f * ((t & 1) ? d_b : d_a);
                float sf[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) { sf[j] = mm_sbyte_f(f0, j); sf[4 + j] = mm_sbyte_f(f1, j); }
#pragma unroll
                for (int a = 0; a < NAMAX; ++a) {
                    if (a < NA) {
                        const uint32_t xa = xsum_s + 4u * (uint32_t)((a * nxs + sb0 + sb) * 16 + 8 * (t >> 1));
                        const float4 x0 = mm_lds128f(xa), x1 = mm_lds128f(xa + 16);
                        float m = sf[0] * x0.x;
                        m = fmaf(sf[1], x0.y, m); m = fmaf(sf[2], x0.z, m); m = fmaf(sf[3], x0.w, m);
                        m = fmaf(sf[4], x1.x, m); m = fmaf(sf[5], x1.y, m); m = fmaf(sf[6], x1.z, m); m = fmaf(sf[7], x1.w, m);
                        ms[a] = fmaf(dd, m, ms[a]);
                    }
                }
            }
            } else {
            uint32_t bsrc[NP];
            bool bon[NP];
#pragma unroll
            for (int ap = 0; ap < NP; ++ap) {
                const int arow = 2 * ap + bcol_row;
                bon[ap] = arow < NA;
                bsrc[ap] = dig_s + (uint32_t)((bon[ap] ? arow : 0) * RS + bcol_dig * PL + (sb0 + sb) * 256) +
                           (FMT == MM_FMT_Q80 ? 8 * t : 4 * t);
            }
            float sgA[NP], sgB[NP];
#pragma unroll
            for (int ap = 0; ap < NP; ++ap) {
                const int ra = min(2 * ap + rowA, NA - 1), rb = min(2 * ap + rowB, NA - 1);
                sgA[ap] = mm_lds32f(sgrp_s + 4u * (uint32_t)(ra * nbp + sb0 + sb));
                sgB[ap] = mm_lds32f(sgrp_s + 4u * (uint32_t)(rb * nbp + sb0 + sb));
            }
            // eight 32-weight blocks, one MMA each; block j of a row starts 2-byte aligned, its
            // quants are word aligned for odd j and two bytes off for even j
            constexpr int BB = MM_BLOCK_BYTES / 8;          // 34 (Q8_0) or 18 (Q4_0)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t a0, a1, a2, a3;                    // rows g / g+8, k 0..15 / 16..31 of the fragment
                const float d_a = mm_lds_half(ba + BB * j), d_b = mm_lds_half(bb + BB * j);
                if constexpr (FMT == MM_FMT_Q80) {
                    // lane t: quant bytes 8t .. 8t+7 of the block
                    const uint32_t oa = ba + BB * j + 2 + 8 * t, ob = bb + BB * j + 2 + 8 * t;
                    if (j & 1) {
                        a0 = mm_lds32(oa); a2 = mm_lds32(oa + 4);
                        a1 = mm_lds32(ob); a3 = mm_lds32(ob + 4);
                    } else {
                        const uint32_t u0 = mm_lds32(oa - 2), u1 = mm_lds32(oa + 2), u2 = mm_lds32(oa + 6);
                        const uint32_t v0 = mm_lds32(ob - 2), v1 = mm_lds32(ob + 2), v2 = mm_lds32(ob + 6);
                        a0 = __byte_perm(u0, u1, 0x5432); a2 = __byte_perm(u1, u2, 0x5432);
                        a1 = __byte_perm(v0, v1, 0x5432); a3 = __byte_perm(v1, v2, 0x5432);
                    }
                } else {
                    // lane t: quant bytes 4t .. 4t+3: low nibbles = weights 4t.., high nibbles = weights 16 + 4t..
                    const uint32_t oa = ba + BB * j + 2 + 4 * t, ob = bb + BB * j + 2 + 4 * t;
                    uint32_t wa, wb;
                    if (j & 1) {
                        wa = mm_lds32(oa); wb = mm_lds32(ob);
                    } else {
                        wa = __byte_perm(mm_lds32(oa - 2), mm_lds32(oa + 2), 0x5432);
                        wb = __byte_perm(mm_lds32(ob - 2), mm_lds32(ob + 2), 0x5432);
                    }
                    a0 = wa & 0x0F0F0F0Fu; a2 = (wa >> 4) & 0x0F0F0F0Fu;
                    a1 = wb & 0x0F0F0F0Fu; a3 = (wb >> 4) & 0x0F0F0F0Fu;
                }
#pragma unroll
                for (int ap = 0; ap < NP; ++ap) {
                    uint32_t b0, b1;
                    if constexpr (FMT == MM_FMT_Q80) {
                        const uint2 b = mm_lds64(bsrc[ap] + j * 32);
                        b0 = b.x; b1 = b.y;
                    } else {
                        b0 = mm_lds32(bsrc[ap] + j * 32);
                        b1 = mm_lds32(bsrc[ap] + j * 32 + 16);
                    }
                    int c[4];
                    if constexpr (FMT == MM_FMT_Q80) skn_mma_s8s8(c, a0, a1, a2, a3, b0, b1);
                    else skn_mma_u8s8(c, a0, a1, a2, a3, b0, b1);
                    accA[ap][0] = fmaf(d_a * sgA[ap], (float)c[0], accA[ap][0]);
                    accA[ap][1] = fmaf(d_b * sgA[ap], (float)c[2], accA[ap][1]);
                    if (!(ODD && ap == NP - 1)) {
                        accB[ap][0] = fmaf(d_a * sgB[ap], (float)c[1], accB[ap][0]);
                        accB[ap][1] = fmaf(d_b * sgB[ap], (float)c[3], accB[ap][1]);
                    }
                }
            }
            if constexpr (FMT == MM_FMT_Q40) {
                // offset term 8 * d * sum(x) per block: this lane covers one weight row and four blocks
                const uint32_t hrow = (t & 1) ? bb : ba;
                const int j0 = 4 * (t >> 1);
                const float d0 = mm_lds_half(hrow + BB * j0), d1 = mm_lds_half(hrow + BB * (j0 + 1));
                const float d2 = mm_lds_half(hrow + BB * (j0 + 2)), d3 = mm_lds_half(hrow + BB * (j0 + 3));
#pragma unroll
                for (int a = 0; a < NAMAX; ++a) {
                    if (a < NA) {
                        const float4 xs = mm_lds128f(xsum_s + 4u * (uint32_t)((a * nxs + sb0 + sb) * 8 + j0));
                        float m = d0 * xs.x;
                        m = fmaf(d1, xs.y, m);
                        m = fmaf(d2, xs.z, m);
                        m = fmaf(d3, xs.w, m);
                        ms[a] = fmaf(8.f, m, ms[a]);
                    }
                }
            }
            }
            // outliers (rare): lane t multiplies outlier t with the weights of rows g and g + 8; the product joins
            // this lane's digit accumulator with the digit's power of two divided out
#pragma unroll
            for (int a = 0; a < NAMAX; ++a) {
                if (ocn[a] != 0) {                                       // warp-uniform
                    if (t < ocn[a]) {
                        const float2 wp = mm_outlier_products<FMT>(ba, bb, oidx_s, oval_s, (uint32_t)(a * nbp + sb0 + sb), t, inv_dw);
                        if (a & 1) { accB[a >> 1][0] += wp.x; accB[a >> 1][1] += wp.y; }
                        else { accA[a >> 1][0] += wp.x; accA[a >> 1][1] += wp.y; }
                    }
                }
            }
        }
        __syncwarp();      // every lane has read its share of the stage
        if (lane == 0) skn_mbar_arrive(&empty[stg]);
        // ---- tile epilogue: lane t holds digit t of both rows of a pair, and the products of their outliers number t
        const float dw = (t == 0) ? 1.f : ((t == 1) ? 256.f : ((t == 2) ? 65536.f : 16777216.f));
#pragma unroll
        for (int ap = 0; ap < NP; ++ap) {
#pragma unroll
            for (int wr = 0; wr < 2; ++wr) {            // weight rows g, g + 8
                float e0 = accA[ap][wr] * dw;
                float e1 = accB[ap][wr] * dw;
                e0 += __shfl_xor_sync(0xffffffffu, e0, 1);
                e1 += __shfl_xor_sync(0xffffffffu, e1, 1);
                e0 += __shfl_xor_sync(0xffffffffu, e0, 2);
                e1 += __shfl_xor_sync(0xffffffffu, e1, 2);
                accA[ap][wr] = e0;                      // now: totals of rows 2 ap and 2 ap + 1 in every lane
                accB[ap][wr] = e1;
            }
        }
#pragma unroll
        for (int a = 0; a < NAMAX; ++a) {
            // both sub-block halves: lanes t = 0, 2 hold weight row g, lanes t = 1, 3 row g + 8
            ms[a] += __shfl_xor_sync(0xffffffffu, ms[a], 2);
            const float mo = __shfl_xor_sync(0xffffffffu, ms[a], 1);
            if (t == 0 && a < NA) {
                const int r0 = rt * 16 + g;
                const float v0 = (a & 1) ? accB[a >> 1][0] : accA[a >> 1][0];
                const float v1 = (a & 1) ? accB[a >> 1][1] : accA[a >> 1][1];
                float *pa = part + (size_t)a * rows * pw;
                if (r0 < rows) pa[(size_t)r0 * pw + ks * W + warp] = v0 - ms[a];
                if (r0 + 8 < rows) pa[(size_t)(r0 + 8) * pw + ks * W + warp] = v1 - mo;
            }
        }
        if (++rt == nrt) { rt = 0; ++ks; }
        if (++stg == nst) { stg = 0; par ^= 1u; }
    }
    MV_STAMP(5);
    // RMSNorm: the scalar 1 / rms of every activation row multiplies its outputs (the products above
    // are linear in x, and the digits were taken of x * gain)
    mm_bar_sync(1, W * 32);
    MV_STAMP(6);
    float nscale[NAMAX];
#pragma unroll
    for (int a = 0; a < NAMAX; ++a) {
        nscale[a] = 1.f;
        if (f_gain && a < NA) {
            float tot = 0.f;
            for (int w2 = 0; w2 < W; ++w2) tot += red[a][w2];
            nscale[a] = rsqrtf(tot / (float)K + grp.norm_eps);
        }
    }
    // L lanes per row (16, 4 or 1, the most that still covers the CTA's rows in about one pass):
    // each adds its share of the row's partials in index order, then a fixed butterfly, so the
    // summation tree depends on the shape only
    const int lsh = (rows * 16 <= W * 32) ? 4 : ((rows * 4 <= W * 32) ? 2 : 0);
    const int L = 1 << lsh;
    const bool push = F_XC && grp.xc_push && grp.xc_world > 1;
    uint32_t xq = 0;
    if (push) xq = *reinterpret_cast<volatile uint32_t *>(grp.xc_state);        // number of this exchange
    const size_t push_off = SKN_COMM_FLAG_BYTES / sizeof(float) + ((size_t)(xq % SKN_COMM_NBUF) * grp.xc_world + grp.xc_rank) * grp.xc_cap;
    for (int a = 0; a < NA; ++a) {
        const float *pa = part + (size_t)a * rows * pw;
        for (int lb = warp * (32 >> lsh); lb < rows; lb += W * (32 >> lsh)) {     // warp-uniform trip count
            const int lr = lb + (lane >> lsh);
            const int sub = lane & (L - 1);
            float s = 0.f;
            if (lr < rows)
                for (int cc = sub; cc < pw; cc += L) s += pa[(size_t)lr * pw + cc];
            for (int o = L >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
#pragma unroll
            for (int k = 0; k < NAMAX; ++k)
                if (k == a) s *= nscale[k];
            const float up = __shfl_xor_sync(0xffffffffu, s, L);      // the next row: the `up` product of a gate row
            if (sub == 0 && lr < rows) {
                int64_t local;
                const int tt = skn_group_row(grp, row_begin + lr, local);
                if (f_swiglu) {
                    if (tt == 0) grp.y[0][(size_t)a * grp.ystride[0] + local] = s / (1.f + expf(-s)) * up;
                } else if (f_rope_hd) {
                    // rotary embedding of the pair (2i, 2i+1) this row belongs to (`up` is the other
                    // row of the pair), k and v straight into the cache
                    const int hd = F_ROPE ? f_rope_hd : 2, seq = grp.rope_a0 + a;
                    int pos = 0, ring0 = 0;
#pragma unroll
                    for (int k = 0; k < NAMAX; ++k)
                        if (k == a) { pos = rp_pos[k]; ring0 = rp_start[k]; }
                    // a full cache (a replayed step the host did not count): nothing is overwritten
                    const bool room = pos < grp.rope_cap;
                    if (!room) atomicExch(status, SKN_ERR_SHAPE);
                    const int slot = (ring0 + pos) % grp.rope_cap;
                    const int h = (int)(local / hd), dd = (int)(local % hd);
                    float o = s;
                    if (tt < 2) {
                        // the angle in double (positions reach thousands of radians), reduced to [-pi, pi] with a
                        // two-term 2 pi, then the fp32 functions: a handful of fp64 instructions instead of a
                        // double-precision sincos
                        const double f = grp.rope_inv_freq ? grp.rope_inv_freq[dd >> 1]
                                                           : exp2(-grp.rope_log2theta * (2.0 * (double)(dd >> 1) / (double)hd));
                        const double ang = (double)pos * f;
                        const double turns = rint(ang * 0.15915494309189535);
                        const float red_ang = (float)fma(-turns, 2.4492935982947064e-16, fma(-turns, 6.283185307179586, ang));
                        float sn, cs;
                        sincosf(red_ang, &sn, &cs);
                        o = (dd & 1) ? (up * sn + s * cs) : (s * cs - up * sn);
                    }
                    if (tt == 0) grp.y[0][(size_t)a * grp.ystride[0] + local] = o;
                    else if (room) (tt == 1 ? grp.rope_kc : grp.rope_vc)[(((size_t)seq * grp.rope_nkv + h) * grp.rope_cap + slot) * hd + dd] = o;
                } else if (push) {
                    // a partial product: slot `rank` of every rank's inbox (ordinary peer stores)
                    const size_t o = push_off + (size_t)a * grp.ystride[tt] + local;
                    for (int r = 0; r < grp.xc_world; ++r) reinterpret_cast<float *>(grp.xc_base[r])[o] = s;
                } else {
                    if (grp.add[tt]) s += grp.add[tt][(size_t)a * grp.addstride[tt] + local];
                    grp.y[tt][(size_t)a * grp.ystride[tt] + local] = s;
                }
            }
        }
    }
    if (push) {
        // the CTA barrier orders every thread's peer stores before thread 0's system-wide fence; the
        // CTA that draws the last ticket counts the exchange and releases the flag on every peer
        mm_bar_sync(1, W * 32);
        if (threadIdx.x == 0) {
            __threadfence_system();
            if (atomicAdd(&grp.xc_state[1], 1u) == gridDim.x - 1) {
                grp.xc_state[1] = 0;
                *reinterpret_cast<volatile uint32_t *>(grp.xc_state) = xq + 1u;
                __threadfence_system();
                for (int r = 0; r < grp.xc_world; ++r) {
                    if (r == grp.xc_rank) continue;
                    uint32_t *flag = reinterpret_cast<uint32_t *>(grp.xc_base[r]) + (xq % SKN_COMM_NBUF) * SKN_COMM_MAX_WORLD + grp.xc_rank;
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(xq + 1u) : "memory");
                }
            }
        }
    }
    MV_STAMP(7);
}

// Launch geometry: compute warps per CTA and ring depth that fit the shared-memory budget.  With
// few tiles the budget is half of an SM's shared memory: the CTA of the next launch can then
// become resident (programmatic dependent launch) and prefetch its weights while this one
// computes.
typedef void (*mm_kernel_t)(const skn_mv_group, int64_t, int, int, const float *, int32_t *, int);

static int mm_fmt_of(int32_t type) {
    switch (type) {
    case SKN_TYPE_Q4_K: return MM_FMT_Q4K;
    case SKN_TYPE_Q8_0: return MM_FMT_Q80;
    case SKN_TYPE_Q4_0: return MM_FMT_Q40;
    case SKN_TYPE_Q6_K: return MM_FMT_Q6K;
    default: return -1;
    }
}

template <int FMT, int SPW, int FEAT>
static mm_kernel_t mm_kernel_na(int n_act) {
    switch (n_act) {
    case 1: return skn_matvec_mma<FMT, SPW, 1, true, FEAT>;
    case 2: return skn_matvec_mma<FMT, SPW, 1, false, FEAT>;
    case 3: return skn_matvec_mma<FMT, SPW, 2, true, FEAT>;
    default: return skn_matvec_mma<FMT, SPW, 2, false, FEAT>;
    }
}

template <int FMT, int SPW>
static mm_kernel_t mm_kernel_feat(int n_act, int feat) {
    switch (feat) {
    case 0: return mm_kernel_na<FMT, SPW, 0>(n_act);
    case 1: return mm_kernel_na<FMT, SPW, 1>(n_act);
    case 2: return mm_kernel_na<FMT, SPW, 2>(n_act);
    default: return mm_kernel_na<FMT, SPW, 3>(n_act);
    }
}

// feat: the smallest feature class (see the kernel) that covers the launch
static mm_kernel_t mm_kernel(int fmt, int warps, int n_act, int feat) {
    if (fmt == MM_FMT_Q80) return mm_kernel_feat<MM_FMT_Q80, 1>(n_act, feat);
    if (fmt == MM_FMT_Q40) return mm_kernel_feat<MM_FMT_Q40, 2>(n_act, feat);
    if (fmt == MM_FMT_Q6K) return mm_kernel_feat<MM_FMT_Q6K, 1>(n_act, feat);
    if (n_act > 1 || warps == 8) return mm_kernel_feat<MM_FMT_Q4K, 2>(n_act, feat);
    return warps == 16 ? skn_matvec_mma<MM_FMT_Q4K, 1, 1, true, 3> : skn_matvec_mma<MM_FMT_Q4K, 4, 1, true, 3>;
}

static size_t mm_fixed_smem(int fmt, int nb, int n_act, int64_t rows_max, int nks, int warps) {
    // three or four rows: digit planes of one K super-chunk at a time; one or two: all of x
    const bool chunked = n_act > 2;
    const int ks = mm_ks(fmt), ksb = chunked ? (nb < ks ? nb : ks) : nb, nxs = chunked ? ks : nb;
    const size_t nbp = (size_t)(nxs + 3) / 4 * 4;
    return ((size_t)n_act * (MM_ND * (ksb * 256 + 32) + 64) + 127) / 128 * 128 + (size_t)n_act * nbp * 4 +
           (size_t)n_act * nxs * mm_xs(fmt) * 4 + (size_t)n_act * nbp * (MM_MAX_OUT * 4 + 4) + ((size_t)n_act * nbp + 15) / 16 * 16 +
           (size_t)n_act * rows_max * nks * warps * 4 + 64;
}

// most activation rows one launch can take for this shape (the digit planes and partial sums of
// every row sit in shared memory next to at least two ring stages)
static int mm_max_acts(const skn_ctx *ctx, int fmt, int64_t n_rows, int64_t n_cols) {
    const int nb = (int)(n_cols / 256);
    int64_t grid = ctx->sm_count;
    if (grid > n_rows) grid = n_rows;
    const int64_t rows_max = (n_rows + grid - 1) / grid + 2;
    for (int a = 4; a > 1; --a)
        if (mm_fixed_smem(fmt, nb, a, rows_max, (nb + mm_ks(fmt) - 1) / mm_ks(fmt), 8) + 2 * (size_t)(mm_stage_bytes(fmt) + 16) <= 200 * 1024)
            return a;
    return 1;
}

static cudaError_t mm_plan(skn_ctx *ctx, int fmt, int64_t n_rows, int64_t n_cols, int n_act, int feat, skn_mv_plan &pl, bool relaxed) {
    pl = skn_mv_plan{-1, 0, 0, 0, 0, 0};
    if (n_cols % 256 || n_cols > (1 << 18) || n_rows < 1 || n_act < 1 || n_act > 4) return cudaSuccess;
    const int nb = (int)(n_cols / 256);
    const int nks = (nb + mm_ks(fmt) - 1) / mm_ks(fmt);
    const size_t stage = (size_t)mm_stage_bytes(fmt) + 16;
    int64_t grid = ctx->sm_count;
    if (grid > n_rows) grid = n_rows;
    const int64_t rows_max = (n_rows + grid - 1) / grid + 2;      // + 2: interleaved launches round to even boundaries
    const int ntiles = (int)((rows_max + 15) / 16) * nks;
    static const int warps_env = env_int("SKN_MM_WARPS", 0);
    static const int nst_env = env_int("SKN_MM_NST", 0);
    static const int budget_env = env_int("SKN_MM_SMEM_KB", 0);
    int warps = warps_env > 0 ? warps_env : 8;
    warps = warps >= 16 ? 16 : (warps >= 8 ? 8 : 4);
    if (n_act > 1 || fmt != MM_FMT_Q4K) warps = 8;
    (void)relaxed;
    // few tiles: half an SM, so that the next launch's CTA is resident early; many tiles: a deeper
    // ring matters more than the neighbour
    const size_t budget = (size_t)(budget_env > 0 ? budget_env : (ntiles >= 6 ? 200 : 110)) * 1024;
    const size_t fixed = mm_fixed_smem(fmt, nb, n_act, rows_max, nks, warps);
    int nst = nst_env > 0 ? nst_env : (ntiles < 4 ? ntiles : 4);
    while (nst > 1 && fixed + (size_t)nst * stage > budget) --nst;
    if (nst < 2 && ntiles > 1 && budget_env <= 0) {
        // long rows or several activation rows: the digit planes leave no room for two stages in
        // half an SM; take all of it
        nst = ntiles < 4 ? ntiles : 4;
        while (nst > 1 && fixed + (size_t)nst * stage > 200 * 1024) --nst;
    }
    const size_t smem = fixed + (size_t)nst * stage;
    if (smem > 220 * 1024) return cudaSuccess;
    mm_kernel_t kern = mm_kernel(fmt, warps, n_act, feat);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return e;
    // all of the SM's L1 / shared memory as shared memory, so that two CTAs (consecutive launches) fit
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    // wg carries the ring depth, nch the compute warps; threads = compute warps + the producer warp
    pl.nch = warps; pl.wg = nst; pl.grid = (int)grid; pl.threads = (warps + 1) * 32; pl.smem = smem;
    pl.state = 1;
    return cudaSuccess;
}

// y[t][a] = W[t] . f(x[a]) (+ add[t]) for n <= 3 Q4_K / Q8_0 / Q4_0 tensors of one type, K and pitch and n_act <= 4
// activation rows (x rows K apart, outputs n_rows apart; add_per_act: add vectors n_rows apart,
// otherwise one bias for all rows).  Returns false when the shapes are not covered (nothing launched).
bool skn_mma_try_group(skn_ctx *ctx, int n, const skn_tensor *const *w, const float *x, float *const *y,
                       const float *const *add, const float *norm_gain, float norm_eps, const float *silu_u,
                       cudaStream_t stream, cudaError_t &err, bool swiglu, int n_act, bool add_per_act,
                       const skn_mv_exchange *xc, const skn_mv_rope *rope) {
    static const int enabled = env_int("SKN_MM", 1);
    err = cudaSuccess;
    const int fmt = mm_fmt_of(w[0]->type);
    if (!enabled || fmt < 0) return false;
    if (swiglu && (n != 2 || w[0]->n_rows != w[1]->n_rows)) return false;
    skn_mv_group grp = {};
    grp.norm_gain = norm_gain; grp.norm_eps = norm_eps; grp.silu_u = silu_u;
    grp.swiglu = swiglu ? 1 : 0;
    grp.n_act = n_act;
    if (rope) {
        if (n != 3 || swiglu || (xc && xc->push) || rope->head_dim < 2 || (rope->head_dim & 1) || w[0]->n_rows % rope->head_dim ||
            w[1]->n_rows != (int64_t)rope->n_kv_heads * rope->head_dim || w[2]->n_rows != w[1]->n_rows)
            return false;
        grp.rope_hd = rope->head_dim; grp.rope_cap = rope->capacity; grp.rope_nkv = rope->n_kv_heads; grp.rope_a0 = rope->seq0;
        grp.rope_len = rope->len_dev; grp.rope_start = rope->start_dev; grp.rope_kc = rope->k_cache; grp.rope_vc = rope->v_cache;
        grp.rope_log2theta = log2((double)rope->theta);
        grp.rope_inv_freq = rope->inv_freq;
    }
    if (xc && xc->view.world > 1) {
        if (xc->push && (swiglu || n != 1)) return false;
        grp.xc_world = xc->view.world; grp.xc_rank = xc->view.rank; grp.xc_cap = xc->view.capacity;
        grp.xc_push = xc->push ? 1 : 0; grp.xc_reduce = xc->reduce ? 1 : 0;
        for (int i = 0; i < SKN_COMM_MAX_WORLD; ++i) grp.xc_base[i] = xc->view.base[i];
        grp.xc_state = xc->view.state;
        grp.xc_wb = xc->writeback;
        // a slot holds n_act outputs of n_rows each (push) or n_act inputs of n_cols each (reduce)
        if (xc->push && (int64_t)n_act * w[0]->n_rows > xc->view.capacity) return false;
        if (xc->reduce && (int64_t)n_act * w[0]->n_cols > xc->view.capacity) return false;
    }
    int64_t tot = 0;
    for (int t = 0; t < n; ++t) {
        tot += w[t]->n_rows;
        grp.W[t] = w[t]->d_blocks; grp.y[t] = y[t]; grp.add[t] = add ? add[t] : nullptr; grp.n_end[t] = tot;
        grp.ystride[t] = w[t]->n_rows;
        grp.addstride[t] = add_per_act ? w[t]->n_rows : 0;
    }
    for (int t = n; t < 3; ++t) grp.n_end[t] = tot;
    grp.count = n;
    if (n_act < 1 || n_act > mm_max_acts(ctx, fmt, tot, w[0]->n_cols)) return false;
    skn_mv_plan pl = skn_mv_plan{0, 0, 0, 0, 0, 0};
    const int feat = ((xc && xc->view.world > 1) || silu_u) ? 3 : (rope ? 2 : ((norm_gain || swiglu) ? 1 : 0));
    const int32_t key_type = 1000 + 256 * feat + 32 * n_act + w[0]->type;       // distinct from the CUDA-core kernels' plans
    for (int i = 0; i < ctx->n_group_plans; ++i) {
        const skn_group_plan &c = ctx->group_plans[i];
        if (c.type == key_type && c.rows == tot && c.cols == w[0]->n_cols && c.relaxed == ctx->relaxed_order) { pl = c.pl; break; }
    }
    if (pl.state == 0) {
        err = mm_plan(ctx, fmt, tot, w[0]->n_cols, n_act, feat, pl, ctx->relaxed_order != 0);
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
    static const int pdl_max_mb = env_int("SKN_PDL_MAX_MB", 1 << 20);   // tuning knob: largest launch (weight bytes) that may start early
    cfg.attrs = attr;
    cfg.numAttrs = (pdl && tot * w[0]->pitch <= (int64_t)pdl_max_mb * (1 << 20)) ? 1 : 0;
    err = cudaLaunchKernelEx(&cfg, mm_kernel(fmt, pl.nch, n_act, feat), grp, w[0]->pitch, (int)w[0]->n_cols, pl.wg, x, ctx->d_status,
                             ctx->relaxed_order);
    return true;
}

int skn_mma_max_acts(const skn_ctx *ctx, int32_t type, int64_t n_rows_total, int64_t n_cols) {
    static const int enabled = env_int("SKN_MM", 1);
    const int fmt = mm_fmt_of(type);
    if (!enabled || fmt < 0 || n_cols % 256 || n_cols > (1 << 18) || n_rows_total < 1) return 0;
    return mm_max_acts(ctx, fmt, n_rows_total, n_cols);
}
