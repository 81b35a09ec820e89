// K2 for small batches (3 to 16 activation rows in ONE launch): Y[M, N] = X[M, K] . W_q[N, K]^T with the weights
// streamed from HBM exactly once.  Same arithmetic as skn_matvec_mma.cu -- exact integer dot products of 32-weight
// sub-blocks with the digit planes of the activations on the tensor cores (mma.sync m16n8k32, one MMA serves two
// activation rows), integer sub-block scales, fp32 across super-blocks -- but organised for many rows:
//
//   * x is prepared ONCE per launch by a kernel of its own (skn_xprep_kernel: one CTA per activation row applies
//     the optional RMSNorm or silu(x) * u, then writes the four digit planes, the block scales, the group sums and
//     the outlier records of every super-block to a scratch buffer), instead of once per CTA: with sixteen rows
//     the preparation would otherwise cost more than the products of a 4096-row projection;
//   * the weight rows are handled in groups of 16 (one MMA's worth); a CTA owns a run of groups; its 8 compute warps
//     are arranged as R row groups x KQ = 8 / R K-parts; a tile is R groups x KSB super-blocks, brought into a
//     shared-memory ring by ONE 2-D tiled TMA load per group (a box of 16 rows x the tile's bytes of each row; no
//     multicast): a bulk copy per row would be bound by the copy unit's request rate at these row lengths
//     (measured: 1 TB/s with 576-byte row copies);
//   * the digit planes of the current K chunk (KSB super-blocks of every activation row) sit in shared memory,
//     double-buffered: a second producer warp fetches the next chunk's planes from L2 while this chunk's tiles run,
//     and all row tiles of the CTA reuse them;
//   * per unit (16 weight rows x one super-block) the A fragments, block headers and scales are decoded once and
//     serve every pair of activation rows;
//   * partial sums live in shared memory per (activation row, weight row, K-part), each slot owned by one warp and
//     accumulated in tile order, so the result does not depend on timing.
#include "skn_mma_common.cuh"

#include <cuda.h>

// ---- prepared activations (global scratch) ------------------------------------------------------------------
// Laid out the way a CTA consumes them, so that the planes and block records of ONE K chunk (KSB super-blocks) of
// ALL activation rows are one contiguous piece and arrive in shared memory with a single bulk copy (a copy per row
// would be bound by the copy unit's request rate):
//   [chunk][row]{ planes [KSB][digit][RW_PLANE bytes] | block records [KSB][RW_META bytes] | padding }
// RW_PLANE = 256 digits + 32 bytes of padding (plane stride 8 words mod 32); a row's slot is padded to 16 words mod
// 32, which keeps the two activation rows of a pair on different banks.
constexpr int RW_PLANE = 256 + 32;
constexpr int RW_SB = MM_ND * RW_PLANE;         // 1152 bytes of planes per (row, super-block)
struct __align__(16) skn_xq_meta {
    float scale;                                // 2^(e-29) of the planes (NaN: the block is not finite)
    uint32_t ocnt, oidx, pad;                   // outliers: count (low byte), positions (one byte each)
    float oval[MM_MAX_OUT];                     // ... and values
    float xsum[16];                             // sums of 32 (first eight) or 16 activations, outliers excluded
};
constexpr int RW_META = (int)sizeof(skn_xq_meta);
static_assert(RW_META == 96, "meta record layout");
// bytes of one (chunk, activation row) slot
static __host__ __device__ inline int rw_slot_bytes(int KSB) {
    const int raw = KSB * (RW_SB + RW_META);
    return raw + ((64 - raw % 128) + 128) % 128;
}

// One CTA per activation row.  f(x) = x, x / rms(x) * gain, or silu(x) * u.
template <bool XS16>
__global__ void __launch_bounds__(1024)
skn_xprep_kernel(const float *__restrict__ x, int K, const float *__restrict__ gain, float eps, const float *__restrict__ silu_u,
                 uint8_t *__restrict__ xq, int KSB) {
    skn_pdl_launch_dependents();                // the product's CTAs may become resident and prefetch their weights
    skn_pdl_wait();                             // x is the previous kernel's output
    const int a = blockIdx.x, nb = K / 256, NA = gridDim.x;
    const int CH = rw_slot_bytes(KSB);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)a * K);
    const float4 *ur = silu_u ? reinterpret_cast<const float4 *>(silu_u + (size_t)a * K) : nullptr;
    __shared__ float s_ss[32];
    float rs = 1.f;
    if (gain) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < K / 4; i += blockDim.x) {
            const float4 v = __ldg(xr + i);
            ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) s_ss[warp] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < nw; ++w) tot += s_ss[w];
        rs = rsqrtf(tot / (float)K + eps);
    }
    auto load = [&](int f) {
        float4 v = __ldg(xr + f);
        if (ur) {
            const float4 u = __ldg(ur + f);
            v.x = v.x / (1.f + expf(-v.x)) * u.x; v.y = v.y / (1.f + expf(-v.y)) * u.y;
            v.z = v.z / (1.f + expf(-v.z)) * u.z; v.w = v.w / (1.f + expf(-v.w)) * u.w;
        }
        if (gain) {
            const float4 g = __ldg(reinterpret_cast<const float4 *>(gain) + f);
            v.x = v.x * rs * g.x; v.y = v.y * rs * g.y; v.z = v.z * rs * g.z; v.w = v.w * rs * g.w;
        }
        return v;
    };
    for (int sb = warp; sb < nb; sb += nw) {
        const float4 v0 = load(sb * 64 + lane), v1 = load(sb * 64 + 32 + lane);
        uint8_t *slot = xq + ((size_t)(sb / KSB) * NA + a) * CH;
        skn_xq_meta *m = reinterpret_cast<skn_xq_meta *>(slot + (size_t)KSB * RW_SB) + sb % KSB;
        mm_digitize<XS16>(v0, v1, 0, lane, slot + (size_t)(sb % KSB) * RW_SB, RW_PLANE, &m->scale, m->xsum, m->oval, &m->oidx,
                          reinterpret_cast<uint8_t *>(&m->ocnt));
    }
}

// ---- the product -------------------------------------------------------------------------------------------
struct skn_rows_geom {
    int R, KSB;             // row groups per tile (2 or 4), super-blocks per tile; KQ = 8 / R K-parts of KSB / KQ = 1 super-block
    int nst;                // ring depth
    int wrow;               // bytes of a weight row in a stage = inner extent of the TMA box (8 or 24 words mod 32)
    int prow;               // bytes of an activation row's slot in a plane buffer (rw_slot_bytes(KSB))
};

// what the launch multiplies: up to three tensors of one type, K and pitch (rows of tensor t: n_rows[t]); their
// 16-row groups are numbered through (gcum[t] = groups before tensor t), or interleaved gate / up for the SwiGLU form
struct skn_rows_args {
    int count, swiglu, n_act;
    int gcum[4];
    int64_t n_rows[3];
    float *y[3];
    const float *add[3];
    int64_t ystride[3], addstride[3];
};

constexpr int RW_W = 8;     // compute warps

template <int FMT> struct RwFmt;
template <> struct RwFmt<MM_FMT_Q4K> { static constexpr int SB_BYTES = 144; };
template <> struct RwFmt<MM_FMT_Q40> { static constexpr int SB_BYTES = 144; };
template <> struct RwFmt<MM_FMT_Q80> { static constexpr int SB_BYTES = 272; };

// group j of the launch -> tensor and first row inside it
__device__ __forceinline__ int rw_group(const skn_rows_args &ar, int j, int &local0) {
    if (ar.swiglu) {
        local0 = 16 * (j >> 1);
        return j & 1;
    }
    const int tt = (j >= ar.gcum[1] ? 1 : 0) + ((ar.count > 2 && j >= ar.gcum[2]) ? 1 : 0);
    local0 = 16 * (j - ar.gcum[tt]);
    return tt;
}

// CTA b's run [gb, ge) of the launch's G sixteen-row groups; the SwiGLU form keeps whole gate / up pairs together
// (even boundaries).  One definition for the kernel and for the host-side query of the layout.
__host__ __device__ __forceinline__ void rw_cta_groups(int b, int grid, int G, bool swiglu, int &gb, int &ge) {
    const int even = swiglu ? ~1 : ~0;
    gb = (int)((int64_t)b * G / grid) & even;
    ge = (b + 1 == grid) ? G : ((int)((int64_t)(b + 1) * G / grid) & even);
}

// 2-D tiled TMA load (no multicast) of a box at element coordinates (x: 8-byte units along the row, y: row)
__device__ __forceinline__ void rw_tma_load_2d(uint32_t dst_smem, const CUtensorMap *tmap, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst_smem),
                 "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(skn_smem_u32(bar))
                 : "memory");
}

template <int FMT, int NP>
__global__ void __launch_bounds__((RW_W + 2) * 32, NP == 2 ? 2 : 1)
skn_matvec_rows(const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1, const __grid_constant__ CUtensorMap tm2,
                const skn_rows_args ar, int K, const skn_rows_geom geo, const uint8_t *__restrict__ xq, int32_t *__restrict__ status) {
    constexpr int SBB = RwFmt<FMT>::SB_BYTES;
    constexpr int NAMAX = 2 * NP;
    constexpr int NPH = NP < 4 ? NP : 4;        // pairs per half-pass over a unit
    const int R = geo.R, KQ = RW_W / R, KSB = geo.KSB, nst = geo.nst;
    const int WROW = geo.wrow, PROW = geo.prow, WSTAGE = 16 * R * WROW;
    const uint32_t MROW = (uint32_t)PROW;               // the block records of consecutive activation rows are a slot apart too
    const bool f_swiglu = ar.swiglu != 0;
    const int NA = ar.n_act;
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nb = K / 256;
    const int nks = (nb + KSB - 1) / KSB;

    // this CTA's run of 16-row groups (whole gate / up pairs in the SwiGLU form)
    const int G = ar.gcum[3];
    int gb, ge;
    rw_cta_groups((int)blockIdx.x, (int)gridDim.x, G, f_swiglu, gb, ge);
    const int ng = ge - gb;
    // A CTA without groups leaves at once (every thread: no barrier has been touched yet).  The SwiGLU form rounds its
    // boundaries to whole gate / up pairs, so with fewer than two groups per CTA some CTAs get none; such a CTA used to
    // stay, and its plane producer waited for compute warps that never take a plane until the bounded wait ran out
    // (two seconds per launch: 224 groups on 148 CTAs, the gate / up shard of an 8-way tensor-parallel decoder).
    if (ng <= 0) return;
    const int rows = 16 * ng;
    const int nrt = (ng + R - 1) / R;
    const int ntiles = nrt * nks;               // tile i: K chunk i / nrt, row tile i % nrt

    // shared memory: ring | plane buffers [2][row] (planes + block records) | partials [row][weight row][KQ] | barriers
    uint8_t *ring = smem;
    uint8_t *pbuf = ring + (size_t)nst * WSTAGE;
    float *part = reinterpret_cast<float *>(pbuf + 2 * (size_t)NA * PROW);
    uint64_t *full = reinterpret_cast<uint64_t *>(part + ((size_t)NA * rows * KQ + 3) / 4 * 4);
    uint64_t *empty = full + nst;
    uint64_t *pfull = empty + nst;
    uint64_t *pempty = pfull + 2;

    if (warp == RW_W) {
        if (lane < nst) {
            skn_mbar_init(&full[lane], 1);
            skn_mbar_init(&empty[lane], RW_W);
        }
        if (lane < 2) {
            skn_mbar_init(&pfull[lane], 1);
            skn_mbar_init(&pempty[lane], RW_W);
        }
        skn_fence_mbar_init();
    }
    __syncthreads();

    if (warp == RW_W) {
        // ---- weight producer: one box (16 rows x the chunk's bytes) per group of a tile, all on the stage's full barrier;
        // rows past a tensor's end and bytes past a row's end arrive as zeros ----
        if (lane == 0) {
            bool failed = false;
            int ks = 0, rt = 0, stg = 0;
            uint32_t par = 0;
            const uint32_t ring_s = skn_smem_u32(ring);
            for (int i = 0; i < ntiles; ++i) {
                if (i >= nst && !failed && !skn_mbar_wait(&empty[stg], par ^ 1u)) {
                    failed = true;
                    atomicExch(status, SKN_ERR_TIMEOUT);
                }
                const int ngt = min(R, ng - rt * R);
                skn_mbar_expect_tx(&full[stg], (uint32_t)ngt * 16u * (uint32_t)WROW);
                skn_fence_proxy_async();
                for (int r = 0; r < ngt; ++r) {
                    int local0;
                    const int tt = rw_group(ar, gb + rt * R + r, local0);
                    const CUtensorMap *tm = tt == 0 ? &tm0 : (tt == 1 ? &tm1 : &tm2);
                    rw_tma_load_2d(ring_s + (uint32_t)stg * WSTAGE + (uint32_t)(16 * r) * WROW, tm, ks * KSB * (SBB / 8), local0, &full[stg]);
                }
                if (i == nst - 1 || i == ntiles - 1) skn_pdl_launch_dependents();   // the first ring-full is on its way
                if (++rt == nrt) { rt = 0; ++ks; }
                if (++stg == nst) { stg = 0; par ^= 1u; }
            }
        }
        return;
    }
    if (warp == RW_W + 1) {
        // ---- plane producer: the planes and block records of K chunk c (all activation rows: one contiguous piece,
        // one copy) go to buffer c & 1 as soon as the compute warps have left chunk c - 2; they are the preparation
        // kernel's output ----
        skn_pdl_wait();
        if (lane == 0) {
            bool failed = false;
            const uint32_t bytes = (uint32_t)NA * (uint32_t)PROW;
            for (int c = 0; c < nks; ++c) {
                const int buf = c & 1;
                if (c >= 2 && !failed && !skn_mbar_wait(&pempty[buf], (uint32_t)((c >> 1) - 1) & 1u)) {
                    failed = true;
                    atomicExch(status, SKN_ERR_TIMEOUT);
                }
                skn_mbar_expect_tx(&pfull[buf], bytes);
                skn_fence_proxy_async();
                skn_bulk_g2s(pbuf + (size_t)buf * bytes, xq + (size_t)c * bytes, bytes, &pfull[buf]);
            }
        }
        return;
    }

    // ---- compute warps ----
    skn_pdl_wait();                             // `add` and y belong to earlier launches of the stream
    const int rg = warp % R, kq = warp / R;
    const uint32_t ring_s = skn_smem_u32(ring), pbuf_s = skn_smem_u32(pbuf);
    const int bcol_row = g & 1, bcol_dig = g >> 1;
    const float inv_dw = (t == 0) ? 1.f : ((t == 1) ? (1.f / 256.f) : ((t == 2) ? (1.f / 65536.f) : (1.f / 16777216.f)));
    const float dw = (t == 0) ? 1.f : ((t == 1) ? 256.f : ((t == 2) ? 65536.f : 16777216.f));
    bool failed = false;
    int ks = 0, rt = 0, stg = 0;
    uint32_t par = 0;
    for (int i = 0; i < ntiles; ++i) {
        const int buf = ks & 1;
        if (rt == 0 && !failed && !skn_mbar_wait(&pfull[buf], (uint32_t)(ks >> 1) & 1u)) {
            failed = true;
            atomicExch(status, SKN_ERR_TIMEOUT);
        }
        if (!failed && !skn_mbar_wait(&full[stg], par)) {
            failed = true;
            atomicExch(status, SKN_ERR_TIMEOUT);
        }
        int nsb = nb - ks * KSB;
        nsb = nsb > KSB ? KSB : nsb;
        const int gi = rt * R + rg;             // this warp's group among the CTA's
        const bool active = gi < ng && kq < nsb;
        // digit t of (activation rows 2 ap, 2 ap + 1) x (weight rows g, g + 8) of this warp's super-block, in units of
        // 2^(8 t): the offset terms and outlier products are folded in with that power of two divided out
        float accA[NP][2], accB[NP][2];
#pragma unroll
        for (int ap = 0; ap < NP; ++ap) accA[ap][0] = accA[ap][1] = accB[ap][0] = accB[ap][1] = 0.f;
        if (active) {
            const int sb = kq;
            const uint32_t ba = ring_s + (uint32_t)stg * WSTAGE + (uint32_t)(16 * rg + g) * WROW + sb * SBB, bb = ba + 8 * WROW;
            const uint32_t pl0 = pbuf_s + (uint32_t)(buf * NA) * PROW + (uint32_t)sb * RW_SB;
            const uint32_t mt0 = pbuf_s + (uint32_t)(buf * NA) * PROW + (uint32_t)KSB * RW_SB + (uint32_t)sb * RW_META;
            // outlier counts per activation row (almost always zero): loaded now, looked at after the MMAs
            int ocn[NAMAX];
#pragma unroll
            for (int a = 0; a < NAMAX; ++a) ocn[a] = (a < NA) ? (int)(mm_lds32(mt0 + (uint32_t)a * MROW + 4) & 0xFFu) : 0;
            // The pairs are taken four at a time (NPH): per step all B fragments are loaded, then all MMAs are
            // issued back to back (their latency is covered by the batch itself), then the integer multiply-adds.
#pragma unroll
            for (int hf = 0; hf < NP / NPH; ++hf) {
                if (8 * hf >= NA) break;                             // warp-uniform: no rows in this half
                // this lane's B column of every pair: activation row 2 ap + (g & 1), digit g >> 1
                uint32_t bsrc[NPH];
#pragma unroll
                for (int ap = 0; ap < NPH; ++ap) {
                    const int arow = min(2 * (NPH * hf + ap) + bcol_row, NA - 1);
                    bsrc[ap] = pl0 + (uint32_t)(arow * PROW + bcol_dig * RW_PLANE) + (FMT == MM_FMT_Q40 ? 4 * t : 8 * t);
                }
                if constexpr (FMT == MM_FMT_Q4K) {
                    const uint4 ha = mm_lds128(ba), hb = mm_lds128(bb);
                    // 6-bit scales as bytes: word 0 = sub-blocks 0..3, word 1 = sub-blocks 4..7
                    const uint32_t sa[2] = {ha.y & 0x3F3F3F3Fu, (ha.w & 0x0F0F0F0Fu) | ((ha.y >> 2) & 0x30303030u)};
                    const uint32_t sq[2] = {hb.y & 0x3F3F3F3Fu, (hb.w & 0x0F0F0F0Fu) | ((hb.y >> 2) & 0x30303030u)};
                    int lo[NPH][4], hi[NPH][4];     // [pair][weight row g col 2t, col 2t+1, weight row g+8 col 2t, col 2t+1]
#pragma unroll
                    for (int ap = 0; ap < NPH; ++ap)
#pragma unroll
                        for (int c = 0; c < 4; ++c) lo[ap][c] = hi[ap][c] = 0;
                    uint2 bl[NPH], bh[NPH];         // B fragments of the step: sub-blocks 2p (low nibbles) and 2p + 1
                    auto load_b = [&](int p) {
#pragma unroll
                        for (int ap = 0; ap < NPH; ++ap) {
                            // (unconditional: a pair without a second row reads its first row again, those columns are never stored)
                            bl[ap] = mm_lds64(bsrc[ap] + (2 * p) * 32);
                            bh[ap] = mm_lds64(bsrc[ap] + (2 * p + 1) * 32);
                        }
                    };
                    load_b(0);
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        const uint2 wa = mm_lds64(ba + 16 + 32 * p + 8 * t);
                        const uint2 wb = mm_lds64(bb + 16 + 32 * p + 8 * t);
                        const uint32_t al0 = wa.x & 0x0F0F0F0Fu, al1 = wb.x & 0x0F0F0F0Fu, al2 = wa.y & 0x0F0F0F0Fu, al3 = wb.y & 0x0F0F0F0Fu;
                        const uint32_t ah0 = wa.x & 0xF0F0F0F0u, ah1 = wb.x & 0xF0F0F0F0u, ah2 = wa.y & 0xF0F0F0F0u, ah3 = wb.y & 0xF0F0F0F0u;
                        int c[NPH][4], h[NPH][4];
#pragma unroll
                        for (int ap = 0; ap < NPH; ++ap) {
                            skn_mma_u8s8(c[ap], al0, al1, al2, al3, bl[ap].x, bl[ap].y);
                            skn_mma_u8s8(h[ap], ah0, ah1, ah2, ah3, bh[ap].x, bh[ap].y);
                        }
                        if (p < 3) load_b(p + 1);                    // next step's fragments arrive under the multiply-adds
                        const int s0a = mm_byte_i(sa[p >> 1], 2 * (p & 1)), s1a = mm_byte_i(sa[p >> 1], 2 * (p & 1) + 1);
                        const int s0b = mm_byte_i(sq[p >> 1], 2 * (p & 1)), s1b = mm_byte_i(sq[p >> 1], 2 * (p & 1) + 1);
#pragma unroll
                        for (int ap = 0; ap < NPH; ++ap) {
                            lo[ap][0] += s0a * c[ap][0]; lo[ap][1] += s0a * c[ap][1]; lo[ap][2] += s0b * c[ap][2]; lo[ap][3] += s0b * c[ap][3];
                            hi[ap][0] += s1a * h[ap][0]; hi[ap][1] += s1a * h[ap][1]; hi[ap][2] += s1b * h[ap][2]; hi[ap][3] += s1b * h[ap][3];
                        }
                    }
                    const float2 da = __half22float2(*reinterpret_cast<const __half2 *>(&ha.x));   // {d, dmin} of row g
                    const float2 db = __half22float2(*reinterpret_cast<const __half2 *>(&hb.x));   // ... of row g + 8
                    // min term: this lane covers weight row g + 8 (t & 1) and sub-blocks 4 (t >> 1) .. + 3
                    const uint4 hm = (t & 1) ? hb : ha;
                    const uint32_t mw = (t & 2) ? (((hm.w >> 4) & 0x0F0F0F0Fu) | ((hm.z >> 2) & 0x30303030u)) : (hm.z & 0x3F3F3F3Fu);
                    const float m0 = mm_byte_f(mw, 0), m1 = mm_byte_f(mw, 1), m2 = mm_byte_f(mw, 2), m3 = mm_byte_f(mw, 3);
                    const float dmin = ((t & 1) ? db.y : da.y) * inv_dw;
                    const float da16 = da.x * 0.0625f, db16 = db.x * 0.0625f;
#pragma unroll
                    for (int ap = 0; ap < NPH; ++ap) {
                        const int pr = NPH * hf + ap;
                        const int ra = min(2 * pr, NA - 1), rb = min(2 * pr + 1, NA - 1);
                        const uint32_t ma = mt0 + (uint32_t)ra * MROW, mb = mt0 + (uint32_t)rb * MROW;
                        const float sgA = mm_lds32f(ma), sgB = mm_lds32f(mb);
                        accA[pr][0] = fmaf(da16 * sgA, (float)(lo[ap][0] * 16 + hi[ap][0]), accA[pr][0]);
                        accA[pr][1] = fmaf(db16 * sgA, (float)(lo[ap][2] * 16 + hi[ap][2]), accA[pr][1]);
                        accB[pr][0] = fmaf(da16 * sgB, (float)(lo[ap][1] * 16 + hi[ap][1]), accB[pr][0]);
                        accB[pr][1] = fmaf(db16 * sgB, (float)(lo[ap][3] * 16 + hi[ap][3]), accB[pr][1]);
                        const float4 xa = mm_lds128f(ma + 32 + 16u * (uint32_t)(t >> 1)), xb = mm_lds128f(mb + 32 + 16u * (uint32_t)(t >> 1));
                        const float va = dmin * fmaf(m3, xa.w, fmaf(m2, xa.z, fmaf(m1, xa.y, m0 * xa.x)));
                        const float vb = dmin * fmaf(m3, xb.w, fmaf(m2, xb.z, fmaf(m1, xb.y, m0 * xb.x)));
                        if (t & 1) { accA[pr][1] -= va; accB[pr][1] -= vb; }
                        else { accA[pr][0] -= va; accB[pr][0] -= vb; }
                    }
                } else {
                    // eight 32-weight blocks, one MMA each; block j of a row starts 2-byte aligned, its
                    // quants are word aligned for odd j and two bytes off for even j
                    constexpr int BB = SBB / 8;             // 34 (Q8_0) or 18 (Q4_0)
                    float sgA[NPH], sgB[NPH];
#pragma unroll
                    for (int ap = 0; ap < NPH; ++ap) {
                        const int pr = NPH * hf + ap;
                        const int ra = min(2 * pr, NA - 1), rb = min(2 * pr + 1, NA - 1);
                        sgA[ap] = mm_lds32f(mt0 + (uint32_t)ra * MROW);
                        sgB[ap] = mm_lds32f(mt0 + (uint32_t)rb * MROW);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint32_t a0, a1, a2, a3;                    // rows g / g+8, k 0..15 / 16..31 of the fragment
                        const float d_a = mm_lds_half(ba + BB * j), d_b = mm_lds_half(bb + BB * j);
                        if constexpr (FMT == MM_FMT_Q80) {
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
                        int c[NPH][4];
#pragma unroll
                        for (int ap = 0; ap < NPH; ++ap) {
                            uint32_t b0, b1;
                            if constexpr (FMT == MM_FMT_Q80) {
                                const uint2 b = mm_lds64(bsrc[ap] + j * 32);
                                b0 = b.x; b1 = b.y;
                            } else {
                                b0 = mm_lds32(bsrc[ap] + j * 32);
                                b1 = mm_lds32(bsrc[ap] + j * 32 + 16);
                            }
                            if constexpr (FMT == MM_FMT_Q80) skn_mma_s8s8(c[ap], a0, a1, a2, a3, b0, b1);
                            else skn_mma_u8s8(c[ap], a0, a1, a2, a3, b0, b1);
                        }
                        // |c| < 2^22: converted through the mantissa of 1.5 * 2^23 + c (no conversion pipe)
#pragma unroll
                        for (int ap = 0; ap < NPH; ++ap) {
                            const int pr = NPH * hf + ap;
                            float f[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) f[i] = __int_as_float(c[ap][i] + 0x4B400000) - 12582912.f;
                            accA[pr][0] = fmaf(d_a * sgA[ap], f[0], accA[pr][0]);
                            accA[pr][1] = fmaf(d_b * sgA[ap], f[2], accA[pr][1]);
                            accB[pr][0] = fmaf(d_a * sgB[ap], f[1], accB[pr][0]);
                            accB[pr][1] = fmaf(d_b * sgB[ap], f[3], accB[pr][1]);
                        }
                    }
                    if constexpr (FMT == MM_FMT_Q40) {
                        // offset term 8 * d * sum(x) per block: this lane covers weight row g + 8 (t & 1) and blocks 4 (t >> 1) .. + 3
                        const uint32_t hrow = (t & 1) ? bb : ba;
                        const int j0 = 4 * (t >> 1);
                        const float d0 = mm_lds_half(hrow + BB * j0), d1 = mm_lds_half(hrow + BB * (j0 + 1));
                        const float d2 = mm_lds_half(hrow + BB * (j0 + 2)), d3 = mm_lds_half(hrow + BB * (j0 + 3));
                        const float e8 = 8.f * inv_dw;
#pragma unroll
                        for (int ap = 0; ap < NPH; ++ap) {
                            const int pr = NPH * hf + ap;
                            const int ra = min(2 * pr, NA - 1), rb = min(2 * pr + 1, NA - 1);
                            const float4 xa = mm_lds128f(mt0 + (uint32_t)ra * MROW + 32 + 4u * (uint32_t)j0);
                            const float4 xb = mm_lds128f(mt0 + (uint32_t)rb * MROW + 32 + 4u * (uint32_t)j0);
                            const float va = e8 * fmaf(d3, xa.w, fmaf(d2, xa.z, fmaf(d1, xa.y, d0 * xa.x)));
                            const float vb = e8 * fmaf(d3, xb.w, fmaf(d2, xb.z, fmaf(d1, xb.y, d0 * xb.x)));
                            if (t & 1) { accA[pr][1] -= va; accB[pr][1] -= vb; }
                            else { accA[pr][0] -= va; accB[pr][0] -= vb; }
                        }
                    }
                }
            }
            // outliers (rare): lane t multiplies outlier t with the weights of rows g and g + 8; the product joins
            // this lane's digit accumulator with the digit's power of two divided out
#pragma unroll
            for (int a = 0; a < NAMAX; ++a) {
                if (ocn[a] != 0) {                                   // warp-uniform
                    if (t < ocn[a]) {
                        const uint32_t mt = mt0 + (uint32_t)a * MROW;
                        const int k = (int)mm_lds8(mt + 8 + (uint32_t)t);
                        const float xv = mm_lds32f(mt + 16 + 4u * (uint32_t)t) * inv_dw;
                        const float wa = mm_weight_at<FMT>(ba, k) * xv, wb = mm_weight_at<FMT>(bb, k) * xv;
                        if (a & 1) { accB[a >> 1][0] += wa; accB[a >> 1][1] += wb; }
                        else { accA[a >> 1][0] += wa; accA[a >> 1][1] += wb; }
                    }
                }
            }
        }
        __syncwarp();      // every lane has read its share of the stage
        if (lane == 0) {
            skn_mbar_arrive(&empty[stg]);
            if (rt == nrt - 1) skn_mbar_arrive(&pempty[buf]);       // the last tile of this K chunk: its planes are free
        }
        // ---- tile epilogue: sum the four digits (lanes t = 0..3); lane t then owns one of the pair's four values
        // (t = 0, 1: first activation row, weight rows g, g + 8; t = 2, 3: second activation row) and accumulates it
        // into this warp's slot: all old values are read before any is written
        if (gi < ng) {
            float mine[NP];
#pragma unroll
            for (int ap = 0; ap < NP; ++ap) {
                float e[4] = {accA[ap][0] * dw, accA[ap][1] * dw, accB[ap][0] * dw, accB[ap][1] * dw};
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    e[v] += __shfl_xor_sync(0xffffffffu, e[v], 1);
                    e[v] += __shfl_xor_sync(0xffffffffu, e[v], 2);
                }
                mine[ap] = (t == 0) ? e[0] : ((t == 1) ? e[1] : ((t == 2) ? e[2] : e[3]));
            }
            const int lr = 16 * gi + g + 8 * (t & 1);
            float *pb = part + ((size_t)(t >> 1) * rows + lr) * KQ + kq;      // slot of pair 0; pair ap is 2 * ap activation rows on
            const size_t pstride = (size_t)2 * rows * KQ;
            float old[NP];
#pragma unroll
            for (int ap = 0; ap < NP; ++ap) old[ap] = (ks != 0 && 2 * ap + (t >> 1) < NA) ? pb[ap * pstride] : 0.f;
#pragma unroll
            for (int ap = 0; ap < NP; ++ap)
                if (2 * ap + (t >> 1) < NA) pb[ap * pstride] = old[ap] + mine[ap];
        }
        if (++rt == nrt) { rt = 0; ++ks; }
        if (++stg == nst) { stg = 0; par ^= 1u; }
    }
    mm_bar_sync(1, RW_W * 32);
    // ---- outputs: K-parts in index order (every slot was written: a warp without a super-block wrote zeros), then
    // bias / residual or the SwiGLU product
    for (int idx = threadIdx.x; idx < NA * rows; idx += RW_W * 32) {
        const int a = idx / rows, lr = idx - a * rows;
        int local0;
        const int tt = rw_group(ar, gb + (lr >> 4), local0);
        const int64_t local = local0 + (lr & 15);
        if (local >= ar.n_rows[tt]) continue;
        const float *p = part + ((size_t)a * rows + lr) * KQ;
        float s = p[0];
        for (int q = 1; q < KQ; ++q) s += p[q];
        if (f_swiglu) {
            if (tt == 0) {
                const float *pu = p + 16 * KQ;  // the `up` rows of these columns are the next group
                float up = pu[0];
                for (int q = 1; q < KQ; ++q) up += pu[q];
                ar.y[0][(size_t)a * ar.ystride[0] + local] = s / (1.f + expf(-s)) * up;
            }
        } else {
            if (ar.add[tt]) s += ar.add[tt][(size_t)a * ar.addstride[tt] + local];
            ar.y[tt][(size_t)a * ar.ystride[tt] + local] = s;
        }
    }
}

// ---- host side ----------------------------------------------------------------------------------------------
typedef void (*rw_kernel_t)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const skn_rows_args, int, const skn_rows_geom,
                            const uint8_t *, int32_t *);

template <int FMT>
static rw_kernel_t rw_kernel_np(int np) {
    switch (np) {
    case 2: return skn_matvec_rows<FMT, 2>;
    case 4: return skn_matvec_rows<FMT, 4>;
    default: return skn_matvec_rows<FMT, 8>;
    }
}

static rw_kernel_t rw_kernel(int fmt, int np) {
    switch (fmt) {
    case MM_FMT_Q4K: return rw_kernel_np<MM_FMT_Q4K>(np);
    case MM_FMT_Q40: return rw_kernel_np<MM_FMT_Q40>(np);
    default: return rw_kernel_np<MM_FMT_Q80>(np);
    }
}

static int rw_fmt_of(int32_t type) {
    switch (type) {
    case SKN_TYPE_Q4_K: return MM_FMT_Q4K;
    case SKN_TYPE_Q8_0: return MM_FMT_Q80;
    case SKN_TYPE_Q4_0: return MM_FMT_Q40;
    default: return -1;
    }
}

struct rw_plan {
    skn_rows_geom geo;
    int grid, np;
    size_t smem;
    bool ok;
};

// n_groups: 16-row groups of the launch (all tensors)
static rw_plan rw_make_plan(const skn_ctx *ctx, int fmt, int64_t n_groups, int64_t n_cols, int n_act) {
    rw_plan pl = {};
    const int sbb = fmt == MM_FMT_Q80 ? 272 : 144;
    const int nb = (int)(n_cols / 256);
    const int np = n_act <= 4 ? 2 : (n_act <= 8 ? 4 : 8);
    // CTAs: one per SM; more when a CTA's partial sums would not fit (very tall matrices)
    // (up to four rows: two CTAs per SM, twice the warps to hide the tensor-core and shared-memory latencies)
    const int per_sm = np == 2 ? 2 : 1;
    const size_t budget = (np == 2 ? 105 : 210) * 1024;
    int64_t grid = (int64_t)ctx->sm_count * per_sm;
    while ((n_groups + grid - 1) / grid > 28) grid += ctx->sm_count;
    if (grid > n_groups) grid = n_groups;
    const int64_t gmax = (n_groups + grid - 1) / grid + 1;         // (+ 1: SwiGLU launches round to even boundaries)
    // many groups per CTA: 4 row groups x 2 K-parts per tile; few: 2 x 4, so that all warps have work
    const int R = gmax > 3 ? 4 : 2, KQ = RW_W / R, KSB = KQ;
    if (KSB > nb && nb < 2) return pl;
    int wrow = KSB * sbb;                                           // row stride 8 or 24 words mod 32: conflict-free fragment loads
    while ((wrow / 4) % 32 != 8 && (wrow / 4) % 32 != 24) wrow += 16;
    if (wrow / 8 > 256) return pl;
    const int prow = rw_slot_bytes(KSB);
    const size_t fixed = 2 * (size_t)n_act * prow +
                         ((size_t)n_act * 16 * gmax * KQ + 3) / 4 * 4 * sizeof(float) + 256;
    const size_t stage = (size_t)16 * R * wrow;
    int nst = 6;
    while (nst > 2 && fixed + (size_t)nst * stage > budget) --nst;
    if (fixed + (size_t)nst * stage > budget) return pl;
    pl.geo = skn_rows_geom{R, KSB, nst, wrow, prow};
    pl.grid = (int)grid;
    pl.np = np;
    pl.smem = fixed + (size_t)nst * stage;
    pl.ok = true;
    return pl;
}

// CTAs of the launch: the plan's, or one per gate / up pair when the SwiGLU form would otherwise leave CTAs without
// a pair (the plan's partial-sum space covers the two or three groups a CTA then owns)
static int rw_launch_grid(const rw_plan &pl, int64_t G, bool swiglu) {
    return (swiglu && pl.grid > G / 2) ? (int)(G / 2 > 0 ? G / 2 : 1) : pl.grid;
}

typedef CUresult (*rw_encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                       const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map of a weight's raw blocks as [n_rows][pitch / 8] 8-byte units: boxes of 16 rows x `wrow` bytes, no swizzle,
// rows past the end and bytes past the pitch read as zeros.  Cached in the tensor per box width.
static cudaError_t rw_tensor_map(const skn_tensor *w, int wrow, CUtensorMap *out) {
    skn_tensor *wm = const_cast<skn_tensor *>(w);
    for (int i = 0; i < 2; ++i)
        if (wm->rows_tmap_wrow[i] == wrow) {
            memcpy(out, wm->rows_tmap[i], sizeof(CUtensorMap));
            return cudaSuccess;
        }
    static rw_encode_tiled_fn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess) return e;
        if (!fn || q != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
        encode = (rw_encode_tiled_fn)fn;
    }
    const cuuint64_t gdim[2] = {(cuuint64_t)(w->pitch / 8), (cuuint64_t)w->n_rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)w->pitch};
    const cuuint32_t box[2] = {(cuuint32_t)(wrow / 8), 16u};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, w->d_blocks, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    const int slot = wm->rows_tmap_wrow[0] == 0 ? 0 : 1;
    memcpy(wm->rows_tmap[slot], out, sizeof(CUtensorMap));
    wm->rows_tmap_wrow[slot] = wrow;
    return cudaSuccess;
}

static int64_t rw_groups(int n, const skn_tensor *const *w) {
    int64_t gsum = 0;
    for (int t = 0; t < n; ++t) gsum += (w[t]->n_rows + 15) / 16;
    return gsum;
}

// most activation rows one launch of this kernel takes for these tensors: 16, 8, 4 or 0 (type or shape not covered)
int skn_rows_max_acts(const skn_ctx *ctx, int n, const skn_tensor *const *w) {
    const int fmt = rw_fmt_of(w[0]->type);
    const int64_t K = w[0]->n_cols;
    if (fmt < 0 || K % 256 || K < 512 || K > (1 << 18) || (w[0]->pitch % 16) || w[0]->n_rows < 1) return 0;
    const int64_t G = rw_groups(n, w);
    // Measured on 4096-column Q4_K tensors: this kernel is ahead of four-row passes of the in-kernel-preparation
    // kernel up to about eight 16-row groups per CTA (4096 to 14336 rows: 21.6 against 40.3 us and 67.5 against 75.2
    // us at sixteen rows) and behind beyond (28672 rows: 136 against 117 us), where that kernel's preparation of x
    // is amortised over many rows per CTA.
    if ((G + ctx->sm_count - 1) / ctx->sm_count > 8) return 0;
    for (int na = 16; na >= 4; na >>= 1)
        if (rw_make_plan(ctx, fmt, G, K, na).ok) return na;
    return 0;
}

// Y[t][m] = W[t] . f(x[m]) (+ add[t]) for n <= 3 tensors of one type, K and pitch and 3 <= M <= skn_rows_max_acts()
// activation rows in one launch pair (preparation of x, then the product); f: identity, RMSNorm (norm_gain) or
// silu(x) * silu_u; swiglu: W[0] = gate, W[1] = up, y[0] receives silu(gate . x) * (up . x).  Returns false when
// the tensors are not covered (nothing launched).
bool skn_rows_try_group(skn_ctx *ctx, int n, const skn_tensor *const *w, const float *x, int M, float *const *y,
                        const float *const *add, bool add_per_act, const float *norm_gain, float norm_eps, const float *silu_u,
                        bool swiglu, cudaStream_t stream, cudaError_t &err) {
    err = cudaSuccess;
    const int fmt = rw_fmt_of(w[0]->type);
    if (fmt < 0 || M < 3 || M > 16 || n < 1 || n > 3) return false;
    if (swiglu && (n != 2 || w[0]->n_rows != w[1]->n_rows)) return false;
    const int64_t K = w[0]->n_cols;
    if (K % 256 || K < 512 || K > (1 << 18) || (w[0]->pitch % 16)) return false;
    skn_rows_args ar = {};
    int64_t G = 0;
    for (int t = 0; t < n; ++t) {
        if (w[t]->type != w[0]->type || w[t]->n_cols != K || w[t]->pitch != w[0]->pitch || w[t]->n_rows < 1) return false;
        ar.gcum[t] = (int)G;
        G += (w[t]->n_rows + 15) / 16;
        ar.n_rows[t] = w[t]->n_rows;
        ar.y[t] = y[t]; ar.add[t] = add ? add[t] : nullptr;
        ar.ystride[t] = w[t]->n_rows;
        ar.addstride[t] = add_per_act ? w[t]->n_rows : 0;
    }
    for (int t = n; t < 4; ++t) ar.gcum[t] = (int)G;
    if (G < 1 || G > (1 << 24)) return false;
    ar.count = n;
    ar.swiglu = swiglu ? 1 : 0;
    ar.n_act = M;
    const rw_plan pl = rw_make_plan(ctx, fmt, G, K, M);
    if (!pl.ok) return false;
    CUtensorMap tm[3];
    for (int t = 0; t < 3; ++t) {
        err = rw_tensor_map(w[t < n ? t : 0], pl.geo.wrow, &tm[t]);
        if (err == cudaErrorNotSupported || err == cudaErrorInvalidValue) { err = cudaSuccess; return false; }
        if (err != cudaSuccess) return true;
    }
    const int nb = (int)(K / 256);
    const int nks = (nb + pl.geo.KSB - 1) / pl.geo.KSB;
    if (skn_stage_reserve(ctx, &ctx->d_xq, &ctx->d_xq_bytes, (size_t)nks * M * pl.geo.prow + 256) != SKN_OK) {
        err = cudaErrorMemoryAllocation;
        return true;
    }
    uint8_t *xq = (uint8_t *)ctx->d_xq;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)M);
        const int warps = nb < 32 ? nb : 32;
        cfg.blockDim = dim3((unsigned)warps * 32);
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        err = cudaLaunchKernelEx(&cfg, skn_xprep_kernel<false>, x, (int)K, norm_gain, norm_eps, silu_u, xq, pl.geo.KSB);
        if (err != cudaSuccess) return true;
    }
    rw_kernel_t kern = rw_kernel(fmt, pl.np);
    // the kernel's shared-memory limit is raised once per context (device) and kernel variant
    const uint32_t cfg_bit = 1u << ((fmt == MM_FMT_Q4K ? 0 : (fmt == MM_FMT_Q40 ? 1 : 2)) * 3 + (pl.np == 2 ? 0 : (pl.np == 4 ? 1 : 2)));
    if (!(ctx->rows_cfg & cfg_bit)) {
        err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (err != cudaSuccess) return true;
        ctx->rows_cfg |= cfg_bit;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rw_launch_grid(pl, G, swiglu));
    cfg.blockDim = dim3((RW_W + 2) * 32);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    err = cudaLaunchKernelEx(&cfg, kern, tm[0], tm[1], tm[2], ar, (int)K, pl.geo, (const uint8_t *)xq, ctx->d_status);
    return true;
}

// Host arithmetic only (no device is touched): the layout a many-row launch of n_groups sixteen-row groups would get
// on a GPU of sm_count SMs.  out[0] = 1 if the shape is covered (else the rest is unset), out[1] = CTAs, out[2] = most
// groups any CTA owns, out[3] = groups a CTA's partial-sum space is sized for, out[4] = CTAs without any group,
// out[5] = K chunks, out[6] = ring stages, out[7] = dynamic shared memory in bytes.
extern "C" int32_t skn_rows_plan_query(int32_t sm_count, int32_t type, int64_t n_groups, int64_t n_cols, int32_t n_act, int32_t swiglu,
                                       int64_t *out) {
    if (!out || sm_count < 1 || n_groups < 1 || n_act < 1 || n_act > 16) return SKN_ERR_ARG;
    for (int i = 0; i < 8; ++i) out[i] = 0;
    const int fmt = rw_fmt_of(type);
    if (fmt < 0 || n_cols % 256 || n_cols < 512 || n_cols > (1 << 18)) return SKN_OK;
    skn_ctx fake = {};
    fake.sm_count = sm_count;
    const rw_plan pl = rw_make_plan(&fake, fmt, n_groups, n_cols, n_act);
    if (!pl.ok) return SKN_OK;
    const int grid = rw_launch_grid(pl, n_groups, swiglu != 0);
    int most = 0, none = 0;
    for (int b = 0; b < grid; ++b) {
        int gb, ge;
        rw_cta_groups(b, grid, (int)n_groups, swiglu != 0, gb, ge);
        most = ge - gb > most ? ge - gb : most;
        none += ge - gb <= 0;
    }
    const int nb = (int)(n_cols / 256);
    const int64_t gmax = (n_groups + pl.grid - 1) / pl.grid + 1;
    out[0] = 1; out[1] = grid; out[2] = most; out[3] = gmax; out[4] = none;
    out[5] = (nb + pl.geo.KSB - 1) / pl.geo.KSB; out[6] = pl.geo.nst; out[7] = (int64_t)pl.smem;
    return SKN_OK;
}
