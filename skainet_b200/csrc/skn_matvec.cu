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

#include <stdlib.h>

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

__device__ __forceinline__ float skn_pow2f(int e) { return __int_as_float((e + 127) << 23); }

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

// ---- Q4_K ------------------------------------------------------------------------------
// chunk = 8 super-blocks (2048 weights, 1152 bytes); lane = (block cb = lane/4, pair p =
// lane%4): the 32 quant bytes whose low nibbles are sub-block 2p and high nibbles
// sub-block 2p+1, i.e. 64 consecutive weights starting at 256*cb + 64*p.
struct Q4KStream {
    static constexpr int CHUNK_BLOCKS = 8;
    static constexpr int BLOCK_BYTES = 144;
    static constexpr int CHUNK_BYTES = CHUNK_BLOCKS * BLOCK_BYTES;
    static constexpr int CHUNK_WEIGHTS = CHUNK_BLOCKS * 256;

    uint64_t x2[32];   // {x_lo[i] * 2^(S - pos_lo), x_hi[i] * 2^(S - pos_hi)}
    float sum_lo, sum_hi;
    float unscale;     // 2^(85 - S); together with the constant 2^64 it undoes 2^(S - 149)
    int cb, p;
    bool active;

    __device__ __forceinline__ void load_x(const float *__restrict__ x, int chunk, int lane, int nblocks_in_chunk) {
        cb = lane >> 2;
        p = lane & 3;
        active = cb < nblocks_in_chunk;
        const float4 *xp = reinterpret_cast<const float4 *>(x + (int64_t)chunk * CHUNK_WEIGHTS + cb * 256 + p * 64);
        float xl[32], xh[32];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 a = active ? __ldg(xp + q) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 b = active ? __ldg(xp + 8 + q) : make_float4(0.f, 0.f, 0.f, 0.f);
            xl[4 * q] = a.x; xl[4 * q + 1] = a.y; xl[4 * q + 2] = a.z; xl[4 * q + 3] = a.w;
            xh[4 * q] = b.x; xh[4 * q + 1] = b.y; xh[4 * q + 2] = b.z; xh[4 * q + 3] = b.w;
        }
        float sl = 0.f, sh = 0.f;
        uint32_t mx = 0;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            sl += xl[i];
            sh += xh[i];
            mx = max(mx, max(__float_as_uint(xl[i]), __float_as_uint(xh[i])) & 0x7fffffffu);
        }
        sum_lo = sl;
        sum_hi = sh;
        // Per-lane power-of-two pre-scale S: the largest |x| of this lane lands near 2^90, so
        // x * 2^S never overflows and the products with k * 2^-149 stay normal numbers whatever
        // the magnitude of the activations.
        int S = 217 - (int)(mx >> 23);
        S = S > 120 ? 120 : (S < -37 ? -37 : S);
        unscale = skn_pow2f(85 - S);
        // byte k of a 32-bit quant word: low nibble sits at bit 8k, high nibble at 8k+4;
        // byte 3 is read from (word >> 8), i.e. at bits 16 / 20
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int k = i & 3;
            const int pos_lo = (k == 3) ? 16 : 8 * k;
            const int pos_hi = pos_lo + 4;
            x2[i] = skn_pack2(xl[i] * skn_pow2f(S - pos_lo), xh[i] * skn_pow2f(S - pos_hi));
        }
    }

    // partial dot of this lane's 64 weights of the row-chunk staged at `sb`
    __device__ __forceinline__ float dot(const uint8_t *sb) const {
        const uint4 hdr = *reinterpret_cast<const uint4 *>(sb + cb * BLOCK_BYTES);
        const uint4 q0 = *reinterpret_cast<const uint4 *>(sb + cb * BLOCK_BYTES + 16 + 32 * p);
        const uint4 q1 = *reinterpret_cast<const uint4 *>(sb + cb * BLOCK_BYTES + 32 + 32 * p);
        const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        uint64_t acc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
        for (int wi = 0; wi < 8; ++wi) {
            const uint32_t w = qw[wi];
            const uint32_t w8 = w >> 8;
            acc[0] = skn_fma2(skn_pack2u(w & 0x0000000Fu, w & 0x000000F0u), x2[4 * wi + 0], acc[0]);
            acc[1] = skn_fma2(skn_pack2u(w & 0x00000F00u, w & 0x0000F000u), x2[4 * wi + 1], acc[1]);
            acc[2] = skn_fma2(skn_pack2u(w & 0x000F0000u, w & 0x00F00000u), x2[4 * wi + 2], acc[2]);
            acc[3] = skn_fma2(skn_pack2u(w8 & 0x000F0000u, w8 & 0x00F00000u), x2[4 * wi + 3], acc[3]);
        }
        float dlo, dhi;
        skn_unpack2(skn_add2(skn_add2(acc[0], acc[1]), skn_add2(acc[2], acc[3])), dlo, dhi);

        // 6-bit scales / mins of sub-blocks 2p and 2p+1 (two adjacent bytes of each group)
        const int sh = (p & 1) * 16;
        const uint32_t a2 = (hdr.y >> sh) & 0xFFFFu, b2 = (hdr.z >> sh) & 0xFFFFu, c2 = (hdr.w >> sh) & 0xFFFFu;
        const uint32_t sc2 = (p < 2) ? (a2 & 0x3F3Fu) : ((c2 & 0x0F0Fu) | ((a2 >> 2) & 0x3030u));
        const uint32_t mn2 = (p < 2) ? (b2 & 0x3F3Fu) : (((c2 >> 4) & 0x0F0Fu) | ((b2 >> 2) & 0x3030u));
        const float d = skn_half_bits_to_float(hdr.x & 0xFFFFu);
        const float dmin = skn_half_bits_to_float(hdr.x >> 16);
        const float t1 = fmaf((float)(sc2 >> 8), dhi, (float)(sc2 & 0xFFu) * dlo) * skn_pow2f(64) * unscale;
        const float t2 = fmaf((float)(mn2 >> 8), sum_hi, (float)(mn2 & 0xFFu) * sum_lo);
        const float r = fmaf(d, t1, -dmin * t2);
        return active ? r : 0.f;
    }
};

// One kernel for every streaming decoder S (a struct with CHUNK_BLOCKS / BLOCK_BYTES /
// CHUNK_BYTES / CHUNK_WEIGHTS, load_x() and dot()).
//   grid  : CTA b owns rows [b*N/grid, (b+1)*N/grid)
//   block : nch * wg warps; warp w -> chunk c = w % nch, row slot g = w / nch
//   smem  : [warps][MV_NST][CHUNK_BYTES] ring | [warps][MV_NST] mbarriers | [rows][nch] partials
template <class S>
__global__ void __launch_bounds__(512, 1)
skn_matvec_stream(const uint8_t *__restrict__ W, int64_t pitch, int64_t N, int nb, int nch, int wg,
                  const float *__restrict__ x, const float *__restrict__ bias, float *__restrict__ y,
                  int32_t *__restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const int c = warp % nch;
    const int g = warp / nch;

    uint8_t *ring = smem + (size_t)warp * MV_NST * S::CHUNK_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)nwarps * MV_NST * S::CHUNK_BYTES) + warp * MV_NST;
    float *part = reinterpret_cast<float *>(smem + (size_t)nwarps * MV_NST * S::CHUNK_BYTES +
                                            (size_t)nwarps * MV_NST * sizeof(uint64_t));

    const int64_t row_begin = (int64_t)blockIdx.x * N / gridDim.x;
    const int64_t row_end = (int64_t)(blockIdx.x + 1) * N / gridDim.x;
    const int rows = (int)(row_end - row_begin);
    const int cnt = (rows > g) ? (rows - g + wg - 1) / wg : 0;   // rows this warp visits

    int nbc = nb - c * S::CHUNK_BLOCKS;
    if (nbc > S::CHUNK_BLOCKS) nbc = S::CHUNK_BLOCKS;
    const uint32_t bytes = (uint32_t)nbc * S::BLOCK_BYTES;
    const uint8_t *src0 = W + (row_begin + g) * pitch + (size_t)c * S::CHUNK_BYTES;
    const int64_t src_step = (int64_t)wg * pitch;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < MV_NST; ++s) skn_mbar_init(&bars[s], 1);
        skn_fence_mbar_init();
        skn_fence_proxy_async();
        // weights never depend on the previous kernel: start streaming them right away
#pragma unroll
        for (int s = 0; s < MV_NST; ++s) {
            if (s < cnt) {
                skn_mbar_expect_tx(&bars[s], bytes);
                skn_bulk_g2s(ring + s * S::CHUNK_BYTES, src0 + s * src_step, bytes, &bars[s]);
            }
        }
    }
    __syncwarp();
    skn_pdl_launch_dependents();
    skn_pdl_wait();   // x (and y) may belong to the previous kernel in the stream

    S dec;
    dec.load_x(x, c, lane, nbc);

    bool failed = false;
    for (int i0 = 0; i0 < cnt; i0 += MV_NST) {
        const uint32_t parity = (uint32_t)(i0 / MV_NST) & 1u;
        float acc[MV_NST];
#pragma unroll
        for (int ii = 0; ii < MV_NST; ++ii) {
            acc[ii] = 0.f;
            const int i = i0 + ii;
            if (i < cnt && !failed) {
                if (!__all_sync(0xffffffffu, skn_mbar_wait(&bars[ii], parity))) {
                    failed = true;
                    if (lane == 0) atomicExch(status, SKN_ERR_TIMEOUT);
                } else {
                    acc[ii] = dec.dot(ring + ii * S::CHUNK_BYTES);
                    __syncwarp();   // every lane has consumed the stage
                    if (lane == 0 && i + MV_NST < cnt) {
                        skn_fence_proxy_async();
                        skn_mbar_expect_tx(&bars[ii], bytes);
                        skn_bulk_g2s(ring + ii * S::CHUNK_BYTES, src0 + (int64_t)(i + MV_NST) * src_step, bytes,
                                     &bars[ii]);
                    }
                }
            }
        }
        const float tot = skn_warp_reduce8(acc, lane);
        const int ii = lane >> 2;
        if ((lane & 3) == 0 && i0 + ii < cnt) part[(size_t)(g + (i0 + ii) * wg) * nch + c] = tot;
    }
    __syncthreads();
    for (int lr = threadIdx.x; lr < rows; lr += blockDim.x) {
        float s = 0.f;
        for (int cc = 0; cc < nch; ++cc) s += part[(size_t)lr * nch + cc];
        if (bias) s += bias[row_begin + lr];
        y[row_begin + lr] = s;
    }
}

static int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}

// Launch geometry of the streaming kernel for one weight tensor; computed on first use and
// cached in the tensor (it depends only on the tensor's shape and the device).
template <class S>
static cudaError_t plan_stream(skn_ctx *ctx, const skn_tensor *w, skn_mv_plan &pl) {
    auto kern = skn_matvec_stream<S>;
    pl.state = -1;  // "no streaming plan" unless everything below works out
    const int64_t nb = w->n_cols / (S::CHUNK_WEIGHTS / S::CHUNK_BLOCKS);  // blocks per row
    const int nch = (int)((nb + S::CHUNK_BLOCKS - 1) / S::CHUNK_BLOCKS);
    if (nch < 1 || nch > 16 || w->n_rows < 1) return cudaSuccess;
    static const int wg_env = env_int("SKN_MV_WG", 0);
    static const int occ_env = env_int("SKN_MV_OCC", 0);
    int wg = wg_env > 0 ? wg_env : (nch <= 8 ? 8 / nch : 1);
    if (wg < 1) wg = 1;
    while (nch * wg > 16) --wg;
    const int warps = nch * wg;
    const int threads = warps * 32;
    const size_t ring = (size_t)warps * MV_NST * S::CHUNK_BYTES + (size_t)warps * MV_NST * sizeof(uint64_t);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return e;
    int occ = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, threads, ring + 1024);
    if (e != cudaSuccess) return e;
    if (occ_env > 0 && occ_env < occ) occ = occ_env;
    if (occ < 1) return cudaSuccess;
    int64_t grid = (int64_t)ctx->sm_count * occ;
    if (grid > w->n_rows) grid = w->n_rows;
    const int64_t rows_max = (w->n_rows + grid - 1) / grid;
    const size_t smem = ring + (size_t)rows_max * nch * sizeof(float);
    if (smem > ring + 1024 || smem > 220 * 1024) {
        // partial-sum area larger than what the occupancy query assumed: use one CTA per SM
        grid = ctx->sm_count < w->n_rows ? ctx->sm_count : w->n_rows;
        const int64_t rm = (w->n_rows + grid - 1) / grid;
        const size_t sm2 = ring + (size_t)rm * nch * sizeof(float);
        if (sm2 > 220 * 1024) return cudaSuccess;
        pl.smem = sm2;
    } else {
        pl.smem = smem;
    }
    pl.nch = nch; pl.wg = wg; pl.grid = (int)grid; pl.threads = threads;
    pl.state = 1;
    return cudaSuccess;
}

template <class S>
static cudaError_t launch_stream(skn_ctx *ctx, const skn_tensor *w, const float *x, const float *bias, float *y,
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
    const int nb = (int)(w->n_cols / (S::CHUNK_WEIGHTS / S::CHUNK_BLOCKS));
    return cudaLaunchKernelEx(&cfg, kern, (const uint8_t *)w->d_blocks, w->pitch, w->n_rows, nb, pl.nch, pl.wg, x,
                              bias, y, ctx->d_status);
}

template <class S>
static bool try_stream(skn_ctx *ctx, const skn_tensor *w, const float *x, const float *bias, float *y,
                       cudaStream_t stream, cudaError_t &err) {
    skn_mv_plan &pl = const_cast<skn_tensor *>(w)->mv_plan;
    if (pl.state == 0) {
        err = plan_stream<S>(ctx, w, pl);
        if (err != cudaSuccess) { pl.state = 0; return true; }
    }
    if (pl.state != 1) return false;
    err = launch_stream<S>(ctx, w, x, bias, y, pl, stream);
    return true;
}

cudaError_t skn_launch_matvec(skn_ctx *ctx, const skn_tensor *w, const float *x, int32_t M, const float *bias,
                              float *y, cudaStream_t stream) {
    static const int force_generic = env_int("SKN_MV_GENERIC", 0);
    if (M == 1 && !force_generic && (w->pitch % 16) == 0) {
        cudaError_t err = cudaSuccess;
        if (w->type == SKN_TYPE_Q4_K && try_stream<Q4KStream>(ctx, w, x, bias, y, stream, err)) return err;
    }
    switch (w->type) {
    case SKN_TYPE_Q4_0: return launch_generic<SKN_TYPE_Q4_0>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_Q8_0: return launch_generic<SKN_TYPE_Q8_0>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_Q4_K: return launch_generic<SKN_TYPE_Q4_K>(w, x, M, bias, y, ctx->sm_count, stream);
    case SKN_TYPE_Q6_K: return launch_generic<SKN_TYPE_Q6_K>(w, x, M, bias, y, ctx->sm_count, stream);
    default: return cudaErrorInvalidValue;
    }
}
