// Pieces shared by the decode matvec kernels (skn_matvec.cu, skn_matvec_mma.cu).
#pragma once
#include "skn_internal.cuh"
#include "skn_ptx.cuh"

#include <stdlib.h>

// SKN_TUNING builds record per-CTA phase timestamps (SM clock and global timer) after the
// status word; used only for profiling experiments, never in the shipped library.
#ifdef SKN_TUNING
#define MV_TRACE_VARS unsigned mv_seq = 0
// (and, for CTA 0, a timeline entry per launch: {launch number, start, dependency wait done, end} in global-timer ns)
#define MV_STAMP(k)                                                                        \
    do {                                                                                   \
        if (threadIdx.x == 0) {                                                            \
            long long *tr = reinterpret_cast<long long *>(status) + 16 + blockIdx.x * 16;  \
            const long long now_ns = (long long)skn_globaltimer_ns();                      \
            if (blockIdx.x == 0) {                                                         \
                long long *tl = reinterpret_cast<long long *>(status) + 2560;              \
                if ((k) == 0) {                                                            \
                    const unsigned sq = atomicAdd(reinterpret_cast<unsigned *>(status) + 2, 1u); \
                    mv_seq = sq;                                                           \
                    tl[(sq % 192u) * 8 + 0] = (long long)sq;                               \
                    tl[(sq % 192u) * 8 + 1] = now_ns;                                      \
                } else if ((k) >= 2) {                                                     \
                    tl[(mv_seq % 192u) * 8 + (k)] = now_ns;                              \
                }                                                                          \
            }                                                                              \
            if ((k) != 1) {                                                                \
                tr[2 * (k)] = clock64();                                                   \
                tr[2 * (k) + 1] = now_ns;                                                  \
            }                                                                              \
        }                                                                                  \
    } while (0)
#else
#define MV_TRACE_VARS
#define MV_STAMP(k) do {} while (0)
#endif


__device__ __forceinline__ float skn_pow2f(int e) { return __int_as_float((e + 127) << 23); }


// Optional transforms applied to x while it is prepared, so that the element-wise ops that
// precede a projection in a decoder need no launch of their own:
//   silu_u != NULL : x <- silu(x) * silu_u      (SwiGLU product feeding the down projection)
//   gain   != NULL : x <- x * scale * gain      (RMSNorm; scale = rsqrt(mean(x^2) + eps) is
//                                                computed by the CTA before the preparation)
struct skn_xform {
    const float *gain;
    const float *silu_u;
    float scale;
    // tensor-parallel consumer: x <- x + sum over ranks of the partial products waiting in this
    // rank's inbox (red_world slots red_stride floats apart, rank order); red_wb != NULL: the sum is
    // also stored there (the new residual stream)
    const float *red;
    int red_world;
    int64_t red_stride;
    float *red_wb;
};

__device__ __forceinline__ float4 skn_load_x4(const float *__restrict__ x, int f, const skn_xform &xf) {
    float4 v;
    if (xf.red_world > 1) {
        v = __ldcg(reinterpret_cast<const float4 *>(x) + f);
        for (int src = 0; src < xf.red_world; ++src) {
            const float4 p = __ldcg(reinterpret_cast<const float4 *>(xf.red + (size_t)src * xf.red_stride) + f);
            v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
        }
        if (xf.red_wb) reinterpret_cast<float4 *>(xf.red_wb)[f] = v;
    } else {
        v = __ldg(reinterpret_cast<const float4 *>(x) + f);
    }
    if (xf.silu_u) {
        const float4 u = __ldg(reinterpret_cast<const float4 *>(xf.silu_u) + f);
        v.x = v.x / (1.f + expf(-v.x)) * u.x;
        v.y = v.y / (1.f + expf(-v.y)) * u.y;
        v.z = v.z / (1.f + expf(-v.z)) * u.z;
        v.w = v.w / (1.f + expf(-v.w)) * u.w;
    }
    if (xf.gain) {
        const float4 g = __ldg(reinterpret_cast<const float4 *>(xf.gain) + f);
        v.x = v.x * xf.scale * g.x;
        v.y = v.y * xf.scale * g.y;
        v.z = v.z * xf.scale * g.z;
        v.w = v.w * xf.scale * g.w;
    }
    return v;
}

// A matvec launch may cover up to three weight tensors of the same type, K and pitch that multiply the
// same x (Q/K/V, gate/up): their rows are concatenated, row r of the concatenation belongs to
// the first tensor whose cumulative end exceeds r.  `add[t]` (may be NULL) is added to tensor
// t's outputs: a bias, or the residual stream when y aliases it.
struct skn_mv_group {
    const uint8_t *W[3];
    float *y[3];
    const float *add[3];
    int64_t n_end[3];       // cumulative row counts
    int count;
    const float *norm_gain; // RMSNorm of x fused into its preparation (NULL: none)
    float norm_eps;
    const float *silu_u;    // x <- silu(x) * silu_u fused into its preparation (NULL: none)
    int n_act;              // tensor-core kernel only: activation rows per launch (x rows K apart, 0 means 1)
    int64_t ystride[3];     // ... distance between the outputs of consecutive activation rows
    int64_t addstride[3];   // ... and between their `add` vectors (0: one bias shared by all rows)
    // tensor-core kernel only, tensor parallelism (both off when xc_world <= 1):
    //   xc_push   : the outputs are partial products: they go to slot xc_rank of every rank's inbox
    //               (y is not written) and the last CTA releases the peers' flags
    //   xc_reduce : x is the residual stream; the partial products pushed by the previous launch of
    //               every rank are added to it while x is prepared; CTA 0 stores the sum to xc_wb
    int xc_world, xc_rank, xc_push, xc_reduce;
    int64_t xc_cap;              // floats per (buffer, source rank) of an inbox
    uint8_t *xc_base[8];         // inboxes of all ranks as mapped here (xc_base[xc_rank] is local)
    uint32_t *xc_state;          // [0] exchanges completed, [1] push tickets
    float *xc_wb;
    // tensor-core kernel only, Q/K/V launch of a single-token decoder step (rope_hd > 0): tensors are
    // (wq, wk, wv); activation row a belongs to sequence rope_a0 + a whose new token has position
    // rope_len[seq]; q is rotated and written to y[0], k is rotated and written straight into the
    // cache slot of that position, v is copied there (cache: [seq][kv head][capacity][head dim])
    int rope_hd, rope_cap, rope_nkv, rope_a0;
    const int32_t *rope_len, *rope_start;
    float *rope_kc, *rope_vc;
    double rope_log2theta;
    const double *rope_inv_freq;
    int swiglu;             // tensor-core kernel only: W[0] = gate, W[1] = up (equal shapes); rows are
                            // interleaved (virtual row v = tensor v & 1, row v >> 1) so that a CTA holds
                            // both products of a column and writes y[0][r] = silu(gate . x) * (up . x)
};

__device__ __forceinline__ int skn_group_find(const skn_mv_group &grp, int64_t r, int64_t &local) {
    const int t = (r >= grp.n_end[0] ? 1 : 0) + ((grp.count > 2 && r >= grp.n_end[1]) ? 1 : 0);
    local = r - (t ? grp.n_end[t - 1] : 0);
    return t;
}

// row v of a launch -> (tensor, row inside it)
__device__ __forceinline__ int skn_group_row(const skn_mv_group &grp, int64_t v, int64_t &local) {
    if (grp.swiglu) {
        local = v >> 1;
        return (int)(v & 1);
    }
    return skn_group_find(grp, v, local);
}

static inline int env_int(const char *name, int dflt) { return skn_tune_int(name, dflt); }

