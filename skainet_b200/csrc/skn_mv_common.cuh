// Pieces shared by the decode matvec kernels (skn_matvec.cu, skn_matvec_mma.cu).
#pragma once
#include "skn_internal.cuh"
#include "skn_ptx.cuh"

#include <stdlib.h>

// SKN_MV_TRACE builds record per-CTA phase timestamps (SM clock and global timer) after the
// status word; used only for profiling experiments, never in the shipped library.
#ifdef SKN_MV_TRACE
#define MV_STAMP(k)                                                                        \
    do {                                                                                   \
        if (threadIdx.x == 0) {                                                            \
            long long *tr = reinterpret_cast<long long *>(status) + 16 + blockIdx.x * 16;  \
            tr[2 * (k)] = clock64();                                                       \
            tr[2 * (k) + 1] = (long long)skn_globaltimer_ns();                             \
        }                                                                                  \
    } while (0)
#else
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
};

__device__ __forceinline__ float4 skn_load_x4(const float *__restrict__ x, int f, const skn_xform &xf) {
    float4 v = __ldg(reinterpret_cast<const float4 *>(x) + f);
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

static inline int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}

