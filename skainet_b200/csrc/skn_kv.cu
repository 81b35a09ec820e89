// K5-K7: device-resident KV cache and decode attention.
//
// Layout (head-major ring of fp32 or, on request, fp16 elements):  K, V : [batch][n_kv_heads][capacity][head_dim].
// Sequence b holds len[b] tokens; logical position p (0 = oldest) lives at ring slot
// (start[b] + p) % capacity.  All tokens of one (sequence, kv head) are contiguous, so the
// attention kernel streams them with fully coalesced 512-byte rows.
//
//  skn_kv_append_kernel   one CTA per sequence writes the new token of every kv head and then
//                         advances len (or start, once the ring is full)
//  skn_kv_gather_kernel   ring -> dense, oldest first (export / verification)
//  skn_attn_split_kernel  grid (splits, kv heads, batch): one CTA attends G = Hq/Hkv query
//                         heads to a chunk of 256 (64, 32 for short contexts) cached tokens.  Pass 1 reads K once and
//                         leaves the chunk's scores in shared memory (lane = 4 head dims;
//                         32 (token, head) partial dots are summed with one transposed
//                         butterfly of 31 shuffles); pass 2 reads V once and accumulates
//                         exp(s - max) * v with the probabilities broadcast from shared
//                         memory.  Writes (max, sum, unnormalised output) per (head, split)
//                         to scratch.
//  skn_attn_stream_kernel the same split for long contexts with the K and V tiles brought into a
//                         shared-memory ring by bulk async copies (a producer warp, mbarriers)
//  skn_attn_merge_kernel  log-sum-exp merge of the splits -> out[b][h][:] (small grids merge in
//                         the split kernel: the CTA that draws the last ticket)
//
// HBM-bound: 2 * head_dim * element size bytes per cached token per kv head, read exactly once.
#include "skn_internal.cuh"
#include "skn_ptx.cuh"

#include <cuda_fp16.h>
#include <math.h>
#include <stdlib.h>
#include <new>

struct skn_kvcache {
    uint32_t magic;
    skn_ctx *ctx;
    int32_t batch, n_kv_heads, head_dim, capacity;
    int32_t dtype;               // SKN_KV_F32, SKN_KV_F16 or SKN_KV_Q8_0: element type of d_k / d_v
    void *d_k, *d_v;
    int32_t *d_len, *d_start;
    unsigned *d_tickets;         // [batch][n_kv_heads], zero between launches: split-attention merge tickets
};

constexpr int ATT_CHUNK = 256;   // cached tokens per CTA (64 when the grid would otherwise leave SMs idle)
constexpr int ATT_WARPS = 4;
constexpr int ATT_MERGE_MAX_SPLITS = 64;   // most splits the in-kernel merge handles (its weights reuse the score buffer)

static bool kv_ok(const skn_kvcache *kv) { return kv && kv->magic == SKN_MAGIC_KV && skn_ctx_ok(kv->ctx); }

// Cache element types: fp32, or fp16 (half the attention traffic; values are rounded to nearest
// even on their way in and widened to fp32 on their way out, all arithmetic stays fp32).
template <class CT> struct KvElem;
template <> struct KvElem<float> {
    static __device__ __forceinline__ void st4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
    static __device__ __forceinline__ void st2(float *p, float2 v) { *reinterpret_cast<float2 *>(p) = v; }
    static __device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
    static __device__ __forceinline__ float4 ldg4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
    static __device__ __forceinline__ float2 ld2(const float *p) { return *reinterpret_cast<const float2 *>(p); }
    static __device__ __forceinline__ float2 ldg2(const float *p) { return __ldg(reinterpret_cast<const float2 *>(p)); }
};
template <> struct KvElem<__half> {
    static __device__ __forceinline__ void st4(__half *p, float4 v) {
        const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<const uint32_t *>(&a);
        u.y = *reinterpret_cast<const uint32_t *>(&b);
        *reinterpret_cast<uint2 *>(p) = u;
    }
    static __device__ __forceinline__ void st2(__half *p, float2 v) { *reinterpret_cast<__half2 *>(p) = __floats2half2_rn(v.x, v.y); }
    static __device__ __forceinline__ float4 widen4(uint2 u) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&u.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&u.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ float4 ld4(const __half *p) { return widen4(*reinterpret_cast<const uint2 *>(p)); }
    static __device__ __forceinline__ float4 ldg4(const __half *p) { return widen4(__ldg(reinterpret_cast<const uint2 *>(p))); }
    static __device__ __forceinline__ float2 ld2(const __half *p) { return __half22float2(*reinterpret_cast<const __half2 *>(p)); }
    static __device__ __forceinline__ float2 ldg2(const __half *p) {
        const uint32_t u = __ldg(reinterpret_cast<const uint32_t *>(p));
        return __half22float2(*reinterpret_cast<const __half2 *>(&u));
    }
};
// VEC (2 or 4) consecutive cache elements -> fp32 registers; GLOBAL: read-only global load, else a plain (shared-memory) load
template <class CT, int VEC, bool GLOBAL> struct KvLoad;
template <class CT, bool GLOBAL> struct KvLoad<CT, 4, GLOBAL> {
    static __device__ __forceinline__ void ld(const CT *p, float (&r)[4]) {
        const float4 v = GLOBAL ? KvElem<CT>::ldg4(p) : KvElem<CT>::ld4(p);
        r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
    }
};
template <class CT, bool GLOBAL> struct KvLoad<CT, 2, GLOBAL> {
    static __device__ __forceinline__ void ld(const CT *p, float (&r)[2]) {
        const float2 v = GLOBAL ? KvElem<CT>::ldg2(p) : KvElem<CT>::ld2(p);
        r[0] = v.x; r[1] = v.y;
    }
};

// Q8_0-style cache: every 32 consecutive head dims of a cached row share one fp16 scale d = max|x| / 127 and are
// kept as int8 q = round(x / d) (ggml's quantize_row_q8_0: the division by the fp32 d, rounding half away from
// zero; the value read back is q * fp16(d)).  Unlike the 34-byte GGUF block the two parts live in two planes of
// the same allocation -- [rows][D] int8, then [rows][D / 32] fp16, rows = batch * kv heads * capacity -- so a
// row's quants stay 16-byte aligned and a lane's four dims are one 32-bit load.
struct skn_q8 { int8_t q; };
template <class CT> struct KvIsQ8 { static constexpr bool value = false; };
template <> struct KvIsQ8<skn_q8> { static constexpr bool value = true; };

// scale plane of a cache tensor with `rows` rows (NULL for the unquantised element types)
template <class CT>
__device__ __forceinline__ __half *kv_scale_plane(CT *plane, size_t rows, int D) {
    if constexpr (KvIsQ8<CT>::value) return reinterpret_cast<__half *>(reinterpret_cast<int8_t *>(plane) + rows * (size_t)D);
    else return nullptr;
}
template <class CT>
__device__ __forceinline__ const __half *kv_scale_plane(const CT *plane, size_t rows, int D) {
    return kv_scale_plane(const_cast<CT *>(plane), rows, D);
}
__device__ __forceinline__ int kv_q8_quant(float x, float id) { return (int)roundf(x * id); }

// Four consecutive dims d .. d + 3 of cache row `row`.  Quantised caches: the eight lanes (lane & ~7) .. + 7 of the
// warp hold the eight quads of one 32-dim block and must call this together.
template <class CT>
__device__ __forceinline__ void kv_store4(CT *plane, __half *scales, size_t row, int D, int d, float4 v) {
    if constexpr (KvIsQ8<CT>::value) {
        const unsigned lane = threadIdx.x & 31u, mask = 0xFFu << (lane & 24u);
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(mask, amax, o));
        const float dq = amax / 127.f, id = dq != 0.f ? 1.f / dq : 0.f;
        const uint32_t pk = (uint32_t)(kv_q8_quant(v.x, id) & 255) | ((uint32_t)(kv_q8_quant(v.y, id) & 255) << 8) |
                            ((uint32_t)(kv_q8_quant(v.z, id) & 255) << 16) | ((uint32_t)(kv_q8_quant(v.w, id) & 255) << 24);
        *reinterpret_cast<uint32_t *>(reinterpret_cast<int8_t *>(plane) + row * (size_t)D + d) = pk;
        if ((lane & 7u) == 0) scales[row * (size_t)(D / 32) + (d >> 5)] = __float2half_rn(dq);
    } else {
        KvElem<CT>::st4(plane + row * (size_t)D + d, v);
    }
}
// Two consecutive dims (a rotated pair).  Quantised caches: the sixteen lanes (lane & ~15) .. + 15 hold one block.
template <class CT>
__device__ __forceinline__ void kv_store2(CT *plane, __half *scales, size_t row, int D, int d, float2 v) {
    if constexpr (KvIsQ8<CT>::value) {
        const unsigned lane = threadIdx.x & 31u, mask = 0xFFFFu << (lane & 16u);
        float amax = fmaxf(fabsf(v.x), fabsf(v.y));
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(mask, amax, o));
        const float dq = amax / 127.f, id = dq != 0.f ? 1.f / dq : 0.f;
        const unsigned short pk = (unsigned short)((kv_q8_quant(v.x, id) & 255) | ((kv_q8_quant(v.y, id) & 255) << 8));
        *reinterpret_cast<unsigned short *>(reinterpret_cast<int8_t *>(plane) + row * (size_t)D + d) = pk;
        if ((lane & 15u) == 0) scales[row * (size_t)(D / 32) + (d >> 5)] = __float2half_rn(dq);
    } else {
        KvElem<CT>::st2(plane + row * (size_t)D + d, v);
    }
}
template <class CT>
__device__ __forceinline__ float4 kv_load4(const CT *plane, const __half *scales, size_t row, int D, int d) {
    if constexpr (KvIsQ8<CT>::value) {
        const uint32_t pk = *reinterpret_cast<const uint32_t *>(reinterpret_cast<const int8_t *>(plane) + row * (size_t)D + d);
        const float sc = __half2float(scales[row * (size_t)(D / 32) + (d >> 5)]);
        return make_float4((float)(int8_t)(pk & 255u) * sc, (float)(int8_t)((pk >> 8) & 255u) * sc,
                           (float)(int8_t)((pk >> 16) & 255u) * sc, (float)(int8_t)(pk >> 24) * sc);
    } else {
        return KvElem<CT>::ld4(plane + row * (size_t)D + d);
    }
}

// The attention kernels' view of one (sequence, kv head): VEC dims per lane of the row in ring slot `slot`.
template <class CT, int D, int VEC> struct KvHeadReader {
    const CT *base;
    const __half *sc;
    __device__ __forceinline__ KvHeadReader(const CT *plane, size_t rows, size_t head_row0, int lane)
        : base(plane + head_row0 * D + lane * VEC), sc(nullptr) {
        if constexpr (KvIsQ8<CT>::value) sc = kv_scale_plane(plane, rows, D) + head_row0 * (D / 32) + ((lane * VEC) >> 5);
    }
    __device__ __forceinline__ void ld(int slot, float (&r)[VEC]) const {
        if constexpr (KvIsQ8<CT>::value) {
            const float s = __half2float(__ldg(sc + (size_t)slot * (D / 32)));
            const int8_t *p = reinterpret_cast<const int8_t *>(base) + (size_t)slot * D;
            if constexpr (VEC == 4) {
                const uint32_t pk = __ldg(reinterpret_cast<const uint32_t *>(p));
                r[0] = (float)(int8_t)(pk & 255u) * s; r[1] = (float)(int8_t)((pk >> 8) & 255u) * s;
                r[2] = (float)(int8_t)((pk >> 16) & 255u) * s; r[3] = (float)(int8_t)(pk >> 24) * s;
            } else {
                const unsigned short pk = __ldg(reinterpret_cast<const unsigned short *>(p));
                r[0] = (float)(int8_t)(pk & 255u) * s; r[1] = (float)(int8_t)(pk >> 8) * s;
            }
        } else {
            KvLoad<CT, VEC, true>::ld(base + (size_t)slot * D, r);
        }
    }
};

// ----------------------------------------------------------------------------------------
template <class CT>
__global__ void skn_kv_append_kernel(CT *__restrict__ kc, CT *__restrict__ vc, int32_t *__restrict__ len,
                                     int32_t *__restrict__ start, const float *__restrict__ k_new,
                                     const float *__restrict__ v_new, int Hkv, int D, int cap) {
    const int b = blockIdx.x;
    const int L = len[b], s0 = start[b];
    const int slot = (L < cap) ? (s0 + L) % cap : s0;   // full ring: overwrite the oldest token
    const int n4 = Hkv * D / 4;
    const size_t rows = (size_t)gridDim.x * Hkv * cap;
    __half *ks = kv_scale_plane(kc, rows, D), *vs = kv_scale_plane(vc, rows, D);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
        const int h = (i * 4) / D, d = (i * 4) % D;
        const size_t dst = ((size_t)b * Hkv + h) * cap + slot;
        const size_t src = ((size_t)b * Hkv + h) * D + d;
        kv_store4(kc, ks, dst, D, d, *reinterpret_cast<const float4 *>(k_new + src));
        kv_store4(vc, vs, dst, D, d, *reinterpret_cast<const float4 *>(v_new + src));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (L < cap) len[b] = L + 1;
        else start[b] = (s0 + 1) % cap;
    }
}

// T new tokens per sequence: k_new, v_new are [batch][T][Hkv][D]; token t goes to ring slot
// (start + len + t) % cap.  The lengths are advanced afterwards by skn_kv_advance_kernel, so
// every CTA of this launch reads the same old length.  The caller guarantees len + T <= cap.
template <class CT>
__global__ void skn_kv_append_many_kernel(CT *__restrict__ kc, CT *__restrict__ vc, const int32_t *__restrict__ len,
                                          const int32_t *__restrict__ start, const float *__restrict__ k_new,
                                          const float *__restrict__ v_new, int Hkv, int D, int cap, int T) {
    const int b = blockIdx.y, t = blockIdx.x;
    const int slot = (start[b] + len[b] + t) % cap;
    const int n4 = Hkv * D / 4;
    const size_t rows = (size_t)gridDim.y * Hkv * cap;
    __half *ks = kv_scale_plane(kc, rows, D), *vs = kv_scale_plane(vc, rows, D);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
        const int h = (i * 4) / D, d = (i * 4) % D;
        const size_t dst = ((size_t)b * Hkv + h) * cap + slot;
        const size_t src = (((size_t)b * T + t) * Hkv + h) * D + d;
        kv_store4(kc, ks, dst, D, d, *reinterpret_cast<const float4 *>(k_new + src));
        kv_store4(vc, vs, dst, D, d, *reinterpret_cast<const float4 *>(v_new + src));
    }
}

__global__ void skn_kv_advance_kernel(int32_t *__restrict__ len, int B, int T, int cap) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) len[b] = min(cap, len[b] + T);
}

// Decoder step, grid (pair blocks + one V block, T, batch): rotary embedding of a new token's
// query heads in place and of its key heads on their way into the ring, V copied alongside.
// Pairs (2i, 2i+1) of a head rotate by pos * theta^(-2i/D) with pos = len[b] + t (angle in double:
// at position 4096 an fp32 angle is already off by ~5e-4 rad); one pair per thread.  The
// lengths are NOT advanced here: the decoder runs attention with `len_extra = T` and advances
// every layer's lengths with one launch at the end of the step.
template <class CT>
__global__ void __launch_bounds__(128)
skn_rope_append_kernel(float *__restrict__ q, const float *__restrict__ k_new, const float *__restrict__ v_new,
                       CT *__restrict__ kc, CT *__restrict__ vc, const int32_t *__restrict__ len,
                       const int32_t *__restrict__ start, int Hq, int Hkv, int D, int cap, int T, double log2_theta,
                       int32_t *__restrict__ status) {
    const int b = blockIdx.z, t = blockIdx.y;
    const int pos = len[b] + t;
    if (pos >= cap) {
        // the cache is full (a replayed step the host did not count): nothing is overwritten, the status word says so
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicExch(status, SKN_ERR_SHAPE);
        return;
    }
    const int slot = (start[b] + pos) % cap;
    const int half = D / 2;
    const size_t row = (size_t)b * T + t;
    const size_t rows = (size_t)gridDim.z * Hkv * cap;
    if (blockIdx.x == gridDim.x - 1) {
        __half *vs = kv_scale_plane(vc, rows, D);
        for (int i = threadIdx.x; i < Hkv * D / 4; i += blockDim.x) {
            const int h = (i * 4) / D, d = (i * 4) % D;
            kv_store4(vc, vs, ((size_t)b * Hkv + h) * cap + slot, D, d, *reinterpret_cast<const float4 *>(v_new + (row * Hkv + h) * D + d));
        }
        return;
    }
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (Hq + Hkv) * half) return;
    const int p = i % half, h = i / half;
    const double ang = (double)pos * exp2(-log2_theta * (2.0 * (double)p / (double)D));
    double sd, cd;
    sincos(ang, &sd, &cd);
    const float sn = (float)sd, cs = (float)cd;
    if (h < Hq) {
        float2 *v = reinterpret_cast<float2 *>(q + (row * Hq + h) * D) + p;
        const float2 a = *v;
        *v = make_float2(a.x * cs - a.y * sn, a.x * sn + a.y * cs);
    } else {
        const int hk = h - Hq;
        const float2 a = reinterpret_cast<const float2 *>(k_new + (row * Hkv + hk) * D)[p];
        // (a block's sixteen pairs sit in sixteen consecutive threads: D / 2 is a multiple of 16 and so is the early exit above)
        kv_store2(kc, kv_scale_plane(kc, rows, D), ((size_t)b * Hkv + hk) * cap + slot, D, 2 * p,
                  make_float2(a.x * cs - a.y * sn, a.x * sn + a.y * cs));
    }
}

// len[l][b] += T for every layer's cache of a decoder (lens: device array of n_layers pointers)
// (a length that would pass the capacity stays at the capacity and SKN_ERR_SHAPE lands in the status word)
__global__ void skn_kv_advance_all_kernel(int32_t *const *__restrict__ lens, int n_layers, int B, int T, int cap,
                                          int32_t *__restrict__ status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_layers * B) {
        int32_t *len = lens[i / B] + (i % B);
        if (*len + T > cap) atomicExch(status, SKN_ERR_SHAPE);
        *len = min(cap, *len + T);
    }
}

// dense fp32 [rows][tokens][D] -> the first `tokens` slots of every (sequence, kv head) of an fp16 or quantised cache
// (total is a multiple of 8 and the stride of 32: the lanes of a block stay together)
template <class CT>
__global__ void skn_kv_load_conv_kernel(const float *__restrict__ src, CT *__restrict__ dst, int64_t rows, int tokens,
                                        int D, int cap) {
    const int64_t per_row = (int64_t)tokens * D / 4, total = rows * per_row;
    __half *sc = kv_scale_plane(dst, (size_t)rows * cap, D);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / per_row, e = (i % per_row) * 4;
        kv_store4(dst, sc, (size_t)r * cap + (size_t)(e / D), D, (int)(e % D), *reinterpret_cast<const float4 *>(src + (size_t)r * tokens * D + e));
    }
}

template <class CT>
__global__ void skn_kv_gather_kernel(const CT *__restrict__ kc, const CT *__restrict__ vc,
                                     const int32_t *__restrict__ start, int b, int Hkv, int D, int cap, int pos0,
                                     int count, float *__restrict__ k_out, float *__restrict__ v_out, int batch) {
    // out: [Hkv][count][D]
    const int s0 = start[b];
    const size_t rows = (size_t)batch * Hkv * cap;
    const __half *ks = kv_scale_plane(kc, rows, D), *vs = kv_scale_plane(vc, rows, D);
    const int d4 = D / 4;
    const int64_t total = (int64_t)Hkv * count * d4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % d4) * 4;
        const int p = (int)((i / d4) % count);
        const int h = (int)(i / ((int64_t)d4 * count));
        const int slot = (s0 + pos0 + p) % cap;
        const size_t src = ((size_t)b * Hkv + h) * cap + slot;
        const size_t dst = ((size_t)h * count + p) * D + d;
        *reinterpret_cast<float4 *>(k_out + dst) = kv_load4(kc, ks, src, D, d);
        *reinterpret_cast<float4 *>(v_out + dst) = kv_load4(vc, vs, src, D, d);
    }
}

// ----------------------------------------------------------------------------------------
// Sum NV per-lane values across the warp.  NV is a power of two <= 32.  On return every lane
// holds the total of value index (lane >> log2(32 / NV)).
template <int NV>
__device__ __forceinline__ float warp_transpose_reduce(float (&v)[NV], int lane) {
    if constexpr (NV >= 32) {
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float send = (lane & 16) ? v[k] : v[k + 16];
            const float keep = (lane & 16) ? v[k + 16] : v[k];
            v[k] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
        }
    }
    constexpr int N16 = NV >= 32 ? 16 : NV;
    constexpr int O16 = NV >= 32 ? 8 : 16;   // xor offset that splits N16 values
    if constexpr (N16 >= 16) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float send = (lane & O16) ? v[k] : v[k + 8];
            const float keep = (lane & O16) ? v[k + 8] : v[k];
            v[k] = keep + __shfl_xor_sync(0xffffffffu, send, O16);
        }
    }
    constexpr int N8 = N16 >= 16 ? 8 : N16;
    constexpr int O8 = N16 >= 16 ? O16 / 2 : 16;
    if constexpr (N8 >= 8) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float send = (lane & O8) ? v[k] : v[k + 4];
            const float keep = (lane & O8) ? v[k + 4] : v[k];
            v[k] = keep + __shfl_xor_sync(0xffffffffu, send, O8);
        }
    }
    constexpr int N4 = N8 >= 8 ? 4 : N8;
    constexpr int O4 = N8 >= 8 ? O8 / 2 : 16;
    if constexpr (N4 >= 4) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float send = (lane & O4) ? v[k] : v[k + 2];
            const float keep = (lane & O4) ? v[k + 2] : v[k];
            v[k] = keep + __shfl_xor_sync(0xffffffffu, send, O4);
        }
    }
    constexpr int N2 = N4 >= 4 ? 2 : N4;
    constexpr int O2 = N4 >= 4 ? O4 / 2 : 16;
    if constexpr (N2 >= 2) {
        const float send = (lane & O2) ? v[0] : v[1];
        const float keep = (lane & O2) ? v[1] : v[0];
        v[0] = keep + __shfl_xor_sync(0xffffffffu, send, O2);
    }
    constexpr int OR = N2 >= 2 ? O2 / 2 : 16;   // remaining plain butterfly steps
    float r = v[0];
#pragma unroll
    for (int o = OR; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

template <int VEC> struct VecLoad;
template <> struct VecLoad<4> {
    static __device__ __forceinline__ void ld(const float *p, float (&r)[4]) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(p));
        r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
    }
};
template <> struct VecLoad<2> {
    static __device__ __forceinline__ void ld(const float *p, float (&r)[2]) {
        const float2 v = __ldg(reinterpret_cast<const float2 *>(p));
        r[0] = v.x; r[1] = v.y;
    }
};

// Log-sum-exp merge of the ns splits of the G query heads of one (query, kv head) by the CTA that drew the last
// ticket: called by the ATT_WARPS compute warps together (named barrier 1), out of line so that the streaming loops
// of its callers keep their registers.  head0 = query * Hq + first head; scratch: ATT_WARPS * G * D floats of shared
// memory that the caller no longer needs.
template <int D, int G>
static __device__ __noinline__ void attn_merge_tail(const float *__restrict__ part, float *__restrict__ out, float *scratch, size_t head0,
                                                    int S, int ns) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // The tail is latency, not bandwidth: every load below is issued before the first one is consumed (a loop
    // of load -> use over the splits would pay one trip to L2 per split).
    // (max, sum) of every (head, split) in one round of loads, into the output staging buffer (free by now)
    float *s_ms = scratch;                          // [G][ns] maxima, then [G][ns] sums, then [G][ns] weights
    float *s_ls = s_ms + G * ns;
    float *s_w = s_ls + G * ns;                     // 3 G ns <= ATT_WARPS G D floats (ns <= 64 <= 4 D / 3)
    for (int i = threadIdx.x; i < G * ns; i += ATT_WARPS * 32) {
        const int g = i / ns, sidx = i - g * ns;
        const float2 ml = __ldcg(reinterpret_cast<const float2 *>(part + ((head0 + g) * S + sidx) * (D + 2)));
        s_ms[i] = ml.x;
        s_ls[i] = ml.y;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(ATT_WARPS * 32) : "memory");
    // weights w = exp(max_s - max) / sum: one warp per head, lanes over the splits
    for (int g = warp; g < G; g += ATT_WARPS) {
        float m = -INFINITY;
        for (int sidx = lane; sidx < ns; sidx += 32) m = fmaxf(m, s_ms[g * ns + sidx]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float l = 0.f;
        for (int sidx = lane; sidx < ns; sidx += 32) {
            const float w = expf(s_ms[g * ns + sidx] - m);
            s_w[g * ns + sidx] = w;
            l = fmaf(s_ls[g * ns + sidx], w, l);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        const float inv = 1.f / l;
        for (int sidx = lane; sidx < ns; sidx += 32) s_w[g * ns + sidx] *= inv;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(ATT_WARPS * 32) : "memory");
    constexpr int MB = 16;                          // splits loaded per batch
    constexpr int NO = (G * D + ATT_WARPS * 32 - 1) / (ATT_WARPS * 32);    // outputs per thread
    float acc[NO];
#pragma unroll
    for (int j = 0; j < NO; ++j) acc[j] = 0.f;
    for (int sb = 0; sb < ns; sb += MB) {
        float r[NO][MB];
#pragma unroll
        for (int j = 0; j < NO; ++j) {
            const int i = min(threadIdx.x + j * ATT_WARPS * 32, G * D - 1), g = i / D, d = i % D;
            const float *rec = part + (head0 + g) * S * (D + 2) + 2 + d;
#pragma unroll
            for (int u = 0; u < MB; ++u) r[j][u] = (sb + u < ns) ? __ldcg(rec + (size_t)(sb + u) * (D + 2)) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < NO; ++j) {
            const int g = min(threadIdx.x + j * ATT_WARPS * 32, G * D - 1) / D;
#pragma unroll
            for (int u = 0; u < MB; ++u) acc[j] = fmaf(r[j][u], (sb + u < ns) ? s_w[g * ns + sb + u] : 0.f, acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < NO; ++j) {
        const int i = threadIdx.x + j * ATT_WARPS * 32;
        if (i < G * D) out[head0 * D + i] = acc[j];
    }
}

// D: head dim (64 or 128); G: query heads per kv head; TT: tokens per warp tile (TT*G <= 32)
template <int D, int G, int TT, int CHUNK, class CT>
__global__ void __launch_bounds__(ATT_WARPS * 32)
skn_attn_split_kernel(const float *__restrict__ q, const CT *__restrict__ kc, const CT *__restrict__ vc,
                      const int32_t *__restrict__ len, const int32_t *__restrict__ start, int Hkv, int cap,
                      float scale, float *__restrict__ part, int S, int tq, int len_extra, float *__restrict__ out,
                      unsigned *__restrict__ tickets) {
    constexpr int VEC = D / 32;
    constexpr int NV = TT * G;
    constexpr int REP = 32 / NV;                 // lanes holding the same (token, head) score
    constexpr int TILES = CHUNK / (ATT_WARPS * TT);
    __shared__ float s_sc[CHUNK][G];         // scores, then probabilities
    __shared__ float s_red[ATT_WARPS][G];
    __shared__ float s_m[G], s_l[G];
    __shared__ float s_o[ATT_WARPS][G][D];

    // blockIdx.z = sequence * tq + t: query t of the tq most recent positions of its sequence
    // sees the cache up to and including its own token (tq = 1: plain decode)
    const int sp = blockIdx.x, kvh = blockIdx.y, bq = blockIdx.z, b = bq / tq;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // the length, the ring start and q are requested together: one trip to L2 instead of three in a row
    const int len_b = __ldg(len + b), s0 = __ldg(start + b);
    const int Hq = Hkv * G;
    float qv[G][VEC];
#pragma unroll
    for (int g = 0; g < G; ++g) VecLoad<VEC>::ld(q + ((size_t)bq * Hq + kvh * G + g) * D + lane * VEC, qv[g]);
    const int L = min(cap, max(0, len_b + len_extra - (tq - 1 - bq % tq)));     // never past the ring: ns <= S
    const int t0 = sp * CHUNK;
    if (t0 >= L) {
        // an empty sequence has no split to merge: its output is zero
        if (tickets && L == 0 && sp == 0)
            for (int i = threadIdx.x; i < G * D; i += ATT_WARPS * 32) out[((size_t)bq * Hkv * G + kvh * G) * D + i] = 0.f;
        return;
    }
    const int nt = min(CHUNK, L - t0);
    const size_t cache_rows = (size_t)(gridDim.z / tq) * Hkv * cap, head_row0 = ((size_t)b * Hkv + kvh) * cap;
    const KvHeadReader<CT, D, VEC> krd(kc, cache_rows, head_row0, lane), vrd(vc, cache_rows, head_row0, lane);
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < VEC; ++e) qv[g][e] *= scale;

    // short chunks (short contexts: latency matters, not bandwidth): the warp's first V tile is
    // requested before the scores are computed, so that its latency overlaps pass 1
    constexpr bool PREV = CHUNK <= 64;
    float v0[PREV ? TT : 1][VEC];
    if constexpr (PREV) {
        const int tl = warp * TT;
        if (tl < nt) {
#pragma unroll
            for (int j = 0; j < TT; ++j) {
                const int t = min(tl + j, nt - 1);
                vrd.ld((s0 + t0 + t) % cap, v0[j]);
            }
        }
    }

    // ---- pass 1: scores ------------------------------------------------------------------
    float mrun = -INFINITY;   // this lane's head only (head = value index % G)
    const int vidx = lane / REP;          // value index held after the transposed reduce
    const int my_j = vidx / G, my_g = vidx % G;
#pragma unroll 2
    for (int ti = 0; ti < TILES; ++ti) {
        const int tl = (ti * ATT_WARPS + warp) * TT;      // first token of the tile within the chunk
        if (tl >= nt) break;
        float kr[TT][VEC];
#pragma unroll
        for (int j = 0; j < TT; ++j) {
            const int t = min(tl + j, nt - 1);            // clamp: the extra scores are discarded
            const int slot = (s0 + t0 + t) % cap;
            krd.ld(slot, kr[j]);
        }
        float pv[NV];
#pragma unroll
        for (int j = 0; j < TT; ++j)
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float a = 0.f;
#pragma unroll
                for (int e = 0; e < VEC; ++e) a = fmaf(qv[g][e], kr[j][e], a);
                pv[j * G + g] = a;
            }
        const float sc = warp_transpose_reduce<NV>(pv, lane);
        const bool valid = tl + my_j < nt;
        if (valid) {
            if ((lane % REP) == 0) s_sc[tl + my_j][my_g] = sc;
            mrun = fmaxf(mrun, sc);
        }
    }
    // max over the lanes that hold the same head: lane bits above log2(REP * G)
#pragma unroll
    for (int o = 16; o >= REP * G; o >>= 1) mrun = fmaxf(mrun, __shfl_xor_sync(0xffffffffu, mrun, o));
    if (lane < REP * G && (lane % REP) == 0) s_red[warp][lane / REP] = mrun;
    __syncthreads();
    if (threadIdx.x < G) {
        float m = s_red[0][threadIdx.x];
#pragma unroll
        for (int w = 1; w < ATT_WARPS; ++w) m = fmaxf(m, s_red[w][threadIdx.x]);
        s_m[threadIdx.x] = m;
    }
    __syncthreads();
    // probabilities in place + their sums
    float lsum[G];
#pragma unroll
    for (int g = 0; g < G; ++g) lsum[g] = 0.f;
    for (int t = threadIdx.x; t < nt; t += ATT_WARPS * 32) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float p = expf(s_sc[t][g] - s_m[g]);
            s_sc[t][g] = p;
            lsum[g] += p;
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lsum[g] += __shfl_xor_sync(0xffffffffu, lsum[g], o);
    }
    __syncthreads();            // s_red is reused
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) s_red[warp][g] = lsum[g];
    }
    __syncthreads();
    if (threadIdx.x < G) {
        float l = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) l += s_red[w][threadIdx.x];
        s_l[threadIdx.x] = l;
    }

    // ---- pass 2: probabilities x V ---------------------------------------------------------
    float o[G][VEC];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[g][e] = 0.f;
#pragma unroll 2
    for (int ti = 0; ti < TILES; ++ti) {
        const int tl = (ti * ATT_WARPS + warp) * TT;
        if (tl >= nt) break;
        float vr[TT][VEC];
        if (PREV && ti == 0) {
#pragma unroll
            for (int j = 0; j < TT; ++j)
#pragma unroll
                for (int e = 0; e < VEC; ++e) vr[j][e] = v0[j][e];
        } else {
#pragma unroll
            for (int j = 0; j < TT; ++j) {
                const int t = min(tl + j, nt - 1);
                const int slot = (s0 + t0 + t) % cap;
                vrd.ld(slot, vr[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < TT; ++j) {
            if (tl + j < nt) {
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float p = s_sc[tl + j][g];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) o[g][e] = fmaf(p, vr[j][e], o[g][e]);
                }
            }
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < VEC; ++e) s_o[warp][g][lane * VEC + e] = o[g][e];
    __syncthreads();
    // partial record per (head, split): [0] = max, [1] = sum, [2 .. 2+D) = unnormalised output
    for (int i = threadIdx.x; i < G * D; i += ATT_WARPS * 32) {
        const int g = i / D, d = i % D;
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) a += s_o[w][g][d];
        float *rec = part + (((size_t)bq * Hq + kvh * G + g) * S + sp) * (D + 2);
        rec[2 + d] = a;
        if (d == 0) { rec[0] = s_m[g]; rec[1] = s_l[g]; }
    }
    if (!tickets) return;
    // merge without a second launch: the CTA that draws the last ticket of its (query, kv head)
    // combines the splits (log-sum-exp) and hands the ticket counter back as zero
    __shared__ bool s_last;
    __threadfence();
    __syncthreads();
    const int ns = (L + CHUNK - 1) / CHUNK;
    if (threadIdx.x == 0) s_last = atomicAdd(&tickets[bq * Hkv + kvh], 1u) == (unsigned)(ns - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    attn_merge_tail<D, G>(part, out, &s_o[0][0][0], (size_t)bq * Hq + kvh * G, S, ns);
    if (threadIdx.x == 0) tickets[bq * Hkv + kvh] = 0;
}

// The same split attention for long contexts (256-token chunks, grids of several CTAs per SM: the
// bandwidth-bound regime), fed by bulk async copies instead of per-lane global loads.  All tokens
// of a (sequence, kv head) are contiguous in the ring, so a tile of ATT_WARPS * TT tokens is one
// copy (two where the ring wraps).  A producer warp streams the chunk's K tiles and then its V tiles
// through `nst` stages of shared memory (full / empty mbarriers); the four compute warps read their
// tokens of a tile from shared memory.  V tiles are already on their way while the scores, the
// chunk maximum and the probabilities are computed, so HBM stays busy across the two passes.
// Writes the (max, sum, unnormalised output) record per (head, split); the merge kernel follows.
template <int D, int G, int TT, class CT>
__global__ void __launch_bounds__((ATT_WARPS + 1) * 32, 5)       // five CTAs per SM (44.5 KB each): at most 80 registers
skn_attn_stream_kernel(const float *__restrict__ q, const CT *__restrict__ kc, const CT *__restrict__ vc,
                       const int32_t *__restrict__ len, const int32_t *__restrict__ start, int Hkv, int cap,
                       float scale, float *__restrict__ part, int S, int tq, int len_extra, int nst,
                       int32_t *__restrict__ status, float *__restrict__ out, unsigned *__restrict__ tickets) {
    constexpr int CHUNK = ATT_CHUNK;
    constexpr int VEC = D / 32;
    constexpr int NV = TT * G;
    constexpr int REP = 32 / NV;
    constexpr int TILE = ATT_WARPS * TT;             // tokens per stage
    constexpr int TILE_BYTES = TILE * D * (int)sizeof(CT);
    extern __shared__ __align__(128) uint8_t att_smem[];
    __shared__ float s_sc[CHUNK][G];
    __shared__ float s_red[ATT_WARPS][G];
    __shared__ float s_m[G], s_l[G];
    __shared__ float s_o[ATT_WARPS][G][D];
    uint64_t *full = reinterpret_cast<uint64_t *>(att_smem + (size_t)nst * TILE_BYTES);
    uint64_t *empty = full + nst;

    const int sp = blockIdx.x, kvh = blockIdx.y, bq = blockIdx.z, b = bq / tq;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int L = min(cap, max(0, len[b] + len_extra - (tq - 1 - bq % tq)));     // never past the ring: ns <= S
    const int t0 = sp * CHUNK;
    if (t0 >= L) {
        // an empty sequence has no split to merge: its output is zero
        if (tickets && L == 0 && sp == 0)
            for (int i = threadIdx.x; i < G * D; i += (ATT_WARPS + 1) * 32) out[((size_t)bq * Hkv * G + kvh * G) * D + i] = 0.f;
        return;
    }
    const int nt = min(CHUNK, L - t0);
    const int ntile = (nt + TILE - 1) / TILE;
    const int s0 = start[b];
    const int Hq = Hkv * G;
    const size_t head = ((size_t)b * Hkv + kvh) * cap * D;

    if (threadIdx.x == 0) {
        for (int i = 0; i < nst; ++i) {
            skn_mbar_init(&full[i], 1);
            skn_mbar_init(&empty[i], ATT_WARPS);
        }
        skn_fence_mbar_init();
    }
    __syncthreads();

    if (warp == ATT_WARPS) {
        // ---- producer: K tiles 0 .. ntile-1, then V tiles 0 .. ntile-1 ----
        if (lane == 0) {
            bool failed = false;
            for (int i = 0; i < 2 * ntile; ++i) {
                const int stg = i % nst;
                if (i >= nst && !failed && !skn_mbar_wait(&empty[stg], (uint32_t)(i / nst - 1) & 1u)) {
                    failed = true;
                    atomicExch(status, SKN_ERR_TIMEOUT);
                }
                const int tile = i < ntile ? i : i - ntile;
                const CT *src = (i < ntile ? kc : vc) + head;
                const int ntok = min(TILE, nt - tile * TILE);
                const int slot0 = (s0 + t0 + tile * TILE) % cap;
                const int n1 = min(ntok, cap - slot0);          // tokens before the ring wraps
                uint8_t *dst = att_smem + (size_t)stg * TILE_BYTES;
                skn_fence_proxy_async();
                constexpr uint32_t ROW = D * (uint32_t)sizeof(CT);
                skn_mbar_expect_tx(&full[stg], (uint32_t)ntok * ROW);
                skn_bulk_g2s(dst, src + (size_t)slot0 * D, (uint32_t)n1 * ROW, &full[stg]);
                if (ntok > n1) skn_bulk_g2s(dst + (size_t)n1 * ROW, src, (uint32_t)(ntok - n1) * ROW, &full[stg]);
            }
        }
        return;
    }

    float qv[G][VEC];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        VecLoad<VEC>::ld(q + ((size_t)bq * Hq + kvh * G + g) * D + lane * VEC, qv[g]);
#pragma unroll
        for (int e = 0; e < VEC; ++e) qv[g][e] *= scale;
    }
    bool failed = false;
    auto wait_full = [&](int i) {
        if (!failed && !skn_mbar_wait(&full[i % nst], (uint32_t)(i / nst) & 1u)) {
            failed = true;
            atomicExch(status, SKN_ERR_TIMEOUT);
        }
    };
    auto tile_row = [&](int i, int local) -> const CT * {
        return reinterpret_cast<const CT *>(att_smem + (size_t)(i % nst) * TILE_BYTES) + (size_t)local * D + lane * VEC;
    };

    // ---- pass 1: scores ------------------------------------------------------------------
    float mrun = -INFINITY;
    const int vidx = lane / REP;
    const int my_j = vidx / G, my_g = vidx % G;
    for (int ti = 0; ti < ntile; ++ti) {
        wait_full(ti);
        const int tl = ti * TILE + warp * TT;             // first token of this warp within the chunk
        const int last = min(TILE, nt - ti * TILE) - 1;   // last valid token of the tile
        if (tl < nt) {
            float kr[TT][VEC];
#pragma unroll
            for (int j = 0; j < TT; ++j) {
                KvLoad<CT, VEC, false>::ld(tile_row(ti, min(warp * TT + j, last)), kr[j]);
            }
            float pv[NV];
#pragma unroll
            for (int j = 0; j < TT; ++j)
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    float a = 0.f;
#pragma unroll
                    for (int e = 0; e < VEC; ++e) a = fmaf(qv[g][e], kr[j][e], a);
                    pv[j * G + g] = a;
                }
            const float sc = warp_transpose_reduce<NV>(pv, lane);
            if (tl + my_j < nt) {
                if ((lane % REP) == 0) s_sc[tl + my_j][my_g] = sc;
                mrun = fmaxf(mrun, sc);
            }
        }
        __syncwarp();
        if (lane == 0) skn_mbar_arrive(&empty[ti % nst]);
    }
    constexpr int NT = ATT_WARPS * 32;
    auto bar = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(NT) : "memory"); };
#pragma unroll
    for (int o = 16; o >= REP * G; o >>= 1) mrun = fmaxf(mrun, __shfl_xor_sync(0xffffffffu, mrun, o));
    if (lane < REP * G && (lane % REP) == 0) s_red[warp][lane / REP] = mrun;
    bar();
    if (threadIdx.x < G) {
        float m = s_red[0][threadIdx.x];
#pragma unroll
        for (int w = 1; w < ATT_WARPS; ++w) m = fmaxf(m, s_red[w][threadIdx.x]);
        s_m[threadIdx.x] = m;
    }
    bar();
    float lsum[G];
#pragma unroll
    for (int g = 0; g < G; ++g) lsum[g] = 0.f;
    for (int t = threadIdx.x; t < nt; t += NT) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float p = expf(s_sc[t][g] - s_m[g]);
            s_sc[t][g] = p;
            lsum[g] += p;
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lsum[g] += __shfl_xor_sync(0xffffffffu, lsum[g], o);
    }
    bar();                      // s_red is reused
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) s_red[warp][g] = lsum[g];
    }
    bar();
    if (threadIdx.x < G) {
        float l = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) l += s_red[w][threadIdx.x];
        s_l[threadIdx.x] = l;
    }

    // ---- pass 2: probabilities x V ---------------------------------------------------------
    float o[G][VEC];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[g][e] = 0.f;
    for (int ti = 0; ti < ntile; ++ti) {
        const int i = ntile + ti;
        wait_full(i);
        const int tl = ti * TILE + warp * TT;
        if (tl < nt) {
#pragma unroll
            for (int j = 0; j < TT; ++j) {
                if (tl + j < nt) {
                    float vr[VEC];
                    KvLoad<CT, VEC, false>::ld(tile_row(i, warp * TT + j), vr);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float pr = s_sc[tl + j][g];
#pragma unroll
                        for (int e = 0; e < VEC; ++e) o[g][e] = fmaf(pr, vr[e], o[g][e]);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) skn_mbar_arrive(&empty[i % nst]);
    }
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < VEC; ++e) s_o[warp][g][lane * VEC + e] = o[g][e];
    bar();
    for (int i = threadIdx.x; i < G * D; i += NT) {
        const int g = i / D, d = i % D;
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) a += s_o[w][g][d];
        float *rec = part + (((size_t)bq * Hq + kvh * G + g) * S + sp) * (D + 2);
        rec[2 + d] = a;
        if (d == 0) { rec[0] = s_m[g]; rec[1] = s_l[g]; }
    }
    if (!tickets) return;
    // merge without a second launch (single-token decode): the CTA that draws the last ticket of its (sequence, kv
    // head) combines the splits; the merge itself is a call, so the loops above keep their register count
    __shared__ bool s_last;
    __threadfence();
    bar();
    const int ns = (L + CHUNK - 1) / CHUNK;
    if (threadIdx.x == 0) s_last = atomicAdd(&tickets[bq * Hkv + kvh], 1u) == (unsigned)(ns - 1);
    bar();
    if (!s_last) return;
    __threadfence();
    attn_merge_tail<D, G>(part, out, &s_o[0][0][0], (size_t)bq * Hq + kvh * G, S, ns);
    if (threadIdx.x == 0) tickets[bq * Hkv + kvh] = 0;
}

// Log-sum-exp merge of the splits of one (query, head): D threads.  The splits' maxima and sums are
// reduced across the block first; every thread then adds up its output element with the loads of eight
// splits in flight at a time (the records sit in L2: the loop is bound by their latency).
template <int D>
__global__ void __launch_bounds__(D)
skn_attn_merge_kernel(const float *__restrict__ part, const int32_t *__restrict__ len, int Hq, int S,
                      float *__restrict__ out, int tq, int chunk, int len_extra, int cap) {
    const int h = blockIdx.x, b = blockIdx.y;          // b = sequence * tq + t
    const int L = min(cap, max(0, len[b / tq] + len_extra - (tq - 1 - b % tq)));
    const int ns = (L + chunk - 1) / chunk;
    const int d = threadIdx.x, lane = d & 31, warp = d >> 5;
    constexpr int NW = D / 32;
    const float *rec = part + ((size_t)b * Hq + h) * S * (D + 2);
    __shared__ float s_red[2][NW];
    if (ns == 0) {
        out[((size_t)b * Hq + h) * D + d] = 0.f;
        return;
    }
    float m = -INFINITY;
    for (int s = d; s < ns; s += D) m = fmaxf(m, rec[(size_t)s * (D + 2)]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) s_red[0][warp] = m;
    __syncthreads();
    m = s_red[0][0];
#pragma unroll
    for (int w = 1; w < NW; ++w) m = fmaxf(m, s_red[0][w]);
    float l = 0.f;
    for (int s = d; s < ns; s += D) l = fmaf(rec[(size_t)s * (D + 2) + 1], expf(rec[(size_t)s * (D + 2)] - m), l);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) s_red[1][warp] = l;
    __syncthreads();
    l = s_red[1][0];
#pragma unroll
    for (int w = 1; w < NW; ++w) l += s_red[1][w];
    float a = 0.f;
    for (int s0 = 0; s0 < ns; s0 += 8) {
        float v[8], e[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int ss = min(s0 + k, ns - 1);
            v[k] = rec[(size_t)ss * (D + 2) + 2 + d];
            e[k] = rec[(size_t)ss * (D + 2)];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (s0 + k < ns) a = fmaf(v[k], expf(e[k] - m), a);
    }
    out[((size_t)b * Hq + h) * D + d] = a / l;
}

template <int D, int G, class CT>
static cudaError_t launch_attn(const skn_kvcache *kv, const float *q, float scale, float *part, int chunk, float *out,
                               cudaStream_t stream, int tq, int len_extra) {
    constexpr int TT = (G >= 8) ? 4 : 8;
    const CT *kc = static_cast<const CT *>(kv->d_k), *vc = static_cast<const CT *>(kv->d_v);
    const int S = (kv->capacity + chunk - 1) / chunk;
    const dim3 grid((unsigned)S, (unsigned)kv->n_kv_heads, (unsigned)(kv->batch * tq));
    // single-token decode: the last split of every (sequence, kv head) merges in the same launch;
    // sequences without any cached token are left to the merge kernel (it writes their zeros)
    // (small grids only: with many CTAs per SM a merge launch costs less than the serial tails)
    const bool small_grid = (int64_t)S * kv->n_kv_heads * kv->batch <= 2 * (int64_t)kv->ctx->sm_count;
    static const int big_tickets = skn_tune_int("SKN_ATTN_BIG_TICKETS", 1);
    const bool streamed_shape = !KvIsQ8<CT>::value && chunk == ATT_CHUNK && !small_grid;
    unsigned *tickets = (tq == 1 && (small_grid || (streamed_shape && big_tickets)) && S <= ATT_MERGE_MAX_SPLITS && S <= chunk) ? kv->d_tickets : nullptr;
    // long contexts: tiles by bulk async copy through a shared-memory ring (quantised caches: per-lane loads at every length)
    const bool streamed = streamed_shape || (!KvIsQ8<CT>::value && chunk == ATT_CHUNK && !tickets);
    if constexpr (!KvIsQ8<CT>::value) if (streamed) {
        constexpr int TILE_BYTES = ATT_WARPS * TT * D * (int)sizeof(CT);
        // two stages: measured, more resident CTAs per SM (five at 44 KB each for D = 128, G = 4) beat a deeper ring
        constexpr int nst = 2;
        const size_t smem = (size_t)nst * TILE_BYTES + 2 * (size_t)nst * sizeof(uint64_t);
        auto kern = skn_attn_stream_kernel<D, G, TT, CT>;
        const uint32_t cfg_bit = 1u << ((sizeof(CT) == 2 ? 8 : 0) + (D == 128 ? 4 : 0) + (G == 1 ? 0 : (G == 2 ? 1 : (G == 4 ? 2 : 3))));
        if (!(kv->ctx->attn_stream_cfg & cfg_bit)) {
            cudaError_t e0 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(100 * 1024));
            if (e0 == cudaSuccess) e0 = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            if (e0 != cudaSuccess) return e0;
            kv->ctx->attn_stream_cfg |= cfg_bit;
        }
        kern<<<grid, (ATT_WARPS + 1) * 32, smem, stream>>>(q, kc, vc, kv->d_len, kv->d_start, kv->n_kv_heads, kv->capacity,
                                                          scale, part, S, tq, len_extra, nst, kv->ctx->d_status, out, tickets);
    }
    if (streamed) {
        // (launched above)
    } else if (chunk == 32)
        // (plain stream order: with a programmatic dependent launch, early or late release of its own dependents, a
        // decode step measured 0.4 to 1.8 % slower)
        skn_attn_split_kernel<D, G, TT, 32, CT><<<grid, ATT_WARPS * 32, 0, stream>>>(q, kc, vc, kv->d_len, kv->d_start,
                                                                                kv->n_kv_heads, kv->capacity, scale, part, S, tq, len_extra, out, tickets);
    else if (chunk == 64)
        skn_attn_split_kernel<D, G, TT, 64, CT><<<grid, ATT_WARPS * 32, 0, stream>>>(q, kc, vc, kv->d_len, kv->d_start,
                                                                                kv->n_kv_heads, kv->capacity, scale, part, S, tq, len_extra, out, tickets);
    else
        skn_attn_split_kernel<D, G, TT, ATT_CHUNK, CT><<<grid, ATT_WARPS * 32, 0, stream>>>(q, kc, vc, kv->d_len, kv->d_start,
                                                                                       kv->n_kv_heads, kv->capacity, scale, part, S, tq, len_extra, out, tickets);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || tickets) return e;
    const dim3 g2((unsigned)(kv->n_kv_heads * G), (unsigned)(kv->batch * tq));
    skn_attn_merge_kernel<D><<<g2, D, 0, stream>>>(part, kv->d_len, kv->n_kv_heads * G, S, out, tq, chunk, len_extra, kv->capacity);
    return cudaGetLastError();
}

static int attn_pick_chunk(const skn_kvcache *kv, int n_q_heads, int tq, size_t scratch_cap) {
    // finer splits while 256-token (then 64-token) chunks leave SMs idle (short contexts, small
    // batches) and the partials of the finer split fit `scratch_cap` bytes
    const int chunks[3] = {ATT_CHUNK, 64, 32};
    int pick = ATT_CHUNK;
    static const int forced = skn_tune_int("SKN_ATTN_CHUNK", 0);
    if (forced == 32 || forced == 64 || forced == ATT_CHUNK) {
        const int64_t S = (kv->capacity + forced - 1) / forced;
        if ((size_t)((int64_t)kv->batch * tq * n_q_heads * S * (kv->head_dim + 2) * 4) <= scratch_cap) return forced;
    }
    for (int i = 0; i < 3; ++i) {
        const int c = chunks[i];
        const int64_t S = (kv->capacity + c - 1) / c;
        const int64_t need = (int64_t)kv->batch * tq * n_q_heads * S * (kv->head_dim + 2) * 4;
        if ((size_t)need > scratch_cap) break;
        pick = c;
        if ((int64_t)kv->batch * tq * kv->n_kv_heads * S >= 2 * (int64_t)kv->ctx->sm_count) break;
    }
    return pick;
}

template <class CT>
static cudaError_t dispatch_attn_t(const skn_kvcache *kv, int G, const float *q, float scale, float *part, int chunk,
                                   float *out, cudaStream_t st, int tq, int len_extra) {
    if (kv->head_dim == 128) {
        switch (G) {
        case 1: return launch_attn<128, 1, CT>(kv, q, scale, part, chunk, out, st, tq, len_extra);
        case 2: return launch_attn<128, 2, CT>(kv, q, scale, part, chunk, out, st, tq, len_extra);
        case 4: return launch_attn<128, 4, CT>(kv, q, scale, part, chunk, out, st, tq, len_extra);
        case 8: return launch_attn<128, 8, CT>(kv, q, scale, part, chunk, out, st, tq, len_extra);
        }
    } else if (kv->head_dim == 64) {
        switch (G) {
        case 1: return launch_attn<64, 1, CT>(kv, q, scale, part, chunk, out, st, tq, len_extra);
        case 2: return launch_attn<64, 2, CT>(kv, q, scale, part, chunk, out, st, tq, len_extra);
        case 4: return launch_attn<64, 4, CT>(kv, q, scale, part, chunk, out, st, tq, len_extra);
        case 8: return launch_attn<64, 8, CT>(kv, q, scale, part, chunk, out, st, tq, len_extra);
        }
    }
    return cudaErrorInvalidValue;
}

static cudaError_t dispatch_attn(const skn_kvcache *kv, int G, const float *q, float scale, float *part, int chunk,
                                 float *out, cudaStream_t st, int tq = 1, int len_extra = 0) {
    if (kv->dtype == SKN_KV_Q8_0) return dispatch_attn_t<skn_q8>(kv, G, q, scale, part, chunk, out, st, tq, len_extra);
    return kv->dtype == SKN_KV_F16 ? dispatch_attn_t<__half>(kv, G, q, scale, part, chunk, out, st, tq, len_extra)
                                   : dispatch_attn_t<float>(kv, G, q, scale, part, chunk, out, st, tq, len_extra);
}

// ----------------------------------------------------------------------------------------
extern "C" {

int32_t skn_kv_create(skn_ctx *ctx, int32_t batch, int32_t n_kv_heads, int32_t head_dim, int32_t capacity,
                      skn_kvcache **out) {
    return skn_kv_create_typed(ctx, batch, n_kv_heads, head_dim, capacity, SKN_KV_F32, out);
}

int32_t skn_kv_create_typed(skn_ctx *ctx, int32_t batch, int32_t n_kv_heads, int32_t head_dim, int32_t capacity,
                            int32_t kv_dtype, skn_kvcache **out) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    SKN_ENTER(ctx);
    if (!out) return skn_fail(ctx, SKN_ERR_ARG, "out is NULL");
    *out = nullptr;
    if (kv_dtype != SKN_KV_F32 && kv_dtype != SKN_KV_F16 && kv_dtype != SKN_KV_Q8_0)
        return skn_fail(ctx, SKN_ERR_TYPE, "cache element type %d is none of fp32, fp16, Q8_0", kv_dtype);
    if (batch < 1 || n_kv_heads < 1 || capacity < 1) return skn_fail(ctx, SKN_ERR_ARG, "batch, heads and capacity must be positive");
    if (head_dim != 64 && head_dim != 128) return skn_fail(ctx, SKN_ERR_SHAPE, "head_dim must be 64 or 128 (got %d)", head_dim);
    skn_kvcache *kv = new (std::nothrow) skn_kvcache();
    if (!kv) return skn_fail(ctx, SKN_ERR_OOM, "host allocation failed");
    memset(kv, 0, sizeof(*kv));
    kv->magic = SKN_MAGIC_KV;
    kv->ctx = ctx;
    kv->batch = batch; kv->n_kv_heads = n_kv_heads; kv->head_dim = head_dim; kv->capacity = capacity;
    kv->dtype = kv_dtype;
    // Q8_0: an int8 plane, then the fp16 scales of its 32-dim blocks
    const size_t elems = (size_t)batch * n_kv_heads * capacity * head_dim;
    const size_t n = kv_dtype == SKN_KV_Q8_0 ? elems + elems / 32 * 2 : elems * (kv_dtype == SKN_KV_F16 ? 2 : sizeof(float));
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e == cudaSuccess) e = cudaMalloc((void **)&kv->d_k, n);
    if (e == cudaSuccess) e = cudaMalloc((void **)&kv->d_v, n);
    const size_t n_ints = (size_t)2 * batch + (size_t)batch * n_kv_heads;     // lengths, starts, merge tickets
    if (e == cudaSuccess) e = cudaMalloc((void **)&kv->d_len, n_ints * sizeof(int32_t));
    if (e == cudaSuccess) {
        kv->d_start = kv->d_len + batch;
        kv->d_tickets = reinterpret_cast<unsigned *>(kv->d_len + 2 * batch);
        e = cudaMemsetAsync(kv->d_len, 0, n_ints * sizeof(int32_t), ctx->stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        if (kv->d_k) cudaFree(kv->d_k);
        if (kv->d_v) cudaFree(kv->d_v);
        if (kv->d_len) cudaFree(kv->d_len);
        kv->magic = 0;
        delete kv;
        return skn_check_cuda(ctx, e, "kv cache allocation");
    }
    *out = kv;
    return SKN_OK;
}

int32_t skn_kv_destroy(skn_kvcache *kv) {
    if (!kv || kv->magic != SKN_MAGIC_KV) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad kv cache handle");
    if (skn_ctx_ok(kv->ctx)) {
        cudaSetDevice(kv->ctx->device);
        cudaStreamSynchronize(kv->ctx->stream);
    }
    cudaFree(kv->d_k);
    cudaFree(kv->d_v);
    cudaFree(kv->d_len);
    kv->magic = 0;
    delete kv;
    return SKN_OK;
}

int32_t skn_kv_reset(skn_kvcache *kv) {
    if (!kv_ok(kv)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad kv cache handle");
    skn_ctx *ctx = kv->ctx;
    SKN_ENTER(ctx);
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    SKN_CUDA(ctx, cudaMemsetAsync(kv->d_len, 0, 2 * sizeof(int32_t) * kv->batch, ctx->stream));
    return SKN_OK;
}

int32_t skn_kv_load(skn_kvcache *kv, const float *k_host, const float *v_host, int32_t tokens,
                    const int32_t *lens_host) {
    if (!kv_ok(kv)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad kv cache handle");
    skn_ctx *ctx = kv->ctx;
    SKN_ENTER(ctx);
    if (tokens < 0 || tokens > kv->capacity) return skn_fail(ctx, SKN_ERR_SHAPE, "tokens (%d) exceeds the capacity (%d)", tokens, kv->capacity);
    if (!lens_host || (tokens > 0 && (!k_host || !v_host))) return skn_fail(ctx, SKN_ERR_ARG, "NULL argument");
    for (int b = 0; b < kv->batch; ++b)
        if (lens_host[b] < 0 || lens_host[b] > tokens)
            return skn_fail(ctx, SKN_ERR_SHAPE, "lens[%d] = %d outside [0, %d]", b, lens_host[b], tokens);
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t row = (size_t)tokens * kv->head_dim * sizeof(float);
    const size_t pitch = (size_t)kv->capacity * kv->head_dim * sizeof(float);
    const size_t nrows = (size_t)kv->batch * kv->n_kv_heads;
    if (tokens > 0 && kv->dtype != SKN_KV_F32) {
        // fp32 rows to a staging buffer, one tensor at a time, then rounded / quantised into the cache
        const int32_t rc = skn_stage_reserve(ctx, &ctx->d_stage_in, &ctx->d_stage_in_bytes, row * nrows);
        if (rc) return rc;
        const int64_t n4 = (int64_t)nrows * tokens * kv->head_dim / 4;
        int blocks = (int)((n4 + 255) / 256 < (int64_t)ctx->sm_count * 16 ? (n4 + 255) / 256 : (int64_t)ctx->sm_count * 16);
        for (int which = 0; which < 2; ++which) {
            SKN_CUDA(ctx, cudaMemcpyAsync(ctx->d_stage_in, which ? v_host : k_host, row * nrows, cudaMemcpyHostToDevice, ctx->stream));
            if (kv->dtype == SKN_KV_F16)
                skn_kv_load_conv_kernel<__half><<<blocks, 256, 0, ctx->stream>>>((const float *)ctx->d_stage_in,
                                                                                 static_cast<__half *>(which ? kv->d_v : kv->d_k),
                                                                                 (int64_t)nrows, tokens, kv->head_dim, kv->capacity);
            else
                skn_kv_load_conv_kernel<skn_q8><<<blocks, 256, 0, ctx->stream>>>((const float *)ctx->d_stage_in,
                                                                                 static_cast<skn_q8 *>(which ? kv->d_v : kv->d_k),
                                                                                 (int64_t)nrows, tokens, kv->head_dim, kv->capacity);
            SKN_CUDA(ctx, cudaGetLastError());
        }
    } else if (tokens > 0) {
        SKN_CUDA(ctx, cudaMemcpy2DAsync(kv->d_k, pitch, k_host, row, row, nrows, cudaMemcpyHostToDevice, ctx->stream));
        SKN_CUDA(ctx, cudaMemcpy2DAsync(kv->d_v, pitch, v_host, row, row, nrows, cudaMemcpyHostToDevice, ctx->stream));
    }
    SKN_CUDA(ctx, cudaMemcpyAsync(kv->d_len, lens_host, sizeof(int32_t) * kv->batch, cudaMemcpyHostToDevice, ctx->stream));
    SKN_CUDA(ctx, cudaMemsetAsync(kv->d_start, 0, sizeof(int32_t) * kv->batch, ctx->stream));
    SKN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return SKN_OK;
}

int32_t skn_kv_lengths(skn_kvcache *kv, int32_t *lens_host, int32_t *start_host) {
    if (!kv_ok(kv)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad kv cache handle");
    skn_ctx *ctx = kv->ctx;
    SKN_ENTER(ctx);
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    SKN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (lens_host) SKN_CUDA(ctx, cudaMemcpy(lens_host, kv->d_len, sizeof(int32_t) * kv->batch, cudaMemcpyDeviceToHost));
    if (start_host) SKN_CUDA(ctx, cudaMemcpy(start_host, kv->d_start, sizeof(int32_t) * kv->batch, cudaMemcpyDeviceToHost));
    return SKN_OK;
}

int32_t skn_kv_append_dev(skn_kvcache *kv, const float *k_new_dev, const float *v_new_dev) {
    if (!kv_ok(kv)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad kv cache handle");
    skn_ctx *ctx = kv->ctx;
    SKN_ENTER(ctx);
    if (!k_new_dev || !v_new_dev) return skn_fail(ctx, SKN_ERR_ARG, "NULL argument");
    if ((((uintptr_t)k_new_dev) | ((uintptr_t)v_new_dev)) & 15) return skn_fail(ctx, SKN_ERR_ALIGN, "k/v must be 16-byte aligned");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    if (kv->dtype == SKN_KV_Q8_0)
        skn_kv_append_kernel<skn_q8><<<kv->batch, 256, 0, ctx->stream>>>(static_cast<skn_q8 *>(kv->d_k), static_cast<skn_q8 *>(kv->d_v),
                                                                         kv->d_len, kv->d_start, k_new_dev, v_new_dev,
                                                                         kv->n_kv_heads, kv->head_dim, kv->capacity);
    else if (kv->dtype == SKN_KV_F16)
        skn_kv_append_kernel<__half><<<kv->batch, 256, 0, ctx->stream>>>(static_cast<__half *>(kv->d_k), static_cast<__half *>(kv->d_v),
                                                                         kv->d_len, kv->d_start, k_new_dev, v_new_dev,
                                                                         kv->n_kv_heads, kv->head_dim, kv->capacity);
    else
        skn_kv_append_kernel<float><<<kv->batch, 256, 0, ctx->stream>>>(static_cast<float *>(kv->d_k), static_cast<float *>(kv->d_v),
                                                                        kv->d_len, kv->d_start, k_new_dev, v_new_dev,
                                                                        kv->n_kv_heads, kv->head_dim, kv->capacity);
    SKN_CUDA(ctx, cudaGetLastError());
    return SKN_OK;
}

int32_t skn_kv_append(skn_kvcache *kv, const float *k_new_host, const float *v_new_host) {
    if (!kv_ok(kv)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad kv cache handle");
    skn_ctx *ctx = kv->ctx;
    SKN_ENTER(ctx);
    if (!k_new_host || !v_new_host) return skn_fail(ctx, SKN_ERR_ARG, "NULL argument");
    const size_t n = (size_t)kv->batch * kv->n_kv_heads * kv->head_dim * sizeof(float);
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    int32_t rc = skn_stage_reserve(ctx, &ctx->d_stage_in, &ctx->d_stage_in_bytes, 2 * n);
    if (rc) return rc;
    float *dk = (float *)ctx->d_stage_in, *dv = (float *)((uint8_t *)ctx->d_stage_in + n);
    SKN_CUDA(ctx, cudaMemcpyAsync(dk, k_new_host, n, cudaMemcpyHostToDevice, ctx->stream));
    SKN_CUDA(ctx, cudaMemcpyAsync(dv, v_new_host, n, cudaMemcpyHostToDevice, ctx->stream));
    rc = skn_kv_append_dev(kv, dk, dv);
    if (rc) return rc;
    return skn_sync(ctx);
}

int32_t skn_kv_gather(skn_kvcache *kv, int32_t b, int32_t pos_begin, int32_t count, float *k_out_host,
                      float *v_out_host) {
    if (!kv_ok(kv)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad kv cache handle");
    skn_ctx *ctx = kv->ctx;
    SKN_ENTER(ctx);
    if (b < 0 || b >= kv->batch) return skn_fail(ctx, SKN_ERR_ARG, "sequence index out of range");
    if (pos_begin < 0 || count < 0) return skn_fail(ctx, SKN_ERR_ARG, "negative range");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    int32_t L = 0;
    SKN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    SKN_CUDA(ctx, cudaMemcpy(&L, kv->d_len + b, sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (pos_begin + count > L) return skn_fail(ctx, SKN_ERR_SHAPE, "range [%d, %d) outside the %d cached tokens", pos_begin, pos_begin + count, L);
    if (count == 0) return SKN_OK;
    if (!k_out_host || !v_out_host) return skn_fail(ctx, SKN_ERR_ARG, "NULL output");
    const size_t n = (size_t)kv->n_kv_heads * count * kv->head_dim * sizeof(float);
    int32_t rc = skn_stage_reserve(ctx, &ctx->d_stage_out, &ctx->d_stage_out_bytes, 2 * n);
    if (rc) return rc;
    float *dk = (float *)ctx->d_stage_out, *dv = (float *)((uint8_t *)ctx->d_stage_out + n);
    const int64_t total = (int64_t)kv->n_kv_heads * count * kv->head_dim / 4;
    int blocks = (int)((total + 255) / 256);
    if (blocks > ctx->sm_count * 16) blocks = ctx->sm_count * 16;
    if (kv->dtype == SKN_KV_Q8_0)
        skn_kv_gather_kernel<skn_q8><<<blocks, 256, 0, ctx->stream>>>(static_cast<const skn_q8 *>(kv->d_k), static_cast<const skn_q8 *>(kv->d_v),
                                                                      kv->d_start, b, kv->n_kv_heads, kv->head_dim, kv->capacity,
                                                                      pos_begin, count, dk, dv, kv->batch);
    else if (kv->dtype == SKN_KV_F16)
        skn_kv_gather_kernel<__half><<<blocks, 256, 0, ctx->stream>>>(static_cast<const __half *>(kv->d_k), static_cast<const __half *>(kv->d_v),
                                                                      kv->d_start, b, kv->n_kv_heads, kv->head_dim, kv->capacity,
                                                                      pos_begin, count, dk, dv, kv->batch);
    else
        skn_kv_gather_kernel<float><<<blocks, 256, 0, ctx->stream>>>(static_cast<const float *>(kv->d_k), static_cast<const float *>(kv->d_v),
                                                                     kv->d_start, b, kv->n_kv_heads, kv->head_dim, kv->capacity,
                                                                     pos_begin, count, dk, dv, kv->batch);
    SKN_CUDA(ctx, cudaGetLastError());
    SKN_CUDA(ctx, cudaMemcpyAsync(k_out_host, dk, n, cudaMemcpyDeviceToHost, ctx->stream));
    SKN_CUDA(ctx, cudaMemcpyAsync(v_out_host, dv, n, cudaMemcpyDeviceToHost, ctx->stream));
    return skn_sync(ctx);
}

int64_t skn_attn_scratch_bytes(const skn_kvcache *kv, int32_t n_q_heads) {
    if (!kv_ok(kv) || n_q_heads < 1) return -1;
    const int64_t S = (kv->capacity + ATT_CHUNK - 1) / ATT_CHUNK;
    return (int64_t)kv->batch * n_q_heads * S * (kv->head_dim + 2) * (int64_t)sizeof(float);
}

static int32_t attn_check(skn_kvcache *kv, int32_t n_q_heads, const void *q, const void *out, int *G) {
    if (!kv_ok(kv)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad kv cache handle");
    skn_ctx *ctx = kv->ctx;
    SKN_ENTER(ctx);
    if (!q || !out) return skn_fail(ctx, SKN_ERR_ARG, "NULL argument");
    if (n_q_heads < 1 || n_q_heads % kv->n_kv_heads) return skn_fail(ctx, SKN_ERR_SHAPE, "Shapes do not align.");
    *G = n_q_heads / kv->n_kv_heads;
    if (*G != 1 && *G != 2 && *G != 4 && *G != 8)
        return skn_fail(ctx, SKN_ERR_SHAPE, "query heads per kv head must be 1, 2, 4 or 8 (got %d)", *G);
    return SKN_OK;
}

// scratch_dev: at least skn_attn_scratch_bytes() bytes of device memory, or NULL to use the
// context's own scratch allocation (grown on demand)
int32_t skn_attn_decode_dev(skn_kvcache *kv, const float *q_dev, int32_t n_q_heads, float scale, float *out_dev,
                            void *scratch_dev) {
    int G = 0;
    int32_t rc = attn_check(kv, n_q_heads, q_dev, out_dev, &G);
    if (rc) return rc;
    skn_ctx *ctx = kv->ctx;
    SKN_ENTER(ctx);
    if ((((uintptr_t)q_dev) | ((uintptr_t)out_dev) | ((uintptr_t)scratch_dev)) & 15)
        return skn_fail(ctx, SKN_ERR_ALIGN, "q, out and scratch must be 16-byte aligned");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    int chunk = ATT_CHUNK;
    float *part = (float *)scratch_dev;
    if (!part) {
        chunk = attn_pick_chunk(kv, n_q_heads, 1, (size_t)64 << 20);
        const int S = (kv->capacity + chunk - 1) / chunk;
        rc = skn_stage_reserve(ctx, &ctx->d_scratch2, &ctx->d_scratch2_bytes,
                               (size_t)kv->batch * n_q_heads * S * (kv->head_dim + 2) * sizeof(float));
        if (rc) return rc;
        part = (float *)ctx->d_scratch2;
    }
    SKN_CUDA(ctx, dispatch_attn(kv, G, q_dev, scale, part, chunk, out_dev, ctx->stream));
    return SKN_OK;
}

int32_t skn_attn_decode(skn_kvcache *kv, const float *q_host, int32_t n_q_heads, float scale, float *out_host) {
    int G = 0;
    int32_t rc = attn_check(kv, n_q_heads, q_host, out_host, &G);
    if (rc) return rc;
    skn_ctx *ctx = kv->ctx;
    SKN_ENTER(ctx);
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t n = (size_t)kv->batch * n_q_heads * kv->head_dim * sizeof(float);
    rc = skn_stage_reserve(ctx, &ctx->d_stage_in, &ctx->d_stage_in_bytes, n);
    if (rc) return rc;
    rc = skn_stage_reserve(ctx, &ctx->d_stage_out, &ctx->d_stage_out_bytes, n);
    if (rc) return rc;
    SKN_CUDA(ctx, cudaMemcpyAsync(ctx->d_stage_in, q_host, n, cudaMemcpyHostToDevice, ctx->stream));
    rc = skn_attn_decode_dev(kv, (const float *)ctx->d_stage_in, n_q_heads, scale, (float *)ctx->d_stage_out, nullptr);
    if (rc) return rc;
    SKN_CUDA(ctx, cudaMemcpyAsync(out_host, ctx->d_stage_out, n, cudaMemcpyDeviceToHost, ctx->stream));
    return skn_sync(ctx);
}

// Append T tokens per sequence (k_new, v_new: [batch][T][n_kv_heads][head_dim] on the device).
// host_len_upper is the caller's knowledge of the longest sequence before the call; the call
// is refused when host_len_upper + T would not fit the ring (a multi-token append never wraps).
int32_t skn_kv_append_many_dev(skn_kvcache *kv, const float *k_new_dev, const float *v_new_dev, int32_t T,
                               int32_t host_len_upper) {
    if (!kv_ok(kv)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad kv cache handle");
    skn_ctx *ctx = kv->ctx;
    SKN_ENTER(ctx);
    if (T < 0 || host_len_upper < 0) return skn_fail(ctx, SKN_ERR_ARG, "negative argument");
    if (T == 0) return SKN_OK;
    if (!k_new_dev || !v_new_dev) return skn_fail(ctx, SKN_ERR_ARG, "NULL argument");
    if ((((uintptr_t)k_new_dev) | ((uintptr_t)v_new_dev)) & 15) return skn_fail(ctx, SKN_ERR_ALIGN, "k/v must be 16-byte aligned");
    if ((int64_t)host_len_upper + T > kv->capacity)
        return skn_fail(ctx, SKN_ERR_SHAPE, "%d cached + %d new tokens exceed the capacity %d", host_len_upper, T, kv->capacity);
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    if (kv->dtype == SKN_KV_Q8_0)
        skn_kv_append_many_kernel<skn_q8><<<dim3((unsigned)T, (unsigned)kv->batch), 128, 0, ctx->stream>>>(
            static_cast<skn_q8 *>(kv->d_k), static_cast<skn_q8 *>(kv->d_v), kv->d_len, kv->d_start, k_new_dev, v_new_dev,
            kv->n_kv_heads, kv->head_dim, kv->capacity, T);
    else if (kv->dtype == SKN_KV_F16)
        skn_kv_append_many_kernel<__half><<<dim3((unsigned)T, (unsigned)kv->batch), 128, 0, ctx->stream>>>(
            static_cast<__half *>(kv->d_k), static_cast<__half *>(kv->d_v), kv->d_len, kv->d_start, k_new_dev, v_new_dev,
            kv->n_kv_heads, kv->head_dim, kv->capacity, T);
    else
        skn_kv_append_many_kernel<float><<<dim3((unsigned)T, (unsigned)kv->batch), 128, 0, ctx->stream>>>(
            static_cast<float *>(kv->d_k), static_cast<float *>(kv->d_v), kv->d_len, kv->d_start, k_new_dev, v_new_dev,
            kv->n_kv_heads, kv->head_dim, kv->capacity, T);
    SKN_CUDA(ctx, cudaGetLastError());
    skn_kv_advance_kernel<<<(kv->batch + 127) / 128, 128, 0, ctx->stream>>>(kv->d_len, kv->batch, T, kv->capacity);
    SKN_CUDA(ctx, cudaGetLastError());
    return SKN_OK;
}

// Causal attention of the T most recent positions of every sequence (after their K/V have been
// appended): q, out are [batch][T][n_q_heads][head_dim]; query t attends to the cache up to its
// own token.  T = 1 is skn_attn_decode_dev.  Scratch: T times skn_attn_scratch_bytes().
static int32_t attn_causal_impl(skn_kvcache *kv, const float *q_dev, int32_t n_q_heads, int32_t T, float scale,
                                float *out_dev, void *scratch_dev, int len_extra) {
    int G = 0;
    int32_t rc = attn_check(kv, n_q_heads, q_dev, out_dev, &G);
    if (rc) return rc;
    skn_ctx *ctx = kv->ctx;
    SKN_ENTER(ctx);
    if (T < 1) return skn_fail(ctx, SKN_ERR_ARG, "T must be positive");
    if ((int64_t)T * kv->batch > 65535) return skn_fail(ctx, SKN_ERR_SHAPE, "batch * T exceeds 65535");
    if ((((uintptr_t)q_dev) | ((uintptr_t)out_dev) | ((uintptr_t)scratch_dev)) & 15)
        return skn_fail(ctx, SKN_ERR_ALIGN, "q, out and scratch must be 16-byte aligned");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    int chunk = ATT_CHUNK;
    float *part = (float *)scratch_dev;
    if (!part) {
        chunk = attn_pick_chunk(kv, n_q_heads, T, (size_t)64 << 20);
        const int S = (kv->capacity + chunk - 1) / chunk;
        rc = skn_stage_reserve(ctx, &ctx->d_scratch2, &ctx->d_scratch2_bytes,
                               (size_t)kv->batch * T * n_q_heads * S * (kv->head_dim + 2) * sizeof(float));
        if (rc) return rc;
        part = (float *)ctx->d_scratch2;
    }
    SKN_CUDA(ctx, dispatch_attn(kv, G, q_dev, scale, part, chunk, out_dev, ctx->stream, T, len_extra));
    return SKN_OK;
}

int32_t skn_attn_causal_dev(skn_kvcache *kv, const float *q_dev, int32_t n_q_heads, int32_t T, float scale,
                            float *out_dev, void *scratch_dev) {
    return attn_causal_impl(kv, q_dev, n_q_heads, T, scale, out_dev, scratch_dev, 0);
}

}  // extern "C"

// ---- decoder-internal forms (skn_llama.cu): append without advancing, attention over the
// cache plus the T pending tokens, one advance for all layers
int32_t skn_kv_rope_append_pending(skn_kvcache *kv, float *q_dev, const float *k_new_dev, const float *v_new_dev,
                                   int32_t n_q_heads, int32_t T, float theta, int32_t host_len_upper) {
    if (!kv_ok(kv)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad kv cache handle");
    skn_ctx *ctx = kv->ctx;
    SKN_ENTER(ctx);
    if ((int64_t)host_len_upper + T > kv->capacity)
        return skn_fail(ctx, SKN_ERR_SHAPE, "%d cached + %d new tokens exceed the capacity %d", host_len_upper, T, kv->capacity);
    if ((int64_t)kv->batch > 65535 || T > 65535) return skn_fail(ctx, SKN_ERR_SHAPE, "batch or T exceeds 65535");
    const int pair_blocks = ((n_q_heads + kv->n_kv_heads) * (kv->head_dim / 2) + 127) / 128;
    const dim3 rgrid((unsigned)pair_blocks + 1, (unsigned)T, (unsigned)kv->batch);
    if (kv->dtype == SKN_KV_Q8_0)
        skn_rope_append_kernel<skn_q8><<<rgrid, 128, 0, ctx->stream>>>(
            q_dev, k_new_dev, v_new_dev, static_cast<skn_q8 *>(kv->d_k), static_cast<skn_q8 *>(kv->d_v), kv->d_len, kv->d_start,
            n_q_heads, kv->n_kv_heads, kv->head_dim, kv->capacity, T, log2((double)theta), ctx->d_status);
    else if (kv->dtype == SKN_KV_F16)
        skn_rope_append_kernel<__half><<<rgrid, 128, 0, ctx->stream>>>(
            q_dev, k_new_dev, v_new_dev, static_cast<__half *>(kv->d_k), static_cast<__half *>(kv->d_v), kv->d_len, kv->d_start,
            n_q_heads, kv->n_kv_heads, kv->head_dim, kv->capacity, T, log2((double)theta), ctx->d_status);
    else
        skn_rope_append_kernel<float><<<rgrid, 128, 0, ctx->stream>>>(
            q_dev, k_new_dev, v_new_dev, static_cast<float *>(kv->d_k), static_cast<float *>(kv->d_v), kv->d_len, kv->d_start,
            n_q_heads, kv->n_kv_heads, kv->head_dim, kv->capacity, T, log2((double)theta), ctx->d_status);
    SKN_CUDA(ctx, cudaGetLastError());
    return SKN_OK;
}

int32_t skn_attn_causal_pending(skn_kvcache *kv, const float *q_dev, int32_t n_q_heads, int32_t T, float scale,
                                float *out_dev) {
    return attn_causal_impl(kv, q_dev, n_q_heads, T, scale, out_dev, nullptr, T);
}

int32_t *skn_kv_len_dev(const skn_kvcache *kv) { return kv_ok(kv) ? kv->d_len : nullptr; }

cudaError_t skn_kv_advance_all(int32_t *const *lens_dev, int n_layers, int B, int T, int cap, int32_t *status_dev,
                               cudaStream_t st) {
    const int n = n_layers * B;
    if (n == 0) return cudaSuccess;
    skn_kv_advance_all_kernel<<<(n + 127) / 128, 128, 0, st>>>(lens_dev, n_layers, B, T, cap, status_dev);
    return cudaGetLastError();
}

extern "C" {

// ---- decode attention without any allocation -----------------------------------------------
// Some hosts may not allocate device memory at the moment they need attention: a serving loop
// whose memory budget was fixed at start-up, a caller inside a region where the CUDA allocator
// must not run (it synchronises the device), or a runtime that hands this library a device
// but no allocator at all.  For them the split partials live in the fixed array below, which
// every GPU that loads the library carries until the process exits.
constexpr int64_t SKN_ATTN_STATIC_SCRATCH_BYTES = 4ll << 20;   // 4 MiB
static __device__ __align__(256) float g_attn_static_scratch[SKN_ATTN_STATIC_SCRATCH_BYTES / sizeof(float)];
// Device address of the array per device.  The symbol's name is only a host-side stand-in;
// kernels must be given the address cudaGetSymbolAddress returns for the current device.
static float *g_attn_static_ptr[64] = {nullptr};

int32_t skn_attn_decode_noalloc_dev(skn_kvcache *kv, const float *q_dev, int32_t n_q_heads, float scale,
                                    float *out_dev) {
    int G = 0;
    int32_t rc = attn_check(kv, n_q_heads, q_dev, out_dev, &G);
    if (rc) return rc;
    skn_ctx *ctx = kv->ctx;
    SKN_ENTER(ctx);
    if ((((uintptr_t)q_dev) | ((uintptr_t)out_dev)) & 15) return skn_fail(ctx, SKN_ERR_ALIGN, "q and out must be 16-byte aligned");
    const int64_t need = skn_attn_scratch_bytes(kv, n_q_heads);
    if (need > SKN_ATTN_STATIC_SCRATCH_BYTES)
        return skn_fail(ctx, SKN_ERR_SHAPE,
                        "attention scratch of %lld bytes exceeds the built-in %lld bytes of the allocation-free "
                        "entry point (batch * query heads * ceil(capacity / 256) * (head_dim + 2) * 4); use "
                        "skn_attn_decode_dev with a caller-provided buffer",
                        (long long)need, (long long)SKN_ATTN_STATIC_SCRATCH_BYTES);
    if (ctx->device < 0 || ctx->device >= 64) return skn_fail(ctx, SKN_ERR_ARG, "device index %d not supported here", ctx->device);
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    float *part = g_attn_static_ptr[ctx->device];
    if (!part) {
        // one-time set-up for this device (it is current): resolve the array's device address
        void *p = nullptr;
        SKN_CUDA(ctx, cudaGetSymbolAddress(&p, g_attn_static_scratch));
        if (!p) return skn_fail(ctx, SKN_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        part = g_attn_static_ptr[ctx->device] = (float *)p;
    }
    SKN_CUDA(ctx, dispatch_attn(kv, G, q_dev, scale, part, attn_pick_chunk(kv, n_q_heads, 1, SKN_ATTN_STATIC_SCRATCH_BYTES),
                                out_dev, ctx->stream));
    return SKN_OK;
}

// element type of the cache buffers (SKN_KV_F32 / SKN_KV_F16 / SKN_KV_Q8_0): what the pointers of skn_kv_info point at
int32_t skn_kv_dtype(const skn_kvcache *kv, int32_t *kv_dtype) {
    if (!kv_ok(kv)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad kv cache handle");
    if (!kv_dtype) return skn_fail(kv->ctx, SKN_ERR_ARG, "kv_dtype is NULL");
    *kv_dtype = kv->dtype;
    return SKN_OK;
}

// device pointers of the cache (for callers that fill it with their own kernels)
int32_t skn_kv_info(const skn_kvcache *kv, int32_t *batch, int32_t *n_kv_heads, int32_t *head_dim, int32_t *capacity,
                    void **k_dev, void **v_dev, void **len_dev, void **start_dev) {
    if (!kv_ok(kv)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad kv cache handle");
    if (batch) *batch = kv->batch;
    if (n_kv_heads) *n_kv_heads = kv->n_kv_heads;
    if (head_dim) *head_dim = kv->head_dim;
    if (capacity) *capacity = kv->capacity;
    if (k_dev) *k_dev = kv->d_k;
    if (v_dev) *v_dev = kv->d_v;
    if (len_dev) *len_dev = kv->d_len;
    if (start_dev) *start_dev = kv->d_start;
    return SKN_OK;
}

}  // extern "C"
