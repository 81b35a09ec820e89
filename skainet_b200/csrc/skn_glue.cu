// Small element-wise kernels around the matmuls (no counterpart in the reference).
#include "skn_internal.cuh"
#include "skn_ptx.cuh"

// h = silu(g) * u, fp32 (the decode-size SwiGLU; the prefill path fuses this into the
// tensor-core epilogue)
__global__ void skn_silu_mul_kernel(const float *__restrict__ g, const float *__restrict__ u, float *__restrict__ h,
                                    int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float a = g[i];
        h[i] = a / (1.f + expf(-a)) * u[i];
    }
}

cudaError_t skn_launch_silu_mul(const float *g, const float *u, float *h, int64_t n, int sm_count, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    int64_t blocks = (n + 255) / 256;
    if (blocks > (int64_t)sm_count * 8) blocks = (int64_t)sm_count * 8;
    skn_silu_mul_kernel<<<(unsigned)blocks, 256, 0, stream>>>(g, u, h, n);
    return cudaGetLastError();
}

// ---- decoder glue (K8) ---------------------------------------------------------------------
// y[m][:] = x[m][:] / sqrt(mean(x[m]^2) + eps) * gain[:]; one CTA per row
__global__ void __launch_bounds__(256)
skn_rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ gain, float *__restrict__ y, int D, float eps) {
    __shared__ float red[8];
    const float *xr = x + (size_t)blockIdx.x * D;
    float *yr = y + (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < D; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4 *>(xr + i);
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
    const float r = rsqrtf(tot / (float)D + eps);
    for (int i = threadIdx.x * 4; i < D; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4 *>(xr + i);
        const float4 g = *reinterpret_cast<const float4 *>(gain + i);
        *reinterpret_cast<float4 *>(yr + i) = make_float4(v.x * r * g.x, v.y * r * g.y, v.z * r * g.z, v.w * r * g.w);
    }
}

// Rotary embedding in place on x [M][H][D]: pairs (2i, 2i+1) of every head rotate by
// pos * theta^(-2i/D); row m = b * T + t has position len[b] + t (len = tokens already cached).
__global__ void skn_rope_kernel(float *__restrict__ x, const int32_t *__restrict__ len, int T, int H, int D,
                                double log2_theta, int64_t total_pairs) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_pairs; i += (int64_t)gridDim.x * blockDim.x) {
        const int p = (int)(i % (D / 2));
        const int64_t mh = i / (D / 2);
        const int64_t m = mh / H;
        const int pos = len[m / T] + (int)(m % T);
        // angle in double: at position 4096 an fp32 angle is already off by ~5e-4 rad
        const double ang = (double)pos * exp2(-(double)log2_theta * (2.0 * (double)p / (double)D));
        double sd, cd;
        sincos(ang, &sd, &cd);
        const float sn = (float)sd, cs = (float)cd;
        float2 *v = reinterpret_cast<float2 *>(x) + i;
        const float2 a = *v;
        *v = make_float2(a.x * cs - a.y * sn, a.x * sn + a.y * cs);
    }
}

__global__ void skn_add_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out, int64_t n4) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const float4 u = reinterpret_cast<const float4 *>(a)[i], v = reinterpret_cast<const float4 *>(b)[i];
        reinterpret_cast<float4 *>(out)[i] = make_float4(u.x + v.x, u.y + v.y, u.z + v.z, u.w + v.w);
    }
}

// out[m][:] = rows[src[m]][:] (row gather of fp32 matrices; used to pick the last position of
// every sequence before the LM head)
__global__ void skn_gather_rows_kernel(const float *__restrict__ in, float *__restrict__ out, int D, int T) {
    const float *src = in + ((size_t)blockIdx.x * T + (T - 1)) * D;
    float *dst = out + (size_t)blockIdx.x * D;
    for (int i = threadIdx.x * 4; i < D; i += blockDim.x * 4)
        *reinterpret_cast<float4 *>(dst + i) = *reinterpret_cast<const float4 *>(src + i);
}

// ids[m] = argmax_v logits[m][v] (first maximum wins, as a sequential scan would give).
// Grid (ARGMAX_SPLIT, M): every CTA scans one slice of the row and leaves its candidate in
// scratch; the CTA that draws the last ticket of its row (threadfence + atomic counter, no
// waiting) picks the winner among the candidates and hands the ticket counter back as zero.
constexpr int ARGMAX_SPLIT = 64;

__device__ __forceinline__ void argmax_take(float &best, int &bi, float v, int i) {
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
}

__global__ void __launch_bounds__(256)
skn_argmax_kernel(const float *__restrict__ logits, int V, int32_t *__restrict__ ids, float *__restrict__ cand_v,
                  int *__restrict__ cand_i, unsigned *__restrict__ tickets) {
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ bool last;
    const int m = blockIdx.y, sp = blockIdx.x;
    const float *row = logits + (size_t)m * V;
    const int per = (V + ARGMAX_SPLIT - 1) / ARGMAX_SPLIT;
    const int lo = sp * per, hi = min(V, lo + per);
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) argmax_take(best, bi, row[i], i);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_take(best, bi, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) argmax_take(best, bi, sv[w], si[w]);
        cand_v[m * ARGMAX_SPLIT + sp] = best;
        cand_i[m * ARGMAX_SPLIT + sp] = bi;
        __threadfence();
        last = atomicAdd(&tickets[m], 1u) == (unsigned)(ARGMAX_SPLIT - 1);
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (threadIdx.x < 32) {
        best = -INFINITY;
        bi = 0x7fffffff;
        for (int i = threadIdx.x; i < ARGMAX_SPLIT; i += 32)
            argmax_take(best, bi, __ldcg(cand_v + m * ARGMAX_SPLIT + i), __ldcg(cand_i + m * ARGMAX_SPLIT + i));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            argmax_take(best, bi, ov, oi);
        }
        if (threadIdx.x == 0) {
            ids[m] = (bi == 0x7fffffff) ? 0 : bi;   // a row of NaNs or -inf: token 0
            tickets[m] = 0;
        }
    }
}

static int glue_blocks(int64_t n, int sm_count) {
    int64_t b = (n + 255) / 256;
    if (b > (int64_t)sm_count * 8) b = (int64_t)sm_count * 8;
    return (int)(b < 1 ? 1 : b);
}

cudaError_t skn_launch_rmsnorm(const float *x, const float *gain, float *y, int M, int D, float eps, cudaStream_t st) {
    if (M == 0) return cudaSuccess;
    skn_rmsnorm_kernel<<<M, 256, 0, st>>>(x, gain, y, D, eps);
    return cudaGetLastError();
}
cudaError_t skn_launch_rope(float *x, const int32_t *len, int M, int T, int H, int D, float theta, int sm_count, cudaStream_t st) {
    const int64_t pairs = (int64_t)M * H * (D / 2);
    if (pairs == 0) return cudaSuccess;
    skn_rope_kernel<<<glue_blocks(pairs, sm_count), 256, 0, st>>>(x, len, T, H, D, log2((double)theta), pairs);
    return cudaGetLastError();
}
// dst[0..n) = src[0..n) in 16-byte words (n a multiple of 4, both 16-byte aligned).  `src` may be page-locked
// host memory mapped into the device's address space: the copy then crosses PCIe inside a kernel, which costs
// a kernel-to-kernel hand-over instead of a copy-engine operation between two kernels.
// Launched with programmatic stream serialisation: the kernel that follows (the product) may become resident
// and prefetch its weights at once; this one waits for everything before it in the stream (the previous
// product may still be reading `dst`) before it copies, and the product waits for this one before it reads.
__global__ void skn_fetch_kernel(const float4 *__restrict__ src, float4 *__restrict__ dst, int64_t n4) {
    skn_pdl_launch_dependents();
    skn_pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) dst[i] = src[i];
}
cudaError_t skn_launch_fetch(const float *src, float *dst, int64_t n, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    const int64_t n4 = n / 4;
    int blocks = (int)((n4 + 255) / 256);
    if (blocks > 32) blocks = 32;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, skn_fetch_kernel, reinterpret_cast<const float4 *>(src), reinterpret_cast<float4 *>(dst), n4);
}
cudaError_t skn_launch_add(const float *a, const float *b, float *out, int64_t n, int sm_count, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    skn_add_kernel<<<glue_blocks(n / 4, sm_count), 256, 0, st>>>(a, b, out, n / 4);
    return cudaGetLastError();
}
cudaError_t skn_launch_last_rows(const float *in, float *out, int B, int T, int D, cudaStream_t st) {
    if (B == 0) return cudaSuccess;
    skn_gather_rows_kernel<<<B, 256, 0, st>>>(in, out, D, T);
    return cudaGetLastError();
}
size_t skn_argmax_scratch_bytes(int M) { return (size_t)M * (ARGMAX_SPLIT * 8 + 4); }
// scratch: skn_argmax_scratch_bytes(M) bytes whose ticket part was zeroed once (the kernel
// leaves it zeroed)
cudaError_t skn_launch_argmax(const float *logits, int M, int V, int32_t *ids, void *scratch, cudaStream_t st) {
    if (M == 0) return cudaSuccess;
    float *cv = (float *)scratch;
    int *ci = (int *)(cv + (size_t)M * ARGMAX_SPLIT);
    unsigned *tk = (unsigned *)(ci + (size_t)M * ARGMAX_SPLIT);
    skn_argmax_kernel<<<dim3(ARGMAX_SPLIT, (unsigned)M), 256, 0, st>>>(logits, V, ids, cv, ci, tk);
    return cudaGetLastError();
}

// Cross-rank greedy choice.  offer: cand[world][B][2] is zero except this rank's slots, which
// hold (best logit of the local slice, its global token id as a float; ids stay below 2^24).
// pick (after the slots of all ranks have been summed together): highest value wins, ties go
// to the lowest id; a slice whose best is NaN never wins.
__global__ void skn_argmax_offer_kernel(const float *__restrict__ logits, const int32_t *__restrict__ ids, int B, int V_local,
                                        int rank, int world, float *__restrict__ cand) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = (world * B * 2 + 3) / 4 * 4;
    if (i >= n) return;
    float v = 0.f;
    const int slot = i / 2, r = slot / B, b = slot % B;
    if (slot < world * B && r == rank) {
        const int id = ids[b];
        v = (i & 1) ? (float)(id + rank * V_local) : logits[(size_t)b * V_local + id];
    }
    cand[i] = v;
}

__global__ void skn_argmax_pick_kernel(const float *__restrict__ cand, int B, int world, int32_t *__restrict__ ids) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int r = 0; r < world; ++r) {
        const float v = cand[((size_t)r * B + b) * 2];
        const int id = (int)cand[((size_t)r * B + b) * 2 + 1];
        argmax_take(best, bi, v, id);
    }
    ids[b] = (bi == 0x7fffffff) ? 0 : bi;
}

cudaError_t skn_launch_argmax_offer(const float *logits, const int32_t *ids, int B, int V_local, int rank, int world,
                                    float *cand, cudaStream_t st) {
    const int n = (world * B * 2 + 3) / 4 * 4;
    skn_argmax_offer_kernel<<<(n + 127) / 128, 128, 0, st>>>(logits, ids, B, V_local, rank, world, cand);
    return cudaGetLastError();
}
cudaError_t skn_launch_argmax_pick(const float *cand, int B, int world, int32_t *ids, cudaStream_t st) {
    skn_argmax_pick_kernel<<<(B + 127) / 128, 128, 0, st>>>(cand, B, world, ids);
    return cudaGetLastError();
}
