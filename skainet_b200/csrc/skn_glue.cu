// Small element-wise kernels around the matmuls (no counterpart in the reference).
#include "skn_internal.cuh"

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
