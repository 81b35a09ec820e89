// K1: raw GGUF blocks -> fp32 weights, bit-exact with gguf-py.  A verification /
// export kernel, not on the decode path (the matvec kernels never materialise fp32
// weights).  One thread decodes one 32-weight group and stores it as eight float4.
#include "skn_blocks.cuh"

template <int TYPE>
__global__ void __launch_bounds__(128)
skn_dequant_kernel(const uint8_t *__restrict__ blocks, int64_t pitch, int64_t n_rows,
                   int64_t groups_per_row, float *__restrict__ out) {
    const int64_t total = n_rows * groups_per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / groups_per_row;
        const int64_t g = i - r * groups_per_row;
        float w[32];
        decode_group<TYPE>(blocks + r * pitch, g, w);
        float4 *o = reinterpret_cast<float4 *>(out + (r * groups_per_row + g) * 32);
#pragma unroll
        for (int q = 0; q < 8; ++q) o[q] = make_float4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    }
}

cudaError_t skn_launch_dequant(int32_t type, const uint8_t *blocks, int64_t pitch, int64_t n_rows,
                               int64_t n_cols, float *out, cudaStream_t stream) {
    const int64_t gpr = n_cols / 32;
    const int64_t total = n_rows * gpr;
    if (total == 0) return cudaSuccess;
    int64_t nblk = (total + 127) / 128;
    if (nblk > 148 * 64) nblk = 148 * 64;
    const dim3 grid((unsigned)nblk), block(128);
    switch (type) {
    case SKN_TYPE_Q4_0: skn_dequant_kernel<SKN_TYPE_Q4_0><<<grid, block, 0, stream>>>(blocks, pitch, n_rows, gpr, out); break;
    case SKN_TYPE_Q8_0: skn_dequant_kernel<SKN_TYPE_Q8_0><<<grid, block, 0, stream>>>(blocks, pitch, n_rows, gpr, out); break;
    case SKN_TYPE_Q4_K: skn_dequant_kernel<SKN_TYPE_Q4_K><<<grid, block, 0, stream>>>(blocks, pitch, n_rows, gpr, out); break;
    case SKN_TYPE_Q6_K: skn_dequant_kernel<SKN_TYPE_Q6_K><<<grid, block, 0, stream>>>(blocks, pitch, n_rows, gpr, out); break;
    case SKN_TYPE_Q4_1: skn_dequant_kernel<SKN_TYPE_Q4_1><<<grid, block, 0, stream>>>(blocks, pitch, n_rows, gpr, out); break;
    case SKN_TYPE_Q5_0: skn_dequant_kernel<SKN_TYPE_Q5_0><<<grid, block, 0, stream>>>(blocks, pitch, n_rows, gpr, out); break;
    case SKN_TYPE_Q5_1: skn_dequant_kernel<SKN_TYPE_Q5_1><<<grid, block, 0, stream>>>(blocks, pitch, n_rows, gpr, out); break;
    case SKN_TYPE_Q5_K: skn_dequant_kernel<SKN_TYPE_Q5_K><<<grid, block, 0, stream>>>(blocks, pitch, n_rows, gpr, out); break;
    case SKN_TYPE_Q2_K: skn_dequant_kernel<SKN_TYPE_Q2_K><<<grid, block, 0, stream>>>(blocks, pitch, n_rows, gpr, out); break;
    case SKN_TYPE_Q3_K: skn_dequant_kernel<SKN_TYPE_Q3_K><<<grid, block, 0, stream>>>(blocks, pitch, n_rows, gpr, out); break;
    case SKN_TYPE_IQ4_NL: skn_dequant_kernel<SKN_TYPE_IQ4_NL><<<grid, block, 0, stream>>>(blocks, pitch, n_rows, gpr, out); break;
    case SKN_TYPE_IQ4_XS: skn_dequant_kernel<SKN_TYPE_IQ4_XS><<<grid, block, 0, stream>>>(blocks, pitch, n_rows, gpr, out); break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// out[m][:] = dequantised row ids[m] of a quantized [vocab][d] table (token embedding lookup)
template <int TYPE>
__global__ void __launch_bounds__(128)
skn_embed_kernel(const uint8_t *__restrict__ blocks, int64_t pitch, int64_t n_rows, int64_t groups_per_row,
                 const int32_t *__restrict__ ids, float *__restrict__ out) {
    int64_t row = ids[blockIdx.x];
    if (row < 0 || row >= n_rows) row = 0;         // out-of-range ids read row 0 (no fault)
    for (int64_t g = threadIdx.x; g < groups_per_row; g += blockDim.x) {
        float w[32];
        decode_group<TYPE>(blocks + row * pitch, g, w);
        float4 *o = reinterpret_cast<float4 *>(out + ((int64_t)blockIdx.x * groups_per_row + g) * 32);
#pragma unroll
        for (int q = 0; q < 8; ++q) o[q] = make_float4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    }
}

cudaError_t skn_launch_embed(const skn_tensor *emb, const int32_t *ids, int M, float *out, cudaStream_t st) {
    if (M == 0) return cudaSuccess;
    const int64_t gpr = emb->n_cols / 32;
    switch (emb->type) {
    case SKN_TYPE_Q4_0: skn_embed_kernel<SKN_TYPE_Q4_0><<<M, 128, 0, st>>>(emb->d_blocks, emb->pitch, emb->n_rows, gpr, ids, out); break;
    case SKN_TYPE_Q8_0: skn_embed_kernel<SKN_TYPE_Q8_0><<<M, 128, 0, st>>>(emb->d_blocks, emb->pitch, emb->n_rows, gpr, ids, out); break;
    case SKN_TYPE_Q4_K: skn_embed_kernel<SKN_TYPE_Q4_K><<<M, 128, 0, st>>>(emb->d_blocks, emb->pitch, emb->n_rows, gpr, ids, out); break;
    case SKN_TYPE_Q6_K: skn_embed_kernel<SKN_TYPE_Q6_K><<<M, 128, 0, st>>>(emb->d_blocks, emb->pitch, emb->n_rows, gpr, ids, out); break;
    case SKN_TYPE_Q4_1: skn_embed_kernel<SKN_TYPE_Q4_1><<<M, 128, 0, st>>>(emb->d_blocks, emb->pitch, emb->n_rows, gpr, ids, out); break;
    case SKN_TYPE_Q5_0: skn_embed_kernel<SKN_TYPE_Q5_0><<<M, 128, 0, st>>>(emb->d_blocks, emb->pitch, emb->n_rows, gpr, ids, out); break;
    case SKN_TYPE_Q5_1: skn_embed_kernel<SKN_TYPE_Q5_1><<<M, 128, 0, st>>>(emb->d_blocks, emb->pitch, emb->n_rows, gpr, ids, out); break;
    case SKN_TYPE_Q5_K: skn_embed_kernel<SKN_TYPE_Q5_K><<<M, 128, 0, st>>>(emb->d_blocks, emb->pitch, emb->n_rows, gpr, ids, out); break;
    case SKN_TYPE_Q2_K: skn_embed_kernel<SKN_TYPE_Q2_K><<<M, 128, 0, st>>>(emb->d_blocks, emb->pitch, emb->n_rows, gpr, ids, out); break;
    case SKN_TYPE_Q3_K: skn_embed_kernel<SKN_TYPE_Q3_K><<<M, 128, 0, st>>>(emb->d_blocks, emb->pitch, emb->n_rows, gpr, ids, out); break;
    case SKN_TYPE_IQ4_NL: skn_embed_kernel<SKN_TYPE_IQ4_NL><<<M, 128, 0, st>>>(emb->d_blocks, emb->pitch, emb->n_rows, gpr, ids, out); break;
    case SKN_TYPE_IQ4_XS: skn_embed_kernel<SKN_TYPE_IQ4_XS><<<M, 128, 0, st>>>(emb->d_blocks, emb->pitch, emb->n_rows, gpr, ids, out); break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}
