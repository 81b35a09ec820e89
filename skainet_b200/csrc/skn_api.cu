// C ABI of libskainet_cuda.so: contexts, error reporting, weight upload, and the
// host-pointer / device-pointer front ends of the kernels.  No exception leaves this file.
#include "skn_internal.cuh"

#include <new>
#include <stdarg.h>
#include <stdlib.h>

static thread_local char g_tls_err[512] = "";

int32_t skn_fail(skn_ctx *ctx, int32_t code, const char *fmt, ...) {
    char *dst = (ctx && ctx->magic == SKN_MAGIC_CTX) ? ctx->err : g_tls_err;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(dst, 512, fmt, ap);
    va_end(ap);
    if (getenv("SKN_LOG")) fprintf(stderr, "[skainet_cuda] error %d: %s\n", code, dst);
    return code;
}

int32_t skn_check_cuda(skn_ctx *ctx, cudaError_t e, const char *what) {
    if (e == cudaSuccess) return SKN_OK;
    const int32_t code = (e == cudaErrorMemoryAllocation) ? SKN_ERR_OOM : SKN_ERR_CUDA;
    return skn_fail(ctx, code, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

uint64_t skn_thread_token() {
    static thread_local char anchor;        // its address is unique among live threads and never 0
    return (uint64_t)(uintptr_t)&anchor;
}

int32_t skn_busy_fail() {
    return skn_fail(nullptr, SKN_ERR_BUSY, "the context is in use by another host thread (one thread at a time)");
}

bool skn_ctx_ok(const skn_ctx *ctx) { return ctx && ctx->magic == SKN_MAGIC_CTX; }
bool skn_tensor_ok(const skn_tensor *t) { return t && t->magic == SKN_MAGIC_TENSOR && skn_ctx_ok(t->ctx); }

int32_t skn_stage_reserve(skn_ctx *ctx, void **buf, size_t *cap, size_t need) {
    if (need <= *cap) return SKN_OK;
    if (*buf) {
        SKN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        SKN_CUDA(ctx, cudaFree(*buf));
        *buf = nullptr;
        *cap = 0;
    }
    size_t want = need < (1u << 20) ? (1u << 20) : need;
    SKN_CUDA(ctx, cudaMalloc(buf, want));
    *cap = want;
    return SKN_OK;
}

extern "C" {

int32_t skn_version(void) { return SKN_VERSION; }

const char *skn_last_error(const skn_ctx *ctx) { return skn_ctx_ok(ctx) ? ctx->err : g_tls_err; }

int32_t skn_ctx_create(int32_t device, skn_ctx **out) {
    if (!out) return skn_fail(nullptr, SKN_ERR_ARG, "skn_ctx_create: out is NULL");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return skn_fail(nullptr, SKN_ERR_CUDA, "no usable CUDA device (%s); this library has no CPU fallback",
                        e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    if (device < 0 || device >= n) return skn_fail(nullptr, SKN_ERR_ARG, "device %d out of range [0,%d)", device, n);
    skn_ctx *ctx = new (std::nothrow) skn_ctx();
    if (!ctx) return skn_fail(nullptr, SKN_ERR_OOM, "host allocation failed");
    memset(ctx, 0, sizeof(*ctx));
    ctx->magic = SKN_MAGIC_CTX;
    ctx->device = device;
#define CTX_TRY(call)                                                \
    do {                                                             \
        cudaError_t e__ = (call);                                    \
        if (e__ != cudaSuccess) {                                    \
            int32_t rc__ = skn_check_cuda(nullptr, e__, #call);      \
            if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream); \
            if (ctx->d_status_base) cudaFree(ctx->d_status_base);    \
            if (ctx->h_status_base) cudaFreeHost(ctx->h_status_base); \
            ctx->magic = 0;                                          \
            delete ctx;                                              \
            return rc__;                                             \
        }                                                            \
    } while (0)
    CTX_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    CTX_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        fprintf(stderr, "[skainet_cuda] warning: device %d is sm_%d%d; kernels are built for sm_100a only\n", device,
                prop.major, prop.minor);
    ctx->sm_count = prop.multiProcessorCount;
    CTX_TRY(cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking));
    ctx->stream = ctx->own_stream;
    ctx->prefill_min_m = 64;
    ctx->fused_exchange = -1;
    CTX_TRY(cudaMalloc((void **)&ctx->d_status_base, SKN_SMALL_OUT_BYTES + 32768));
    ctx->d_status = reinterpret_cast<int32_t *>(ctx->d_status_base + SKN_SMALL_OUT_BYTES);
    CTX_TRY(cudaMemset(ctx->d_status, 0, 32768));
    CTX_TRY(cudaMallocHost((void **)&ctx->h_status_base, SKN_SMALL_OUT_BYTES + 256));
    ctx->h_status = reinterpret_cast<int32_t *>(ctx->h_status_base + SKN_SMALL_OUT_BYTES);
    {
        void *hd = nullptr;
        if (cudaHostGetDevicePointer(&hd, ctx->h_status, 0) == cudaSuccess) ctx->h_status_dev = (int32_t *)hd;
        else cudaGetLastError();
    }
#undef CTX_TRY
    *ctx->h_status = 0;
    *out = ctx;
    return SKN_OK;
}

int32_t skn_ctx_destroy(skn_ctx *ctx) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "skn_ctx_destroy: bad context handle");
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->d_stage_in) cudaFree(ctx->d_stage_in);
    if (ctx->d_stage_out) cudaFree(ctx->d_stage_out);
    if (ctx->d_scratch) cudaFree(ctx->d_scratch);
    if (ctx->d_scratch2) cudaFree(ctx->d_scratch2);
    if (ctx->d_xq) cudaFree(ctx->d_xq);
    if (ctx->d_status_base) cudaFree(ctx->d_status_base);
    if (ctx->h_status_base) cudaFreeHost(ctx->h_status_base);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    ctx->magic = 0;
    delete ctx;
    return SKN_OK;
}

int32_t skn_ctx_set_stream(skn_ctx *ctx, void *cuda_stream) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    SKN_ENTER(ctx);
    ctx->stream = cuda_stream ? (cudaStream_t)cuda_stream : ctx->own_stream;
    return SKN_OK;
}

int32_t skn_ctx_set_option(skn_ctx *ctx, int32_t option, int64_t value) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    SKN_ENTER(ctx);
    switch (option) {
    case SKN_OPT_RELAXED_ORDER: ctx->relaxed_order = value ? 1 : 0; return SKN_OK;
    case SKN_OPT_PREFILL_MIN_M:
        if (value < 0 || value > (1 << 30)) return skn_fail(ctx, SKN_ERR_ARG, "prefill threshold out of range");
        ctx->prefill_min_m = (int)value;
        return SKN_OK;
    case SKN_OPT_FUSED_EXCHANGE: ctx->fused_exchange = value < 0 ? -1 : (value ? 1 : 0); return SKN_OK;
    case SKN_OPT_KV_F16: ctx->kv_f16 = value ? SKN_KV_F16 : SKN_KV_F32; return SKN_OK;
    case SKN_OPT_KV_DTYPE:
        if (value != SKN_KV_F32 && value != SKN_KV_F16 && value != SKN_KV_Q8_0) return skn_fail(ctx, SKN_ERR_TYPE, "cache element type %lld is none of fp32, fp16, Q8_0", (long long)value);
        ctx->kv_f16 = (int)value;
        return SKN_OK;
    case SKN_OPT_WAIT_LIMIT_MS: {
        if (value < 0 || value > 600000) return skn_fail(ctx, SKN_ERR_ARG, "wait limit outside [0, 600000] ms");
        const int32_t ms = (int32_t)value;
        SKN_CUDA(ctx, cudaSetDevice(ctx->device));
        SKN_CUDA(ctx, cudaMemcpyAsync(ctx->d_status + SKN_STATUS_WAIT_MS, &ms, sizeof(ms), cudaMemcpyHostToDevice, ctx->stream));
        SKN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        return SKN_OK;
    }
    default: return skn_fail(ctx, SKN_ERR_ARG, "unknown option %d", option);
    }
}

int32_t skn_sync(skn_ctx *ctx) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    SKN_ENTER(ctx);
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    SKN_CUDA(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    SKN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return skn_status_check(ctx);
}

}  // extern "C"

// the status word has just arrived in the pinned mirror: report it (and clear it on the device)
int32_t skn_status_check(skn_ctx *ctx) {
    const int32_t st = *ctx->h_status;
    if (st != 0) {
        cudaMemsetAsync(ctx->d_status, 0, sizeof(int32_t), ctx->stream);
        cudaStreamSynchronize(ctx->stream);
        return skn_fail(ctx, st, "a kernel reported device-side status %d (%s)", st,
                        st == SKN_ERR_TIMEOUT ? "a bounded wait ran out"
                        : st == SKN_ERR_SHAPE ? "a KV cache was asked to hold more tokens than its capacity; nothing was overwritten"
                                              : "see status codes");
    }
    return SKN_OK;
}

extern "C" {

int32_t skn_quant_geometry(int32_t ggml_type, int32_t *block_elems, int32_t *block_bytes) {
    int32_t e, b;
    if (!skn_geometry(ggml_type, &e, &b)) return skn_fail(nullptr, SKN_ERR_TYPE, "unsupported GGML type id %d", ggml_type);
    if (block_elems) *block_elems = e;
    if (block_bytes) *block_bytes = b;
    return SKN_OK;
}

int32_t skn_quant_row_bytes(int32_t ggml_type, int64_t n_cols, int64_t *row_bytes) {
    int32_t e, b;
    if (!skn_geometry(ggml_type, &e, &b)) return skn_fail(nullptr, SKN_ERR_TYPE, "unsupported GGML type id %d", ggml_type);
    if (n_cols < 0 || n_cols % e)
        return skn_fail(nullptr, SKN_ERR_SHAPE, "Quantized tensor row size (%lld) is not a multiple of block size (%d)",
                        (long long)n_cols, e);
    if (row_bytes) *row_bytes = n_cols / e * b;
    return SKN_OK;
}

int32_t skn_tensor_upload_quant_shard(skn_ctx *ctx, int32_t ggml_type, int64_t n_rows_total, int64_t n_cols_total,
                                      const void *host_blocks, int64_t n_bytes, int64_t row_begin, int64_t row_count,
                                      int64_t col_begin, int64_t col_count, skn_tensor **out) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    SKN_ENTER(ctx);
    if (!out) return skn_fail(ctx, SKN_ERR_ARG, "out is NULL");
    *out = nullptr;
    int32_t e, b;
    if (!skn_geometry(ggml_type, &e, &b)) return skn_fail(ctx, SKN_ERR_TYPE, "unsupported GGML type id %d", ggml_type);
    if (n_rows_total < 0 || n_cols_total < 0) return skn_fail(ctx, SKN_ERR_ARG, "negative shape");
    if (n_cols_total % e)
        return skn_fail(ctx, SKN_ERR_SHAPE, "Quantized tensor row size (%lld) is not a multiple of block size (%d)",
                        (long long)n_cols_total, e);
    const int64_t row_bytes_total = n_cols_total / e * b;
    if (n_bytes != n_rows_total * row_bytes_total)
        return skn_fail(ctx, SKN_ERR_SHAPE, "byte length %lld does not match %lld rows x %lld bytes", (long long)n_bytes,
                        (long long)n_rows_total, (long long)row_bytes_total);
    if (row_begin < 0 || row_count < 0 || row_begin + row_count > n_rows_total || col_begin < 0 || col_count < 0 ||
        col_begin + col_count > n_cols_total)
        return skn_fail(ctx, SKN_ERR_SHAPE, "shard range outside the tensor");
    if (col_begin % e || col_count % e) return skn_fail(ctx, SKN_ERR_SHAPE, "shard columns must be whole blocks");
    if (!host_blocks && n_bytes > 0) return skn_fail(ctx, SKN_ERR_ARG, "host_blocks is NULL");

    skn_tensor *t = new (std::nothrow) skn_tensor();
    if (!t) return skn_fail(ctx, SKN_ERR_OOM, "host allocation failed");
    memset(t, 0, sizeof(*t));
    t->magic = SKN_MAGIC_TENSOR;
    t->ctx = ctx;
    t->type = ggml_type;
    t->n_rows = row_count;
    t->n_cols = col_count;
    t->row_bytes = col_count / e * b;
    t->pitch = (t->row_bytes + 15) / 16 * 16;
    const size_t dev_bytes = (size_t)(t->pitch * t->n_rows);
    cudaError_t err = cudaSetDevice(ctx->device);
    // a few spare bytes so that vector loads of the last row may over-read safely
    if (err == cudaSuccess) err = cudaMalloc((void **)&t->d_blocks, dev_bytes + 256);
    if (err == cudaSuccess && dev_bytes > 0) {
        if (t->pitch != t->row_bytes) err = cudaMemsetAsync(t->d_blocks, 0, dev_bytes + 256, ctx->stream);
        const uint8_t *src = (const uint8_t *)host_blocks + row_begin * row_bytes_total + col_begin / e * b;
        if (err == cudaSuccess)
            err = cudaMemcpy2DAsync(t->d_blocks, (size_t)t->pitch, src, (size_t)row_bytes_total, (size_t)t->row_bytes,
                                    (size_t)t->n_rows, cudaMemcpyHostToDevice, ctx->stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(ctx->stream);
    }
    if (err != cudaSuccess) {
        if (t->d_blocks) cudaFree(t->d_blocks);
        t->magic = 0;
        delete t;
        return skn_check_cuda(ctx, err, "weight upload");
    }
    *out = t;
    return SKN_OK;
}

int32_t skn_tensor_upload_quant(skn_ctx *ctx, int32_t ggml_type, int64_t n_rows, int64_t n_cols, const void *host_blocks,
                                int64_t n_bytes, skn_tensor **out) {
    return skn_tensor_upload_quant_shard(ctx, ggml_type, n_rows, n_cols, host_blocks, n_bytes, 0, n_rows, 0, n_cols, out);
}

int32_t skn_tensor_destroy(skn_tensor *t) {
    if (!t || t->magic != SKN_MAGIC_TENSOR) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad tensor handle");
    if (skn_ctx_ok(t->ctx)) {
        SKN_ENTER(t->ctx);
        cudaSetDevice(t->ctx->device);
        cudaStreamSynchronize(t->ctx->stream);
    }
    if (t->d_blocks) cudaFree(t->d_blocks);
    t->magic = 0;
    delete t;
    return SKN_OK;
}

int32_t skn_tensor_info(const skn_tensor *t, int32_t *ggml_type, int64_t *n_rows, int64_t *n_cols, int64_t *row_bytes,
                        int64_t *row_pitch_bytes, void **device_blocks) {
    if (!skn_tensor_ok(t)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad tensor handle");
    if (ggml_type) *ggml_type = t->type;
    if (n_rows) *n_rows = t->n_rows;
    if (n_cols) *n_cols = t->n_cols;
    if (row_bytes) *row_bytes = t->row_bytes;
    if (row_pitch_bytes) *row_pitch_bytes = t->pitch;
    if (device_blocks) *device_blocks = t->d_blocks;
    return SKN_OK;
}

int32_t skn_dequantize_dev(skn_ctx *ctx, const skn_tensor *t, float *out_dev) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    SKN_ENTER(ctx);
    if (!skn_tensor_ok(t) || t->ctx != ctx) return skn_fail(ctx, SKN_ERR_BAD_HANDLE, "bad tensor handle");
    if (!out_dev) return skn_fail(ctx, SKN_ERR_ARG, "out is NULL");
    if (((uintptr_t)out_dev) & 15) return skn_fail(ctx, SKN_ERR_ALIGN, "output must be 16-byte aligned");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    SKN_CUDA(ctx, skn_launch_dequant(t->type, t->d_blocks, t->pitch, t->n_rows, t->n_cols, out_dev, ctx->stream));
    return SKN_OK;
}

int32_t skn_dequantize(skn_ctx *ctx, const skn_tensor *t, float *out_host) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    SKN_ENTER(ctx);
    if (!skn_tensor_ok(t) || t->ctx != ctx) return skn_fail(ctx, SKN_ERR_BAD_HANDLE, "bad tensor handle");
    if (!out_host) return skn_fail(ctx, SKN_ERR_ARG, "out is NULL");
    const size_t bytes = (size_t)t->n_rows * (size_t)t->n_cols * sizeof(float);
    if (bytes == 0) return SKN_OK;
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    int32_t rc = skn_stage_reserve(ctx, &ctx->d_stage_out, &ctx->d_stage_out_bytes, bytes);
    if (rc) return rc;
    rc = skn_dequantize_dev(ctx, t, (float *)ctx->d_stage_out);
    if (rc) return rc;
    SKN_CUDA(ctx, cudaMemcpyAsync(out_host, ctx->d_stage_out, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return skn_sync(ctx);
}

static int32_t check_matmul_args(skn_ctx *ctx, const skn_tensor *w, const void *x, int32_t M, int64_t K, const void *y) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    if (!skn_tensor_ok(w) || w->ctx != ctx) return skn_fail(ctx, SKN_ERR_BAD_HANDLE, "bad tensor handle");
    if (M < 0) return skn_fail(ctx, SKN_ERR_ARG, "M is negative");
    if (K != w->n_cols) return skn_fail(ctx, SKN_ERR_SHAPE, "Shapes do not align.");
    if (M > 0 && (!x || !y)) return skn_fail(ctx, SKN_ERR_ARG, "x or y is NULL");
    return SKN_OK;
}

int32_t skn_matmul_dev(skn_ctx *ctx, const skn_tensor *w, const float *x_dev, int32_t M, int64_t K,
                       const float *bias_dev, float *y_dev) {
    int32_t rc = check_matmul_args(ctx, w, x_dev, M, K, y_dev);
    if (rc) return rc;
    SKN_ENTER(ctx);
    if (M == 0 || w->n_rows == 0) return SKN_OK;
    if ((((uintptr_t)x_dev) & 15) || (((uintptr_t)y_dev) & 15))
        return skn_fail(ctx, SKN_ERR_ALIGN, "x and y must be 16-byte aligned device pointers");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    if (K == 0) {
        // empty reduction: y = bias (or 0)
        SKN_CUDA(ctx, cudaMemsetAsync(y_dev, 0, (size_t)M * w->n_rows * sizeof(float), ctx->stream));
        if (bias_dev)
            for (int32_t m = 0; m < M; ++m)
                SKN_CUDA(ctx, cudaMemcpyAsync(y_dev + (size_t)m * w->n_rows, bias_dev, w->n_rows * sizeof(float),
                                              cudaMemcpyDeviceToDevice, ctx->stream));
        return SKN_OK;
    }
    if (ctx->prefill_min_m > 0 && M >= ctx->prefill_min_m && skn_tc_supported(w, M)) {
        // prefill: bf16 copy of the activations, tensor-core matmul with fp32 accumulation
        const size_t ab = (size_t)M * (size_t)K * 2;
        int32_t rc2 = skn_stage_reserve(ctx, &ctx->d_scratch, &ctx->d_scratch_bytes, ab);
        if (rc2) return rc2;
        SKN_CUDA(ctx, skn_launch_f32_to_bf16(x_dev, ctx->d_scratch, (int64_t)M * K, ctx->sm_count, ctx->stream));
        SKN_CUDA(ctx, skn_launch_matmul_tc(ctx, w, ctx->d_scratch, M, bias_dev, y_dev, ctx->stream));
        return SKN_OK;
    }
    SKN_CUDA(ctx, skn_launch_matvec(ctx, w, x_dev, M, bias_dev, y_dev, ctx->stream));
    return SKN_OK;
}

// y[t] = W[t] . x (+ add[t]) for up to three weights that share the activation vector x
int32_t skn_matvec_group_dev(skn_ctx *ctx, int32_t n, const skn_tensor *const *w, const float *x_dev,
                             float *const *y_dev, const float *const *add_dev) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    SKN_ENTER(ctx);
    if (n < 1 || n > 3 || !w || !y_dev || !x_dev) return skn_fail(ctx, SKN_ERR_ARG, "1 to 3 tensors, non-NULL arrays");
    for (int32_t t = 0; t < n; ++t) {
        if (!skn_tensor_ok(w[t]) || w[t]->ctx != ctx) return skn_fail(ctx, SKN_ERR_BAD_HANDLE, "bad tensor handle");
        if (w[t]->n_cols != w[0]->n_cols) return skn_fail(ctx, SKN_ERR_SHAPE, "Shapes do not align.");
        if (!y_dev[t] || (((uintptr_t)y_dev[t]) & 15)) return skn_fail(ctx, SKN_ERR_ALIGN, "outputs must be 16-byte aligned");
    }
    if (((uintptr_t)x_dev) & 15) return skn_fail(ctx, SKN_ERR_ALIGN, "x must be 16-byte aligned");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    SKN_CUDA(ctx, skn_launch_matvec_group(ctx, n, w, x_dev, y_dev, add_dev, ctx->stream));
    return SKN_OK;
}

int32_t skn_matvec_fused_dev(skn_ctx *ctx, int32_t n, const skn_tensor *const *w, const float *x_dev,
                             float *const *y_dev, const float *const *add_dev, const float *norm_gain_dev,
                             float norm_eps, const float *silu_u_dev) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    SKN_ENTER(ctx);
    if (n < 1 || n > 3 || !w || !y_dev || !x_dev) return skn_fail(ctx, SKN_ERR_ARG, "1 to 3 tensors, non-NULL arrays");
    if (norm_gain_dev && silu_u_dev) return skn_fail(ctx, SKN_ERR_ARG, "either a norm gain or a SwiGLU partner, not both");
    for (int32_t t = 0; t < n; ++t) {
        if (!skn_tensor_ok(w[t]) || w[t]->ctx != ctx) return skn_fail(ctx, SKN_ERR_BAD_HANDLE, "bad tensor handle");
        if (w[t]->n_cols != w[0]->n_cols) return skn_fail(ctx, SKN_ERR_SHAPE, "Shapes do not align.");
        if (!y_dev[t] || (((uintptr_t)y_dev[t]) & 15)) return skn_fail(ctx, SKN_ERR_ALIGN, "outputs must be 16-byte aligned");
    }
    if ((((uintptr_t)x_dev) | ((uintptr_t)norm_gain_dev) | ((uintptr_t)silu_u_dev)) & 15)
        return skn_fail(ctx, SKN_ERR_ALIGN, "x, gain and partner must be 16-byte aligned");
    const int64_t K = w[0]->n_cols;
    if (K % 4) return skn_fail(ctx, SKN_ERR_SHAPE, "Shapes do not align.");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaError_t e = skn_launch_matvec_fused(ctx, n, w, x_dev, y_dev, add_dev, norm_gain_dev, norm_eps, silu_u_dev, ctx->stream);
    if (e == cudaErrorNotSupported) {
        // shapes outside the streaming kernel: transform x with the element-wise kernels first
        const float *xin = x_dev;
        if (norm_gain_dev || silu_u_dev) {
            int32_t rc = skn_stage_reserve(ctx, &ctx->d_scratch, &ctx->d_scratch_bytes, (size_t)K * sizeof(float));
            if (rc) return rc;
            float *t = (float *)ctx->d_scratch;
            if (norm_gain_dev) SKN_CUDA(ctx, skn_launch_rmsnorm(x_dev, norm_gain_dev, t, 1, (int)K, norm_eps, ctx->stream));
            else SKN_CUDA(ctx, skn_launch_silu_mul(x_dev, silu_u_dev, t, K, ctx->sm_count, ctx->stream));
            xin = t;
        }
        e = skn_launch_matvec_group(ctx, n, w, xin, y_dev, add_dev, ctx->stream);
    }
    SKN_CUDA(ctx, e);
    return SKN_OK;
}

int32_t skn_ffn_swiglu_dev(skn_ctx *ctx, const skn_tensor *wg, const skn_tensor *wu, const skn_tensor *wd,
                           const float *x_dev, int32_t M, float *y_dev) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    SKN_ENTER(ctx);
    if (!skn_tensor_ok(wg) || !skn_tensor_ok(wu) || !skn_tensor_ok(wd) || wg->ctx != ctx || wu->ctx != ctx || wd->ctx != ctx)
        return skn_fail(ctx, SKN_ERR_BAD_HANDLE, "bad tensor handle");
    if (M < 0) return skn_fail(ctx, SKN_ERR_ARG, "M is negative");
    if (wg->n_rows != wu->n_rows || wg->n_cols != wu->n_cols || wd->n_cols != wg->n_rows || wg->type != wu->type)
        return skn_fail(ctx, SKN_ERR_SHAPE, "Shapes do not align.");
    if (M == 0 || wd->n_rows == 0) return SKN_OK;
    if (!x_dev || !y_dev) return skn_fail(ctx, SKN_ERR_ARG, "x or y is NULL");
    if ((((uintptr_t)x_dev) | ((uintptr_t)y_dev)) & 15) return skn_fail(ctx, SKN_ERR_ALIGN, "x and y must be 16-byte aligned");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    const int64_t F = wg->n_rows, K = wg->n_cols;
    if (ctx->prefill_min_m > 0 && M >= ctx->prefill_min_m && skn_tc_supported(wg, M) && skn_tc_supported(wd, M)) {
        // [A bf16 | H bf16] in the context scratch
        const size_t ab = ((size_t)M * K * 2 + 255) / 256 * 256, hb = (size_t)M * F * 2;
        int32_t rc = skn_stage_reserve(ctx, &ctx->d_scratch, &ctx->d_scratch_bytes, ab + hb);
        if (rc) return rc;
        void *a16 = ctx->d_scratch, *h16 = (uint8_t *)ctx->d_scratch + ab;
        SKN_CUDA(ctx, skn_launch_f32_to_bf16(x_dev, a16, (int64_t)M * K, ctx->sm_count, ctx->stream));
        SKN_CUDA(ctx, skn_launch_gate_up_tc(ctx, wg, wu, a16, M, h16, ctx->stream));
        SKN_CUDA(ctx, skn_launch_matmul_tc(ctx, wd, h16, M, nullptr, y_dev, ctx->stream));
        return SKN_OK;
    }
    // decode-size path: three fp32 fused dequant-dot products and an element-wise SwiGLU
    const size_t gb = ((size_t)M * F * sizeof(float) + 255) / 256 * 256;
    int32_t rc = skn_stage_reserve(ctx, &ctx->d_scratch, &ctx->d_scratch_bytes, 2 * gb);
    if (rc) return rc;
    float *g = (float *)ctx->d_scratch, *u = (float *)((uint8_t *)ctx->d_scratch + gb);
    SKN_CUDA(ctx, skn_launch_matvec(ctx, wg, x_dev, M, nullptr, g, ctx->stream));
    SKN_CUDA(ctx, skn_launch_matvec(ctx, wu, x_dev, M, nullptr, u, ctx->stream));
    SKN_CUDA(ctx, skn_launch_silu_mul(g, u, g, (int64_t)M * F, ctx->sm_count, ctx->stream));
    SKN_CUDA(ctx, skn_launch_matvec(ctx, wd, g, M, nullptr, y_dev, ctx->stream));
    return SKN_OK;
}

int32_t skn_ffn_swiglu(skn_ctx *ctx, const skn_tensor *wg, const skn_tensor *wu, const skn_tensor *wd,
                       const float *x_host, int32_t M, float *y_host) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    SKN_ENTER(ctx);
    if (!skn_tensor_ok(wg) || !skn_tensor_ok(wd)) return skn_fail(ctx, SKN_ERR_BAD_HANDLE, "bad tensor handle");
    if (M < 0) return skn_fail(ctx, SKN_ERR_ARG, "M is negative");
    if (M == 0) return SKN_OK;
    if (!x_host || !y_host) return skn_fail(ctx, SKN_ERR_ARG, "x or y is NULL");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t xb = (size_t)M * wg->n_cols * sizeof(float), yb = (size_t)M * wd->n_rows * sizeof(float);
    int32_t rc = skn_stage_reserve(ctx, &ctx->d_stage_in, &ctx->d_stage_in_bytes, xb);
    if (rc) return rc;
    rc = skn_stage_reserve(ctx, &ctx->d_stage_out, &ctx->d_stage_out_bytes, yb);
    if (rc) return rc;
    SKN_CUDA(ctx, cudaMemcpyAsync(ctx->d_stage_in, x_host, xb, cudaMemcpyHostToDevice, ctx->stream));
    rc = skn_ffn_swiglu_dev(ctx, wg, wu, wd, (const float *)ctx->d_stage_in, M, (float *)ctx->d_stage_out);
    if (rc) return rc;
    SKN_CUDA(ctx, cudaMemcpyAsync(y_host, ctx->d_stage_out, yb, cudaMemcpyDeviceToHost, ctx->stream));
    return skn_sync(ctx);
}

// device-side address of a page-locked host buffer (registered or allocated by the CUDA runtime), or NULL for
// pageable memory
static void *host_mapped(const void *p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return a.type == cudaMemoryTypeHost ? a.devicePointer : nullptr;
}

// sync: return when y_host holds the result (and report the device status); otherwise return once the
// copies and the launch are enqueued on the context's stream
static int32_t matmul_host(skn_ctx *ctx, const skn_tensor *w, const float *x_host, int32_t M, int64_t K, const float *bias_host,
                           float *y_host, bool sync) {
    int32_t rc = check_matmul_args(ctx, w, x_host, M, K, y_host);
    if (rc) return rc;
    SKN_ENTER(ctx);
    if (M == 0 || w->n_rows == 0) return SKN_OK;
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    // The product reads what the fetch kernel (or the staged copy) of this very call wrote: that chain keeps
    // stream order whatever SKN_OPT_RELAXED_ORDER says about the caller's consecutive calls.
    skn_order_guard guard(ctx);
    const size_t xb = (size_t)M * (size_t)K * sizeof(float);
    const size_t bb = bias_host ? (size_t)w->n_rows * sizeof(float) : 0;
    const size_t xb_al = (xb + 255) / 256 * 256;
    const size_t yb = (size_t)M * (size_t)w->n_rows * sizeof(float);
    rc = skn_stage_reserve(ctx, &ctx->d_stage_in, &ctx->d_stage_in_bytes, xb_al + bb + 256);
    if (rc) return rc;
    float *dx = (float *)ctx->d_stage_in;
    float *db = bias_host ? (float *)((uint8_t *)ctx->d_stage_in + xb_al) : nullptr;
    if (yb <= (64 << 10) && xb <= (1 << 20) && (K % 4) == 0 && ((w->n_rows * (int64_t)M) % 4) == 0 && (!sync || ctx->h_status_dev)) {
        // Decode-size call on page-locked buffers: no copy-engine operation at all.  A one-CTA-per-4-KB kernel
        // fetches x over PCIe into device memory (every CTA of the matvec reads all of x: that must not cross
        // the bus 148 times), and the matvec writes y straight into the caller's mapped buffer.  A copy-engine
        // operation between two kernels costs several microseconds of hand-over each way; kernels hand over
        // to one another in one or two, and the matvec prefetches its weights under the fetch.
        void *xm = host_mapped(x_host), *ym = host_mapped(y_host), *bm = bias_host ? host_mapped(bias_host) : nullptr;
        if (xm && ym && (!bias_host || bm) && !((((uintptr_t)xm) | ((uintptr_t)ym) | ((uintptr_t)bm)) & 15)) {
            SKN_CUDA(ctx, skn_launch_fetch((const float *)xm, dx, (int64_t)M * K, ctx->stream));
            if (db) SKN_CUDA(ctx, skn_launch_fetch((const float *)bm, db, w->n_rows, ctx->stream));
            // (measured: 12.8 us per 4096 x 4096 call this way, 14.8 with a second kernel pushing y out of device
            // memory, 20.2 with a copy-engine transfer of y)
            rc = skn_matmul_dev(ctx, w, dx, M, K, db, (float *)ym);
            if (rc || !sync) return rc;
            // the blocking call: the status word follows through a kernel as well (16 bytes into the pinned mirror)
            SKN_CUDA(ctx, skn_launch_fetch((const float *)ctx->d_status, (float *)ctx->h_status_dev, 4, ctx->stream));
            SKN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            return skn_status_check(ctx);
        }
    }
    if (sync && yb <= SKN_SMALL_OUT_BYTES) {
        // decode-size result: it is written right below the status word and comes back with it in ONE copy
        // (a separate copy of the status costs as much as the matvec itself)
        const size_t yb_al = (yb + 255) / 256 * 256;
        float *dys = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(ctx->d_status) - yb_al);
        uint8_t *hys = reinterpret_cast<uint8_t *>(ctx->h_status) - yb_al;
        if (xb) SKN_CUDA(ctx, cudaMemcpyAsync(dx, x_host, xb, cudaMemcpyHostToDevice, ctx->stream));
        if (db) SKN_CUDA(ctx, cudaMemcpyAsync(db, bias_host, bb, cudaMemcpyHostToDevice, ctx->stream));
        rc = skn_matmul_dev(ctx, w, dx, M, K, db, dys);
        if (rc) return rc;
        SKN_CUDA(ctx, cudaMemcpyAsync(hys, dys, yb_al + sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
        SKN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        rc = skn_status_check(ctx);
        if (rc) return rc;
        memcpy(y_host, hys, yb);
        return SKN_OK;
    }
    rc = skn_stage_reserve(ctx, &ctx->d_stage_out, &ctx->d_stage_out_bytes, yb);
    if (rc) return rc;
    if (xb) SKN_CUDA(ctx, cudaMemcpyAsync(dx, x_host, xb, cudaMemcpyHostToDevice, ctx->stream));
    if (db) SKN_CUDA(ctx, cudaMemcpyAsync(db, bias_host, bb, cudaMemcpyHostToDevice, ctx->stream));
    rc = skn_matmul_dev(ctx, w, dx, M, K, db, (float *)ctx->d_stage_out);
    if (rc) return rc;
    SKN_CUDA(ctx, cudaMemcpyAsync(y_host, ctx->d_stage_out, yb, cudaMemcpyDeviceToHost, ctx->stream));
    return sync ? skn_sync(ctx) : SKN_OK;
}

int32_t skn_matmul(skn_ctx *ctx, const skn_tensor *w, const float *x_host, int32_t M, int64_t K, const float *bias_host,
                   float *y_host) {
    return matmul_host(ctx, w, x_host, M, K, bias_host, y_host, true);
}

int32_t skn_matmul_async(skn_ctx *ctx, const skn_tensor *w, const float *x_host, int32_t M, int64_t K,
                         const float *bias_host, float *y_host) {
    return matmul_host(ctx, w, x_host, M, K, bias_host, y_host, false);
}

}  // extern "C"

#ifdef SKN_TUNING
// Profiling builds only (never in the shipped library): copies the raw status/trace area.
extern "C" int32_t skn_debug_read_status(skn_ctx *ctx, void *out_host, int64_t bytes) {
    if (!skn_ctx_ok(ctx) || bytes > 32768) return SKN_ERR_ARG;
    SKN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    SKN_CUDA(ctx, cudaMemcpy(out_host, ctx->d_status, (size_t)bytes, cudaMemcpyDeviceToHost));
    return SKN_OK;
}
#endif
