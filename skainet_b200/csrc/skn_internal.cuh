// Internal declarations shared by the translation units of libskainet_cuda.so.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "skainet_cuda.h"

#define SKN_MAGIC_CTX 0x736b6e63u     // 'sknc'
#define SKN_MAGIC_TENSOR 0x736b6e74u  // 'sknt'
#define SKN_MAGIC_KV 0x736b6e6bu      // 'sknk'

// cached launch geometry of the streaming matvec (state: 0 = not planned yet,
// 1 = valid, -1 = shape not covered by the streaming kernel)
struct skn_mv_plan {
    int state;
    int nch, wg, grid, threads;
    size_t smem;
};

// plan of a grouped launch, cached in the context by (block type, total rows, columns, order)
struct skn_group_plan {
    int32_t type;
    int relaxed;
    int64_t rows, cols;
    skn_mv_plan pl;
};

constexpr size_t SKN_SMALL_OUT_BYTES = 96 * 1024;

struct skn_ctx {
    uint32_t magic;
    int device;
    cudaStream_t own_stream;
    cudaStream_t stream;        // stream `_dev` calls enqueue on
    int sm_count;
    int relaxed_order;          // SKN_OPT_RELAXED_ORDER
    int prefill_min_m;          // SKN_OPT_PREFILL_MIN_M: batch size from which the tensor-core path runs
    int fused_exchange;         // SKN_OPT_FUSED_EXCHANGE
    int kv_f16;                 // SKN_OPT_KV_F16 / SKN_OPT_KV_DTYPE: SKN_KV_* element type of the caches of new decoders
    int32_t *d_status;          // device status word written by bounded waits
    int32_t *h_status;          // pinned mirror
    // Small results of the host-pointer calls sit directly BELOW the status word, on the device and in the
    // pinned mirror alike, so that one device-to-host copy brings a result and the status together.
    uint8_t *d_status_base;     // allocation: [SKN_SMALL_OUT_BYTES of result area][status / trace area]
    uint8_t *h_status_base;     // pinned:     [SKN_SMALL_OUT_BYTES of result area][status word]
    int32_t *h_status_dev;      // device-side address of h_status (page-locked memory is mapped)
    // staging for the host-pointer entry points (grown on demand)
    void *d_stage_in;  size_t d_stage_in_bytes;
    void *d_stage_out; size_t d_stage_out_bytes;
    void *d_scratch;   size_t d_scratch_bytes;   // kernel scratch (bf16 operands, FFN intermediates)
    void *d_scratch2;  size_t d_scratch2_bytes;  // attention split partials
    void *d_xq;        size_t d_xq_bytes;        // prepared activations of the many-row matvec (digit planes, block records)
    uint32_t rows_cfg;                           // many-row matvec variants whose attributes are set on this device
    skn_group_plan group_plans[32];
    int n_group_plans;
    uint32_t attn_stream_cfg;   // bit per (head_dim, group size): the streamed attention kernel's attributes are set on this device
    // one host thread at a time: the thread inside an entry point (0: none) and its nesting depth
    // (entry points call one another); a second thread gets SKN_ERR_BUSY
    uint64_t owner;
    int owner_depth;
    char err[512];
};

// Entry-point guard of the one-thread-at-a-time rule.  Re-entrant for the owning thread.
uint64_t skn_thread_token();
struct skn_busy_guard {
    skn_ctx *c;
    bool ok;
    explicit skn_busy_guard(skn_ctx *cx) : c(cx), ok(false) {
        const uint64_t me = skn_thread_token();
        uint64_t expected = 0;
        if (__atomic_compare_exchange_n(&c->owner, &expected, me, false, __ATOMIC_ACQUIRE, __ATOMIC_RELAXED)) {
            ok = true;
            c->owner_depth = 1;
        } else if (expected == me) {
            ok = true;
            ++c->owner_depth;
        }
    }
    ~skn_busy_guard() {
        if (ok && --c->owner_depth == 0) __atomic_store_n(&c->owner, (uint64_t)0, __ATOMIC_RELEASE);
    }
    skn_busy_guard(const skn_busy_guard &) = delete;
    skn_busy_guard &operator=(const skn_busy_guard &) = delete;
};
int32_t skn_busy_fail();
// after the handle checks of an entry point: claim the context for this thread or answer SKN_ERR_BUSY
#define SKN_ENTER(ctx)                 \
    skn_busy_guard busy_guard__(ctx);  \
    if (!busy_guard__.ok) return skn_busy_fail()

// the status area on the device: word 0 = status of bounded waits and capacity checks, word 1 = limit of the
// flag waits of the inter-GPU exchange in milliseconds (0: the default of two seconds)
constexpr int SKN_STATUS_WAIT_MS = 1;
__device__ __forceinline__ uint64_t skn_wait_limit_ns(const int32_t *status) {
    const int32_t ms = reinterpret_cast<const volatile int32_t *>(status)[SKN_STATUS_WAIT_MS];
    return ms > 0 ? (uint64_t)ms * 1000000ull : 2000000000ull;
}

struct skn_tensor {
    uint32_t magic;
    skn_ctx *ctx;
    int32_t type;
    int64_t n_rows, n_cols;
    int64_t row_bytes;   // n_cols / block_elems * block_bytes
    int64_t pitch;       // device row pitch in bytes (multiple of 16)
    uint8_t *d_blocks;
    skn_mv_plan mv_plan[2];      // [0] stream order, [1] relaxed order
    // tensor maps of the raw blocks for the many-row matvec (opaque CUtensorMap images), by box width in bytes (0: unset)
    alignas(64) unsigned char rows_tmap[2][128];
    int rows_tmap_wrow[2];
};

// Forces stream order on the context for the lifetime of the guard: call sequences whose launches depend on
// one another (a decoder step; the fetch -> product chain inside a host-pointer call) must not inherit
// SKN_OPT_RELAXED_ORDER, which only describes the caller's consecutive calls.
struct skn_order_guard {
    skn_ctx *c;
    int saved;
    explicit skn_order_guard(skn_ctx *cx) : c(cx), saved(cx->relaxed_order) { c->relaxed_order = 0; }
    ~skn_order_guard() { c->relaxed_order = saved; }
    skn_order_guard(const skn_order_guard &) = delete;
    skn_order_guard &operator=(const skn_order_guard &) = delete;
};

// error plumbing (skn_api.cu)
int32_t skn_fail(skn_ctx *ctx, int32_t code, const char *fmt, ...);
int32_t skn_check_cuda(skn_ctx *ctx, cudaError_t e, const char *what);
bool skn_ctx_ok(const skn_ctx *ctx);
bool skn_tensor_ok(const skn_tensor *t);
int32_t skn_stage_reserve(skn_ctx *ctx, void **buf, size_t *cap, size_t need);
int32_t skn_status_check(skn_ctx *ctx);

#define SKN_CUDA(ctx, call)                                            \
    do {                                                               \
        cudaError_t e__ = (call);                                      \
        if (e__ != cudaSuccess) return skn_check_cuda(ctx, e__, #call); \
    } while (0)

static inline bool skn_geometry(int32_t type, int32_t *elems, int32_t *bytes) {
    switch (type) {
    case SKN_TYPE_Q4_0: *elems = 32;  *bytes = 18;  return true;
    case SKN_TYPE_Q8_0: *elems = 32;  *bytes = 34;  return true;
    case SKN_TYPE_Q4_K: *elems = 256; *bytes = 144; return true;
    case SKN_TYPE_Q6_K: *elems = 256; *bytes = 210; return true;
    case SKN_TYPE_Q4_1: *elems = 32;  *bytes = 20;  return true;
    case SKN_TYPE_Q5_0: *elems = 32;  *bytes = 22;  return true;
    case SKN_TYPE_Q5_1: *elems = 32;  *bytes = 24;  return true;
    case SKN_TYPE_Q5_K: *elems = 256; *bytes = 176; return true;
    case SKN_TYPE_Q2_K: *elems = 256; *bytes = 84;  return true;
    case SKN_TYPE_Q3_K: *elems = 256; *bytes = 110; return true;
    case SKN_TYPE_IQ4_NL: *elems = 32;  *bytes = 18;  return true;
    case SKN_TYPE_IQ4_XS: *elems = 256; *bytes = 136; return true;
    default: return false;
    }
}

// kernel launchers (one per translation unit); all enqueue on `stream` and return the
// launch status
cudaError_t skn_launch_dequant(int32_t type, const uint8_t *blocks, int64_t pitch, int64_t n_rows,
                               int64_t n_cols, float *out, cudaStream_t stream);
cudaError_t skn_launch_matvec(skn_ctx *ctx, const skn_tensor *w, const float *x, int32_t M,
                              const float *bias, float *y, cudaStream_t stream);
cudaError_t skn_launch_matvec_fused(skn_ctx *ctx, int n, const skn_tensor *const *w, const float *x, float *const *y,
                                    const float *const *add, const float *norm_gain, float norm_eps,
                                    const float *silu_u, cudaStream_t stream);
// integer tensor-core matvec (skn_matvec_mma.cu); false = shapes or type not covered
bool skn_mma_try_group(skn_ctx *ctx, int n, const skn_tensor *const *w, const float *x, float *const *y,
                       const float *const *add, const float *norm_gain, float norm_eps, const float *silu_u,
                       cudaStream_t stream, cudaError_t &err, bool swiglu = false, int n_act = 1, bool add_per_act = false,
                       const struct skn_mv_exchange *xc = nullptr, const struct skn_mv_rope *rope = nullptr);
// activation rows one tensor-core matvec launch can take for this tensor (0: not covered)
int skn_mma_max_acts(const skn_ctx *ctx, int32_t type, int64_t n_rows_total, int64_t n_cols);
// many-row tensor-core matvec (skn_matvec_rows.cu): x prepared once per launch by its own kernel, 3 to 16 rows
int skn_rows_max_acts(const skn_ctx *ctx, int n, const skn_tensor *const *w);
bool skn_rows_try_group(skn_ctx *ctx, int n, const skn_tensor *const *w, const float *x, int M, float *const *y,
                        const float *const *add, bool add_per_act, const float *norm_gain, float norm_eps, const float *silu_u,
                        bool swiglu, cudaStream_t stream, cudaError_t &err);
// y[t][m] = W[t] . f(x[m]) (+ add) for M activation rows through the tensor-core matvec, in launches
// of as many rows as fit; cudaErrorNotSupported (nothing launched) when it does not cover the tensors.
// x rows are K apart, outputs (and per-row add vectors) n_rows apart.
cudaError_t skn_launch_matvec_acts(skn_ctx *ctx, int n, const skn_tensor *const *w, const float *x, int M, float *const *y,
                                   const float *const *add, bool add_per_act, const float *norm_gain, float norm_eps,
                                   const float *silu_u, bool swiglu, cudaStream_t stream, const struct skn_mv_exchange *xc = nullptr,
                                   const struct skn_mv_rope *rope = nullptr);
// h = silu(Wg . f(x)) * (Wu . f(x)) in one launch (f: optional RMSNorm); cudaErrorNotSupported when
// the tensor-core matvec does not cover the tensors (nothing launched)
cudaError_t skn_launch_gate_up_swiglu(skn_ctx *ctx, const skn_tensor *wg, const skn_tensor *wu, const float *x, float *h,
                                      const float *norm_gain, float norm_eps, cudaStream_t stream);
cudaError_t skn_launch_matvec_group(skn_ctx *ctx, int n, const skn_tensor *const *w, const float *x, float *const *y,
                                    const float *const *add, cudaStream_t stream);

// tensor-core prefill path (skn_matmul_tc.cu)
bool skn_tc_supported(const skn_tensor *w, int32_t M);
cudaError_t skn_launch_f32_to_bf16(const float *in, void *out_bf16, int64_t n, int sm_count, cudaStream_t stream);
cudaError_t skn_launch_matmul_tc(skn_ctx *ctx, const skn_tensor *w, const void *a_bf16, int32_t M, const float *bias,
                                 float *y, cudaStream_t stream);
cudaError_t skn_launch_gate_up_tc(skn_ctx *ctx, const skn_tensor *wg, const skn_tensor *wu, const void *a_bf16,
                                  int32_t M, void *h_bf16, cudaStream_t stream);
cudaError_t skn_launch_silu_mul(const float *g, const float *u, float *h, int64_t n, int sm_count, cudaStream_t stream);

// decoder glue (skn_glue.cu)
cudaError_t skn_launch_rmsnorm(const float *x, const float *gain, float *y, int M, int D, float eps, cudaStream_t st);
cudaError_t skn_launch_rope(float *x, const int32_t *len, int M, int T, int H, int D, float theta, int sm_count, cudaStream_t st);
cudaError_t skn_launch_add(const float *a, const float *b, float *out, int64_t n, int sm_count, cudaStream_t st);
cudaError_t skn_launch_fetch(const float *src, float *dst, int64_t n, cudaStream_t st);
cudaError_t skn_launch_last_rows(const float *in, float *out, int B, int T, int D, cudaStream_t st);
size_t skn_argmax_scratch_bytes(int M);
cudaError_t skn_launch_argmax(const float *logits, int M, int V, int32_t *ids, void *scratch, cudaStream_t st);
cudaError_t skn_launch_argmax_offer(const float *logits, const int32_t *ids, int B, int V_local, int rank, int world,
                                    float *cand, cudaStream_t st);
cudaError_t skn_launch_argmax_pick(const float *cand, int B, int world, int32_t *ids, cudaStream_t st);
cudaError_t skn_launch_embed(const skn_tensor *emb, const int32_t *ids, int M, float *out, cudaStream_t st);

// decoder-internal forms of the cache operations (skn_kv.cu): K/V rotated and written without
// advancing the lengths, attention over the cache plus those T pending tokens, and one advance
// for all layers at the end of a step
int32_t skn_kv_rope_append_pending(skn_kvcache *kv, float *q_dev, const float *k_new_dev, const float *v_new_dev,
                                   int32_t n_q_heads, int32_t T, float theta, int32_t host_len_upper);
int32_t skn_attn_causal_pending(skn_kvcache *kv, const float *q_dev, int32_t n_q_heads, int32_t T, float scale,
                                float *out_dev);
int32_t *skn_kv_len_dev(const skn_kvcache *kv);
cudaError_t skn_kv_advance_all(int32_t *const *lens_dev, int n_layers, int B, int T, int cap, int32_t *status_dev,
                               cudaStream_t st);

// inter-GPU exchange (skn_comm.cu): layout constants and the device-side view the matvec kernels
// use to push partial products from their epilogue and to add them up while they prepare x
constexpr int SKN_COMM_NBUF = 2;
constexpr int SKN_COMM_MAX_WORLD = 8;
constexpr size_t SKN_COMM_FLAG_BYTES = 4096;
struct skn_comm_view {
    int32_t rank, world;
    int64_t capacity;                       // floats per (buffer, source rank)
    uint8_t *base[SKN_COMM_MAX_WORLD];      // inbox of every rank as mapped on this device
    uint32_t *state;                        // [0] exchanges completed, [1] push tickets, [2] finish tickets
};
bool skn_comm_get_view(const skn_comm *c, skn_comm_view *v);
// Sweep knobs exist only in SKN_TUNING builds; the shipped library compiles every one down to its default.
#ifdef SKN_TUNING
#include <stdlib.h>
static inline int skn_tune_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}
#else
static inline int skn_tune_int(const char *, int dflt) { return dflt; }
#endif

struct skn_mv_rope {                        // optional argument of skn_launch_matvec_acts: (wq, wk, wv) of a single-token step
    int head_dim, n_kv_heads, capacity, seq0;   // seq0: sequence of the first activation row
    const int32_t *len_dev, *start_dev;         // cache lengths (= positions of the new tokens) and ring starts
    float *k_cache, *v_cache;
    float theta;
    const double *inv_freq;                     // optional device table theta^(-2i / head_dim), i < head_dim / 2 (NULL: computed per element)
};
struct skn_mv_exchange {                    // optional argument of skn_launch_matvec_acts
    skn_comm_view view;
    bool push;                              // outputs are partial products: push them, y is not written
    bool reduce;                            // x is the residual stream: add the partials pushed before
    float *writeback;                       // reduce: the summed residual stream goes here (may be NULL)
};
