/*
 * libskainet_cuda.so -- C ABI of the B200 (sm_100a) quantized-inference backend for
 * sk-ai-net/skainet.
 *
 * Every entry point takes plain pointers and sizes, returns an int32 status
 * (0 = SKN_OK) and never lets a C++ exception cross the boundary.  Handles are opaque
 * pointers created and destroyed explicitly.  Host buffers are borrowed for the
 * duration of one call.  Entry points whose name ends in `_dev` take DEVICE pointers
 * and only enqueue work on the context's stream (call skn_sync to wait); all others
 * take HOST pointers and return when the result is in the caller's buffer.
 *
 * The reference (Kotlin multiplatform, v0.0.7) has no FFI of its own; each function
 * cites the reference interface it stands behind.  Paths are relative to the
 * reference's repository root.
 *
 * A context is bound to one CUDA device and must be used by one host thread at a
 * time: an entry point called while another thread is inside a call on the same context
 * (directly, or through one of its tensors, caches, exchanges or decoders) returns
 * SKN_ERR_BUSY without touching the context; its message is read with skn_last_error(NULL)
 * on the refused thread.  The reference is single-threaded (no counterpart).  There is no
 * CPU fallback: without a usable CUDA device every compute entry point fails with
 * SKN_ERR_CUDA.
 */
#ifndef SKAINET_CUDA_H
#define SKAINET_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SKN_VERSION 100 /* 0.1.0 */

/* status codes */
#define SKN_OK 0
#define SKN_ERR_SHAPE 1      /* maps to IllegalArgumentException("Shapes do not align.") */
#define SKN_ERR_TYPE 2       /* unknown / unsupported GGML type id */
#define SKN_ERR_ALIGN 3      /* pointer or pitch alignment */
#define SKN_ERR_OOM 4
#define SKN_ERR_CUDA 5
#define SKN_ERR_TIMEOUT 6    /* a bounded device-side wait ran out */
#define SKN_ERR_BAD_HANDLE 7
#define SKN_ERR_ARG 8        /* null pointer, negative size, ... */
#define SKN_ERR_COMM 9
#define SKN_ERR_BUSY 10      /* the context is inside a call made by another host thread */

/* GGML type ids: gguf/src/commonMain/kotlin/sk/ai/net/gguf/Constants.kt:14-52 */
#define SKN_TYPE_Q4_0 2
#define SKN_TYPE_Q8_0 8
#define SKN_TYPE_Q4_K 12
#define SKN_TYPE_Q6_K 14
/* Further block types of the reference's table (Constants.kt:62-80), served by the dequantiser
 * and the generic fused dequant-dot (any M, fp32); they have no streaming / tensor-core kernels. */
#define SKN_TYPE_Q4_1 3   /* 32 weights, 20 bytes: d, m (fp16), 16 nibble bytes: q * d + m */
#define SKN_TYPE_Q5_0 6   /* 32 weights, 22 bytes: d, 32 high bits, 16 nibble bytes: (q - 16) * d */
#define SKN_TYPE_Q5_1 7   /* 32 weights, 24 bytes: d, m, 32 high bits, 16 nibble bytes: q * d + m */
#define SKN_TYPE_Q5_K 13  /* 256 weights, 176 bytes: d, dmin, 12 scale bytes, 32 high-bit bytes, 128 nibble bytes */
#define SKN_TYPE_Q2_K 10  /* 256 weights, 84 bytes: 16 scale/min nibble pairs, 64 bytes of 2-bit quants, d, dmin */
#define SKN_TYPE_Q3_K 11  /* 256 weights, 110 bytes: 32 high-bit bytes, 64 bytes of 2-bit quants, 12 scale bytes, d */
#define SKN_TYPE_IQ4_NL 20 /* 32 weights, 18 bytes: d, 16 nibble bytes indexing the 16-entry IQ4 codebook */
#define SKN_TYPE_IQ4_XS 23 /* 256 weights, 136 bytes: d, 16 scale high bits, 4 scale nibble bytes, 128 codebook nibbles */

typedef struct skn_ctx skn_ctx;
typedef struct skn_tensor skn_tensor;
typedef struct skn_kvcache skn_kvcache;

/* ---- library / context ------------------------------------------------------------- */

/* Library version (SKN_VERSION of the build). */
int32_t skn_version(void);

/* Message of the last failure on `ctx` (or, with ctx == NULL, of the last failing call
 * on this thread that had no context).  Never NULL.  Plays the role of the exception
 * message in the reference (core/src/commonMain/kotlin/sk/ai/net/impl/DoublesTensor.kt:256). */
const char *skn_last_error(const skn_ctx *ctx);

/* Create a context on CUDA device `device` with its own non-blocking stream.
 * Stands where the reference constructs its one backend,
 * core/src/commonMain/kotlin/sk/ai/net/impl/DefaultTensorFactory.kt:9-17. */
int32_t skn_ctx_create(int32_t device, skn_ctx **out);
int32_t skn_ctx_destroy(skn_ctx *ctx);

/* Make `_dev` entry points enqueue on `cuda_stream` (a cudaStream_t) instead of the
 * context's own stream; NULL restores the context's stream. */
int32_t skn_ctx_set_stream(skn_ctx *ctx, void *cuda_stream);

/* Context options.
 * SKN_OPT_RELAXED_ORDER (default 0): with value 1 the caller promises that consecutive
 * `_dev` launches on this context are independent of one another -- no launch reads a
 * buffer that the launch before it writes, nor writes one that it reads or writes (as for
 * the Q/K/V or gate/up projections of one activation, or a stack of unrelated layers).
 * Launches may then overlap on the GPU instead of running in stream order; everything is
 * still complete when skn_sync (or a later operation on the stream) returns.  The reference
 * is single-threaded and has no notion of ordering (Tensor.kt:6-33): no counterpart. */
#define SKN_OPT_RELAXED_ORDER 1
/* SKN_OPT_PREFILL_MIN_M (default 64): batch size M from which skn_matmul / skn_ffn_swiglu run on
 * the tensor cores with bf16 operands and fp32 accumulation (relative error up to 1e-2 against
 * the fp64 oracle); below it, and always with value 0, products are fp32 fused dequant-dot
 * (1e-5). */
#define SKN_OPT_PREFILL_MIN_M 2
/* SKN_OPT_FUSED_EXCHANGE (1 on, 0 off, -1 automatic = default): tensor-parallel decoder with one or two rows per step: the
 * K-sharded projections push their partial products into every rank's inbox from the matvec
 * epilogue and the next projection adds them to the residual stream while it prepares x,
 * instead of a separate exchange launch (skn_allreduce_dev) after each of them.  Same results
 * bit for bit.  Automatic means off: the separate exchange of decode-size vectors is a single
 * trip over NVLink (tagged words, no fence) started early by programmatic dependent launch, and
 * measures faster than the fused form, in which every CTA of the consuming launch repeats the sum. */
#define SKN_OPT_FUSED_EXCHANGE 3
/* SKN_OPT_KV_F16 (default 0): with value 1, decoders created afterwards (skn_llama_create, skn_llama_create_tp)
 * keep their KV caches in fp16 (see skn_kv_create_typed).  SKN_OPT_KV_DTYPE is the general form: its value is
 * the SKN_KV_* element type of the caches of decoders created afterwards. */
#define SKN_OPT_KV_F16 4
#define SKN_OPT_KV_DTYPE 6
/* SKN_OPT_WAIT_LIMIT_MS (default 0 = 2000): how long a kernel of the inter-GPU exchange waits for its
 * peers' flags before it gives up, records SKN_ERR_TIMEOUT and returns (1 .. 600000 milliseconds). */
#define SKN_OPT_WAIT_LIMIT_MS 5
int32_t skn_ctx_set_option(skn_ctx *ctx, int32_t option, int64_t value);

/* Wait for everything enqueued on the context's stream; reports a pending device-side status if a
 * kernel recorded one, and clears it: SKN_ERR_TIMEOUT (a bounded wait ran out) or SKN_ERR_SHAPE (a
 * decoder step found its KV cache full: nothing was overwritten, the step's results are invalid). */
int32_t skn_sync(skn_ctx *ctx);

/* ---- block geometry ---------------------------------------------------------------- */

/* (elements per block, bytes per block) of a GGML type:
 * GGML_QUANT_SIZES, gguf/src/commonMain/kotlin/sk/ai/net/gguf/Constants.kt:58-90. */
int32_t skn_quant_geometry(int32_t ggml_type, int32_t *block_elems, int32_t *block_bytes);

/* Bytes of one row of `n_cols` weights; SKN_ERR_SHAPE when n_cols is not a multiple of
 * the block size: quantShapeToByteShape, gguf/src/commonMain/kotlin/sk/ai/net/gguf/Quants.kt:10-20. */
int32_t skn_quant_row_bytes(int32_t ggml_type, int64_t n_cols, int64_t *row_bytes);

/* ---- quantized weight tensors ------------------------------------------------------ */

/* Upload the raw blocks of a [n_rows, n_cols] weight (GGUF order: n_cols contiguous,
 * i.e. Linear's [out, in], core/src/commonMain/kotlin/sk/ai/net/nn/Linear.kt:43-49) to
 * HBM, unchanged.  `host_blocks` is what GGUFReader hands out for a quantized tensor
 * (gguf/src/commonMain/kotlin/sk/ai/net/gguf/GGUFReader.kt:370-398); n_bytes must equal
 * n_rows * row_bytes.  Replaces the branch that skips quantized tensors,
 * samples/mnist-mlp-cli/src/jvmMain/kotlin/sk/ai/net/samples/mnist/mlp/Main.kt:229-232. */
int32_t skn_tensor_upload_quant(skn_ctx *ctx, int32_t ggml_type, int64_t n_rows, int64_t n_cols,
                                const void *host_blocks, int64_t n_bytes, skn_tensor **out);

/* Upload the sub-matrix rows [row_begin, row_begin+row_count) x columns
 * [col_begin, col_begin+col_count) of a [n_rows_total, n_cols_total] weight whose full
 * raw blocks are at host_blocks: the shard one GPU owns under column (row range) or row
 * (column range) parallelism.  col_begin / col_count must be multiples of the block
 * size.  Blocks are copied unchanged; the device row pitch is padded to 16 bytes.
 * No counterpart in the reference (it has no multi-device notion, Tensor.kt:6-33). */
int32_t skn_tensor_upload_quant_shard(skn_ctx *ctx, int32_t ggml_type, int64_t n_rows_total,
                                      int64_t n_cols_total, const void *host_blocks, int64_t n_bytes,
                                      int64_t row_begin, int64_t row_count, int64_t col_begin,
                                      int64_t col_count, skn_tensor **out);

int32_t skn_tensor_destroy(skn_tensor *t);

/* shape / type / device layout of a tensor (any out pointer may be NULL):
 * Tensor.shape / dataDescriptor, core/src/commonMain/kotlin/sk/ai/net/Tensor.kt:12-33. */
int32_t skn_tensor_info(const skn_tensor *t, int32_t *ggml_type, int64_t *n_rows, int64_t *n_cols,
                        int64_t *row_bytes, int64_t *row_pitch_bytes, void **device_blocks);

/* Dequantise the whole tensor to fp32 [n_rows, n_cols] (bit-exact with gguf-py 0.19.0's
 * dequantize, the code the reference's gguf module transliterates, Quants.kt:3-8). */
int32_t skn_dequantize(skn_ctx *ctx, const skn_tensor *t, float *out_host);
int32_t skn_dequantize_dev(skn_ctx *ctx, const skn_tensor *t, float *out_dev);

/* Y[M, n_rows] = X[M, K] . W^T with W the quantized [n_rows, K] tensor, fp32
 * accumulation; M = 1 is the decode matvec.  This is Linear.forward's
 * input.matmul(weight.t()) (core/src/commonMain/kotlin/sk/ai/net/nn/Linear.kt:48) i.e.
 * DoublesTensor.matmul's vector x matrix and matrix x matrix cases
 * (core/src/commonMain/kotlin/sk/ai/net/impl/DoublesTensor.kt:255-279) without the
 * per-call transposed copy (DoublesTensor.kt:362-387).  K != n_cols fails with
 * SKN_ERR_SHAPE ("Shapes do not align.", DoublesTensor.kt:256).  `bias` ([n_rows]
 * fp32, may be NULL) is added as Linear does. */
int32_t skn_matmul(skn_ctx *ctx, const skn_tensor *w, const float *x_host, int32_t M, int64_t K,
                   const float *bias_host, float *y_host);
int32_t skn_matmul_dev(skn_ctx *ctx, const skn_tensor *w, const float *x_dev, int32_t M, int64_t K,
                       const float *bias_dev, float *y_dev);
/* skn_matmul for a loop over layers: returns as soon as the copy of x (and bias), the kernel and the copy of y
 * are enqueued on the context's stream.  x_host and bias_host must stay unchanged and y_host must not be read
 * until skn_sync(ctx) has returned (it also reports the kernels' status).  Calls on one context run in the order
 * they were made, so a result may be the next call's x_host.  Page-locked host buffers keep the copies
 * asynchronous; pageable ones work, with the copies staged by the driver. */
int32_t skn_matmul_async(skn_ctx *ctx, const skn_tensor *w, const float *x_host, int32_t M, int64_t K,
                         const float *bias_host, float *y_host);

/* y[t] = W[t] . x (+ add[t]) for n <= 3 weights that multiply the same activation vector x (Q/K/V,
 * gate/up): one launch when the weights share type and K, separate launches otherwise.  add[t]
 * ([n_rows of W[t]], may be NULL, the array itself may be NULL) is a bias or a residual; y[t] may
 * alias add[t].  Several Linear.forward calls on one input (nn/Linear.kt:43-49) in one step. */
int32_t skn_matvec_group_dev(skn_ctx *ctx, int32_t n, const skn_tensor *const *w, const float *x_dev,
                             float *const *y_dev, const float *const *add_dev);

/* skn_matvec_group_dev with an element-wise step folded into the preparation of x (no extra
 * launch, no intermediate vector in HBM).  Exactly one of:
 *   norm_gain_dev != NULL : x <- x / sqrt(mean(x^2) + norm_eps) * gain   (RMSNorm before Q/K/V or gate/up)
 *   silu_u_dev    != NULL : x <- silu(x) * u                              (SwiGLU before the down projection)
 * or neither (then identical to skn_matvec_group_dev).  x itself is not modified, so y[t] may
 * alias add[t] but not x.  The reference would run these as separate tensor ops around
 * Linear.forward (nn/Linear.kt:43-49); it has neither RMSNorm nor SiLU. */
int32_t skn_matvec_fused_dev(skn_ctx *ctx, int32_t n, const skn_tensor *const *w, const float *x_dev,
                             float *const *y_dev, const float *const *add_dev, const float *norm_gain_dev,
                             float norm_eps, const float *silu_u_dev);

/* Y[M, N] = (silu(X . Wg^T) * (X . Wu^T)) . Wd^T -- the SwiGLU feed-forward block; Wg, Wu are
 * [F, K] (same block type), Wd is [N, F].  The reference has neither SiLU nor SwiGLU (its
 * sigmoid(), core/src/commonMain/kotlin/sk/ai/net/impl/DoublesTensor.kt:448-449, computes
 * 1/exp(-x)); this is Linear.forward (nn/Linear.kt:43-49) applied three times around the
 * textbook activation.  M >= SKN_OPT_PREFILL_MIN_M runs on the tensor cores (the intermediate
 * is kept in bf16, never fp16). */
int32_t skn_ffn_swiglu(skn_ctx *ctx, const skn_tensor *wg, const skn_tensor *wu, const skn_tensor *wd,
                       const float *x_host, int32_t M, float *y_host);
int32_t skn_ffn_swiglu_dev(skn_ctx *ctx, const skn_tensor *wg, const skn_tensor *wu, const skn_tensor *wd,
                           const float *x_dev, int32_t M, float *y_dev);

/* ---- KV cache and decode attention ------------------------------------------------------
 * The reference has no KV cache, no attention and no usable softmax (its softmax(dim),
 * core/src/commonMain/kotlin/sk/ai/net/impl/DoublesTensor.kt:491-519, indexes the wrong axis);
 * the nearest ancestor of a gather is the range slice DoublesTensor.get(vararg IntRange),
 * DoublesTensor.kt:52-68.  These entry points are new surface in the style of the rest. */

/* fp32 cache for `batch` sequences: K, V [batch][n_kv_heads][capacity][head_dim] (head-major
 * ring buffer, device resident).  head_dim is 64 or 128. */
int32_t skn_kv_create(skn_ctx *ctx, int32_t batch, int32_t n_kv_heads, int32_t head_dim, int32_t capacity,
                      skn_kvcache **out);
/* The same cache with a chosen element type.  SKN_KV_F16 stores K and V as IEEE fp16 (rounded to nearest
 * even on their way in, widened on their way out; every sum stays fp32), which halves the bytes attention
 * reads per cached token.  SKN_KV_Q8_0 stores them the way GGUF's Q8_0 stores weights
 * (gguf/src/commonMain/kotlin/sk/ai/net/gguf/Constants.kt:60: 32 values per block, one fp16 scale): per 32 head
 * dims d = max|x| / 127 and int8 q = round(x / d), read back as q * fp16(d) -- 1.0625 bytes per value instead of
 * four.  In memory the quants and the scales are two planes of one allocation ([rows][head_dim] int8, then
 * [rows][head_dim / 32] fp16, rows = batch * n_kv_heads * capacity), not interleaved 34-byte blocks.
 * Every entry point below keeps its fp32 interface: appends, loads, gathers, q and the attention output are
 * fp32 whatever the cache holds.  SKN_ERR_TYPE for any other value. */
#define SKN_KV_F32 0
#define SKN_KV_F16 1
#define SKN_KV_Q8_0 2
int32_t skn_kv_create_typed(skn_ctx *ctx, int32_t batch, int32_t n_kv_heads, int32_t head_dim, int32_t capacity,
                            int32_t kv_dtype, skn_kvcache **out);
/* element type of the cache (what k_dev / v_dev of skn_kv_info point at) */
int32_t skn_kv_dtype(const skn_kvcache *kv, int32_t *kv_dtype);
int32_t skn_kv_destroy(skn_kvcache *kv);
/* forget every cached token */
int32_t skn_kv_reset(skn_kvcache *kv);
/* Pre-fill: k_host, v_host are [batch][n_kv_heads][tokens][head_dim]; sequence b keeps its
 * first lens_host[b] tokens (lens_host[b] <= tokens <= capacity). */
int32_t skn_kv_load(skn_kvcache *kv, const float *k_host, const float *v_host, int32_t tokens,
                    const int32_t *lens_host);
/* Current length and ring start of every sequence (either pointer may be NULL). */
int32_t skn_kv_lengths(skn_kvcache *kv, int32_t *lens_host, int32_t *start_host);
/* Append one token per sequence: k_new, v_new are [batch][n_kv_heads][head_dim] (no rotary
 * embedding is applied here).  A full ring overwrites its oldest token. */
int32_t skn_kv_append(skn_kvcache *kv, const float *k_new_host, const float *v_new_host);
int32_t skn_kv_append_dev(skn_kvcache *kv, const float *k_new_dev, const float *v_new_dev);
/* Copy tokens [pos_begin, pos_begin+count) of sequence b, oldest first, to dense host arrays
 * [n_kv_heads][count][head_dim]. */
int32_t skn_kv_gather(skn_kvcache *kv, int32_t b, int32_t pos_begin, int32_t count, float *k_out_host,
                      float *v_out_host);
/* geometry and device pointers of the cache (any out pointer may be NULL) */
int32_t skn_kv_info(const skn_kvcache *kv, int32_t *batch, int32_t *n_kv_heads, int32_t *head_dim,
                    int32_t *capacity, void **k_dev, void **v_dev, void **len_dev, void **start_dev);

/* out[b][h][:] = softmax(q[b][h] . K^T * scale) . V over the cached tokens of sequence b, with
 * query head h reading kv head h / (n_q_heads / n_kv_heads); q and out are
 * [batch][n_q_heads][head_dim] fp32.  A sequence without tokens gives zeros.  n_q_heads must
 * be 1, 2, 4 or 8 times n_kv_heads ("Shapes do not align." otherwise).
 * The device form needs skn_attn_scratch_bytes() bytes of device scratch for the partial
 * results of its sequence splits: pass a buffer, or NULL to let the context allocate one. */
int32_t skn_attn_decode(skn_kvcache *kv, const float *q_host, int32_t n_q_heads, float scale, float *out_host);
int32_t skn_attn_decode_dev(skn_kvcache *kv, const float *q_dev, int32_t n_q_heads, float scale, float *out_dev,
                            void *scratch_dev);
/* bytes of scratch skn_attn_decode_dev needs for this cache and head count (-1 on bad arguments) */
int64_t skn_attn_scratch_bytes(const skn_kvcache *kv, int32_t n_q_heads);

/* skn_attn_decode_dev for callers that cannot allocate device memory when they call it (a
 * server whose memory plan is frozen after start-up, code running where the CUDA allocator's
 * implicit device synchronisation is not acceptable, an embedding runtime that passes a device
 * but no allocator).  It has no counterpart in the reference.  Same inputs, outputs and
 * results as skn_attn_decode_dev, but the split partials go to a 4 MiB array built into the
 * library (held by every GPU that loads it, until the process exits) and the call performs
 * no cudaMalloc / cudaFree of any kind.
 *  - Limit: skn_attn_scratch_bytes(kv, n_q_heads) <= 4 MiB (4 194 304), i.e.
 *    batch * n_q_heads * ceil(capacity / 256) * (head_dim + 2) * 4 bytes; larger problems are
 *    refused with SKN_ERR_SHAPE and a message naming both sizes.
 *  - The first call on each device looks up the array's device address (one
 *    cudaGetSymbolAddress with that device current); make that first call before any stream
 *    capture begins.
 *  - All calls, from every context on the device, share the one array and it keeps whatever
 *    the last call left in it.  Nothing in it needs clearing: each call writes every record
 *    it later reads.  Two calls that overlap on the GPU (different streams, or relaxed order)
 *    race on it; keep them in one stream's order. */
int32_t skn_attn_decode_noalloc_dev(skn_kvcache *kv, const float *q_dev, int32_t n_q_heads, float scale,
                                    float *out_dev);

/* Multi-token forms used by prefill (no counterpart in the reference).
 * skn_kv_append_many_dev: T tokens per sequence, k_new / v_new [batch][T][n_kv_heads][head_dim];
 *   never wraps the ring: host_len_upper (the caller's bound on the current lengths) + T must
 *   fit the capacity.
 * skn_attn_causal_dev: q, out [batch][T][n_q_heads][head_dim]; query t of the T most recent
 *   positions attends to the cache up to its own token (T = 1 is skn_attn_decode_dev).  Scratch:
 *   T * skn_attn_scratch_bytes() bytes, or NULL for the context's own. */
int32_t skn_kv_append_many_dev(skn_kvcache *kv, const float *k_new_dev, const float *v_new_dev, int32_t T,
                               int32_t host_len_upper);
int32_t skn_attn_causal_dev(skn_kvcache *kv, const float *q_dev, int32_t n_q_heads, int32_t T, float scale,
                            float *out_dev, void *scratch_dev);

/* Host arithmetic only (no device is touched, no context needed): the launch geometry the many-row
 * matvec (3 to 16 activation rows, weights streamed once) would get for n_groups sixteen-row groups of
 * n_cols columns on a GPU of sm_count SMs; swiglu: the interleaved gate / up form.  No reference
 * counterpart (introspection for hosts that size shards, and for this library's CPU tests).
 * out[8]: [0] 1 if the shape is covered, [1] CTAs, [2] most groups one CTA owns, [3] groups a CTA's
 * partial-sum space holds, [4] CTAs without a group, [5] K chunks, [6] ring stages, [7] bytes of
 * dynamic shared memory. */
int32_t skn_rows_plan_query(int32_t sm_count, int32_t type, int64_t n_groups, int64_t n_cols, int32_t n_act,
                            int32_t swiglu, int64_t *out);

/* ---- Exchange between the GPUs of one box ------------------------------------------------------
 * Sum of per-rank partial products of a K-sharded (row-parallel) layer, and, with zero-filled
 * slots, the concatenation of the slices of an N-sharded (column-parallel) one.  The reference
 * has no multi-device notion (core/src/commonMain/kotlin/sk/ai/net/Tensor.kt:6-33): new surface.
 * Every rank owns an inbox that its peers write with ordinary peer stores; one kernel per rank
 * pushes, waits (bounded: about two seconds, then SKN_ERR_TIMEOUT is reported by the next
 * skn_sync and later exchanges stop waiting) and sums in rank order, so every rank obtains the
 * same bits.  Vectors of up to 65536 floats travel as tagged 8-byte words {value, exchange number}
 * that the receiver polls, so that an exchange of decode size is a single trip over NVLink (no
 * fence, no flag behind the data); the bound on the wait is SKN_OPT_WAIT_LIMIT_MS either way.
 * No library collective is involved and the sequence is CUDA-graph capturable.
 *   one process per GPU : skn_comm_create on every rank, exchange skn_comm_handle() blobs
 *                         (skn_comm_handle_bytes() each) by any host channel, skn_comm_connect;
 *   one process, n GPUs : skn_comm_create per device, then skn_comm_connect_local(all of them).
 * capacity_floats bounds the element count of one skn_allreduce_dev call. */
typedef struct skn_comm skn_comm;
int32_t skn_comm_create(skn_ctx *ctx, int32_t rank, int32_t world, int64_t capacity_floats, skn_comm **out);
int32_t skn_comm_destroy(skn_comm *c);
int32_t skn_comm_handle_bytes(void);
int32_t skn_comm_handle(skn_comm *c, void *handle_out);
int32_t skn_comm_connect(skn_comm *c, const void *handles_in_rank_order);
int32_t skn_comm_connect_local(skn_comm *const *comms, int32_t n);
int32_t skn_comm_info(const skn_comm *c, int32_t *rank, int32_t *world, int64_t *capacity_floats);
/* out = resid + sum over ranks of partial: n floats (multiple of 4), 16-byte aligned device
 * pointers; resid may be NULL; out may alias resid or partial.  Collective: every rank calls it
 * the same number of times with the same n. */
int32_t skn_allreduce_dev(skn_comm *c, const float *partial_dev, const float *resid_dev, float *out_dev, int64_t n);

/* ---- Llama-style decoder ---------------------------------------------------------------------
 * RMSNorm -> Q/K/V -> rotary embedding (interleaved pairs) -> KV append -> grouped-query
 * attention -> output projection -> residual -> RMSNorm -> SwiGLU FFN -> residual; final norm,
 * LM head, greedy argmax.  The reference contains no decoder, attention, RoPE or RMSNorm
 * (model-zoo holds only an MNIST loader, model-zoo/src/commonMain/kotlin/sk/ai/net/io/data/mnist);
 * this is the loop of Module.forward calls (core/src/commonMain/kotlin/sk/ai/net/nn/Module.kt:6-16,
 * nn/topology/MLP.kt:13-19) a caller would write, kept in the library so that a step is a
 * fixed launch sequence.  Every forward processes all `max_batch` sequences with the same
 * number of new tokens.  Weight tensors are borrowed and must outlive the decoder. */
typedef struct skn_llama skn_llama;
int32_t skn_llama_create(skn_ctx *ctx, int32_t n_layers, int32_t d_model, int32_t n_heads, int32_t n_kv_heads,
                         int32_t head_dim, int32_t ffn_dim, int32_t vocab, float rope_theta, float rms_eps,
                         int32_t max_batch, int32_t max_tokens, int32_t max_ctx, skn_llama **out);
/* Tensor-parallel form: the geometry arguments stay those of the WHOLE model; rank r of the
 * exchange owns n_heads / world query heads and n_kv_heads / world KV heads (with their cache),
 * ffn_dim / world FFN columns and vocab / world LM-head rows, all contiguous ranges in rank
 * order.  skn_llama_set_layer then takes wq [n_heads*head_dim/world, d_model], wk, wv
 * [n_kv_heads*head_dim/world, d_model], wo [d_model, n_heads*head_dim/world] (a K-shard),
 * w_gate, w_up [ffn_dim/world, d_model], w_down [d_model, ffn_dim/world] (a K-shard);
 * skn_llama_set_head takes the full embedding table and output [vocab/world, d_model].  The
 * partial products of wo and w_down are summed through the exchange (two per layer), the
 * greedy token is chosen across the ranks' vocabulary slices, and logits_host of
 * skn_llama_forward receives this rank's slice [max_batch][vocab/world].  comm == NULL or a
 * world of one is skn_llama_create. */
int32_t skn_llama_create_tp(skn_ctx *ctx, int32_t n_layers, int32_t d_model, int32_t n_heads, int32_t n_kv_heads,
                            int32_t head_dim, int32_t ffn_dim, int32_t vocab, float rope_theta, float rms_eps,
                            int32_t max_batch, int32_t max_tokens, int32_t max_ctx, skn_comm *comm, skn_llama **out);
int32_t skn_llama_destroy(skn_llama *m);
int32_t skn_llama_set_layer(skn_llama *m, int32_t layer, const skn_tensor *wq, const skn_tensor *wk,
                            const skn_tensor *wv, const skn_tensor *wo, const skn_tensor *w_gate,
                            const skn_tensor *w_up, const skn_tensor *w_down, const float *attn_norm_host,
                            const float *ffn_norm_host);
int32_t skn_llama_set_head(skn_llama *m, const skn_tensor *tok_embd, const float *out_norm_host,
                           const skn_tensor *output);
int32_t skn_llama_reset(skn_llama *m);
/* tokens [max_batch][T] int32; NULL with T == 1 feeds back the ids of the previous forward.
 * next (greedy token per sequence) and logits ([max_batch][vocab], last position) may be NULL. */
int32_t skn_llama_forward(skn_llama *m, const int32_t *tokens_host, int32_t T, int32_t *next_host,
                          float *logits_host);
/* The device form only enqueues.  A single-token step (tokens_dev == NULL) is a fixed launch sequence and may
 * be captured into a CUDA graph once an uncaptured call has sized the scratch buffers; REPLAYING the graph
 * advances the caches on the device but not skn_llama_position, so the host must count its replays against
 * max_ctx itself.  A step that finds a cache full appends nothing, leaves the lengths at the capacity and
 * makes the next skn_sync return SKN_ERR_SHAPE; skn_llama_reset starts over. */
int32_t skn_llama_forward_dev(skn_llama *m, const int32_t *tokens_dev, int32_t T);
/* tokens cached per sequence so far as counted by the host-side calls (-1 on a bad handle) */
int32_t skn_llama_position(const skn_llama *m);

/* ---- GGUF container --------------------------------------------------------------------------
 * Memory-mapped GGUF v2 / v3 reader with 64-bit offsets; tensor data is handed out as pointers
 * into the mapping (no copy, no boxing) and quantized tensors upload straight from it.  Stands
 * where the reference parses the file, gguf/src/commonMain/kotlin/sk/ai/net/gguf/GGUFReader.kt:82-112
 * (fields: GGUFReader.kt:285-318, tensors: GGUFReader.kt:332-401), without its whole-file
 * ByteArray (:83), Int byte counts (:359) and F16 rejection (:363).  Host code; needs no GPU
 * except skn_gguf_upload. */
typedef struct skn_gguf skn_gguf;
int32_t skn_gguf_open(const char *path, skn_gguf **out);
int32_t skn_gguf_close(skn_gguf *g);
int32_t skn_gguf_counts(const skn_gguf *g, int32_t *version, int64_t *n_tensors, int64_t *n_kv, int64_t *alignment,
                        int64_t *data_offset);
/* Metadata entry i: key (NUL-terminated), GGUFValueType ids (Constants.kt, GGUFValueType; elem_type
 * is -1 unless the value is an array), a pointer to the value inside the mapping and a count
 * (string: byte length; array: elements, string elements being u64 length + bytes each). */
int32_t skn_gguf_kv(const skn_gguf *g, int64_t i, const char **key, int32_t *value_type, int32_t *elem_type,
                    const void **value, int64_t *count);
/* Tensor i: name, dims in file order (dims[0] contiguous; unused dims are 1), GGML type id, absolute
 * file offset, byte length and a pointer to the data inside the mapping: ReaderTensor,
 * GGUFReader.kt:35-44. */
int32_t skn_gguf_tensor(const skn_gguf *g, int64_t i, const char **name, int32_t *n_dims, int64_t *dims4,
                        int32_t *ggml_type, int64_t *data_offset, int64_t *n_bytes, const void **data);
int32_t skn_gguf_find_tensor(const skn_gguf *g, const char *name, int64_t *index);
/* Upload quantized tensor i as a [dims[1], dims[0]] weight (the step the reference's loader
 * skips, samples/mnist-mlp-cli/src/jvmMain/kotlin/sk/ai/net/samples/mnist/mlp/Main.kt:229-232). */
int32_t skn_gguf_upload(skn_ctx *ctx, const skn_gguf *g, int64_t i, skn_tensor **out);

#ifdef __cplusplus
}
#endif
#endif /* SKAINET_CUDA_H */
