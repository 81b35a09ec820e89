// Llama-style decoder over the quantized kernels (configuration 5): RMSNorm -> Q/K/V ->
// RoPE -> KV append -> attention -> output projection -> residual -> RMSNorm -> SwiGLU FFN ->
// residual, then final norm, LM head and greedy argmax.  The reference has no decoder of
// any kind (model-zoo holds only an MNIST loader); this is the host-side loop a Kotlin
// caller would otherwise write over the individual entry points, kept in the library so
// that one forward is a fixed sequence of launches on the context's stream (capturable in a
// CUDA graph once the first call has sized the scratch buffers).
#include "skn_internal.cuh"

#include <new>
#include <vector>

#define SKN_MAGIC_LLAMA 0x736b6e6cu   // 'sknl'

struct skn_llama_layer {
    const skn_tensor *wq, *wk, *wv, *wo, *wg, *wu, *wd;
    float *attn_norm, *ffn_norm;      // device, [d_model]
    skn_kvcache *kv;
};

struct skn_llama {
    uint32_t magic;
    skn_ctx *ctx;
    int32_t n_layers, d_model, n_heads, n_kv_heads, head_dim, ffn_dim, vocab, max_batch, max_ctx;
    float rope_theta, rms_eps;
    std::vector<skn_llama_layer> layers;
    const skn_tensor *tok_embd, *output;
    float *out_norm;
    // activations for up to max_rows = max_batch * max_tokens rows
    int32_t max_rows;
    float *x, *h, *q, *k, *v, *att, *proj, *last, *logits, *ffn_g, *ffn_u;
    int32_t *ids_in, *ids_out;
    int32_t **len_ptrs;               // device array: the length vector of every layer's cache
    void *argmax_scratch;             // candidates and tickets of the two-level argmax
    int32_t host_len;                 // tokens cached so far (the same for every sequence)
    int32_t kv_f16;                   // SKN_KV_* element type of the layers' caches (SKN_OPT_KV_F16 / SKN_OPT_KV_DTYPE at creation)
    // tensor parallelism: this rank's share of heads, FFN columns and vocabulary rows
    skn_comm *comm;
    int32_t world, rank, heads_l, kv_heads_l, ffn_l, vocab_l;
    float *cand;                      // [world][max_batch][2] (value, global id) of the cross-rank argmax
    double *inv_freq;                 // rope_theta^(-2i / head_dim), i < head_dim / 2, for the fused rotary epilogue
};

// from skn_kv.cu
extern "C" int32_t skn_kv_append_many_dev(skn_kvcache *kv, const float *k, const float *v, int32_t T, int32_t host_len_upper);
extern "C" int32_t skn_attn_causal_dev(skn_kvcache *kv, const float *q, int32_t n_q_heads, int32_t T, float scale,
                                       float *out, void *scratch);
extern "C" int32_t skn_comm_info(const skn_comm *c, int32_t *rank, int32_t *world, int64_t *capacity_floats);
extern "C" int32_t skn_allreduce_dev(skn_comm *c, const float *partial, const float *resid, float *out, int64_t n);
extern "C" int32_t skn_kv_info(const skn_kvcache *kv, int32_t *, int32_t *, int32_t *, int32_t *capacity, void **k_dev,
                               void **v_dev, void **len_dev, void **start_dev);

static bool llama_ok(const skn_llama *m) { return m && m->magic == SKN_MAGIC_LLAMA && skn_ctx_ok(m->ctx); }

static cudaError_t dev_alloc(float **p, size_t n) { return cudaMalloc((void **)p, n * sizeof(float)); }

extern "C" {

int32_t skn_llama_destroy(skn_llama *m);

int32_t skn_llama_create(skn_ctx *ctx, int32_t n_layers, int32_t d_model, int32_t n_heads, int32_t n_kv_heads,
                         int32_t head_dim, int32_t ffn_dim, int32_t vocab, float rope_theta, float rms_eps,
                         int32_t max_batch, int32_t max_tokens, int32_t max_ctx, skn_llama **out) {
    return skn_llama_create_tp(ctx, n_layers, d_model, n_heads, n_kv_heads, head_dim, ffn_dim, vocab, rope_theta, rms_eps,
                               max_batch, max_tokens, max_ctx, nullptr, out);
}

int32_t skn_llama_create_tp(skn_ctx *ctx, int32_t n_layers, int32_t d_model, int32_t n_heads, int32_t n_kv_heads,
                            int32_t head_dim, int32_t ffn_dim, int32_t vocab, float rope_theta, float rms_eps,
                            int32_t max_batch, int32_t max_tokens, int32_t max_ctx, skn_comm *comm, skn_llama **out) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    if (!out) return skn_fail(ctx, SKN_ERR_ARG, "out is NULL");
    *out = nullptr;
    int32_t world = 1, rank = 0;
    int64_t comm_cap = 0;
    if (comm) {
        if (skn_comm_info(comm, &rank, &world, &comm_cap)) return skn_fail(ctx, SKN_ERR_BAD_HANDLE, "bad exchange handle");
        if (world == 1) comm = nullptr;
    }
    if (n_layers < 1 || d_model < 4 || n_heads < 1 || n_kv_heads < 1 || ffn_dim < 1 || vocab < 1 || max_batch < 1 ||
        max_tokens < 1 || max_ctx < max_tokens)
        return skn_fail(ctx, SKN_ERR_ARG, "invalid model geometry");
    if (d_model % 4 || n_heads % n_kv_heads || (head_dim != 64 && head_dim != 128))
        return skn_fail(ctx, SKN_ERR_SHAPE, "Shapes do not align.");
    if (n_heads % world || n_kv_heads % world || ffn_dim % world || vocab % world)
        return skn_fail(ctx, SKN_ERR_SHAPE, "heads, FFN width and vocabulary must divide by the %d ranks", world);
    if (comm && comm_cap < (int64_t)max_batch * max_tokens * d_model)
        return skn_fail(ctx, SKN_ERR_SHAPE, "exchange capacity %lld below max_batch * max_tokens * d_model = %lld floats",
                        (long long)comm_cap, (long long)max_batch * max_tokens * d_model);
    skn_llama *m = new (std::nothrow) skn_llama();
    if (!m) return skn_fail(ctx, SKN_ERR_OOM, "host allocation failed");
    m->magic = SKN_MAGIC_LLAMA;
    m->ctx = ctx;
    m->n_layers = n_layers; m->d_model = d_model; m->n_heads = n_heads; m->n_kv_heads = n_kv_heads;
    m->head_dim = head_dim; m->ffn_dim = ffn_dim; m->vocab = vocab; m->max_batch = max_batch; m->max_ctx = max_ctx;
    m->kv_f16 = ctx->kv_f16;
    m->rope_theta = rope_theta; m->rms_eps = rms_eps;
    m->comm = comm; m->world = world; m->rank = rank;
    m->heads_l = n_heads / world; m->kv_heads_l = n_kv_heads / world; m->ffn_l = ffn_dim / world; m->vocab_l = vocab / world;
    m->cand = nullptr;
    m->tok_embd = m->output = nullptr;
    m->out_norm = nullptr;
    m->max_rows = max_batch * max_tokens;
    m->host_len = 0;
    m->x = m->h = m->q = m->k = m->v = m->att = m->proj = m->last = m->logits = m->ffn_g = m->ffn_u = nullptr;
    m->ids_in = m->ids_out = nullptr;
    m->len_ptrs = nullptr;
    m->argmax_scratch = nullptr;
    m->layers.resize(n_layers);
    for (auto &l : m->layers) l = skn_llama_layer{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    cudaError_t e = cudaSetDevice(ctx->device);
    const size_t R = (size_t)m->max_rows, qd = (size_t)m->heads_l * head_dim, kd = (size_t)m->kv_heads_l * head_dim;
    if (e == cudaSuccess) e = dev_alloc(&m->x, R * d_model);
    if (e == cudaSuccess) e = dev_alloc(&m->h, R * d_model);
    if (e == cudaSuccess) e = dev_alloc(&m->q, R * qd);
    if (e == cudaSuccess) e = dev_alloc(&m->k, R * kd);
    if (e == cudaSuccess) e = dev_alloc(&m->v, R * kd);
    if (e == cudaSuccess) e = dev_alloc(&m->att, R * qd);
    if (e == cudaSuccess) e = dev_alloc(&m->proj, R * d_model);
    if (e == cudaSuccess) e = dev_alloc(&m->last, (size_t)max_batch * d_model);
    if (e == cudaSuccess) e = dev_alloc(&m->logits, (size_t)max_batch * m->vocab_l);
    if (e == cudaSuccess) e = dev_alloc(&m->cand, ((size_t)world * max_batch * 2 + 3) / 4 * 4);
    if (e == cudaSuccess) e = dev_alloc(&m->out_norm, d_model);
    // gate / up outputs of the decode-size path (rows below the prefill threshold only)
    const size_t small_rows = R < 64 ? R : 64;
    if (e == cudaSuccess) e = dev_alloc(&m->ffn_g, small_rows * m->ffn_l);
    if (e == cudaSuccess) e = dev_alloc(&m->ffn_u, small_rows * m->ffn_l);
    if (e == cudaSuccess) e = cudaMalloc((void **)&m->ids_in, sizeof(int32_t) * R);
    if (e == cudaSuccess) e = cudaMalloc((void **)&m->ids_out, sizeof(int32_t) * max_batch);
    if (e == cudaSuccess) e = cudaMalloc((void **)&m->len_ptrs, sizeof(int32_t *) * n_layers);
    if (e == cudaSuccess) e = cudaMalloc(&m->argmax_scratch, skn_argmax_scratch_bytes(max_batch));
    if (e == cudaSuccess) e = cudaMemset(m->argmax_scratch, 0, skn_argmax_scratch_bytes(max_batch));
    if (e == cudaSuccess) e = cudaMalloc((void **)&m->inv_freq, sizeof(double) * (size_t)(head_dim / 2 + 1));
    if (e == cudaSuccess) {
        std::vector<double> fr((size_t)head_dim / 2 + 1);
        for (int i = 0; i < head_dim / 2; ++i) fr[i] = pow((double)rope_theta, -2.0 * (double)i / (double)head_dim);
        e = cudaMemcpy(m->inv_freq, fr.data(), sizeof(double) * fr.size(), cudaMemcpyHostToDevice);
    }
    int32_t rc = SKN_OK;
    if (e != cudaSuccess) rc = skn_check_cuda(ctx, e, "decoder activation buffers");
    for (int l = 0; l < n_layers && rc == SKN_OK; ++l) {
        e = dev_alloc(&m->layers[l].attn_norm, d_model);
        if (e == cudaSuccess) e = dev_alloc(&m->layers[l].ffn_norm, d_model);
        if (e != cudaSuccess) { rc = skn_check_cuda(ctx, e, "decoder norm gains"); break; }
        rc = skn_kv_create_typed(ctx, max_batch, m->kv_heads_l, head_dim, max_ctx, ctx->kv_f16, &m->layers[l].kv);
    }
    if (rc == SKN_OK) {
        std::vector<int32_t *> lens(n_layers);
        for (int l = 0; l < n_layers; ++l) lens[l] = skn_kv_len_dev(m->layers[l].kv);
        e = cudaMemcpy(m->len_ptrs, lens.data(), sizeof(int32_t *) * n_layers, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) rc = skn_check_cuda(ctx, e, "decoder length table");
    }
    if (rc != SKN_OK) {
        skn_llama_destroy(m);
        return rc;
    }
    *out = m;
    return SKN_OK;
}

int32_t skn_llama_destroy(skn_llama *m) {
    if (!m || m->magic != SKN_MAGIC_LLAMA) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad decoder handle");
    if (skn_ctx_ok(m->ctx)) {
        cudaSetDevice(m->ctx->device);
        cudaStreamSynchronize(m->ctx->stream);
    }
    float *bufs[] = {m->x, m->h, m->q, m->k, m->v, m->att, m->proj, m->last, m->logits, m->out_norm, m->ffn_g, m->ffn_u, m->cand};
    for (float *b : bufs) if (b) cudaFree(b);
    if (m->ids_in) cudaFree(m->ids_in);
    if (m->ids_out) cudaFree(m->ids_out);
    if (m->len_ptrs) cudaFree(m->len_ptrs);
    if (m->argmax_scratch) cudaFree(m->argmax_scratch);
    if (m->inv_freq) cudaFree(m->inv_freq);
    for (auto &l : m->layers) {
        if (l.attn_norm) cudaFree(l.attn_norm);
        if (l.ffn_norm) cudaFree(l.ffn_norm);
        if (l.kv) skn_kv_destroy(l.kv);
    }
    m->magic = 0;
    delete m;
    return SKN_OK;
}

}  // extern "C"

static int32_t upload_gain(skn_llama *m, float *dst, const float *host) {
    skn_ctx *ctx = m->ctx;
    SKN_CUDA(ctx, cudaMemcpyAsync(dst, host, sizeof(float) * m->d_model, cudaMemcpyHostToDevice, ctx->stream));
    SKN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return SKN_OK;
}

static bool shape_is(const skn_tensor *t, const skn_ctx *ctx, int64_t rows, int64_t cols) {
    return skn_tensor_ok(t) && t->ctx == ctx && t->n_rows == rows && t->n_cols == cols;
}

extern "C" {

// Weights of one layer (borrowed: the tensors must outlive the decoder).  Norm gains are fp32
// host vectors of length d_model.
int32_t skn_llama_set_layer(skn_llama *m, int32_t layer, const skn_tensor *wq, const skn_tensor *wk,
                            const skn_tensor *wv, const skn_tensor *wo, const skn_tensor *w_gate,
                            const skn_tensor *w_up, const skn_tensor *w_down, const float *attn_norm_host,
                            const float *ffn_norm_host) {
    if (!llama_ok(m)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad decoder handle");
    skn_ctx *ctx = m->ctx;
    SKN_ENTER(ctx);
    if (layer < 0 || layer >= m->n_layers) return skn_fail(ctx, SKN_ERR_ARG, "layer index out of range");
    if (!attn_norm_host || !ffn_norm_host) return skn_fail(ctx, SKN_ERR_ARG, "NULL norm gain");
    const int64_t d = m->d_model, qd = (int64_t)m->heads_l * m->head_dim, kd = (int64_t)m->kv_heads_l * m->head_dim;
    if (!shape_is(wq, ctx, qd, d) || !shape_is(wk, ctx, kd, d) || !shape_is(wv, ctx, kd, d) || !shape_is(wo, ctx, d, qd) ||
        !shape_is(w_gate, ctx, m->ffn_l, d) || !shape_is(w_up, ctx, m->ffn_l, d) || !shape_is(w_down, ctx, d, m->ffn_l))
        return skn_fail(ctx, SKN_ERR_SHAPE, "Shapes do not align.");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    skn_llama_layer &l = m->layers[layer];
    l.wq = wq; l.wk = wk; l.wv = wv; l.wo = wo; l.wg = w_gate; l.wu = w_up; l.wd = w_down;
    int32_t rc = upload_gain(m, l.attn_norm, attn_norm_host);
    if (rc) return rc;
    return upload_gain(m, l.ffn_norm, ffn_norm_host);
}

// Token embedding table [vocab, d_model], final norm gain and LM head [vocab, d_model].
int32_t skn_llama_set_head(skn_llama *m, const skn_tensor *tok_embd, const float *out_norm_host,
                           const skn_tensor *output) {
    if (!llama_ok(m)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad decoder handle");
    skn_ctx *ctx = m->ctx;
    SKN_ENTER(ctx);
    if (!out_norm_host) return skn_fail(ctx, SKN_ERR_ARG, "NULL norm gain");
    if (!shape_is(tok_embd, ctx, m->vocab, m->d_model) || !shape_is(output, ctx, m->vocab_l, m->d_model))
        return skn_fail(ctx, SKN_ERR_SHAPE, "Shapes do not align.");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    m->tok_embd = tok_embd;
    m->output = output;
    return upload_gain(m, m->out_norm, out_norm_host);
}

// Forget all cached tokens.
int32_t skn_llama_reset(skn_llama *m) {
    if (!llama_ok(m)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad decoder handle");
    SKN_ENTER(m->ctx);
    for (auto &l : m->layers) {
        int32_t rc = skn_kv_reset(l.kv);
        if (rc) return rc;
    }
    m->host_len = 0;
    return SKN_OK;
}

// Enqueue one forward over T new tokens for each of the max_batch sequences.  tokens_dev
// ([batch][T] int32 on the device) may be NULL with T == 1: the ids produced by the previous
// forward are then fed back (greedy decoding without a host round trip).
int32_t skn_llama_forward_dev(skn_llama *m, const int32_t *tokens_dev, int32_t T) {
    if (!llama_ok(m)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad decoder handle");
    skn_ctx *ctx = m->ctx;
    SKN_ENTER(ctx);
    const int B = m->max_batch;
    if (T < 1 || (int64_t)B * T > m->max_rows) return skn_fail(ctx, SKN_ERR_SHAPE, "T outside [1, max_tokens]");
    if (!tokens_dev && T != 1) return skn_fail(ctx, SKN_ERR_ARG, "tokens may be NULL only for single-token steps");
    if (m->host_len + T > m->max_ctx) return skn_fail(ctx, SKN_ERR_SHAPE, "context of %d tokens exceeded", m->max_ctx);
    if (!m->tok_embd || !m->output) return skn_fail(ctx, SKN_ERR_ARG, "model head not set");
    for (auto &l : m->layers)
        if (!l.wq) return skn_fail(ctx, SKN_ERR_ARG, "a layer has no weights");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaStream_t st = ctx->stream;
    const int M = B * T, d = m->d_model, Hq = m->heads_l, Hkv = m->kv_heads_l, D = m->head_dim;
    const bool tp = m->comm != nullptr;
    const float scale = 1.0f / sqrtf((float)D);
    const int32_t *ids = tokens_dev ? tokens_dev : m->ids_out;
    // below the prefill threshold every product is an fp32 streaming matvec per activation row
    const bool small = M <= 64 && !(ctx->prefill_min_m > 0 && M >= ctx->prefill_min_m);
    // the step is a dependent chain: every launch keeps stream order whatever the context's
    // launch-order option says
    skn_order_guard guard(ctx);
    SKN_CUDA(ctx, skn_launch_embed(m->tok_embd, ids, M, m->x, st));
    int32_t rc;
    const int64_t qd = (int64_t)Hq * D, kd = (int64_t)Hkv * D, F = m->ffn_l;
    // fused form of one matvec launch; `fell_back` reports a shape the streaming kernel does not
    // cover.  Folding the norm / SwiGLU into the preparation of x saves a launch per layer but
    // adds a few microseconds to every row's launch: it pays for one or two rows, beyond that
    // one batched element-wise launch is cheaper.
    // (from three rows on, the many-row kernel's preparation pass applies the norm / SwiGLU product for all rows at
    // once, when it covers the layer's projections)
    bool fold = M <= 2;
    if (M >= 3 && small) {
        fold = true;
        for (auto &l : m->layers) {
            const skn_tensor *qkv[3] = {l.wq, l.wk, l.wv}, *gu[2] = {l.wg, l.wu};
            fold = fold && l.wk->type == l.wq->type && l.wv->type == l.wq->type && l.wq->pitch == l.wk->pitch &&
                   l.wq->pitch == l.wv->pitch && skn_rows_max_acts(ctx, 3, qkv) >= 4 && l.wu->type == l.wg->type &&
                   l.wu->pitch == l.wg->pitch && skn_rows_max_acts(ctx, 2, gu) >= 4;
        }
    }
    auto fused = [&](int n, const skn_tensor *const *ws, const float *x, float *const *ys, const float *const *add,
                     const float *gain, const float *silu_u, bool &fell_back) -> cudaError_t {
        if (!fold) { fell_back = true; return cudaSuccess; }
        const cudaError_t e = skn_launch_matvec_fused(ctx, n, ws, x, ys, add, gain, m->rms_eps, silu_u, st);
        fell_back = (e == cudaErrorNotSupported);
        return fell_back ? cudaSuccess : e;
    };
    // residual stream: m->x, or alternately m->x / m->h while exchanges are fused into the matvecs
    float *xcur = m->x, *xalt = m->h;
    bool pending = false;
    skn_comm_view xview = {};
    // (automatic = off: since the exchange launch became a single trip over NVLink, started early by programmatic
    // dependent launch, it measures faster than the fused form at every rank count)
    const bool want_fused = ctx->fused_exchange > 0;
    // (the fused exchange rides on the single-launch tensor-core matvec: one or two rows)
    bool fusedx = tp && fold && M <= 2 && want_fused && skn_comm_get_view(m->comm, &xview) && xview.capacity >= (int64_t)M * d;
    if (fusedx) {
        // only when every layer takes the multi-row tensor-core path (a pending exchange is consumed
        // by the next layer's first projection)
        for (auto &l : m->layers)
            fusedx = fusedx && small && skn_mma_max_acts(ctx, l.wq->type, 2 * kd + qd, d) > 0 && l.wk->type == l.wq->type &&
                     l.wv->type == l.wq->type && l.wq->pitch == l.wk->pitch && l.wq->pitch == l.wv->pitch &&
                     skn_mma_max_acts(ctx, l.wo->type, d, qd) > 0 && skn_mma_max_acts(ctx, l.wg->type, 2 * F, d) > 0 &&
                     l.wu->type == l.wg->type && l.wu->pitch == l.wg->pitch && skn_mma_max_acts(ctx, l.wd->type, d, F) > 0;
    }
    for (auto &l : m->layers) {
        // Decode-size batches whose projections the tensor-core matvec covers: every product takes
        // all M activation rows (a few rows per launch, the weights of the later launches come
        // from L2), Q/K/V grouped, gate / up / SwiGLU in one launch, residuals in the epilogues.
        const bool rows_path =
            small && skn_mma_max_acts(ctx, l.wq->type, 2 * kd + qd, d) > 0 && l.wk->type == l.wq->type && l.wv->type == l.wq->type &&
            l.wq->pitch == l.wk->pitch && l.wq->pitch == l.wv->pitch && skn_mma_max_acts(ctx, l.wo->type, d, qd) > 0 &&
            skn_mma_max_acts(ctx, l.wg->type, 2 * F, d) > 0 && l.wu->type == l.wg->type && l.wu->pitch == l.wg->pitch &&
            skn_mma_max_acts(ctx, l.wd->type, d, F) > 0;
        if (rows_path) {
            // Tensor parallelism with one or two rows: the K-sharded projections push their partial
            // products into every rank's inbox from their epilogue, and the next projection adds
            // them to the residual stream while it prepares x (no exchange launch); the summed
            // stream alternates between two buffers (xcur is read, xalt written by CTA 0).
            skn_mv_exchange xpush = {}, xred = {};
            if (fusedx) {
                xpush.view = xview; xpush.push = true;
                xred.view = xview; xred.reduce = true;
            }
            const bool last_layer = (&l == &m->layers.back());
            const float *src = xcur;
            if (!fold) {
                SKN_CUDA(ctx, skn_launch_rmsnorm(xcur, l.attn_norm, m->h, M, d, m->rms_eps, st));
                src = m->h;
            }
            // single-token steps: the Q/K/V launch rotates q and k in its epilogue and writes k and v
            // straight into the cache (row a of the batch is sequence a, its position the cache length)
            skn_mv_rope rope = {};
            // larger batches: the separate kernel spreads the sincos work better; the epilogue writes fp32 cache slots only
            const bool rope_fused = (T == 1 && M <= 4 && !m->kv_f16);
            if (rope_fused) {
                void *kdev = nullptr, *vdev = nullptr, *ldev = nullptr, *sdev = nullptr;
                int32_t cap = 0;
                if ((rc = skn_kv_info(l.kv, nullptr, nullptr, nullptr, &cap, &kdev, &vdev, &ldev, &sdev))) return rc;
                if (m->host_len + 1 > cap) return skn_fail(ctx, SKN_ERR_SHAPE, "context of %d tokens exceeded", cap);
                rope.head_dim = D; rope.n_kv_heads = Hkv; rope.capacity = cap; rope.seq0 = 0;
                rope.len_dev = (const int32_t *)ldev; rope.start_dev = (const int32_t *)sdev;
                rope.k_cache = (float *)kdev; rope.v_cache = (float *)vdev; rope.theta = m->rope_theta;
                rope.inv_freq = m->inv_freq;
            }
            {
                const skn_tensor *ws[3] = {l.wq, l.wk, l.wv};
                float *ys[3] = {m->q, m->k, m->v};
                xred.writeback = xalt;
                SKN_CUDA(ctx, skn_launch_matvec_acts(ctx, 3, ws, src, M, ys, nullptr, false, fold ? l.attn_norm : nullptr, m->rms_eps,
                                                     nullptr, false, st, pending ? &xred : nullptr, rope_fused ? &rope : nullptr));
                if (pending) { float *tmp = xcur; xcur = xalt; xalt = tmp; pending = false; }
            }
            if (!rope_fused && (rc = skn_kv_rope_append_pending(l.kv, m->q, m->k, m->v, Hq, T, m->rope_theta, m->host_len))) return rc;
            if ((rc = skn_attn_causal_pending(l.kv, m->q, Hq, T, scale, m->att))) return rc;
            {
                const skn_tensor *ws[1] = {l.wo};
                float *ys[1] = {tp ? m->proj : xcur};
                const float *as[1] = {tp ? nullptr : xcur};
                SKN_CUDA(ctx, skn_launch_matvec_acts(ctx, 1, ws, m->att, M, ys, as, true, nullptr, 0.f, nullptr, false, st,
                                                     fusedx ? &xpush : nullptr));
                if (fusedx) pending = true;
                else if (tp && (rc = skn_allreduce_dev(m->comm, m->proj, xcur, xcur, (int64_t)M * d))) return rc;
            }
            src = xcur;
            if (!fold) {
                SKN_CUDA(ctx, skn_launch_rmsnorm(xcur, l.ffn_norm, m->h, M, d, m->rms_eps, st));
                src = m->h;
            }
            {
                const skn_tensor *ws[2] = {l.wg, l.wu};
                float *ys[2] = {m->ffn_g, m->ffn_g};
                xred.writeback = xalt;
                SKN_CUDA(ctx, skn_launch_matvec_acts(ctx, 2, ws, src, M, ys, nullptr, false, fold ? l.ffn_norm : nullptr, m->rms_eps,
                                                     nullptr, true, st, pending ? &xred : nullptr));
                if (pending) { float *tmp = xcur; xcur = xalt; xalt = tmp; pending = false; }
            }
            {
                // the last layer's partial sums meet in the exchange kernel: the LM head that follows
                // need not be a tensor-core matvec
                const bool fuse_down = fusedx && !last_layer;
                const skn_tensor *ws[1] = {l.wd};
                float *ys[1] = {tp ? m->proj : xcur};
                const float *as[1] = {tp ? nullptr : xcur};
                SKN_CUDA(ctx, skn_launch_matvec_acts(ctx, 1, ws, m->ffn_g, M, ys, as, true, nullptr, 0.f, nullptr, false, st,
                                                     fuse_down ? &xpush : nullptr));
                if (fuse_down) pending = true;
                else if (tp && (rc = skn_allreduce_dev(m->comm, m->proj, xcur, xcur, (int64_t)M * d))) return rc;
            }
            continue;
        }
        if (small) {
            // decode-size batches, per activation row: RMSNorm folded into the preparation of x
            // for Q/K/V (one launch) ...
            bool fb = false;
            for (int r = 0; r < M && !fb; ++r) {
                const skn_tensor *ws[3] = {l.wq, l.wk, l.wv};
                float *ys[3] = {m->q + r * qd, m->k + r * kd, m->v + r * kd};
                SKN_CUDA(ctx, fused(3, ws, m->x + (int64_t)r * d, ys, nullptr, l.attn_norm, nullptr, fb));
            }
            if (fb) {
                SKN_CUDA(ctx, skn_launch_rmsnorm(m->x, l.attn_norm, m->h, M, d, m->rms_eps, st));
                for (int r = 0; r < M; ++r) {
                    const skn_tensor *ws[3] = {l.wq, l.wk, l.wv};
                    float *ys[3] = {m->q + r * qd, m->k + r * kd, m->v + r * kd};
                    SKN_CUDA(ctx, skn_launch_matvec_group(ctx, 3, ws, m->h + (int64_t)r * d, ys, nullptr, st));
                }
            }
        } else {
            SKN_CUDA(ctx, skn_launch_rmsnorm(m->x, l.attn_norm, m->h, M, d, m->rms_eps, st));
            if ((rc = skn_matmul_dev(ctx, l.wq, m->h, M, d, nullptr, m->q))) return rc;
            if ((rc = skn_matmul_dev(ctx, l.wk, m->h, M, d, nullptr, m->k))) return rc;
            if ((rc = skn_matmul_dev(ctx, l.wv, m->h, M, d, nullptr, m->v))) return rc;
        }
        // rotary embedding of q in place and of k on its way into the cache, v alongside; the
        // lengths advance once for all layers at the end of the step
        if ((rc = skn_kv_rope_append_pending(l.kv, m->q, m->k, m->v, Hq, T, m->rope_theta, m->host_len))) return rc;
        if ((rc = skn_attn_causal_pending(l.kv, m->q, Hq, T, scale, m->att))) return rc;
        if (small) {
            // ... output projection with the residual added in its epilogue (x += att . Wo^T); with
            // K-sharded weights the partial products meet in the exchange, which adds the residual ...
            for (int r = 0; r < M; ++r) {
                float *xr = m->x + (int64_t)r * d;
                SKN_CUDA(ctx, skn_launch_matvec(ctx, l.wo, m->att + r * qd, 1, tp ? nullptr : xr, tp ? m->proj + (int64_t)r * d : xr, st));
            }
            if (tp && (rc = skn_allreduce_dev(m->comm, m->proj, m->x, m->x, (int64_t)M * d))) return rc;
            // ... gate, up and silu(g) * u in one launch (second RMSNorm folded in for one or two
            // rows), then the down projection with the residual in its epilogue ...
            float *gbuf = m->ffn_g, *ubuf = m->ffn_u;
            bool fused_ffn = true;
            if (!fold) SKN_CUDA(ctx, skn_launch_rmsnorm(m->x, l.ffn_norm, m->h, M, d, m->rms_eps, st));
            for (int r = 0; r < M && fused_ffn; ++r) {
                const float *src = fold ? m->x + (int64_t)r * d : m->h + (int64_t)r * d;
                const cudaError_t e = skn_launch_gate_up_swiglu(ctx, l.wg, l.wu, src, gbuf + r * F, fold ? l.ffn_norm : nullptr,
                                                                m->rms_eps, st);
                if (e == cudaErrorNotSupported) fused_ffn = false;       // only ever on the first row
                else SKN_CUDA(ctx, e);
            }
            if (fused_ffn) {
                for (int r = 0; r < M; ++r) {
                    float *xr = m->x + (int64_t)r * d;
                    SKN_CUDA(ctx, skn_launch_matvec(ctx, l.wd, gbuf + r * F, 1, tp ? nullptr : xr, tp ? m->proj + (int64_t)r * d : xr, st));
                }
            } else {
                // ... or, for block types the fused kernel does not cover: gate and up grouped, the
                // SwiGLU product formed while the down projection prepares x
                bool fb = false;
                for (int r = 0; r < M && !fb; ++r) {
                    const skn_tensor *ws[2] = {l.wg, l.wu};
                    float *ys[2] = {gbuf + r * F, ubuf + r * F};
                    SKN_CUDA(ctx, fused(2, ws, m->x + (int64_t)r * d, ys, nullptr, l.ffn_norm, nullptr, fb));
                }
                if (fb) {
                    if (fold) SKN_CUDA(ctx, skn_launch_rmsnorm(m->x, l.ffn_norm, m->h, M, d, m->rms_eps, st));
                    for (int r = 0; r < M; ++r) {
                        const skn_tensor *ws[2] = {l.wg, l.wu};
                        float *ys[2] = {gbuf + r * F, ubuf + r * F};
                        SKN_CUDA(ctx, skn_launch_matvec_group(ctx, 2, ws, m->h + (int64_t)r * d, ys, nullptr, st));
                    }
                }
                fb = false;
                for (int r = 0; r < M && !fb; ++r) {
                    const skn_tensor *ws[1] = {l.wd};
                    float *ys[1] = {tp ? m->proj + (int64_t)r * d : m->x + (int64_t)r * d};
                    const float *adds[1] = {tp ? nullptr : m->x + (int64_t)r * d};
                    SKN_CUDA(ctx, fused(1, ws, gbuf + r * F, ys, adds, nullptr, ubuf + r * F, fb));
                }
                if (fb) {
                    SKN_CUDA(ctx, skn_launch_silu_mul(gbuf, ubuf, gbuf, (int64_t)M * F, ctx->sm_count, st));
                    for (int r = 0; r < M; ++r) {
                        float *xr = m->x + (int64_t)r * d;
                        SKN_CUDA(ctx, skn_launch_matvec(ctx, l.wd, gbuf + r * F, 1, tp ? nullptr : xr, tp ? m->proj + (int64_t)r * d : xr, st));
                    }
                }
            }
            if (tp && (rc = skn_allreduce_dev(m->comm, m->proj, m->x, m->x, (int64_t)M * d))) return rc;
        } else {
            if ((rc = skn_matmul_dev(ctx, l.wo, m->att, M, qd, nullptr, m->proj))) return rc;
            if (tp) { if ((rc = skn_allreduce_dev(m->comm, m->proj, m->x, m->x, (int64_t)M * d))) return rc; }
            else SKN_CUDA(ctx, skn_launch_add(m->x, m->proj, m->x, (int64_t)M * d, ctx->sm_count, st));
            SKN_CUDA(ctx, skn_launch_rmsnorm(m->x, l.ffn_norm, m->h, M, d, m->rms_eps, st));
            if ((rc = skn_ffn_swiglu_dev(ctx, l.wg, l.wu, l.wd, m->h, M, m->proj))) return rc;
            if (tp) { if ((rc = skn_allreduce_dev(m->comm, m->proj, m->x, m->x, (int64_t)M * d))) return rc; }
            else SKN_CUDA(ctx, skn_launch_add(m->x, m->proj, m->x, (int64_t)M * d, ctx->sm_count, st));
        }
    }
    SKN_CUDA(ctx, skn_kv_advance_all(m->len_ptrs, m->n_layers, B, T, m->max_ctx, ctx->d_status, st));
    m->host_len += T;
    // final norm + LM head on the last position of every sequence
    bool fb = !(B <= 64 && !(ctx->prefill_min_m > 0 && B >= ctx->prefill_min_m));
    for (int b = 0; b < B && !fb; ++b) {
        const skn_tensor *ws[1] = {m->output};
        float *ys[1] = {m->logits + (int64_t)b * m->vocab_l};
        SKN_CUDA(ctx, fused(1, ws, xcur + ((int64_t)b * T + (T - 1)) * d, ys, nullptr, m->out_norm, nullptr, fb));
    }
    if (fb) {
        SKN_CUDA(ctx, skn_launch_last_rows(xcur, m->last, B, T, d, st));
        SKN_CUDA(ctx, skn_launch_rmsnorm(m->last, m->out_norm, m->h, B, d, m->rms_eps, st));
        if ((rc = skn_matmul_dev(ctx, m->output, m->h, B, d, nullptr, m->logits))) return rc;
    }
    SKN_CUDA(ctx, skn_launch_argmax(m->logits, B, m->vocab_l, m->ids_out, m->argmax_scratch, st));
    if (tp) {
        // every rank offers the best token of its vocabulary slice; zero-filled slots make the
        // exchange's sum a concatenation, and every rank then picks the same winner
        const int64_t nc = ((int64_t)m->world * B * 2 + 3) / 4 * 4;
        SKN_CUDA(ctx, skn_launch_argmax_offer(m->logits, m->ids_out, B, m->vocab_l, m->rank, m->world, m->cand, st));
        if ((rc = skn_allreduce_dev(m->comm, m->cand, nullptr, m->cand, nc))) return rc;
        SKN_CUDA(ctx, skn_launch_argmax_pick(m->cand, B, m->world, m->ids_out, st));
    }
    return SKN_OK;
}

// Host-pointer form: tokens_host [batch][T] (NULL with T == 1 feeds back the previous ids);
// returns the greedy next token of every sequence and, optionally, the logits of the last
// position ([batch][vocab]).
int32_t skn_llama_forward(skn_llama *m, const int32_t *tokens_host, int32_t T, int32_t *next_host, float *logits_host) {
    if (!llama_ok(m)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad decoder handle");
    skn_ctx *ctx = m->ctx;
    SKN_ENTER(ctx);
    const int B = m->max_batch;
    if (T < 1 || (int64_t)B * T > m->max_rows) return skn_fail(ctx, SKN_ERR_SHAPE, "T outside [1, max_tokens]");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    if (tokens_host)
        SKN_CUDA(ctx, cudaMemcpyAsync(m->ids_in, tokens_host, sizeof(int32_t) * B * T, cudaMemcpyHostToDevice, ctx->stream));
    int32_t rc = skn_llama_forward_dev(m, tokens_host ? m->ids_in : nullptr, T);
    if (rc) return rc;
    if (next_host)
        SKN_CUDA(ctx, cudaMemcpyAsync(next_host, m->ids_out, sizeof(int32_t) * B, cudaMemcpyDeviceToHost, ctx->stream));
    if (logits_host)
        SKN_CUDA(ctx, cudaMemcpyAsync(logits_host, m->logits, sizeof(float) * B * m->vocab_l, cudaMemcpyDeviceToHost, ctx->stream));
    return skn_sync(ctx);
}

// number of tokens cached per sequence
int32_t skn_llama_position(const skn_llama *m) { return llama_ok(m) ? m->host_len : -1; }

}  // extern "C"
