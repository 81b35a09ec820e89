// C1/C2: exchange between the GPUs of one box without a library collective.
//
// Every rank owns one "inbox" allocation that its peers map (CUDA IPC between processes, peer
// access inside one process):
//
//   [ flags : uint32 flag[NBUF][MAX_WORLD] ]  4 KiB
//   [ data  : float  inbox[NBUF][world][capacity] ]
//
// Reduce number q (q = 0, 1, 2, ... counted on the device, so that a captured CUDA graph can be
// replayed) uses buffer q % NBUF.  One kernel per rank does the whole exchange:
//   1. push    every CTA copies its share of the local partial into inbox[q % NBUF][rank] of
//              every peer with plain peer stores, then a system-wide fence and a ticket; the CTA
//              that draws the last ticket releases flag[q % NBUF][rank] = q + 1 on every peer;
//   2. wait    one thread per peer polls the local flags with acquire loads; the wait is bounded
//              (about two seconds, then SKN_ERR_TIMEOUT lands in the context's status word and
//              later exchanges do not wait at all);
//   3. sum     out = resid + partial_0 + partial_1 + ... in rank order, the same on every rank,
//              so the replicated residual stream stays bit-identical across ranks.
// The kernel runs with one CTA per SM at most, so all its CTAs are resident while any of them
// waits.  Two buffers suffice: a peer can push reduce q + 2 only after it has finished reduce
// q + 1, which needs this rank's push of q + 1, which this rank issues after its own reduce q
// has completed.
//
// Decode-size vectors (up to COMM_LL_MAX floats) take a second, lower-latency form of the same exchange
// (skn_allreduce_ll_kernel): every float travels as an 8-byte word {value, q + 1} written with one store, and the
// receiver polls the words themselves.  No fence, no flag store behind the data: the exchange costs one trip
// over NVLink instead of three (data, the acknowledgement the system fence waits for, the flag).  Its inbox
// follows the first one in the same allocation: uint2 ll[NBUF][world][COMM_LL_MAX].
//
// No multicast, no bulk-async loads from peer memory: only ordinary stores to peers and loads
// from local memory.
#include "skn_internal.cuh"
#include "skn_ptx.cuh"

#include <new>
#include <stdlib.h>

#define SKN_MAGIC_COMM 0x736b6e6du   // 'sknm'

constexpr int COMM_NBUF = SKN_COMM_NBUF;
constexpr int COMM_MAX_WORLD = SKN_COMM_MAX_WORLD;
constexpr size_t COMM_FLAG_BYTES = SKN_COMM_FLAG_BYTES;
constexpr int64_t COMM_LL_MAX = 65536;            // floats per (buffer, source rank) of the low-latency inbox

struct skn_comm {
    uint32_t magic;
    skn_ctx *ctx;
    int32_t rank, world;
    int64_t capacity;                  // floats per (buffer, source rank)
    uint8_t *local;                    // this rank's inbox allocation
    uint8_t *peer[COMM_MAX_WORLD];     // peers' inboxes as mapped here (peer[rank] == local)
    bool ipc_mapped[COMM_MAX_WORLD];
    uint32_t *d_state;                 // [0] reduce counter q, [1] push tickets, [2] finish tickets
    bool connected;
};

struct comm_peers {
    uint8_t *base[COMM_MAX_WORLD];
};

static bool comm_ok(const skn_comm *c) { return c && c->magic == SKN_MAGIC_COMM && skn_ctx_ok(c->ctx); }

bool skn_comm_get_view(const skn_comm *c, skn_comm_view *v) {
    if (!comm_ok(c) || !c->connected || !v) return false;
    v->rank = c->rank;
    v->world = c->world;
    v->capacity = c->capacity;
    for (int i = 0; i < COMM_MAX_WORLD; ++i) v->base[i] = c->peer[i];
    v->state = c->d_state;
    return true;
}

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ float *comm_inbox(uint8_t *base, int buf, int world, int src, int64_t cap) {
    return reinterpret_cast<float *>(base + COMM_FLAG_BYTES) + ((int64_t)buf * world + src) * cap;
}
__device__ __forceinline__ uint32_t *comm_flag(uint8_t *base, int buf, int src) {
    return reinterpret_cast<uint32_t *>(base) + buf * COMM_MAX_WORLD + src;
}

// The low-latency form for n <= COMM_LL_MAX: out[i] = resid[i] + sum over ranks of partial_r[i], ranks in order.
// ll_off: byte offset of the low-latency inbox inside every rank's allocation.
__global__ void __launch_bounds__(1024)
skn_allreduce_ll_kernel(comm_peers peers, size_t ll_off, int rank, int world, uint32_t *__restrict__ state,
                        int32_t *__restrict__ status, const float *__restrict__ partial, const float *__restrict__ resid,
                        float *__restrict__ out, int64_t n, int early) {
    // programmatic dependent launch on both sides (steps of a few rows): this kernel is resident when the producer of
    // `partial` finishes, and the projection behind it starts at once and fetches its weights while the exchange
    // is under way.  Measured on two GPUs: batch 1 +6 %, batch 16 -3 % (hence not for the larger vectors).
    if (early) skn_pdl_launch_dependents();
    skn_pdl_wait();
    const uint32_t q = *reinterpret_cast<volatile uint32_t *>(state);
    const uint32_t tag = q + 1u;
    const int buf = (int)(q % COMM_NBUF);
    const int64_t n4 = n / 4;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (int64_t)gridDim.x * blockDim.x;
    auto inbox = [&](int owner, int src) {
        return reinterpret_cast<uint2 *>(peers.base[owner] + ll_off) + ((int64_t)buf * world + src) * COMM_LL_MAX;
    };
    // 1. push: four tagged words per thread and peer
    for (int64_t i = tid; i < n4; i += nthr) {
        const float4 v = reinterpret_cast<const float4 *>(partial)[i];
        const uint32_t w[4] = {__float_as_uint(v.x), __float_as_uint(v.y), __float_as_uint(v.z), __float_as_uint(v.w)};
        for (int p = 1; p < world; ++p) {
            uint2 *to = inbox((rank + p) % world, rank) + 4 * i;      // start with a different peer on every rank
#pragma unroll
            for (int j = 0; j < 4; ++j)
                asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(to + j), "r"(w[j]), "r"(tag) : "memory");
        }
    }
    // 2. + 3. poll the words of every peer (bounded) and sum in rank order
    const bool waiting = *reinterpret_cast<volatile int32_t *>(status) == 0;
    const uint64_t t0 = skn_globaltimer_ns(), limit = skn_wait_limit_ns(status);
    bool gave_up = !waiting;
    for (int64_t i = tid; i < n4; i += nthr) {
        float4 acc = resid ? reinterpret_cast<const float4 *>(resid)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        for (int src = 0; src < world; ++src) {
            float4 v;
            if (src == rank) {
                v = reinterpret_cast<const float4 *>(partial)[i];
            } else {
                const uint2 *from = inbox(rank, src) + 4 * i;
                uint2 a, b, c, d;
                uint32_t spins = 0;
                for (;;) {
                    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(a.x), "=r"(a.y) : "l"(from) : "memory");
                    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(b.x), "=r"(b.y) : "l"(from + 1) : "memory");
                    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(c.x), "=r"(c.y) : "l"(from + 2) : "memory");
                    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(d.x), "=r"(d.y) : "l"(from + 3) : "memory");
                    if ((a.y == tag && b.y == tag && c.y == tag && d.y == tag) || gave_up) break;
                    if ((++spins & 255u) == 0 && skn_globaltimer_ns() - t0 > limit) {
                        atomicExch(status, SKN_ERR_TIMEOUT);
                        gave_up = true;
                    }
                }
                v = make_float4(__uint_as_float(a.x), __uint_as_float(b.x), __uint_as_float(c.x), __uint_as_float(d.x));
            }
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        reinterpret_cast<float4 *>(out)[i] = acc;
    }
    __syncthreads();
    // the CTA that finishes last moves the counter on
    if (threadIdx.x == 0) {
        if (gridDim.x == 1) {
            *reinterpret_cast<volatile uint32_t *>(state) = q + 1;
        } else {
            __threadfence();
            if (atomicAdd(&state[2], 1u) == gridDim.x - 1) {
                state[2] = 0;
                *reinterpret_cast<volatile uint32_t *>(state) = q + 1;
            }
        }
    }
}

// out[i] = resid[i] + sum over ranks of partial_r[i]   (resid may be NULL, out may alias resid
// or partial); n is a multiple of 4.
__global__ void __launch_bounds__(1024)
skn_allreduce_push_kernel(comm_peers peers, int rank, int world, int64_t cap, uint32_t *__restrict__ state,
                          int32_t *__restrict__ status, const float *__restrict__ partial,
                          const float *__restrict__ resid, float *__restrict__ out, int64_t n) {
    __shared__ uint32_t s_q;
    __shared__ bool s_last;
    if (threadIdx.x == 0) s_q = *reinterpret_cast<volatile uint32_t *>(state);
    __syncthreads();
    const uint32_t q = s_q;
    const int buf = (int)(q % COMM_NBUF);
    const int64_t n4 = n / 4;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (int64_t)gridDim.x * blockDim.x;

    // 1. push
    for (int p = 1; p < world; ++p) {
        const int dst = (rank + p) % world;           // start with a different peer on every rank
        float4 *to = reinterpret_cast<float4 *>(comm_inbox(peers.base[dst], buf, world, rank, cap));
        for (int64_t i = tid; i < n4; i += nthr) to[i] = reinterpret_cast<const float4 *>(partial)[i];
    }
    // the CTA barrier orders every thread's peer stores before thread 0's system-wide fence
    // (fences are cumulative), so one fence per CTA is enough
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        s_last = gridDim.x == 1 || atomicAdd(&state[1], 1u) == gridDim.x - 1;
        if (s_last) {
            if (gridDim.x > 1) {
                state[1] = 0;
                __threadfence_system();
            }
            for (int p = 1; p < world; ++p) st_release_sys(comm_flag(peers.base[(rank + p) % world], buf, rank), q + 1);
        }
    }

    // 2. wait for every peer's push of reduce q
    if (threadIdx.x < world && threadIdx.x != rank) {
        const uint32_t *flag = comm_flag(peers.base[rank], buf, threadIdx.x);
        if (*reinterpret_cast<volatile int32_t *>(status) == 0) {
            const uint64_t t0 = skn_globaltimer_ns(), limit = skn_wait_limit_ns(status);
            uint32_t spins = 0;
            while (ld_acquire_sys(flag) != q + 1) {
                if ((++spins & 1023u) == 0 && skn_globaltimer_ns() - t0 > limit) {
                    atomicExch(status, SKN_ERR_TIMEOUT);
                    break;
                }
            }
        }
    }
    __syncthreads();

    // 3. sum in rank order
    for (int64_t i = tid; i < n4; i += nthr) {
        float4 acc = resid ? reinterpret_cast<const float4 *>(resid)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        for (int src = 0; src < world; ++src) {
            const float4 v = (src == rank)
                                 ? reinterpret_cast<const float4 *>(partial)[i]
                                 : __ldcg(reinterpret_cast<const float4 *>(comm_inbox(peers.base[rank], buf, world, src, cap)) + i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        reinterpret_cast<float4 *>(out)[i] = acc;
    }
    __syncthreads();
    // the CTA that finishes last moves the counter on
    if (threadIdx.x == 0) {
        if (gridDim.x == 1) {
            *reinterpret_cast<volatile uint32_t *>(state) = q + 1;
        } else {
            __threadfence();
            if (atomicAdd(&state[2], 1u) == gridDim.x - 1) {
                state[2] = 0;
                *reinterpret_cast<volatile uint32_t *>(state) = q + 1;
            }
        }
    }
}

extern "C" {

int32_t skn_comm_destroy(skn_comm *c);

int32_t skn_comm_create(skn_ctx *ctx, int32_t rank, int32_t world, int64_t capacity_floats, skn_comm **out) {
    if (!skn_ctx_ok(ctx)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad context handle");
    if (!out) return skn_fail(ctx, SKN_ERR_ARG, "out is NULL");
    *out = nullptr;
    if (world < 1 || world > COMM_MAX_WORLD || rank < 0 || rank >= world)
        return skn_fail(ctx, SKN_ERR_ARG, "rank %d outside a world of %d (at most %d ranks)", rank, world, COMM_MAX_WORLD);
    if (capacity_floats < 4) return skn_fail(ctx, SKN_ERR_ARG, "capacity must be at least 4 floats");
    skn_comm *c = new (std::nothrow) skn_comm();
    if (!c) return skn_fail(ctx, SKN_ERR_OOM, "host allocation failed");
    c->magic = SKN_MAGIC_COMM;
    c->ctx = ctx;
    c->rank = rank;
    c->world = world;
    c->capacity = (capacity_floats + 63) / 64 * 64;
    c->local = nullptr;
    c->d_state = nullptr;
    c->connected = (world == 1);
    for (int i = 0; i < COMM_MAX_WORLD; ++i) { c->peer[i] = nullptr; c->ipc_mapped[i] = false; }
    // flags | inbox | low-latency inbox (zero-filled: tag 0 never matches q + 1)
    const size_t ll_off = COMM_FLAG_BYTES + (size_t)COMM_NBUF * world * c->capacity * sizeof(float);
    const size_t ll_bytes = (size_t)COMM_NBUF * world * COMM_LL_MAX * sizeof(uint2);
    const size_t bytes = ll_off + ll_bytes;
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e == cudaSuccess) e = cudaMalloc((void **)&c->local, bytes);
    if (e == cudaSuccess) e = cudaMemset(c->local, 0, COMM_FLAG_BYTES);
    if (e == cudaSuccess) e = cudaMemset(c->local + ll_off, 0, ll_bytes);
    if (e == cudaSuccess) e = cudaMalloc((void **)&c->d_state, 64);
    if (e == cudaSuccess) e = cudaMemset(c->d_state, 0, 64);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        const int32_t rc = skn_check_cuda(ctx, e, "exchange buffers");
        skn_comm_destroy(c);
        return rc;
    }
    c->peer[rank] = c->local;
    *out = c;
    return SKN_OK;
}

int32_t skn_comm_destroy(skn_comm *c) {
    if (!c || c->magic != SKN_MAGIC_COMM) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad exchange handle");
    if (skn_ctx_ok(c->ctx)) {
        cudaSetDevice(c->ctx->device);
        cudaStreamSynchronize(c->ctx->stream);
    }
    for (int i = 0; i < COMM_MAX_WORLD; ++i)
        if (c->ipc_mapped[i] && c->peer[i]) cudaIpcCloseMemHandle(c->peer[i]);
    if (c->local) cudaFree(c->local);
    if (c->d_state) cudaFree(c->d_state);
    c->magic = 0;
    delete c;
    return SKN_OK;
}

int32_t skn_comm_handle_bytes(void) { return (int32_t)sizeof(cudaIpcMemHandle_t); }

// Writes the inter-process handle of this rank's inbox (skn_comm_handle_bytes() bytes).
int32_t skn_comm_handle(skn_comm *c, void *handle_out) {
    if (!comm_ok(c)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad exchange handle");
    if (!handle_out) return skn_fail(c->ctx, SKN_ERR_ARG, "handle_out is NULL");
    SKN_CUDA(c->ctx, cudaSetDevice(c->ctx->device));
    cudaIpcMemHandle_t h;
    SKN_CUDA(c->ctx, cudaIpcGetMemHandle(&h, c->local));
    memcpy(handle_out, &h, sizeof(h));
    return SKN_OK;
}

// One process per GPU: `handles` holds the world's handles in rank order (this rank's own
// entry is ignored).  Every rank must have created its exchange with the same capacity.
int32_t skn_comm_connect(skn_comm *c, const void *handles) {
    if (!comm_ok(c)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad exchange handle");
    skn_ctx *ctx = c->ctx;
    if (!handles) return skn_fail(ctx, SKN_ERR_ARG, "handles is NULL");
    if (c->connected) return skn_fail(ctx, SKN_ERR_ARG, "exchange already connected");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t *)handles + (size_t)r * sizeof(h), sizeof(h));
        void *p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return skn_fail(ctx, SKN_ERR_COMM, "cannot map the inbox of rank %d: %s", r, cudaGetErrorString(e));
        }
        c->peer[r] = (uint8_t *)p;
        c->ipc_mapped[r] = true;
    }
    c->connected = true;
    return SKN_OK;
}

// One process driving several GPUs: connects the n = world exchanges of that process (rank
// order) through peer access.
int32_t skn_comm_connect_local(skn_comm *const *comms, int32_t n) {
    if (!comms || n < 1 || n > COMM_MAX_WORLD) return skn_fail(nullptr, SKN_ERR_ARG, "1 to %d exchanges", COMM_MAX_WORLD);
    for (int i = 0; i < n; ++i)
        if (!comm_ok(comms[i]) || comms[i]->world != n || comms[i]->rank != i || comms[i]->capacity != comms[0]->capacity)
            return skn_fail(nullptr, SKN_ERR_ARG, "exchanges must be given in rank order with equal world and capacity");
    for (int i = 0; i < n; ++i) {
        skn_ctx *ctx = comms[i]->ctx;
        SKN_CUDA(ctx, cudaSetDevice(ctx->device));
        for (int j = 0; j < n; ++j) {
            if (j == i) continue;
            if (getenv("SKN_FAKE_NO_PEER_ACCESS"))
                return skn_fail(ctx, SKN_ERR_COMM, "device %d cannot access device %d", ctx->device, comms[j]->ctx->device);
            if (comms[j]->ctx->device != ctx->device) {
                int can = 0;
                SKN_CUDA(ctx, cudaDeviceCanAccessPeer(&can, ctx->device, comms[j]->ctx->device));
                if (!can) return skn_fail(ctx, SKN_ERR_COMM, "device %d cannot access device %d", ctx->device, comms[j]->ctx->device);
                const cudaError_t e = cudaDeviceEnablePeerAccess(comms[j]->ctx->device, 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return skn_check_cuda(ctx, e, "peer access");
                cudaGetLastError();
            }
            comms[i]->peer[j] = comms[j]->local;
        }
        comms[i]->connected = true;
    }
    return SKN_OK;
}

int32_t skn_comm_info(const skn_comm *c, int32_t *rank, int32_t *world, int64_t *capacity_floats) {
    if (!comm_ok(c)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad exchange handle");
    if (rank) *rank = c->rank;
    if (world) *world = c->world;
    if (capacity_floats) *capacity_floats = c->capacity;
    return SKN_OK;
}

// out = resid + sum over ranks of partial (all device pointers, n floats, n % 4 == 0, 16-byte
// aligned; resid may be NULL; out may alias resid or partial).  Every rank must call this the
// same number of times with the same n.  Enqueued on the context's stream.
int32_t skn_allreduce_dev(skn_comm *c, const float *partial_dev, const float *resid_dev, float *out_dev, int64_t n) {
    if (!comm_ok(c)) return skn_fail(nullptr, SKN_ERR_BAD_HANDLE, "bad exchange handle");
    skn_ctx *ctx = c->ctx;
    SKN_ENTER(ctx);
    if (!c->connected) return skn_fail(ctx, SKN_ERR_COMM, "exchange not connected");
    if (n < 0 || n % 4) return skn_fail(ctx, SKN_ERR_SHAPE, "element count must be a non-negative multiple of 4");
    if (n > c->capacity) return skn_fail(ctx, SKN_ERR_SHAPE, "%lld floats exceed the exchange capacity %lld", (long long)n, (long long)c->capacity);
    if (n == 0) return SKN_OK;
    if (!partial_dev || !out_dev) return skn_fail(ctx, SKN_ERR_ARG, "NULL argument");
    if ((((uintptr_t)partial_dev) | ((uintptr_t)resid_dev) | ((uintptr_t)out_dev)) & 15)
        return skn_fail(ctx, SKN_ERR_ALIGN, "buffers must be 16-byte aligned");
    SKN_CUDA(ctx, cudaSetDevice(ctx->device));
    comm_peers peers;
    for (int i = 0; i < COMM_MAX_WORLD; ++i) peers.base[i] = c->peer[i];
    if (n <= COMM_LL_MAX) {
        // decode sizes: the low-latency form (tagged 8-byte words); a CTA per 1024 quads, all resident
        const size_t ll_off = COMM_FLAG_BYTES + (size_t)COMM_NBUF * c->world * c->capacity * sizeof(float);
        const int64_t quads = n / 4;
        const int threads_ll = quads >= 1024 ? 1024 : (int)((quads + 31) / 32 * 32);
        const unsigned blocks_ll = (unsigned)((quads + 1023) / 1024);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(blocks_ll);
        cfg.blockDim = dim3((unsigned)threads_ll);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        const int early = n <= 16384 ? 1 : 0;
        cfg.attrs = attr;
        cfg.numAttrs = early;
        SKN_CUDA(ctx, cudaLaunchKernelEx(&cfg, skn_allreduce_ll_kernel, peers, ll_off, (int)c->rank, (int)c->world, c->d_state,
                                         ctx->d_status, partial_dev, resid_dev, out_dev, n, early));
        return SKN_OK;
    }
    // a decode-size vector: one CTA (no tickets, one fence); otherwise at most one CTA per SM, so
    // that every CTA is resident while any of them waits
    int threads = 256;
    int64_t blocks = (n / 4 + 255) / 256;
    if (n <= 16384) {
        blocks = 1;
        threads = n / 4 >= 1024 ? 1024 : (int)((n / 4 + 31) / 32 * 32);
    }
    if (blocks > ctx->sm_count) blocks = ctx->sm_count;
    skn_allreduce_push_kernel<<<(unsigned)blocks, threads, 0, ctx->stream>>>(peers, c->rank, c->world, c->capacity, c->d_state,
                                                                       ctx->d_status, partial_dev, resid_dev, out_dev, n);
    SKN_CUDA(ctx, cudaGetLastError());
    return SKN_OK;
}

}  // extern "C"
