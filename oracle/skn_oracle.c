/*
 * CPU oracle for the quantized-inference hot path.  TEST INFRASTRUCTURE ONLY:
 * this file is the checker the CUDA library is compared against and the timed
 * CPU baseline; nothing in the product library links, calls or falls back to it.
 *
 * Parity status: UNPINNED BY THE REFERENCE.  sk-ai-net/skainet v0.0.7 holds no
 * dequantizer, no quantized dot product and no golden vector for a quantized
 * block (gguf/src/commonMain/kotlin/sk/ai/net/gguf/Quants.kt:8 is a TODO).  Its
 * gguf module declares itself a transliteration of llama.cpp's gguf-py
 * (Constants.kt:3-6, Quants.kt:3-6); the block arithmetic below restates that
 * published format and is pinned against gguf-py 0.19.0 (`gguf.quants.dequantize`)
 * through the fixtures under tests/golden/.  What the reference does pin is
 * followed to the letter:
 *   - block geometry:  gguf/src/commonMain/kotlin/sk/ai/net/gguf/Constants.kt:55-90
 *   - row byte length and the "K multiple of block" rule:  Quants.kt:10-20
 *   - Linear = x * W^T + b with W stored [out, in] row-major:
 *       core/src/commonMain/kotlin/sk/ai/net/nn/Linear.kt:43-49
 *   - matmul loop order, fp64 accumulation:
 *       core/src/commonMain/kotlin/sk/ai/net/impl/DoublesTensor.kt:255-279
 *   - per-call transposed copy of the weight:  DoublesTensor.kt:362-387
 * Attention, SwiGLU, RMSNorm and RoPE have no counterpart in the reference (its
 * softmax(dim), DoublesTensor.kt:491-519, indexes the wrong axis); they are the
 * textbook definitions evaluated in fp64.
 *
 * Build:  make -C oracle      (gcc -O2 -fopenmp -ffp-contract=off)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* GGML type ids, Constants.kt:14-52 */
enum { T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8, T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12, T_Q5_K = 13,
       T_Q6_K = 14, T_IQ4_NL = 20, T_IQ4_XS = 23 };

/* (elements per block, bytes per block): Constants.kt:58-90 */
int skn_oracle_geometry(int type, int *elems, int *bytes) {
    switch (type) {
    case T_Q4_0: *elems = 32;  *bytes = 2 + 16; return 0;                     /* Constants.kt:61 */
    case T_Q8_0: *elems = 32;  *bytes = 2 + 32; return 0;                     /* Constants.kt:65 */
    case T_Q4_K: *elems = 256; *bytes = 2 + 2 + 256 / 2 + 12; return 0;       /* Constants.kt:69 */
    case T_Q6_K: *elems = 256; *bytes = 2 + 256 / 2 + 256 / 4 + 256 / 16; return 0; /* Constants.kt:71 */
    case T_Q4_1: *elems = 32;  *bytes = 2 + 2 + 16; return 0;                 /* Constants.kt:62 */
    case T_Q5_0: *elems = 32;  *bytes = 2 + 4 + 16; return 0;                 /* Constants.kt:63 */
    case T_Q5_1: *elems = 32;  *bytes = 2 + 2 + 4 + 16; return 0;             /* Constants.kt:64 */
    case T_Q5_K: *elems = 256; *bytes = 2 + 2 + 12 + 256 / 8 + 256 / 2; return 0; /* Constants.kt:70 */
    case T_Q2_K: *elems = 256; *bytes = 2 + 2 + 256 / 16 + 256 / 4; return 0; /* Constants.kt:67 */
    case T_Q3_K: *elems = 256; *bytes = 2 + 256 / 4 + 256 / 8 + 12; return 0; /* Constants.kt:68 */
    case T_IQ4_NL: *elems = 32; *bytes = 2 + 16; return 0;                    /* Constants.kt:77 */
    case T_IQ4_XS: *elems = 256; *bytes = 2 + 2 + 256 / 2 + 256 / 64; return 0; /* Constants.kt:80 */
    default: return -1;
    }
}

/* Quants.kt:10-20: bytes of one row of n_cols weights, -1 if n_cols is not a
 * multiple of the block size (the reference throws IllegalArgumentException). */
int64_t skn_oracle_row_bytes(int type, int64_t n_cols) {
    int e, b;
    if (skn_oracle_geometry(type, &e, &b)) return -1;
    if (n_cols % e) return -1;
    return n_cols / e * b;
}

/* IEEE binary16 -> binary32, exact (handles subnormals, inf, nan). */
static float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int shift = 0;
            while (!(man & 0x400u)) { man <<= 1; ++shift; }
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* One block -> fp32 weights.  All arithmetic in fp32, in the evaluation order of
 * gguf-py 0.19.0 so that results are bit-identical to it. */
static void dq_q4_0(const uint8_t *b, float *out) {
    const float d = half_to_float(rd16(b));
    const uint8_t *qs = b + 2;
    for (int e = 0; e < 16; ++e) {
        out[e]      = (float)((int)(qs[e] & 15) - 8) * d;
        out[e + 16] = (float)((int)(qs[e] >> 4) - 8) * d;
    }
}

static void dq_q8_0(const uint8_t *b, float *out) {
    const float d = half_to_float(rd16(b));
    const int8_t *q = (const int8_t *)(b + 2);
    for (int e = 0; e < 32; ++e) out[e] = (float)q[e] * d;
}

/* 6-bit (scale, min) pair of sub-block j from the 12 packed bytes. */
static void q4k_scale_min(const uint8_t *s, int j, int *sc, int *mn) {
    if (j < 4) {
        *sc = s[j] & 63;
        *mn = s[j + 4] & 63;
    } else {
        *sc = (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4);
        *mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

static void dq_q4_k(const uint8_t *b, float *out) {
    const float d = half_to_float(rd16(b));
    const float dmin = half_to_float(rd16(b + 2));
    const uint8_t *s = b + 4;
    const uint8_t *qs = b + 16;
    for (int j = 0; j < 8; ++j) {
        int sc, mn;
        q4k_scale_min(s, j, &sc, &mn);
        const float dl = d * (float)sc;
        const float ml = dmin * (float)mn;
        const uint8_t *q = qs + 32 * (j >> 1);
        for (int l = 0; l < 32; ++l) {
            const int nib = (j & 1) ? (q[l] >> 4) : (q[l] & 15);
            out[32 * j + l] = dl * (float)nib - ml;
        }
    }
}

static void dq_q6_k(const uint8_t *b, float *out) {
    const uint8_t *ql = b;
    const uint8_t *qh = b + 128;
    const int8_t *sc = (const int8_t *)(b + 192);
    const float d = half_to_float(rd16(b + 208));
    for (int h = 0; h < 2; ++h) {
        for (int g = 0; g < 4; ++g) {
            for (int l = 0; l < 32; ++l) {
                const uint8_t lo = ql[64 * h + l + 32 * (g & 1)];
                const int nib = (g < 2) ? (lo & 15) : (lo >> 4);
                const int hi2 = (qh[32 * h + l] >> (2 * g)) & 3;
                const int q = (nib | (hi2 << 4)) - 32;
                const float dl = d * (float)sc[8 * h + 2 * g + l / 16];
                out[128 * h + 32 * g + l] = dl * (float)q;
            }
        }
    }
}

/* q * d + m (two roundings, as gguf-py's `(d * qs) + m`). */
static void dq_q4_1(const uint8_t *b, float *out) {
    const float d = half_to_float(rd16(b)), m = half_to_float(rd16(b + 2));
    const uint8_t *qs = b + 4;
    for (int e = 0; e < 16; ++e) {
        out[e]      = d * (float)(qs[e] & 15) + m;
        out[e + 16] = d * (float)(qs[e] >> 4) + m;
    }
}

/* The fifth bit of weight i is bit i of the little-endian 32-bit word that follows the scale(s). */
static uint32_t rd32(const uint8_t *p) { return (uint32_t)rd16(p) | ((uint32_t)rd16(p + 2) << 16); }

static void dq_q5_0(const uint8_t *b, float *out) {
    const float d = half_to_float(rd16(b));
    const uint32_t qh = rd32(b + 2);
    const uint8_t *qs = b + 6;
    for (int e = 0; e < 16; ++e) {
        const int lo = (qs[e] & 15) | (int)(((qh >> e) & 1u) << 4);
        const int hi = (qs[e] >> 4) | (int)(((qh >> (e + 16)) & 1u) << 4);
        out[e]      = d * (float)(lo - 16);
        out[e + 16] = d * (float)(hi - 16);
    }
}

static void dq_q5_1(const uint8_t *b, float *out) {
    const float d = half_to_float(rd16(b)), m = half_to_float(rd16(b + 2));
    const uint32_t qh = rd32(b + 4);
    const uint8_t *qs = b + 8;
    for (int e = 0; e < 16; ++e) {
        const int lo = (qs[e] & 15) | (int)(((qh >> e) & 1u) << 4);
        const int hi = (qs[e] >> 4) | (int)(((qh >> (e + 16)) & 1u) << 4);
        out[e]      = d * (float)lo + m;
        out[e + 16] = d * (float)hi + m;
    }
}

/* Q4_K's layout with a fifth bit per weight: bit j of byte qh[l] belongs to weight l of sub-block j. */
static void dq_q5_k(const uint8_t *b, float *out) {
    const float d = half_to_float(rd16(b));
    const float dmin = half_to_float(rd16(b + 2));
    const uint8_t *s = b + 4;
    const uint8_t *qh = b + 16;
    const uint8_t *qs = b + 48;
    for (int j = 0; j < 8; ++j) {
        int sc, mn;
        q4k_scale_min(s, j, &sc, &mn);
        const float dl = d * (float)sc;
        const float ml = dmin * (float)mn;
        const uint8_t *q = qs + 32 * (j >> 1);
        for (int l = 0; l < 32; ++l) {
            const int nib = (j & 1) ? (q[l] >> 4) : (q[l] & 15);
            const int v = nib | (((qh[l] >> j) & 1) << 4);
            out[32 * j + l] = dl * (float)v - ml;
        }
    }
}

/* Q2_K: 16 scale bytes (low nibble scale, high nibble min), 64 bytes of 2-bit quants, d, dmin.
 * Weight 128h + 32s + l sits in byte qs[32h + l] at bit 2s; its scale byte is number (128h + 32s + l) / 16. */
static void dq_q2_k(const uint8_t *b, float *out) {
    const uint8_t *sc = b, *qs = b + 16;
    const float d = half_to_float(rd16(b + 80)), dmin = half_to_float(rd16(b + 82));
    for (int e = 0; e < 256; ++e) {
        const int h = e >> 7, s = (e >> 5) & 3, l = e & 31;
        const float dl = d * (float)(sc[e >> 4] & 15);
        const float ml = dmin * (float)(sc[e >> 4] >> 4);
        const int q = (qs[32 * h + l] >> (2 * s)) & 3;
        out[e] = dl * (float)q - ml;
    }
}

/* Q3_K: 32 bytes of high bits (bit g of hmask[l] belongs to weight 32g + l; a CLEAR bit subtracts 4),
 * 64 bytes of 2-bit quants laid out as in Q2_K, 12 bytes holding sixteen 6-bit scales (offset 32), d.
 * Scale i: low nibble from byte i & 7 (upper nibble when i >= 8), two high bits from byte 8 + (i & 3) at bit 2(i / 4). */
static void dq_q3_k(const uint8_t *b, float *out) {
    const uint8_t *hm = b, *qs = b + 32, *sp = b + 96;
    const float d = half_to_float(rd16(b + 108));
    for (int e = 0; e < 256; ++e) {
        const int i = e >> 4, h = e >> 7, s = (e >> 5) & 3, l = e & 31, g = e >> 5;
        const int lo = (i < 8) ? (sp[i] & 15) : (sp[i - 8] >> 4);
        const int hi = (sp[8 + (i & 3)] >> (2 * (i >> 2))) & 3;
        const float dl = d * (float)((lo | (hi << 4)) - 32);
        const int q = ((qs[32 * h + l] >> (2 * s)) & 3) - ((((hm[l] >> g) & 1) ^ 1) << 2);
        out[e] = dl * (float)q;
    }
}

/* The 16-entry non-linear codebook of the IQ4 formats (part of the published format). */
static const int8_t iq4_codebook[16] = { -127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113 };

/* IQ4_NL: Q4_0's layout; the nibble indexes the codebook. */
static void dq_iq4_nl(const uint8_t *b, float *out) {
    const float d = half_to_float(rd16(b));
    const uint8_t *qs = b + 2;
    for (int e = 0; e < 16; ++e) {
        out[e]      = d * (float)iq4_codebook[qs[e] & 15];
        out[e + 16] = d * (float)iq4_codebook[qs[e] >> 4];
    }
}

/* IQ4_XS: d, 16 bits of scale high parts (2 per sub-block), 4 bytes of scale low nibbles, 128 nibble bytes.
 * Sub-block i (32 weights): bytes qs[16i .. 16i+15], low nibbles first; scale = (low | high << 4) - 32. */
static void dq_iq4_xs(const uint8_t *b, float *out) {
    const float d = half_to_float(rd16(b));
    const uint32_t sh = rd16(b + 2);
    const uint8_t *sl = b + 4, *qs = b + 8;
    for (int i = 0; i < 8; ++i) {
        const int lo = (sl[i >> 1] >> (4 * (i & 1))) & 15;
        const int hi = (int)((sh >> (2 * i)) & 3u);
        const float dl = d * (float)((lo | (hi << 4)) - 32);
        for (int l = 0; l < 16; ++l) {
            out[32 * i + l]      = dl * (float)iq4_codebook[qs[16 * i + l] & 15];
            out[32 * i + l + 16] = dl * (float)iq4_codebook[qs[16 * i + l] >> 4];
        }
    }
}

static void dq_block(int type, const uint8_t *b, float *out) {
    switch (type) {
    case T_Q4_0: dq_q4_0(b, out); break;
    case T_Q8_0: dq_q8_0(b, out); break;
    case T_Q4_K: dq_q4_k(b, out); break;
    case T_Q4_1: dq_q4_1(b, out); break;
    case T_Q5_0: dq_q5_0(b, out); break;
    case T_Q5_1: dq_q5_1(b, out); break;
    case T_Q5_K: dq_q5_k(b, out); break;
    case T_Q2_K: dq_q2_k(b, out); break;
    case T_Q3_K: dq_q3_k(b, out); break;
    case T_IQ4_NL: dq_iq4_nl(b, out); break;
    case T_IQ4_XS: dq_iq4_xs(b, out); break;
    default:     dq_q6_k(b, out); break;
    }
}

/* n_blocks raw blocks -> n_blocks*elems fp32 values. */
int skn_oracle_dequant(int type, const uint8_t *blocks, int64_t n_blocks, float *out) {
    int e, bb;
    if (skn_oracle_geometry(type, &e, &bb)) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n_blocks; ++i) dq_block(type, blocks + i * bb, out + i * e);
    return 0;
}

/* Reference-faithful Linear.forward on quantized weights, single thread:
 *   W (fp64 copy of the dequantised [N,K] weight)  ->  Wt = W.t()  ([K,N], a fresh
 *   copy per call, DoublesTensor.kt:362-387)  ->  matmul in the reference's loop
 *   order (vec x mat: DoublesTensor.kt:255-264, k outer / n inner;
 *   mat x mat: DoublesTensor.kt:267-279, i-j-k)  ->  + bias (Linear.kt:48).
 * `dequantised` (fp64 [N,K]) is passed in so that the caller decides whether the
 * dequantisation is inside its timed region.  Y is fp64 [M,N]. */
int skn_oracle_linear_ref(const double *W, int64_t N, int64_t K, const float *X, int64_t M,
                          const float *bias, double *Y) {
    double *Wt = (double *)malloc(sizeof(double) * (size_t)N * (size_t)K);
    if (!Wt) return -2;
    for (int64_t n = 0; n < N; ++n)
        for (int64_t k = 0; k < K; ++k) Wt[k * N + n] = W[n * K + k];
    if (M == 1) {
        for (int64_t n = 0; n < N; ++n) Y[n] = 0.0;
        for (int64_t k = 0; k < K; ++k) {
            const double xv = (double)X[k];
            for (int64_t n = 0; n < N; ++n) Y[n] += xv * Wt[k * N + n];
        }
    } else {
        for (int64_t i = 0; i < M; ++i)
            for (int64_t n = 0; n < N; ++n) {
                double acc = 0.0;
                for (int64_t k = 0; k < K; ++k) acc += (double)X[i * K + k] * Wt[k * N + n];
                Y[i * N + n] = acc;
            }
    }
    if (bias)
        for (int64_t i = 0; i < M; ++i)
            for (int64_t n = 0; n < N; ++n) Y[i * N + n] += (double)bias[n];
    free(Wt);
    return 0;
}

/* Dequantise a [N,K] quantized weight (row pitch = row bytes) to fp64. */
int skn_oracle_dequant_f64(int type, const uint8_t *blocks, int64_t N, int64_t K, double *W) {
    int e, bb;
    if (skn_oracle_geometry(type, &e, &bb) || K % e) return -1;
    const int64_t nb = K / e;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        float tmp[256];
        for (int64_t j = 0; j < nb; ++j) {
            dq_block(type, blocks + (n * nb + j) * bb, tmp);
            for (int t = 0; t < e; ++t) W[n * K + j * e + t] = (double)tmp[t];
        }
    }
    return 0;
}

/* Same numbers as skn_oracle_linear_ref without the transposed copy: per output
 * row, dequantise block by block and accumulate x*w in fp64 in ascending k (the
 * order both reference loops use), rows spread over `threads` OpenMP threads.
 * Also returns, when `absdot` is non-NULL, sum_k |x_k * w_k| per output (the
 * denominator the fp32 tolerance is stated against). */
int skn_oracle_matmul(int type, const uint8_t *blocks, int64_t row_pitch, int64_t N, int64_t K,
                      const float *X, int64_t M, double *Y, double *absdot, int threads) {
    int e, bb;
    if (skn_oracle_geometry(type, &e, &bb) || K % e) return -1;
    const int64_t nb = K / e;
    if (row_pitch < nb * bb) return -1;
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        float tmp[256];
        double acc[64];
        double aacc[64];
        for (int64_t m0 = 0; m0 < M; m0 += 64) {
            const int64_t mc = (M - m0 < 64) ? (M - m0) : 64;
            for (int64_t i = 0; i < mc; ++i) { acc[i] = 0.0; aacc[i] = 0.0; }
            for (int64_t j = 0; j < nb; ++j) {
                dq_block(type, blocks + n * row_pitch + j * bb, tmp);
                for (int64_t i = 0; i < mc; ++i) {
                    const float *x = X + (m0 + i) * K + j * e;
                    double a = acc[i], aa = aacc[i];
                    for (int t = 0; t < e; ++t) {
                        const double p = (double)x[t] * (double)tmp[t];
                        a += p;
                        aa += fabs(p);
                    }
                    acc[i] = a;
                    aacc[i] = aa;
                }
            }
            for (int64_t i = 0; i < mc; ++i) {
                Y[(m0 + i) * N + n] = acc[i];
                if (absdot) absdot[(m0 + i) * N + n] = aacc[i];
            }
        }
    }
    return 0;
}

/* SwiGLU feed-forward, fp64:  H = silu(X Wg^T) * (X Wu^T)  ([M,F]),  Y = H Wd^T.
 * Wg, Wu: [F,K] blocks of type_gu;  Wd: [N,F] blocks of type_d.  H (fp64 [M,F]) is
 * returned too when non-NULL.  No counterpart in the reference (no SiLU; its
 * sigmoid(), DoublesTensor.kt:448-449, computes 1/exp(-x)). */
int skn_oracle_ffn_swiglu(int type_gu, const uint8_t *wg, const uint8_t *wu, int type_d,
                          const uint8_t *wd, int64_t F, int64_t K, int64_t N, const float *X,
                          int64_t M, double *Y, double *H_out, int threads) {
    double *G = (double *)malloc(sizeof(double) * (size_t)M * (size_t)F);
    double *U = (double *)malloc(sizeof(double) * (size_t)M * (size_t)F);
    if (!G || !U) { free(G); free(U); return -2; }
    const int64_t pg = skn_oracle_row_bytes(type_gu, K), pd = skn_oracle_row_bytes(type_d, F);
    if (pg < 0 || pd < 0) { free(G); free(U); return -1; }
    skn_oracle_matmul(type_gu, wg, pg, F, K, X, M, G, NULL, threads);
    skn_oracle_matmul(type_gu, wu, pg, F, K, X, M, U, NULL, threads);
    for (int64_t i = 0; i < M * F; ++i) {
        const double g = G[i];
        G[i] = g / (1.0 + exp(-g)) * U[i];
    }
    if (H_out) memcpy(H_out, G, sizeof(double) * (size_t)M * (size_t)F);
    /* second product with fp64 activations */
    int e, bb;
    skn_oracle_geometry(type_d, &e, &bb);
    const int64_t nb = F / e;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        float tmp[256];
        for (int64_t i = 0; i < M; ++i) Y[i * N + n] = 0.0;
        for (int64_t j = 0; j < nb; ++j) {
            dq_block(type_d, wd + n * pd + j * bb, tmp);
            for (int64_t i = 0; i < M; ++i) {
                double a = Y[i * N + n];
                const double *h = G + i * F + j * e;
                for (int t = 0; t < e; ++t) a += h[t] * (double)tmp[t];
                Y[i * N + n] = a;
            }
        }
    }
    free(G);
    free(U);
    return 0;
}

/* Decode attention with grouped queries over a head-major cache, fp64:
 *   K, V caches: [B, Hkv, capacity, D] fp32;  q: [B, Hq, D];  lens[b] tokens valid
 *   (positions 0..lens[b]-1 of the ring, the caller having already appended);
 *   out[b,h,:] = softmax(q . K^T * scale) . V with kv head = h / (Hq/Hkv).
 * `start[b]` is the ring position of the oldest valid token (0 when the ring has
 * not wrapped).  Textbook definition; the reference has no attention. */
int skn_oracle_attn_decode(const float *q, const float *kc, const float *vc, const int32_t *lens,
                           const int32_t *start, int64_t B, int64_t Hq, int64_t Hkv, int64_t D,
                           int64_t capacity, double scale, double *out) {
    if (Hq % Hkv) return -1;
    const int64_t grp = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < B; ++b) {
        for (int64_t h = 0; h < Hq; ++h) {
            const int64_t L = lens[b];
            const int64_t s0 = start ? start[b] : 0;
            const int64_t kvh = h / grp;
            const float *Kb = kc + ((b * Hkv + kvh) * capacity) * D;
            const float *Vb = vc + ((b * Hkv + kvh) * capacity) * D;
            const float *qv = q + (b * Hq + h) * D;
            double *o = out + (b * Hq + h) * D;
            for (int64_t d = 0; d < D; ++d) o[d] = 0.0;
            if (L <= 0) continue;
            double *sc = (double *)malloc(sizeof(double) * (size_t)L);
            double mx = -INFINITY;
            for (int64_t t = 0; t < L; ++t) {
                const float *kr = Kb + ((s0 + t) % capacity) * D;
                double a = 0.0;
                for (int64_t d = 0; d < D; ++d) a += (double)qv[d] * (double)kr[d];
                sc[t] = a * scale;
                if (sc[t] > mx) mx = sc[t];
            }
            double den = 0.0;
            for (int64_t t = 0; t < L; ++t) { sc[t] = exp(sc[t] - mx); den += sc[t]; }
            for (int64_t t = 0; t < L; ++t) {
                const float *vr = Vb + ((s0 + t) % capacity) * D;
                const double p = sc[t] / den;
                for (int64_t d = 0; d < D; ++d) o[d] += p * (double)vr[d];
            }
            free(sc);
        }
    }
    return 0;
}

/* RMSNorm, fp64:  y = x / sqrt(mean(x^2) + eps) * gain. */
int skn_oracle_rmsnorm(const float *x, const float *gain, int64_t M, int64_t D, double eps,
                       double *y) {
    for (int64_t i = 0; i < M; ++i) {
        double ss = 0.0;
        for (int64_t d = 0; d < D; ++d) ss += (double)x[i * D + d] * (double)x[i * D + d];
        const double r = 1.0 / sqrt(ss / (double)D + eps);
        for (int64_t d = 0; d < D; ++d) y[i * D + d] = (double)x[i * D + d] * r * (double)gain[d];
    }
    return 0;
}

/* Rotary embedding on [M, H, D] with positions pos[M]; pairs (2i, 2i+1) rotate by
 * pos * theta^(-2i/D)  (interleaved-pair convention). */
int skn_oracle_rope(const float *x, const int32_t *pos, int64_t M, int64_t H, int64_t D,
                    double theta, double *y) {
    for (int64_t i = 0; i < M; ++i)
        for (int64_t h = 0; h < H; ++h)
            for (int64_t p = 0; p < D / 2; ++p) {
                const double ang = (double)pos[i] * pow(theta, -2.0 * (double)p / (double)D);
                const double c = cos(ang), s = sin(ang);
                const double a = x[(i * H + h) * D + 2 * p], b = x[(i * H + h) * D + 2 * p + 1];
                y[(i * H + h) * D + 2 * p] = a * c - b * s;
                y[(i * H + h) * D + 2 * p + 1] = a * s + b * c;
            }
    return 0;
}

int skn_oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
