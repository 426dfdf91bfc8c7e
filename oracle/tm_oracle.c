/*
 * tm_oracle.c -- CPU restatement of TuckCore's scalar Q8_0 arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is
 * compared against; the product never links, imports or calls it.  Only the
 * test-suite, the smoke check and the bench's CPU-baseline leg may load it.
 *
 * Every function names the reference source it follows (path inside the
 * withhull/tuckmill tree).  Compile with -ffp-contract=off and without
 * -ffast-math: the reference is plain Rust f32 arithmetic, which never fuses
 * a multiply and an add, so neither may this file.
 *
 * Parity pin: the known-answer vectors of the reference's own unit tests for
 * f16 decode/encode, Q8_0 dequantisation, the one-block GEMV, rmsnorm, rope
 * and argmax are replayed against this file by the CPU test-suite.  The
 * reference has no Q8_0 model fixture and no CPU executor for the Gemma-3
 * graph, so model-level parity of this file is "parity unpinned": it follows
 * the reference's graph and block semantics but no runnable golden output
 * exists for it.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define TMO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ f16 -- */

/* crates/tuckcore/src/tensor.rs:12-28 -- binary16 decode; subnormals are
 * m * 2^-24, normals (1 + m/1024) * 2^(e-15); both exact in f32. */
TMO_API float tmo_f16_to_f32(uint16_t bits) {
    const uint32_t sign = (bits >> 15) & 1u;
    const uint32_t exp = (bits >> 10) & 0x1fu;
    const uint32_t mant = bits & 0x3ffu;
    float value;
    if (exp == 0 && mant == 0) {
        value = 0.0f;
    } else if (exp == 0) {
        value = (float)mant * ldexpf(1.0f, -24);
    } else if (exp == 31 && mant == 0) {
        value = INFINITY;
    } else if (exp == 31) {
        value = NAN;
    } else {
        value = (1.0f + (float)mant / 1024.0f) * ldexpf(1.0f, (int)exp - 15);
    }
    return sign ? -value : value;
}

/* crates/tuckcore/src/tensor.rs:145-178 -- binary16 encode, round to nearest
 * even, overflow saturates to infinity, below 2^-25 flushes to signed zero.
 * (NaN inputs take the overflow branch, as in the reference.) */
TMO_API uint16_t tmo_f32_to_f16_bits(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    int exp = (int)((bits >> 23) & 0xffu) - 127 + 15;
    const uint32_t mant = bits & 0x7fffffu;
    if (exp >= 0x1f) {
        return sign | 0x7c00u;
    }
    if (exp <= 0) {
        if (exp < -10) {
            return sign;
        }
        const uint32_t m = mant | 0x800000u;
        const uint32_t shift = (uint32_t)(14 - exp);
        uint32_t half = (m >> shift) & 0x3ffu;
        const uint32_t rem = m & ((1u << shift) - 1u);
        const uint32_t halfway = 1u << (shift - 1u);
        const int round_up = rem > halfway || (rem == halfway && (half & 1u) == 1u);
        half += (uint32_t)round_up;
        return sign | (uint16_t)half;
    }
    const uint32_t rounded = mant + 0x0fffu + ((mant >> 13) & 1u);
    if (rounded & 0x800000u) {
        exp += 1;
        if (exp >= 0x1f) {
            return sign | 0x7c00u;
        }
        return sign | (uint16_t)(exp << 10);
    }
    return sign | (uint16_t)(exp << 10) | (uint16_t)(rounded >> 13);
}

/* crates/tuckcore/src/forward.rs:186-191 -- KvPrecision::F16::round. */
static inline float round_f16(float v) { return tmo_f16_to_f32(tmo_f32_to_f16_bits(v)); }

static inline uint16_t read_u16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* ---------------------------------------------------------------- Q8_0 -- */

/* crates/tuckcore/src/tensor.rs:94-104 -- [f16 d][i8 q x 32], w = d * q. */
TMO_API void tmo_dequant_q8_0(const uint8_t *bytes, size_t blocks, float *out) {
    for (size_t b = 0; b < blocks; ++b) {
        const uint8_t *blk = bytes + b * 34;
        const float d = tmo_f16_to_f32(read_u16(blk));
        for (int q = 0; q < 32; ++q) {
            out[b * 32 + q] = d * (float)(int8_t)blk[2 + q];
        }
    }
}

/* crates/tuckcore/src/kernels.rs:186-204 -- scalar::dot_q8_0_x_f32: per block
 * a sequential sum from 0.0 of (q as f32) * x, then acc += d * block_sum, the
 * blocks in order. */
TMO_API float tmo_dot_q8_0_x_f32(const uint8_t *row, size_t blocks, const float *x) {
    float acc = 0.0f;
    for (size_t b = 0; b < blocks; ++b) {
        const uint8_t *blk = row + b * 34;
        const float d = tmo_f16_to_f32(read_u16(blk));
        const float *xb = x + b * 32;
        float block_sum = 0.0f;
        for (int q = 0; q < 32; ++q) {
            const float w = (float)(int8_t)blk[2 + q];
            block_sum += w * xb[q];
        }
        acc += d * block_sum;
    }
    return acc;
}

/* crates/tuckcore/src/kernels.rs:139-149 -- validate_q8_0_row: the row is a
 * positive multiple of 34 bytes and x holds blocks*32 values.  Returns the
 * block count, or -1 (InvalidArtifact) / -2 (Internal: activation width). */
TMO_API long tmo_validate_q8_0_row(size_t row_len, size_t x_len) {
    if (row_len == 0 || row_len % 34 != 0) {
        return -1;
    }
    const size_t blocks = row_len / 34;
    if (x_len != blocks * 32) {
        return -2;
    }
    return (long)blocks;
}

/* ------------------------------------------------------- row-loop matvec -- */

#define TMO_TB 8 /* tokens advanced together; per-token order is unchanged */

typedef struct {
    const uint8_t *w;
    size_t rows, cols, batch;
    const float *x; /* [batch, cols] */
    float *y;       /* [batch, rows] */
    size_t r0, r1;
} mv_job;

/* One weight row against TMO_TB tokens.  Each token's accumulator runs the
 * exact sequence of tmo_dot_q8_0_x_f32; the tokens are merely independent
 * lanes, so every result is bit-identical to the one-token call. */
__attribute__((target_clones("avx2", "default")))
static void row_times_tokens(const uint8_t *row, size_t blocks, const float *xt /* [cols][TB] */,
                             float *acc /* [TB] */) {
    float a[TMO_TB];
    for (int t = 0; t < TMO_TB; ++t) a[t] = 0.0f;
    for (size_t b = 0; b < blocks; ++b) {
        const uint8_t *blk = row + b * 34;
        const float d = tmo_f16_to_f32(read_u16(blk));
        float s[TMO_TB];
        for (int t = 0; t < TMO_TB; ++t) s[t] = 0.0f;
        const float *xb = xt + b * 32 * TMO_TB;
        for (int q = 0; q < 32; ++q) {
            const float w = (float)(int8_t)blk[2 + q];
            for (int t = 0; t < TMO_TB; ++t) {
                s[t] += w * xb[q * TMO_TB + t];
            }
        }
        for (int t = 0; t < TMO_TB; ++t) a[t] += d * s[t];
    }
    for (int t = 0; t < TMO_TB; ++t) acc[t] = a[t];
}

static void *mv_worker(void *arg) {
    mv_job *j = (mv_job *)arg;
    const size_t blocks = j->cols / 32;
    const size_t row_bytes = blocks * 34;
    size_t t0 = 0;
    float *xt = NULL;
    if (j->batch >= TMO_TB) {
        xt = (float *)malloc(j->cols * TMO_TB * sizeof(float));
    }
    for (; xt && t0 + TMO_TB <= j->batch; t0 += TMO_TB) {
        for (size_t c = 0; c < j->cols; ++c)
            for (int t = 0; t < TMO_TB; ++t) xt[c * TMO_TB + t] = j->x[(t0 + t) * j->cols + c];
        for (size_t r = j->r0; r < j->r1; ++r) {
            float acc[TMO_TB];
            row_times_tokens(j->w + r * row_bytes, blocks, xt, acc);
            for (int t = 0; t < TMO_TB; ++t) j->y[(t0 + t) * j->rows + r] = acc[t];
        }
    }
    free(xt);
    /* crates/tuckcore/src/forward.rs:719-727 -- the row loop, one token. */
    for (; t0 < j->batch; ++t0) {
        for (size_t r = j->r0; r < j->r1; ++r) {
            j->y[t0 * j->rows + r] =
                tmo_dot_q8_0_x_f32(j->w + r * row_bytes, blocks, j->x + t0 * j->cols);
        }
    }
    return NULL;
}

/* crates/tuckcore/src/forward.rs:562-737 -- Forward::matvec over a resident
 * Q8_0 matrix: y[b][r] = dot(row_r, x[b]).  `threads` row-partitions the loop
 * (the reference runs it on one thread; more threads change no result). */
TMO_API int tmo_matmul_q8_0(const uint8_t *w, size_t rows, size_t cols, const float *x,
                            size_t batch, float *y, int threads) {
    if (rows == 0 || cols == 0 || cols % 32 != 0 || batch == 0) {
        return -1;
    }
    if (threads < 1) threads = 1;
    if ((size_t)threads > rows) threads = (int)rows;
    if (threads > 256) threads = 256;
    mv_job jobs[256];
    pthread_t tids[256];
    const size_t per = (rows + (size_t)threads - 1) / (size_t)threads;
    int n = 0;
    for (int t = 0; t < threads; ++t) {
        const size_t r0 = (size_t)t * per;
        if (r0 >= rows) break;
        const size_t r1 = r0 + per < rows ? r0 + per : rows;
        jobs[n] = (mv_job){w, rows, cols, batch, x, y, r0, r1};
        ++n;
    }
    if (n == 1) {
        mv_worker(&jobs[0]);
        return 0;
    }
    for (int t = 0; t < n; ++t) pthread_create(&tids[t], NULL, mv_worker, &jobs[t]);
    for (int t = 0; t < n; ++t) pthread_join(tids[t], NULL);
    return 0;
}

/* crates/tuckcore/src/kernels.rs:223-232 -- scalar::dot_f16_x_f32: one sequential
 * sum from 0.0 of f16_to_f32(w_i) * x_i. */
TMO_API float tmo_dot_f16_x_f32(const uint8_t *row, size_t cols, const float *x) {
    float acc = 0.0f;
    for (size_t i = 0; i < cols; ++i) {
        const float w = tmo_f16_to_f32(read_u16(row + 2 * i));
        acc += w * x[i];
    }
    return acc;
}

typedef struct {
    const uint8_t *w;
    size_t rows, cols, batch;
    const float *x;
    float *y;
    size_t r0, r1;
} mvh_job;

static void *mvh_worker(void *arg) {
    mvh_job *j = (mvh_job *)arg;
    for (size_t t = 0; t < j->batch; ++t)
        for (size_t r = j->r0; r < j->r1; ++r)
            j->y[t * j->rows + r] = tmo_dot_f16_x_f32(j->w + r * j->cols * 2, j->cols, j->x + t * j->cols);
    return NULL;
}

/* The row loop of crates/tuckcore/src/forward.rs:562-737 over an F16 matrix
 * (rows * cols binary16 values, row-major). */
TMO_API int tmo_matmul_f16(const uint8_t *w, size_t rows, size_t cols, const float *x, size_t batch,
                           float *y, int threads) {
    if (rows == 0 || cols == 0 || batch == 0) return -1;
    if (threads < 1) threads = 1;
    if ((size_t)threads > rows) threads = (int)rows;
    if (threads > 256) threads = 256;
    mvh_job jobs[256];
    pthread_t tids[256];
    const size_t per = (rows + (size_t)threads - 1) / (size_t)threads;
    int n = 0;
    for (int t = 0; t < threads; ++t) {
        const size_t r0 = (size_t)t * per;
        if (r0 >= rows) break;
        const size_t r1 = r0 + per < rows ? r0 + per : rows;
        jobs[n] = (mvh_job){w, rows, cols, batch, x, y, r0, r1};
        ++n;
    }
    if (n == 1) {
        mvh_worker(&jobs[0]);
        return 0;
    }
    for (int t = 0; t < n; ++t) pthread_create(&tids[t], NULL, mvh_worker, &jobs[t]);
    for (int t = 0; t < n; ++t) pthread_join(tids[t], NULL);
    return 0;
}

/* ------------------------------------------------------------ small ops -- */

/* crates/tuckcore/src/forward.rs:917-926 -- rmsnorm_in_place. */
TMO_API void tmo_rmsnorm(const float *x, const float *w, float eps, size_t n, float *y) {
    float ss = 0.0f;
    for (size_t i = 0; i < n; ++i) ss += x[i] * x[i];
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (size_t i = 0; i < n; ++i) y[i] = x[i] * inv * w[i];
}

/* crates/tuckcore/src/qwen35_ops.rs:265-272 (and forward.rs:272-279):
 * inv_freq[i] = (1 / base^(2i/rope_dims) in f64) as f32; base is an f32. */
TMO_API void tmo_rope_inv_freq(size_t rope_dims, float base, float *out) {
    for (size_t i = 0; i < rope_dims / 2; ++i) {
        const double exponent = 2.0 * (double)i / (double)rope_dims;
        out[i] = (float)(1.0 / pow((double)base, exponent));
    }
}

/* crates/tuckcore/src/forward.rs:930-941 -- rope_apply: pairs (i, i+half),
 * theta = pos as f32 * inv_freq[i]. */
TMO_API void tmo_rope_apply(float *x, size_t rope_dims, size_t pos, const float *inv_freq) {
    const size_t half = rope_dims / 2;
    for (size_t i = 0; i < half; ++i) {
        const float theta = (float)pos * inv_freq[i];
        const float s = sinf(theta), c = cosf(theta);
        const float x0 = x[i], x1 = x[i + half];
        x[i] = x0 * c - x1 * s;
        x[i + half] = x0 * s + x1 * c;
    }
}

/* crates/tuckcore/src/forward.rs:906-908 -- silu. */
TMO_API float tmo_silu(float x) { return x / (1.0f + expf(-x)); }

/* native/metal/kernels.metal:382-393 -- tm_gelu_tanh_mul_f32's gate: ggml's
 * tanh GELU, 0.5 x (1 + tanh(sqrt(2/pi) x (1 + 0.044715 x^2))). */
TMO_API float tmo_gelu_tanh(float x) {
    const float inner = 0.7978845608028654f * x * (1.0f + 0.044715f * x * x);
    return 0.5f * x * (1.0f + tanhf(inner));
}

/* crates/backend/src/sampling.rs:68-82 -- greedy argmax: NaN skipped, strict
 * '>' so ties keep the lowest index; 0xFFFFFFFF when every entry is NaN. */
TMO_API uint32_t tmo_argmax(const float *logits, size_t n) {
    int have = 0;
    size_t bi = 0;
    float bv = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        const float v = logits[i];
        if (isnan(v)) continue;
        if (!have || v > bv) {
            have = 1;
            bi = i;
            bv = v;
        }
    }
    return have ? (uint32_t)bi : 0xFFFFFFFFu;
}

/* crates/tuckcore/src/forward.rs:459-498 -- one query head's causal attention
 * over keys [start, seq): sequential dot, running max, exp(s - max), then
 * w = e / sum and out += w * v_j.  `start` is 0 for full attention and
 * seq - window for a sliding window (native/metal/kernels.metal:1032-1034).
 * K and V planes are [cap][head_dim] f32 holding the cache's stored values. */
TMO_API void tmo_attend_head(const float *qh, const float *k_plane, const float *v_plane,
                             size_t head_dim, size_t start, size_t seq, float scale,
                             float *scores /* [seq] scratch */, float *out) {
    float max = -INFINITY;
    for (size_t j = start; j < seq; ++j) {
        const float *kj = k_plane + j * head_dim;
        float dot = 0.0f;
        for (size_t i = 0; i < head_dim; ++i) dot += qh[i] * kj[i];
        scores[j] = dot * scale;
        if (scores[j] > max) max = scores[j];
    }
    float sum = 0.0f;
    for (size_t j = start; j < seq; ++j) {
        scores[j] = expf(scores[j] - max);
        sum += scores[j];
    }
    for (size_t i = 0; i < head_dim; ++i) out[i] = 0.0f;
    if (sum > 0.0f) {
        for (size_t j = start; j < seq; ++j) {
            const float w = scores[j] / sum;
            const float *vj = v_plane + j * head_dim;
            for (size_t i = 0; i < head_dim; ++i) out[i] += w * vj[i];
        }
    }
}

/* ------------------------------------------------------ dense decoder -- */

/* One layer of the typed graph (crates/tuckcore/src/engine/graph.rs:119-132,
 * 12-37): weights are raw GGUF Q8_0 bytes, norm vectors f32. */
typedef struct {
    const uint8_t *q, *k, *v, *o, *gate, *up, *down;
    const float *pre_norm, *post_norm, *q_norm, *k_norm;
    const float *mixer_out_norm; /* NULL unless the artifact has it (Gemma) */
    const float *ffn_out_norm;   /* NULL unless the artifact has it (Gemma) */
    float rope_base;
    uint32_t window;   /* 0 = full causal attention */
    uint32_t act_gelu; /* 0 = SwiGLU, 1 = GeGLU */
} tmo_layer;

typedef struct {
    uint32_t layers, hidden, ffn, heads, kv_heads, head_dim, vocab;
    float eps;
    float embedding_scale; /* 0 = none */
    uint32_t kv_f16;       /* 1: KV values rounded through f16 at store */
    const uint8_t *embedding; /* [vocab][hidden] Q8_0 */
    const uint8_t *head;      /* [vocab][hidden] Q8_0 (may equal embedding) */
    const float *final_norm;
    const tmo_layer *layer;
    uint32_t weight_type; /* GGML type of every matrix: 8 = Q8_0 (also when 0), 1 = F16 */
} tmo_model;

/* y = W x for the model's matrix type. */
static int model_matmul(const tmo_model *m, const uint8_t *w, size_t rows, size_t cols, const float *x,
                        size_t batch, float *y, int threads) {
    if (m->weight_type == 1) return tmo_matmul_f16(w, rows, cols, x, batch, y, threads);
    return tmo_matmul_q8_0(w, rows, cols, x, batch, y, threads);
}

typedef struct {
    float *k, *v; /* [layer][kv_head][cap][head_dim] */
    size_t cap;
} tmo_kv;

TMO_API tmo_kv *tmo_kv_new(const tmo_model *m, size_t cap) {
    tmo_kv *kv = (tmo_kv *)calloc(1, sizeof(tmo_kv));
    const size_t n = (size_t)m->layers * m->kv_heads * cap * m->head_dim;
    kv->k = (float *)calloc(n, sizeof(float));
    kv->v = (float *)calloc(n, sizeof(float));
    kv->cap = cap;
    if (!kv->k || !kv->v) {
        free(kv->k);
        free(kv->v);
        free(kv);
        return NULL;
    }
    return kv;
}

TMO_API void tmo_kv_free(tmo_kv *kv) {
    if (kv) {
        free(kv->k);
        free(kv->v);
        free(kv);
    }
}

static float *falloc(size_t n) { return (float *)malloc((n ? n : 1) * sizeof(float)); }

/*
 * Forward `n` tokens at positions pos0..pos0+n-1 through the graph and write
 * the logits of the LAST token (vocab f32) when `logits` is non-NULL.
 *
 * Qwen3 follows crates/tuckcore/src/forward.rs:391-549 step by step.  The
 * Gemma-3 additions follow the engine's block order, the only executor the
 * reference has for that graph: embedding scale
 * (crates/tuckcore/src/engine/metal.rs:2057-2064), an RMS norm on the mixer
 * and FFN outputs before each residual add (:1478-1498, :505-512), GeGLU, and
 * the sliding-window start.  Tokens of a chunk are processed together only in
 * the projections (same per-token arithmetic); attention runs per token after
 * the chunk's K/V rows are stored, which yields the token-by-token values
 * because a query never reads a later position.
 *
 * Returns 0, -1 for a token outside the vocabulary, -2 when a position
 * reaches the KV capacity (forward.rs:399-413), -3 on allocation failure.
 */
TMO_API int tmo_forward(const tmo_model *m, tmo_kv *kv, const uint32_t *tokens, size_t n,
                        size_t pos0, float *logits, int threads) {
    const size_t hidden = m->hidden, heads = m->heads, kvh = m->kv_heads, hd = m->head_dim;
    const size_t ffn = m->ffn, group = heads / kvh;
    for (size_t t = 0; t < n; ++t) {
        if (tokens[t] >= m->vocab) return -1;
        if (pos0 + t >= kv->cap) return -2;
    }
    float *x = falloc(n * hidden), *h = falloc(n * hidden), *q = falloc(n * heads * hd);
    float *k = falloc(n * kvh * hd), *v = falloc(n * kvh * hd), *att = falloc(n * heads * hd);
    float *proj = falloc(n * hidden), *g = falloc(n * ffn), *u = falloc(n * ffn);
    float *scores = falloc(pos0 + n), *inv_freq = falloc(hd / 2);
    if (!x || !h || !q || !k || !v || !att || !proj || !g || !u || !scores || !inv_freq) return -3;

    /* forward.rs:552-558 -- embedding row dequant */
    for (size_t t = 0; t < n; ++t) {
        if (m->weight_type == 1) {
            const uint8_t *row = m->embedding + (size_t)tokens[t] * hidden * 2;
            for (size_t i = 0; i < hidden; ++i) x[t * hidden + i] = tmo_f16_to_f32(read_u16(row + 2 * i));
        } else {
            tmo_dequant_q8_0(m->embedding + (size_t)tokens[t] * (hidden / 32) * 34, hidden / 32,
                             x + t * hidden);
        }
        if (m->embedding_scale != 0.0f)
            for (size_t i = 0; i < hidden; ++i) x[t * hidden + i] *= m->embedding_scale;
    }
    const float scale = 1.0f / sqrtf((float)hd);
    for (uint32_t l = 0; l < m->layers; ++l) {
        const tmo_layer *L = &m->layer[l];
        tmo_rope_inv_freq(hd, L->rope_base, inv_freq);
        for (size_t t = 0; t < n; ++t)
            tmo_rmsnorm(x + t * hidden, L->pre_norm, m->eps, hidden, h + t * hidden);
        model_matmul(m, L->q, heads * hd, hidden, h, n, q, threads);
        model_matmul(m, L->k, kvh * hd, hidden, h, n, k, threads);
        model_matmul(m, L->v, kvh * hd, hidden, h, n, v, threads);
        float *kplane = kv->k + (size_t)l * kvh * kv->cap * hd;
        float *vplane = kv->v + (size_t)l * kvh * kv->cap * hd;
        for (size_t t = 0; t < n; ++t) {
            const size_t pos = pos0 + t;
            for (size_t hh = 0; hh < heads; ++hh) {
                float *qh = q + (t * heads + hh) * hd;
                tmo_rmsnorm(qh, L->q_norm, m->eps, hd, qh);
                tmo_rope_apply(qh, hd, pos, inv_freq);
            }
            for (size_t hh = 0; hh < kvh; ++hh) {
                float *kh = k + (t * kvh + hh) * hd;
                tmo_rmsnorm(kh, L->k_norm, m->eps, hd, kh);
                tmo_rope_apply(kh, hd, pos, inv_freq);
                const float *vh = v + (t * kvh + hh) * hd;
                float *kd = kplane + (hh * kv->cap + pos) * hd;
                float *vd = vplane + (hh * kv->cap + pos) * hd;
                for (size_t i = 0; i < hd; ++i) {
                    kd[i] = m->kv_f16 ? round_f16(kh[i]) : kh[i];
                    vd[i] = m->kv_f16 ? round_f16(vh[i]) : vh[i];
                }
            }
        }
        for (size_t t = 0; t < n; ++t) {
            const size_t seq = pos0 + t + 1;
            const size_t start = (L->window != 0 && seq > L->window) ? seq - L->window : 0;
            for (size_t hh = 0; hh < heads; ++hh) {
                const size_t kvhh = hh / group;
                tmo_attend_head(q + (t * heads + hh) * hd, kplane + kvhh * kv->cap * hd,
                                vplane + kvhh * kv->cap * hd, hd, start, seq, scale, scores,
                                att + (t * heads + hh) * hd);
            }
        }
        model_matmul(m, L->o, hidden, heads * hd, att, n, proj, threads);
        for (size_t t = 0; t < n; ++t) {
            float *p = proj + t * hidden;
            if (L->mixer_out_norm) tmo_rmsnorm(p, L->mixer_out_norm, m->eps, hidden, p);
            for (size_t i = 0; i < hidden; ++i) x[t * hidden + i] += p[i];
            tmo_rmsnorm(x + t * hidden, L->post_norm, m->eps, hidden, h + t * hidden);
        }
        model_matmul(m, L->gate, ffn, hidden, h, n, g, threads);
        model_matmul(m, L->up, ffn, hidden, h, n, u, threads);
        for (size_t i = 0; i < n * ffn; ++i)
            g[i] = (L->act_gelu ? tmo_gelu_tanh(g[i]) : tmo_silu(g[i])) * u[i];
        model_matmul(m, L->down, hidden, ffn, g, n, proj, threads);
        for (size_t t = 0; t < n; ++t) {
            float *p = proj + t * hidden;
            if (L->ffn_out_norm) tmo_rmsnorm(p, L->ffn_out_norm, m->eps, hidden, p);
            for (size_t i = 0; i < hidden; ++i) x[t * hidden + i] += p[i];
        }
    }
    if (logits) {
        tmo_rmsnorm(x + (n - 1) * hidden, m->final_norm, m->eps, hidden, h);
        model_matmul(m, m->head, m->vocab, hidden, h, 1, logits, threads);
    }
    free(x); free(h); free(q); free(k); free(v); free(att);
    free(proj); free(g); free(u); free(scores); free(inv_freq);
    return 0;
}
