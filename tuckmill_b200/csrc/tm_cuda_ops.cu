// Dense-decoder support operators: elementwise utilities, RMS norm, greedy
// argmax, RoPE, f16 KV store and causal (optionally sliding-window) GQA
// attention.  Semantics follow the reference's device kernels
// (native/metal/kernels.metal:15-58 utilities, :142-226 argmax, :341-362
// rmsnorm, :382-406 gates, :887-930 rope / kv store, :944-1085 attention) and,
// through them, the scalar executor (crates/tuckcore/src/forward.rs:391-549,
// 906-941).  Launch shapes and reductions are this library's own.
#include "tm_cuda_internal.cuh"
#include "tm_cuda_device.cuh"

namespace {

using tmdev::kThreads;
using tmdev::kWarps;

constexpr uint32_t kArgmaxNone = 0xFFFFFFFFu;
constexpr int kArgmaxGroups = 64;

inline int grid_for(size_t n, int threads = 256, int cap = 148 * 16) {
    size_t g = (n + threads - 1) / threads;
    return (int)(g < 1 ? 1 : g > (size_t)cap ? (size_t)cap : g);
}

__global__ void scale_kernel(const float *x, float *y, float f, uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        y[i] = x[i] * f;
}
__global__ void axpy_kernel(const float *a, float *y, float alpha, uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        y[i] = y[i] + alpha * a[i];
}
__global__ void copy_kernel(const float *s, float *d, uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        d[i] = s[i];
}
__global__ void f16_to_f32_kernel(const __half *x, float *y, uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        y[i] = __half2float(x[i]);
}
__global__ void f32_to_f16_kernel(const float *x, __half *y, uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        y[i] = __float2half_rn(x[i]);
}
__global__ void silu_mul_kernel(const float *g, const float *u, float *o, uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        o[i] = tmdev::silu_f(g[i]) * u[i];
}
__global__ void gelu_mul_kernel(const float *g, const float *u, float *o, uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        o[i] = tmdev::gelu_tanh_f(g[i]) * u[i];
}
__global__ void u32_add_kernel(uint32_t *p, uint32_t delta) { *p += delta; }

// y[row] = x[row] * rsqrt(mean(x^2) + eps) * w; one CTA per row; in place is safe.
__global__ void __launch_bounds__(kThreads) rmsnorm_kernel(const float *x, const float *w, float *y,
                                                           uint32_t cols, float eps) {
    __shared__ float red[kWarps];
    const float *xr = x + (size_t)blockIdx.x * cols;
    float *yr = y + (size_t)blockIdx.x * cols;
    const float ss = tmdev::block_sumsq(xr, cols, red);
    const float inv = 1.0f / sqrtf(ss / (float)cols + eps);
    for (uint32_t i = threadIdx.x; i < cols; i += kThreads) yr[i] = xr[i] * inv * w[i];
}

// ---- greedy argmax (crates/backend/src/sampling.rs:68-82) -------------------
__device__ __forceinline__ bool better(float av, uint32_t ai, float bv, uint32_t bi) {
    if (ai == kArgmaxNone) return false;
    if (bi == kArgmaxNone) return true;
    return av > bv || (av == bv && ai < bi);
}
__device__ void argmax_block(float &v, uint32_t &i, float *tv, uint32_t *ti) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_down_sync(0xffffffffu, v, o);
        const uint32_t oi = __shfl_down_sync(0xffffffffu, i, o);
        if (better(ov, oi, v, i)) { v = ov; i = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { tv[warp] = v; ti[warp] = i; }
    __syncthreads();
    if (warp == 0) {
        v = lane < kWarps ? tv[lane] : -INFINITY;
        i = lane < kWarps ? ti[lane] : kArgmaxNone;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_down_sync(0xffffffffu, v, o);
            const uint32_t oi = __shfl_down_sync(0xffffffffu, i, o);
            if (better(ov, oi, v, i)) { v = ov; i = oi; }
        }
    }
}
__global__ void __launch_bounds__(kThreads) argmax_partial_kernel(const float *x, float *pv,
                                                                  uint32_t *pi, uint32_t n) {
    __shared__ float tv[kWarps];
    __shared__ uint32_t ti[kWarps];
    float v = -INFINITY;
    uint32_t i = kArgmaxNone;
    for (uint32_t k = blockIdx.x * kThreads + threadIdx.x; k < n; k += kArgmaxGroups * kThreads) {
        const float xv = x[k];
        if (!isnan(xv) && better(xv, k, v, i)) { v = xv; i = k; }
    }
    argmax_block(v, i, tv, ti);
    if (threadIdx.x == 0) { pv[blockIdx.x] = v; pi[blockIdx.x] = i; }
}
__global__ void __launch_bounds__(kThreads) argmax_final_kernel(const float *pv, const uint32_t *pi,
                                                                uint32_t *out, uint32_t out_index,
                                                                const uint32_t *pos, uint32_t out_cap,
                                                                uint32_t *mirror) {
    __shared__ float tv[kWarps];
    __shared__ uint32_t ti[kWarps];
    float v = threadIdx.x < kArgmaxGroups ? pv[threadIdx.x] : -INFINITY;
    uint32_t i = threadIdx.x < kArgmaxGroups ? pi[threadIdx.x] : kArgmaxNone;
    argmax_block(v, i, tv, ti);
    if (threadIdx.x == 0) {
        const uint32_t slot = pos ? out_index + *pos : out_index;
        if (slot < out_cap) {
            out[slot] = i;
            if (mirror) mirror[slot] = i;
        }
    }
}

// ---- RoPE / KV store ---------------------------------------------------------
// Split-half rotation of the first n_rot dims of `row`; pairs (i, i + n_rot/2).
__device__ __forceinline__ void rope_pair(float *row, uint32_t i, uint32_t half_rot, uint32_t pos,
                                          const float *inv_freq) {
    const float angle = (float)pos * inv_freq[i];
    const float c = cosf(angle), s = sinf(angle);
    const float a = row[i], b = row[i + half_rot];
    row[i] = a * c - b * s;
    row[i + half_rot] = a * s + b * c;
}

// grid (n_q_heads + n_kv_heads, n tokens): q [n][n_q][hd], k [n][n_kv][hd].
__global__ void rope_kernel(float *q, float *k, const float *inv_freq, uint32_t pos0, uint32_t n_q,
                            uint32_t n_kv, uint32_t hd, uint32_t n_rot) {
    const uint32_t head = blockIdx.x, t = blockIdx.y;
    float *row = head < n_q ? q + ((size_t)t * n_q + head) * hd
                            : k + ((size_t)t * n_kv + (head - n_q)) * hd;
    for (uint32_t i = threadIdx.x; i < n_rot / 2; i += blockDim.x)
        rope_pair(row, i, n_rot / 2, pos0 + t, inv_freq);
}

// cache[h][pos0+t][d] = (half) src[t][h][d]
__global__ void kv_store_kernel(const float *ks, const float *vs, __half *kc, __half *vc,
                                uint32_t pos0, uint32_t cap, uint32_t hd, uint32_t kvh, uint32_t n) {
    const size_t total = (size_t)n * kvh * hd;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t d = (uint32_t)(i % hd);
        const uint32_t h = (uint32_t)((i / hd) % kvh);
        const uint32_t t = (uint32_t)(i / ((size_t)hd * kvh));
        const size_t dst = ((size_t)h * cap + pos0 + t) * hd + d;
        kc[dst] = __float2half_rn(ks[i]);
        vc[dst] = __float2half_rn(vs[i]);
    }
}

// ---- attention ---------------------------------------------------------------
// One query head over keys [start, seq) of one KV head's f16 planes.  Scores go
// to `sc` (global scratch row or shared memory), softmax weights are normalised
// in place (w = e / sum, forward.rs:484-489), then every value dim accumulates.
// `k_new`/`v_new`, when non-null, stand for position seq-1 (the token being
// decoded, already rounded to f16) so the caller need not wait for its store.
__device__ void attend_row(const float *qh, const __half *kc, const __half *vc, float *oh, float *sc,
                           uint32_t start, uint32_t seq, uint32_t hd, float scale, float *red,
                           const __half *k_new, const __half *v_new) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t j = start + warp; j < seq; j += kWarps) {
        const __half *kr = (k_new && j == seq - 1) ? k_new : kc + (size_t)j * hd;
        float part = 0.0f;
        for (uint32_t d = lane * 2; d < hd; d += 64) {
            const float2 kk = __half22float2(*(const __half2 *)(kr + d));
            part = fmaf(qh[d], kk.x, part);
            part = fmaf(qh[d + 1], kk.y, part);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (lane == 0) sc[j] = part * scale;
    }
    __syncthreads();
    float m = -INFINITY;
    for (uint32_t j = start + threadIdx.x; j < seq; j += kThreads) m = fmaxf(m, sc[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    float s = 0.0f;
    for (uint32_t j = start + threadIdx.x; j < seq; j += kThreads) {
        const float e = expf(sc[j] - m);
        sc[j] = e;
        s += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) red[warp] = s;
    __syncthreads();
    float sum = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) sum += red[w];
    __syncthreads();
    for (uint32_t j = start + threadIdx.x; j < seq; j += kThreads) sc[j] = sc[j] / sum;
    __syncthreads();
    // Values: thread pairs (d, d+1); key ranges split across the CTA's slices.
    const uint32_t pairs = hd / 2;               // half2 columns
    const uint32_t slices = kThreads / pairs;     // >= 1 for hd <= 512
    const uint32_t slice = threadIdx.x / pairs, col = (threadIdx.x % pairs) * 2;
    float ax = 0.0f, ay = 0.0f;
    if (slice < slices) {
        for (uint32_t j = start + slice; j < seq; j += slices) {
            const __half *vr = (v_new && j == seq - 1) ? v_new : vc + (size_t)j * hd;
            const float2 vv = __half22float2(*(const __half2 *)(vr + col));
            const float w = sc[j];
            ax = fmaf(w, vv.x, ax);
            ay = fmaf(w, vv.y, ay);
        }
    }
    // Combine the slices in a fixed order through shared memory (reuses sc's
    // CTA only after everyone finished reading it).
    __shared__ float part_o[kThreads * 2];
    part_o[threadIdx.x * 2] = ax;
    part_o[threadIdx.x * 2 + 1] = ay;
    __syncthreads();
    if (threadIdx.x < pairs) {
        float ox = 0.0f, oy = 0.0f;
        for (uint32_t s2 = 0; s2 < slices; ++s2) {
            ox += part_o[(s2 * pairs + threadIdx.x) * 2];
            oy += part_o[(s2 * pairs + threadIdx.x) * 2 + 1];
        }
        oh[threadIdx.x * 2] = ox;
        oh[threadIdx.x * 2 + 1] = oy;
    }
    __syncthreads();
}

__device__ __forceinline__ uint32_t attn_start(uint32_t seq, uint32_t window) {
    return (window != 0u && seq > window) ? seq - window : 0u;
}

// grid (heads, n): query row t of a chunk at pos0 attends keys [start, pos0+t].
__global__ void __launch_bounds__(kThreads) attention_chunk_kernel(
    const float *q, const __half *kc, const __half *vc, float *out, float *scratch, uint32_t heads,
    uint32_t pos0, uint32_t cap, uint32_t hd, uint32_t group, float scale, uint32_t window) {
    __shared__ float red[kWarps];
    const uint32_t head = blockIdx.x, t = blockIdx.y, kvh = head / group;
    const size_t row = (size_t)t * heads + head;
    const uint32_t seq = pos0 + t + 1u;
    attend_row(q + row * hd, kc + (size_t)kvh * cap * hd, vc + (size_t)kvh * cap * hd,
               out + row * hd, scratch + row * cap, attn_start(seq, window), seq, hd, scale, red,
               nullptr, nullptr);
}

// One CTA per query head: q/k RMS norm, RoPE, KV store (by the first head of
// each group) and attention at the device-held position.
__global__ void __launch_bounds__(kThreads) attention_decode_kernel(
    float *q, const float *k, const float *v, const float *q_norm, const float *k_norm,
    const float *inv_freq, __half *kc, __half *vc, float *out, float *scratch, const uint32_t *pos_p,
    uint32_t *status, uint32_t heads, uint32_t kv_heads, uint32_t hd, uint32_t n_rot, uint32_t cap,
    uint32_t window, float eps, float scale) {
    __shared__ float red[kWarps];
    __shared__ __align__(16) float qs[512];
    __shared__ __align__(16) float ks[512];
    __shared__ __align__(16) __half kh[512];
    __shared__ __align__(16) __half vh[512];
    const uint32_t head = blockIdx.x, group = heads / kv_heads, kvh = head / group;
    const uint32_t pos = *pos_p;
    if (pos >= cap) {
        if (threadIdx.x == 0) atomicOr(status, 1u);
        return;
    }
    // per-head RMS norm of q and of this group's k (same tree as rmsnorm_kernel)
    const float *qsrc = q + (size_t)head * hd;
    const float *ksrc = k + (size_t)kvh * hd;
    const float qss = tmdev::block_sumsq(qsrc, hd, red);
    const float kss = tmdev::block_sumsq(ksrc, hd, red);
    const float qinv = 1.0f / sqrtf(qss / (float)hd + eps);
    const float kinv = 1.0f / sqrtf(kss / (float)hd + eps);
    for (uint32_t i = threadIdx.x; i < hd; i += kThreads) {
        qs[i] = qsrc[i] * qinv * q_norm[i];
        ks[i] = ksrc[i] * kinv * k_norm[i];
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < n_rot / 2; i += kThreads) {
        rope_pair(qs, i, n_rot / 2, pos, inv_freq);
        rope_pair(ks, i, n_rot / 2, pos, inv_freq);
    }
    __syncthreads();
    const float *vsrc = v + (size_t)kvh * hd;
    for (uint32_t i = threadIdx.x; i < hd; i += kThreads) {
        kh[i] = __float2half_rn(ks[i]);
        vh[i] = __float2half_rn(vsrc[i]);
        if (head % group == 0) {
            const size_t dst = ((size_t)kvh * cap + pos) * hd + i;
            kc[dst] = kh[i];
            vc[dst] = vh[i];
        }
    }
    __syncthreads();
    const uint32_t seq = pos + 1u;
    attend_row(qs, kc + (size_t)kvh * cap * hd, vc + (size_t)kvh * cap * hd, out + (size_t)head * hd,
               scratch + (size_t)head * cap, attn_start(seq, window), seq, hd, scale, red, kh, vh);
}

}  // namespace

#define TM_EW_CHECK_N()                                                                      \
    if (n == 0) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "element count must be positive")

extern "C" {

int tm_cuda_f32_scale(tm_cuda_ctx *ctx, tm_cuda_buffer *x, tm_cuda_buffer *y, float factor,
                      uint32_t n, char *err, size_t err_cap) {
    TM_ENTER();
    TM_EW_CHECK_N();
    TM_CHECK_BUF(x, (size_t)n * 4, "x");
    TM_CHECK_BUF(y, (size_t)n * 4, "y");
    TM_OP_BEGIN("f32_scale");
    scale_kernel<<<grid_for(n), 256, 0, ctx->stream>>>((const float *)x->dev, (float *)y->dev, factor, n);
    TM_OP_END(1);
}

int tm_cuda_f32_axpy(tm_cuda_ctx *ctx, tm_cuda_buffer *a, tm_cuda_buffer *y, float alpha,
                     uint32_t n, char *err, size_t err_cap) {
    TM_ENTER();
    TM_EW_CHECK_N();
    TM_CHECK_BUF(a, (size_t)n * 4, "a");
    TM_CHECK_BUF(y, (size_t)n * 4, "y");
    TM_OP_BEGIN("f32_axpy");
    axpy_kernel<<<grid_for(n), 256, 0, ctx->stream>>>((const float *)a->dev, (float *)y->dev, alpha, n);
    TM_OP_END(1);
}

int tm_cuda_copy_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *src, uint32_t src_off, tm_cuda_buffer *dst,
                     uint32_t dst_off, uint32_t n, char *err, size_t err_cap) {
    TM_ENTER();
    TM_EW_CHECK_N();
    TM_CHECK_BUF(src, ((size_t)src_off + n) * 4, "copy source");
    TM_CHECK_BUF(dst, ((size_t)dst_off + n) * 4, "copy target");
    TM_OP_BEGIN("copy_f32");
    copy_kernel<<<grid_for(n), 256, 0, ctx->stream>>>((const float *)src->dev + src_off,
                                                       (float *)dst->dev + dst_off, n);
    TM_OP_END(1);
}

int tm_cuda_cast_f16_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t n,
                         char *err, size_t err_cap) {
    TM_ENTER();
    TM_EW_CHECK_N();
    TM_CHECK_BUF(x, (size_t)n * 2, "x");
    TM_CHECK_BUF(y, (size_t)n * 4, "y");
    TM_OP_BEGIN("cast_f16_f32");
    f16_to_f32_kernel<<<grid_for(n), 256, 0, ctx->stream>>>((const __half *)x->dev, (float *)y->dev, n);
    TM_OP_END(1);
}

int tm_cuda_cast_f32_f16(tm_cuda_ctx *ctx, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t n,
                         char *err, size_t err_cap) {
    TM_ENTER();
    TM_EW_CHECK_N();
    TM_CHECK_BUF(x, (size_t)n * 4, "x");
    TM_CHECK_BUF(y, (size_t)n * 2, "y");
    TM_OP_BEGIN("cast_f32_f16");
    f32_to_f16_kernel<<<grid_for(n), 256, 0, ctx->stream>>>((const float *)x->dev, (__half *)y->dev, n);
    TM_OP_END(1);
}

int tm_cuda_silu_mul_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *gate, tm_cuda_buffer *up,
                         tm_cuda_buffer *out, uint32_t n, char *err, size_t err_cap) {
    TM_ENTER();
    TM_EW_CHECK_N();
    TM_CHECK_BUF(gate, (size_t)n * 4, "gate");
    TM_CHECK_BUF(up, (size_t)n * 4, "up");
    TM_CHECK_BUF(out, (size_t)n * 4, "out");
    TM_OP_BEGIN("silu_mul");
    silu_mul_kernel<<<grid_for(n), 256, 0, ctx->stream>>>((const float *)gate->dev,
                                                           (const float *)up->dev, (float *)out->dev, n);
    TM_OP_END(1);
}

int tm_cuda_gelu_tanh_mul_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *gate, tm_cuda_buffer *up,
                              tm_cuda_buffer *out, uint32_t n, char *err, size_t err_cap) {
    TM_ENTER();
    TM_EW_CHECK_N();
    TM_CHECK_BUF(gate, (size_t)n * 4, "gate");
    TM_CHECK_BUF(up, (size_t)n * 4, "up");
    TM_CHECK_BUF(out, (size_t)n * 4, "out");
    TM_OP_BEGIN("gelu_tanh_mul");
    gelu_mul_kernel<<<grid_for(n), 256, 0, ctx->stream>>>((const float *)gate->dev,
                                                           (const float *)up->dev, (float *)out->dev, n);
    TM_OP_END(1);
}

int tm_cuda_u32_add(tm_cuda_ctx *ctx, tm_cuda_buffer *buf, uint32_t index, uint32_t delta,
                    char *err, size_t err_cap) {
    TM_ENTER();
    TM_CHECK_BUF(buf, ((size_t)index + 1) * 4, "counter");
    TM_OP_BEGIN("u32_add");
    u32_add_kernel<<<1, 1, 0, ctx->stream>>>((uint32_t *)buf->dev + index, delta);
    TM_OP_END(1);
}

int tm_cuda_rmsnorm_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *x, tm_cuda_buffer *weight,
                        tm_cuda_buffer *y, uint32_t rows, uint32_t cols, float eps, char *err,
                        size_t err_cap) {
    TM_ENTER();
    if (rows == 0 || cols == 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "rmsnorm geometry %u x %u", rows, cols);
    TM_CHECK_BUF(x, (size_t)rows * cols * 4, "x");
    TM_CHECK_BUF(y, (size_t)rows * cols * 4, "y");
    TM_CHECK_BUF(weight, (size_t)cols * 4, "norm weight");
    TM_OP_BEGIN("rmsnorm");
    rmsnorm_kernel<<<rows, kThreads, 0, ctx->stream>>>((const float *)x->dev,
                                                       (const float *)weight->dev, (float *)y->dev,
                                                       cols, eps);
    TM_OP_END(1);
}

static int argmax_common(tm_cuda_ctx *ctx, tm_cuda_buffer *x, uint32_t n, tm_cuda_buffer *partial,
                         tm_cuda_buffer *out, uint32_t out_index, const uint32_t *pos,
                         uint32_t out_cap, uint32_t *mirror, char *err, size_t err_cap) {
    if (n == 0) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "argmax over zero elements");
    TM_CHECK_BUF(x, (size_t)n * 4, "logits");
    TM_CHECK_BUF(partial, 512, "argmax partials");
    TM_OP_BEGIN("argmax");
    float *pv = (float *)partial->dev;
    uint32_t *pi = (uint32_t *)(partial->dev + 256);
    argmax_partial_kernel<<<kArgmaxGroups, kThreads, 0, ctx->stream>>>((const float *)x->dev, pv, pi, n);
    argmax_final_kernel<<<1, kThreads, 0, ctx->stream>>>(pv, pi, (uint32_t *)out->dev, out_index, pos,
                                                         out_cap, mirror);
    TM_OP_END(2);
}

int tm_cuda_argmax_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *x, uint32_t n, tm_cuda_buffer *partial,
                       tm_cuda_buffer *out, uint32_t out_index, char *err, size_t err_cap) {
    TM_ENTER();
    TM_CHECK_BUF(out, ((size_t)out_index + 1) * 4, "argmax output");
    return argmax_common(ctx, x, n, partial, out, out_index, nullptr, (uint32_t)(out->len / 4),
                         nullptr, err, err_cap);
}

int tm_cuda_argmax_f32_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *x, uint32_t n,
                           tm_cuda_buffer *partial, tm_cuda_buffer *out, uint32_t base,
                           tm_cuda_buffer *pos_buf, uint32_t pos_index, uint32_t out_cap,
                           tm_cuda_buffer *mirror, char *err, size_t err_cap) {
    TM_ENTER();
    if (mirror) TM_CHECK_BUF(mirror, (size_t)out_cap * 4, "token log mirror");
    if (out_cap == 0) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "empty token log");
    TM_CHECK_BUF(out, (size_t)out_cap * 4, "token log");
    TM_CHECK_BUF(pos_buf, ((size_t)pos_index + 1) * 4, "position");
    return argmax_common(ctx, x, n, partial, out, base, (const uint32_t *)pos_buf->dev + pos_index,
                         out_cap, mirror ? (uint32_t *)mirror->dev : nullptr, err, err_cap);
}

static int rope_common(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k,
                       tm_cuda_buffer *inv_freq, uint32_t pos0, uint32_t n_q, uint32_t n_kv,
                       uint32_t hd, uint32_t n_rot, uint32_t n, char *err, size_t err_cap) {
    if (n == 0 || n_q == 0 || n_kv == 0 || hd == 0 || n_rot == 0 || n_rot > hd || n_rot % 2 != 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "rope geometry: heads %u/%u, head_dim %u, n_rot %u, tokens %u", n_q, n_kv, hd,
                       n_rot, n);
    TM_CHECK_BUF(q, (size_t)n * n_q * hd * 4, "q");
    TM_CHECK_BUF(k, (size_t)n * n_kv * hd * 4, "k");
    TM_CHECK_BUF(inv_freq, (size_t)(n_rot / 2) * 4, "inv_freq");
    TM_OP_BEGIN("rope");
    const int threads = n_rot / 2 >= 128 ? 128 : n_rot / 2 >= 64 ? 64 : 32;
    rope_kernel<<<dim3(n_q + n_kv, n), threads, 0, ctx->stream>>>(
        (float *)q->dev, (float *)k->dev, (const float *)inv_freq->dev, pos0, n_q, n_kv, hd, n_rot);
    TM_OP_END(1);
}

int tm_cuda_qwen35_rope_partial(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k,
                                tm_cuda_buffer *inv_freq, uint32_t pos, uint32_t n_q_heads,
                                uint32_t n_kv_heads, uint32_t head_dim, uint32_t n_rot, char *err,
                                size_t err_cap) {
    TM_ENTER();
    return rope_common(ctx, q, k, inv_freq, pos, n_q_heads, n_kv_heads, head_dim, n_rot, 1, err, err_cap);
}

int tm_cuda_qwen35_rope_partial_chunk(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k,
                                      tm_cuda_buffer *inv_freq, uint32_t pos0, uint32_t n_q_heads,
                                      uint32_t n_kv_heads, uint32_t head_dim, uint32_t n_rot,
                                      uint32_t n, char *err, size_t err_cap) {
    TM_ENTER();
    return rope_common(ctx, q, k, inv_freq, pos0, n_q_heads, n_kv_heads, head_dim, n_rot, n, err, err_cap);
}

static int kv_store_common(tm_cuda_ctx *ctx, tm_cuda_buffer *k_src, tm_cuda_buffer *v_src,
                           tm_cuda_buffer *k_cache, tm_cuda_buffer *v_cache, uint32_t pos0,
                           uint32_t cap, uint32_t hd, uint32_t kvh, uint32_t n, char *err,
                           size_t err_cap) {
    if (n == 0 || hd == 0 || kvh == 0 || cap == 0 || pos0 >= cap || n > cap - pos0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "kv store of %u rows at position %u exceeds capacity %u", n, pos0, cap);
    const size_t plane = (size_t)kvh * cap * hd * 2;
    TM_CHECK_BUF(k_src, (size_t)n * kvh * hd * 4, "k rows");
    TM_CHECK_BUF(v_src, (size_t)n * kvh * hd * 4, "v rows");
    TM_CHECK_BUF(k_cache, plane, "k cache");
    TM_CHECK_BUF(v_cache, plane, "v cache");
    TM_OP_BEGIN("kv_store");
    kv_store_kernel<<<grid_for((size_t)n * kvh * hd), 256, 0, ctx->stream>>>(
        (const float *)k_src->dev, (const float *)v_src->dev, (__half *)k_cache->dev,
        (__half *)v_cache->dev, pos0, cap, hd, kvh, n);
    TM_OP_END(1);
}

int tm_cuda_qwen35_kv_store_f16(tm_cuda_ctx *ctx, tm_cuda_buffer *k_src, tm_cuda_buffer *v_src,
                                tm_cuda_buffer *k_cache, tm_cuda_buffer *v_cache, uint32_t pos,
                                uint32_t cap, uint32_t head_dim, uint32_t kv_heads, char *err,
                                size_t err_cap) {
    TM_ENTER();
    return kv_store_common(ctx, k_src, v_src, k_cache, v_cache, pos, cap, head_dim, kv_heads, 1, err, err_cap);
}

int tm_cuda_qwen35_kv_store_f16_chunk(tm_cuda_ctx *ctx, tm_cuda_buffer *k_src,
                                      tm_cuda_buffer *v_src, tm_cuda_buffer *k_cache,
                                      tm_cuda_buffer *v_cache, uint32_t pos0, uint32_t cap,
                                      uint32_t head_dim, uint32_t kv_heads, uint32_t n, char *err,
                                      size_t err_cap) {
    TM_ENTER();
    return kv_store_common(ctx, k_src, v_src, k_cache, v_cache, pos0, cap, head_dim, kv_heads, n, err, err_cap);
}

static int attention_common(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k_cache,
                            tm_cuda_buffer *v_cache, tm_cuda_buffer *out, tm_cuda_buffer *scratch,
                            uint32_t heads, uint32_t pos0, uint32_t cap, uint32_t hd, uint32_t group,
                            float scale, uint32_t n, uint32_t window, char *err, size_t err_cap) {
    if (n == 0 || heads == 0 || group == 0 || heads % group != 0 || hd == 0 || hd % 2 != 0 ||
        hd > 512 || cap == 0 || pos0 >= cap || n > cap - pos0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "attention geometry: heads %u, group %u, head_dim %u (even, <= 512), rows %u at "
                       "position %u, capacity %u", heads, group, hd, n, pos0, cap);
    const size_t plane = (size_t)(heads / group) * cap * hd * 2;
    TM_CHECK_BUF(q, (size_t)n * heads * hd * 4, "q");
    TM_CHECK_BUF(out, (size_t)n * heads * hd * 4, "attention output");
    TM_CHECK_BUF(k_cache, plane, "k cache");
    TM_CHECK_BUF(v_cache, plane, "v cache");
    TM_CHECK_BUF(scratch, (size_t)n * heads * cap * 4, "attention scratch");
    TM_OP_BEGIN("attention");
    attention_chunk_kernel<<<dim3(heads, n), kThreads, 0, ctx->stream>>>(
        (const float *)q->dev, (const __half *)k_cache->dev, (const __half *)v_cache->dev,
        (float *)out->dev, (float *)scratch->dev, heads, pos0, cap, hd, group, scale, window);
    TM_OP_END(1);
}

int tm_cuda_qwen35_attention_f16(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k_cache,
                                 tm_cuda_buffer *v_cache, tm_cuda_buffer *out,
                                 tm_cuda_buffer *scratch, uint32_t heads, uint32_t pos,
                                 uint32_t cap, uint32_t head_dim, uint32_t group, float scale,
                                 char *err, size_t err_cap) {
    TM_ENTER();
    return attention_common(ctx, q, k_cache, v_cache, out, scratch, heads, pos, cap, head_dim, group,
                            scale, 1, 0, err, err_cap);
}

int tm_cuda_qwen35_attention_f16_chunk(tm_cuda_ctx *ctx, tm_cuda_buffer *q,
                                       tm_cuda_buffer *k_cache, tm_cuda_buffer *v_cache,
                                       tm_cuda_buffer *out, tm_cuda_buffer *scratch,
                                       uint32_t heads, uint32_t pos0, uint32_t cap,
                                       uint32_t head_dim, uint32_t group, float scale, uint32_t n,
                                       uint32_t window, char *err, size_t err_cap) {
    TM_ENTER();
    return attention_common(ctx, q, k_cache, v_cache, out, scratch, heads, pos0, cap, head_dim, group,
                            scale, n, window, err, err_cap);
}

int tm_cuda_attention_decode_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k,
                                 tm_cuda_buffer *v, tm_cuda_buffer *q_norm, tm_cuda_buffer *k_norm,
                                 tm_cuda_buffer *inv_freq, tm_cuda_buffer *k_cache,
                                 tm_cuda_buffer *v_cache, tm_cuda_buffer *out,
                                 tm_cuda_buffer *scratch, tm_cuda_buffer *pos_buf,
                                 uint32_t pos_index, tm_cuda_buffer *status, uint32_t heads,
                                 uint32_t kv_heads, uint32_t head_dim, uint32_t n_rot,
                                 uint32_t cap, uint32_t window, float eps, float scale, char *err,
                                 size_t err_cap) {
    TM_ENTER();
    if (heads == 0 || kv_heads == 0 || heads % kv_heads != 0 || head_dim == 0 || head_dim % 2 != 0 ||
        head_dim > 512 || n_rot == 0 || n_rot > head_dim || n_rot % 2 != 0 || cap == 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "decode attention geometry: heads %u/%u, head_dim %u (even, <= 512), n_rot %u, "
                       "capacity %u", heads, kv_heads, head_dim, n_rot, cap);
    const size_t plane = (size_t)kv_heads * cap * head_dim * 2;
    TM_CHECK_BUF(q, (size_t)heads * head_dim * 4, "q");
    TM_CHECK_BUF(k, (size_t)kv_heads * head_dim * 4, "k");
    TM_CHECK_BUF(v, (size_t)kv_heads * head_dim * 4, "v");
    TM_CHECK_BUF(q_norm, (size_t)head_dim * 4, "q norm");
    TM_CHECK_BUF(k_norm, (size_t)head_dim * 4, "k norm");
    TM_CHECK_BUF(inv_freq, (size_t)(n_rot / 2) * 4, "inv_freq");
    TM_CHECK_BUF(k_cache, plane, "k cache");
    TM_CHECK_BUF(v_cache, plane, "v cache");
    TM_CHECK_BUF(out, (size_t)heads * head_dim * 4, "attention output");
    TM_CHECK_BUF(scratch, (size_t)heads * cap * 4, "attention scratch");
    TM_CHECK_BUF(pos_buf, ((size_t)pos_index + 1) * 4, "position");
    TM_CHECK_BUF(status, 4, "status");
    TM_OP_BEGIN("attention_decode");
    attention_decode_kernel<<<heads, kThreads, 0, ctx->stream>>>(
        (float *)q->dev, (const float *)k->dev, (const float *)v->dev, (const float *)q_norm->dev,
        (const float *)k_norm->dev, (const float *)inv_freq->dev, (__half *)k_cache->dev,
        (__half *)v_cache->dev, (float *)out->dev, (float *)scratch->dev,
        (const uint32_t *)pos_buf->dev + pos_index, (uint32_t *)status->dev, heads, kv_heads,
        head_dim, n_rot, cap, window, eps, scale);
    TM_OP_END(1);
}

}  // extern "C"
