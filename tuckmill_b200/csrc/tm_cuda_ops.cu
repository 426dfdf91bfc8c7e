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
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
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
__global__ void u32_add_kernel(uint32_t *p, uint32_t delta) {
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    *p += delta;
}

// y[row] = x[row] * rsqrt(mean(x^2) + eps) * w; one CTA per row; in place is safe.
__global__ void __launch_bounds__(kThreads) rmsnorm_kernel(const float *x, const float *w, float *y,
                                                           uint32_t cols, float eps) {
    __shared__ float red[kWarps];
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    const float *xr = x + (size_t)blockIdx.x * cols;
    float *yr = y + (size_t)blockIdx.x * cols;
    const float ss = tmdev::block_sumsq(xr, cols, red);
    const float inv = 1.0f / sqrtf(ss / (float)cols + eps);
    for (uint32_t i = threadIdx.x; i < cols; i += kThreads) yr[i] = xr[i] * inv * w[i];
}

// x[row] += p[row] * rsqrt(mean(p^2) + eps) * w: the output norm and the residual add of a layer as one
// launch, rounded exactly like rmsnorm_kernel followed by axpy_kernel(alpha = 1): the product is
// formed with two multiplies and added with one rounding.
__global__ void __launch_bounds__(kThreads) rmsnorm_add_kernel(const float *p, const float *w, float *x,
                                                               uint32_t cols, float eps) {
    __shared__ float red[kWarps];
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    const float *pr = p + (size_t)blockIdx.x * cols;
    float *xr = x + (size_t)blockIdx.x * cols;
    const float ss = tmdev::block_sumsq(pr, cols, red);
    const float inv = 1.0f / sqrtf(ss / (float)cols + eps);
    for (uint32_t i = threadIdx.x; i < cols; i += kThreads)
        xr[i] = __fadd_rn(xr[i], __fmul_rn(__fmul_rn(pr[i], inv), w[i]));
}

// x[row] += sum over ranks r (in rank order) of slots[r][row] -- or, with a norm weight, += rmsnorm of
// that sum: the reduction of a column-split projection's partial products and the residual add (and a
// layer's output norm) as one launch.  With a norm the sum is written over slot 0 first.
__global__ void __launch_bounds__(kThreads) reduce_ranks_add_kernel(float *slots, float *x, const float *w,
                                                                    uint32_t world, uint32_t n_rows, uint32_t cols,
                                                                    float eps) {
    __shared__ float red[kWarps];
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    const size_t stride = (size_t)n_rows * cols, base = (size_t)blockIdx.x * cols;
    float *xr = x + base, *p0 = slots + base;
    // A thread's loads of one column from every rank's slot are issued together (up to 8 ranks at a
    // time), then added in rank order: one memory round trip per column instead of one per rank.
    for (uint32_t i = blockIdx.y * kThreads + threadIdx.x; i < cols; i += gridDim.y * kThreads) {
        float p = p0[i];
        for (uint32_t r0 = 1; r0 < world; r0 += 8) {
            float v[8];
#pragma unroll
            for (uint32_t k = 0; k < 8; ++k) v[k] = r0 + k < world ? p0[(size_t)(r0 + k) * stride + i] : 0.0f;
#pragma unroll
            for (uint32_t k = 0; k < 8; ++k)
                if (r0 + k < world) p = __fadd_rn(p, v[k]);
        }
        if (w) p0[i] = p;
        else xr[i] = __fadd_rn(xr[i], p);
    }
    if (!w) return;
    __syncthreads();
    const float ss = tmdev::block_sumsq(p0, cols, red);
    const float inv = 1.0f / sqrtf(ss / (float)cols + eps);
    for (uint32_t i = threadIdx.x; i < cols; i += kThreads)
        xr[i] = __fadd_rn(xr[i], __fmul_rn(__fmul_rn(p0[i], inv), w[i]));
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
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
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
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
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

// The same two passes for several rows in one launch each (blockIdx.y = row): row r of `x` is n
// values; its winner goes to out[r * out_stride + base + pos[r]].
__global__ void __launch_bounds__(kThreads) argmax_rows_partial_kernel(const float *x, float *pv, uint32_t *pi,
                                                                       uint32_t n) {
    __shared__ float tv[kWarps];
    __shared__ uint32_t ti[kWarps];
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    const float *xr = x + (size_t)blockIdx.y * n;
    float v = -INFINITY;
    uint32_t i = kArgmaxNone;
    for (uint32_t k = blockIdx.x * kThreads + threadIdx.x; k < n; k += kArgmaxGroups * kThreads) {
        const float xv = xr[k];
        if (!isnan(xv) && better(xv, k, v, i)) { v = xv; i = k; }
    }
    argmax_block(v, i, tv, ti);
    if (threadIdx.x == 0) {
        pv[blockIdx.y * kArgmaxGroups + blockIdx.x] = v;
        pi[blockIdx.y * kArgmaxGroups + blockIdx.x] = i;
    }
}
__global__ void __launch_bounds__(kThreads) argmax_rows_final_kernel(const float *pv, const uint32_t *pi, uint32_t *out,
                                                                     uint32_t out_stride, uint32_t base,
                                                                     const uint32_t *pos, uint32_t out_cap,
                                                                     uint32_t *mirror) {
    __shared__ float tv[kWarps];
    __shared__ uint32_t ti[kWarps];
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    const uint32_t r = blockIdx.x;
    float v = threadIdx.x < kArgmaxGroups ? pv[r * kArgmaxGroups + threadIdx.x] : -INFINITY;
    uint32_t i = threadIdx.x < kArgmaxGroups ? pi[r * kArgmaxGroups + threadIdx.x] : kArgmaxNone;
    argmax_block(v, i, tv, ti);
    if (threadIdx.x == 0) {
        const uint32_t slot = base + pos[r];
        if (slot < out_cap) {
            out[(size_t)r * out_stride + slot] = i;
            if (mirror) mirror[(size_t)r * out_stride + slot] = i;
        }
    }
}
__global__ void u32_add_sat_kernel(uint32_t *p, uint32_t count, uint32_t delta, uint32_t limit) {
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) {
        const uint32_t v = p[i];
        p[i] = v >= limit || limit - v < delta ? limit : v + delta;
    }
}

// ---- RoPE / KV store ---------------------------------------------------------
// (x, y) = (a c - b s, a s + b c), with the fused multiply-adds spelled out so
// every kernel that rotates rounds the same way.
__device__ __forceinline__ void rope_rotate(float a, float b, float c, float s, float &x, float &y) {
    x = fmaf(a, c, -__fmul_rn(b, s));
    y = fmaf(a, s, __fmul_rn(b, c));
}

// Split-half rotation of the first n_rot dims of `row`; pairs (i, i + n_rot/2).
__device__ __forceinline__ void rope_pair(float *row, uint32_t i, uint32_t half_rot, uint32_t pos,
                                          const float *inv_freq) {
    const float angle = (float)pos * inv_freq[i];
    const float c = cosf(angle), s = sinf(angle);
    const float a = row[i], b = row[i + half_rot];
    rope_rotate(a, b, c, s, row[i], row[i + half_rot]);
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
// Causal (optionally sliding-window) GQA attention over a packed f16 cache.
// The arithmetic is the scalar executor's (crates/tuckcore/src/forward.rs:
// 464-498: score = dot * scale, softmax over the attended keys, weighted sum of
// values) evaluated blockwise so it parallelises and streams:
//   * keys are taken in blocks of 32 aligned to absolute positions; lane j of a
//     warp owns key j of the block (whole dot product, fixed order), the block
//     yields m = max score, l = sum exp(s - m), o[d] = sum exp(s - m) v[d];
//   * blocks are merged in increasing order with the running-max recurrence
//     M' = max(M, m), L = L e^(M-M') + l e^(m-M'), O likewise; out = O / L.
// Both entry points -- one query row of a prefill chunk per warp, and the decode
// step with one warp per key block plus a last-arrival merge -- call the same
// two device functions, so prefill and decode agree bit for bit.
constexpr int kAttnBlock = 32;

// Sum of squares with the tree of tmdev::block_sumsq (256 threads), evaluated
// by one warp, so a per-head RMS norm computed here matches rmsnorm_kernel.
__device__ float warp_sumsq_as_block(const float *x, uint32_t n, int lane) {
    float total = 0.0f;
#pragma unroll 1
    for (int w = 0; w < kWarps; ++w) {
        float s = 0.0f;
        for (uint32_t i = w * 32 + lane; i < n; i += kThreads) s += x[i] * x[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        total += s;
    }
    return total;
}

// Value dim held in slot i of lane `lane`: with an even number of slots the
// lane owns adjacent pairs (one 4-byte load per pair), otherwise single dims.
template <int DPL>
__device__ __forceinline__ uint32_t attn_dim(int lane, int i) {
    return DPL % 2 == 0 ? 2u * lane + 64u * (i / 2) + (i & 1) : (uint32_t)lane + 32u * i;
}

// Partial attention of G query heads (shared memory qs[G][hd]) over the keys
// [lo, hi) of the 32-key block starting at j0.  Slot i of o[g] holds value dim
// attn_dim(lane, i).  Per head the arithmetic does not depend on G.
template <int G, int DPL>
__device__ __forceinline__ void attend_block(const float *qs, const __half *kc, const __half *vc, uint32_t hd,
                                             uint32_t j0, uint32_t lo, uint32_t hi, float scale,
                                             const __half *k_new, const __half *v_new, uint32_t pos_new,
                                             int lane, float (&m)[G], float (&l)[G], float (&o)[G][DPL]) {
    const uint32_t j = j0 + lane;
    const bool valid = j >= lo && j < hi;
    // Four interleaved partial sums per head (chunk c of 8 dims goes to sum
    // c % 4), added as (s0 + s1) + (s2 + s3).
    float dot[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g) dot[g][0] = dot[g][1] = dot[g][2] = dot[g][3] = 0.0f;
    if (valid) {
        const __half *kr = (k_new && j == pos_new) ? k_new : kc + (size_t)j * hd;
        constexpr int KB = DPL * 4 < 16 ? DPL * 4 : 16;  // 16-byte loads in flight (hd/8, at most 16)
        for (uint32_t d0 = 0; d0 < hd; d0 += KB * 8) {
            int4 raw[KB];
#pragma unroll
            for (int c = 0; c < KB; ++c) raw[c] = *(const int4 *)(kr + d0 + c * 8);
#pragma unroll
            for (int c = 0; c < KB; ++c) {
                const uint32_t d = d0 + c * 8;
                const __half2 *h2 = (const __half2 *)&raw[c];
                float kf[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(h2[e]);
                    kf[2 * e] = f.x;
                    kf[2 * e + 1] = f.y;
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float4 q0 = *(const float4 *)(qs + g * hd + d), q1 = *(const float4 *)(qs + g * hd + d + 4);
                    float t = dot[g][c & 3];
                    t = fmaf(q0.x, kf[0], t); t = fmaf(q0.y, kf[1], t); t = fmaf(q0.z, kf[2], t); t = fmaf(q0.w, kf[3], t);
                    t = fmaf(q1.x, kf[4], t); t = fmaf(q1.y, kf[5], t); t = fmaf(q1.z, kf[6], t); t = fmaf(q1.w, kf[7], t);
                    dot[g][c & 3] = t;
                }
            }
        }
    }
    float p[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float dsum = __fadd_rn(__fadd_rn(dot[g][0], dot[g][1]), __fadd_rn(dot[g][2], dot[g][3]));
        const float sc = valid ? __fmul_rn(dsum, scale) : -INFINITY;
        float mx = sc;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        p[g] = valid ? expf(sc - mx) : 0.0f;
        float sum = p[g];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        m[g] = mx;
        l[g] = sum;
#pragma unroll
        for (int i = 0; i < DPL; ++i) o[g][i] = 0.0f;
    }
    const uint32_t jj0 = lo > j0 ? lo - j0 : 0, jj1 = (hi < j0 + kAttnBlock ? hi : j0 + kAttnBlock) - j0;
    // Keys in increasing order; the value rows of VB keys are loaded before use.
    constexpr int VB = DPL <= 4 ? 16 : 8;
    for (uint32_t jb = jj0; jb < jj1; jb += VB) {
        float vf[VB][DPL];
#pragma unroll
        for (int c = 0; c < VB; ++c) {
            const uint32_t jk = j0 + jb + c;
            const bool ok = jb + c < jj1;
            const __half *vr = (v_new && jk == pos_new) ? v_new : vc + (size_t)(ok ? jk : j0 + jj0) * hd;
            if (DPL % 2 == 0) {
#pragma unroll
                for (int i = 0; i < DPL; i += 2) {
                    const float2 f = __half22float2(*(const __half2 *)(vr + attn_dim<DPL>(lane, i)));
                    vf[c][i] = f.x;
                    vf[c][i + 1] = f.y;
                }
            } else {
#pragma unroll
                for (int i = 0; i < DPL; ++i) vf[c][i] = __half2float(vr[attn_dim<DPL>(lane, i)]);
            }
        }
#pragma unroll
        for (int c = 0; c < VB; ++c) {
            if (jb + c >= jj1) break;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float pj = __shfl_sync(0xffffffffu, p[g], (int)(jb + c));
#pragma unroll
                for (int i = 0; i < DPL; ++i) o[g][i] = fmaf(pj, vf[c][i], o[g][i]);
            }
        }
    }
}

// Running-max merge of one block partial into (M, L, O).
template <int DPL>
__device__ __forceinline__ void attend_merge(float &M, float &L, float (&O)[DPL], float m, float l,
                                             const float (&o)[DPL]) {
    const float Mn = fmaxf(M, m);
    const float a = expf(M - Mn), b = expf(m - Mn);
    L = fmaf(L, a, l * b);
#pragma unroll
    for (int i = 0; i < DPL; ++i) O[i] = fmaf(O[i], a, o[i] * b);
    M = Mn;
}

__device__ __forceinline__ uint32_t attn_start(uint32_t seq, uint32_t window) {
    return (window != 0u && seq > window) ? seq - window : 0u;
}

// Prefill: grid (kv_heads, n), one warp: query row t of a chunk at pos0 attends
// keys [start, pos0+t] for the G heads of its KV head.  q, out: [n][heads][hd].
template <int G, int DPL>
__global__ void __launch_bounds__(32) attention_chunk_kernel(const float *q, const __half *kc, const __half *vc,
                                                             float *out, uint32_t heads, uint32_t pos0,
                                                             uint32_t cap, uint32_t hd, uint32_t group0,
                                                             uint32_t group, float scale, uint32_t window) {
    __shared__ __align__(16) float qs[G * 32 * DPL];
    const int lane = threadIdx.x;
    const uint32_t kvh = blockIdx.x, t = blockIdx.y;
    const uint32_t seq = pos0 + t + 1u, start = attn_start(seq, window);
    const uint32_t head0 = kvh * group + group0;  // first of the G heads handled here
    const float *qrow = q + ((size_t)t * heads + head0) * hd;
    for (uint32_t i = lane; i < G * hd; i += 32) qs[i] = qrow[i];
    __syncwarp();
    const __half *kp = kc + (size_t)kvh * cap * hd, *vp = vc + (size_t)kvh * cap * hd;
    float M[G], L[G], O[G][DPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        M[g] = -INFINITY;
        L[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) O[g][i] = 0.0f;
    }
    for (uint32_t j0 = start / kAttnBlock * kAttnBlock; j0 < seq; j0 += kAttnBlock) {
        float m[G], l[G], o[G][DPL];
        attend_block<G, DPL>(qs, kp, vp, hd, j0, start, seq, scale, nullptr, nullptr, 0u, lane, m, l, o);
#pragma unroll
        for (int g = 0; g < G; ++g) attend_merge<DPL>(M[g], L[g], O[g], m[g], l[g], o[g]);
    }
    float *orow = out + ((size_t)t * heads + head0) * hd;
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < DPL; ++i) orow[g * hd + attn_dim<DPL>(lane, i)] = O[g][i] / L[g];
}

// Decode: grid (heads, ceil(cap/32)), one warp per (query head, key block).
// Every warp norms and rotates its query head (cheap, avoids a dependency); the
// warps whose block holds the new position also norm, rotate and round the new
// K/V row (the first head of each group stores it), each warp writes its block
// partial to `scratch`, and the last warp to arrive for a head merges that
// head's blocks in order.
//   scratch: float part[heads][nblk][hd + 2], then u32 count[heads]
// Several sequences in one launch (blockIdx.z = sequence): element strides between the sequences'
// q / k / v / out rows, cache planes and scratch regions; positions are consecutive u32.  All zero
// (and a grid of depth 1) is the single-sequence call.
struct decode_seq_strides {
    size_t q = 0, k = 0, v = 0, out = 0, cache = 0, scratch = 0;
};
#define TM_DECODE_SEQ_OFFSETS(st)                    \
    {                                                \
        const size_t sq_ = blockIdx.z;               \
        q += sq_ * (st).q;                           \
        k += sq_ * (st).k;                           \
        v += sq_ * (st).v;                           \
        out += sq_ * (st).out;                       \
        kc += sq_ * (st).cache;                      \
        vc += sq_ * (st).cache;                      \
        scratch += sq_ * (st).scratch;               \
        pos_p += sq_;                                \
    }

template <int DPL>
__global__ void __launch_bounds__(32) attention_decode_kernel(
    const float *q, const float *k, const float *v, const float *q_norm, const float *k_norm,
    const float *inv_freq, __half *kc, __half *vc, float *out, float *scratch, const uint32_t *pos_p,
    uint32_t *status, uint32_t heads, uint32_t kv_heads, uint32_t hd, uint32_t n_rot, uint32_t cap,
    uint32_t window, float eps, float scale, const decode_seq_strides seqs) {
    TM_DECODE_SEQ_OFFSETS(seqs)
    __shared__ __align__(16) float qs[32 * DPL];
    __shared__ __align__(16) float ks[32 * DPL];
    __shared__ __align__(16) __half kh[32 * DPL];
    __shared__ __align__(16) __half vh[32 * DPL];
    const int lane = threadIdx.x;
    const uint32_t head = blockIdx.x, blk = blockIdx.y, group = heads / kv_heads, kvh = head / group;
    const uint32_t nblk = (cap + kAttnBlock - 1) / kAttnBlock;
    const __half *kp = kc + (size_t)kvh * cap * hd, *vp = vc + (size_t)kvh * cap * hd;
    // The cache rows of this block do not depend on the predecessor's output
    // (except the new row, taken from shared memory below): pull them close now.
    // Only as far as L2, which is coherent: a kernel two places back in a chain of
    // programmatic launches (the previous token's attention) may still be storing
    // its row, and a copy of that line taken into L1 now would be read stale later.
    {
        const uint32_t j = min(blk * kAttnBlock + lane, cap - 1u);
        for (uint32_t off = 0; off < hd * 2u; off += 128u) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"((const char *)(kp + (size_t)j * hd) + off));
            asm volatile("prefetch.global.L2 [%0];" ::"l"((const char *)(vp + (size_t)j * hd) + off));
        }
    }
    tmdev::pdl_wait();
    // The successor may start only now, when this kernel's own predecessor has finished: a kernel that
    // let its successor start at once would let a whole chain of launches run ahead, and a later
    // attention call could read cache rows early that a call several places back is still storing.
    // This way only the call directly before can still be running: the row it stores is read again below.
    tmdev::pdl_trigger();
    // Every small input is fetched in one trip, before the position is needed.
    // Lane l holds quads l and l + 32 of a row.
    constexpr int QW = DPL > 4 ? 2 : 1;
    constexpr int RP = (DPL + 1) / 2;
    const uint32_t nquad = hd / 4, half_rot = n_rot / 2;
    float4 qv[QW], qnv[QW], kv4[QW], knv[QW], vv4[QW];
    float fr[RP];
#pragma unroll
    for (int w = 0; w < QW; ++w) {
        const uint32_t quad = w * 32 + lane;
        const bool ok = quad < nquad;
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        qnv[w] = ok ? ((const float4 *)q_norm)[quad] : z;
        knv[w] = ok ? ((const float4 *)k_norm)[quad] : z;
        kv4[w] = ok ? ((const float4 *)(k + (size_t)kvh * hd))[quad] : z;
        vv4[w] = ok ? ((const float4 *)(v + (size_t)kvh * hd))[quad] : z;
        qv[w] = ok ? ((const float4 *)(q + (size_t)head * hd))[quad] : z;
    }
#pragma unroll
    for (int r = 0; r < RP; ++r) fr[r] = lane + 32 * r < half_rot ? inv_freq[lane + 32 * r] : 0.0f;
    const uint32_t pos = *pos_p;
    if (pos >= cap) {
        if (lane == 0 && blk == 0 && head == 0) atomicOr(status, 1u);
        return;
    }
    const uint32_t seq = pos + 1u, start = attn_start(seq, window);
    const uint32_t first = start / kAttnBlock, last = pos / kAttnBlock;
    if (blk < first || blk > last) return;
    float rc[RP], rs[RP];
#pragma unroll
    for (int r = 0; r < RP; ++r) {
        const float angle = (float)pos * fr[r];
        rc[r] = cosf(angle);
        rs[r] = sinf(angle);
    }
    // Per-head RMS norm (the canonical sum-of-squares tree: quads of virtual
    // warps 0 and 1, ordered sum) into shared memory, then RoPE in place.
    auto norm_rope = [&](const float4 (&x)[QW], const float4 (&nw)[QW], float *dst) {
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < QW; ++w) {
            float sq = tmdev::sumsq_quad(0.0f, x[w]);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
            total += sq;
        }
        const float inv = 1.0f / sqrtf(total / (float)hd + eps);
#pragma unroll
        for (int w = 0; w < QW; ++w) {
            const uint32_t quad = w * 32 + lane;
            if (quad < nquad) {
                float4 y;
                y.x = x[w].x * inv * nw[w].x;
                y.y = x[w].y * inv * nw[w].y;
                y.z = x[w].z * inv * nw[w].z;
                y.w = x[w].w * inv * nw[w].w;
                ((float4 *)dst)[quad] = y;
            }
        }
        __syncwarp();
#pragma unroll
        for (int r = 0; r < RP; ++r) {
            const uint32_t i = lane + 32 * r;
            if (i < half_rot) {
                const float a0 = dst[i], b0 = dst[i + half_rot];
                rope_rotate(a0, b0, rc[r], rs[r], dst[i], dst[i + half_rot]);
            }
        }
        __syncwarp();
    };
    norm_rope(qv, qnv, qs);
    const bool owns_new = blk == last;
    if (owns_new) {
        norm_rope(kv4, knv, ks);
#pragma unroll
        for (int w = 0; w < QW; ++w) {
            const uint32_t quad = w * 32 + lane;
            if (quad < nquad) {
                const float4 kq = ((const float4 *)ks)[quad];
                const __half2 k01 = __floats2half2_rn(kq.x, kq.y), k23 = __floats2half2_rn(kq.z, kq.w);
                const __half2 v01 = __floats2half2_rn(vv4[w].x, vv4[w].y), v23 = __floats2half2_rn(vv4[w].z, vv4[w].w);
                ((__half2 *)kh)[quad * 2] = k01;
                ((__half2 *)kh)[quad * 2 + 1] = k23;
                ((__half2 *)vh)[quad * 2] = v01;
                ((__half2 *)vh)[quad * 2 + 1] = v23;
                if (head % group == 0) {
                    __half2 *kd = (__half2 *)(kc + ((size_t)kvh * cap + pos) * hd) + quad * 2;
                    __half2 *vd = (__half2 *)(vc + ((size_t)kvh * cap + pos) * hd) + quad * 2;
                    kd[0] = k01;
                    kd[1] = k23;
                    vd[0] = v01;
                    vd[1] = v23;
                }
            }
        }
    }
    __syncwarp();
    float m[1], l[1], o[1][DPL];
    attend_block<1, DPL>(qs, kp, vp, hd, blk * kAttnBlock, start, seq, scale, owns_new ? kh : nullptr,
                         owns_new ? vh : nullptr, pos, lane, m, l, o);
    float *orow = out + (size_t)head * hd;
    if (first == last) {  // a single block: merge it into the empty state and finish
        float M = -INFINITY, L = 0.0f, O[DPL];
#pragma unroll
        for (int i = 0; i < DPL; ++i) O[i] = 0.0f;
        attend_merge<DPL>(M, L, O, m[0], l[0], o[0]);
#pragma unroll
        for (int i = 0; i < DPL; ++i) orow[attn_dim<DPL>(lane, i)] = O[i] / L;
        return;
    }
    const uint32_t stride = hd + 2;
    float *part = scratch + ((size_t)head * nblk + blk) * stride;
    if (lane == 0) {
        part[0] = m[0];
        part[1] = l[0];
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) part[2 + attn_dim<DPL>(lane, i)] = o[0][i];
    __threadfence();
    __syncwarp();
    uint32_t *count = (uint32_t *)(scratch + (size_t)heads * nblk * stride) + head;
    uint32_t arrived = 0;
    if (lane == 0) arrived = atomicAdd(count, 1u);
    arrived = __shfl_sync(0xffffffffu, arrived, 0);
    if (arrived != last - first) return;
    __threadfence();
    float M = -INFINITY, L = 0.0f, O[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) O[i] = 0.0f;
    // Partials of 8 blocks are fetched together, then merged in block order.
    for (uint32_t b0 = first; b0 <= last; b0 += 8) {
        float mb[8], lb[8], ob[8][DPL];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint32_t b = b0 + c <= last ? b0 + c : last;
            const float *pb = scratch + ((size_t)head * nblk + b) * stride;
            mb[c] = __ldcg(pb);
            lb[c] = __ldcg(pb + 1);
#pragma unroll
            for (int i = 0; i < DPL; ++i) ob[c][i] = __ldcg(pb + 2 + attn_dim<DPL>(lane, i));
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            if (b0 + c > last) break;
            attend_merge<DPL>(M, L, O, mb[c], lb[c], ob[c]);
        }
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) orow[attn_dim<DPL>(lane, i)] = O[i] / L;
    if (lane == 0) *count = 0u;  // ready for the next launch on this stream
}

// ---- decode attention, latency-optimised form ---------------------------------
// Same mathematics as attention_decode_kernel, tolerance-qualified instead of
// bit-identical to the prefill kernel (the engine uses it unless `exact` is
// asked): one CTA of 128 threads per (KV head, 64-key split) serves all G query
// heads of the group, so K and V are read once; the per-thread instruction
// chain is short (two threads share a key's dot product, the value sum is
// spread over dim pairs x key halves) and the last CTA to arrive for a KV head
// merges the splits with a two-pass softmax, one thread per value dim.
//   scratch: float part[kv_heads][nsplit][G][HD + 2], then u32 count[kv_heads]
constexpr int kFastSplit = 64;
constexpr int kFastThreads = 128;

template <int G, int HD>
__global__ void __launch_bounds__(kFastThreads) attention_decode_fast_kernel(
    const float *q, const float *k, const float *v, const float *q_norm, const float *k_norm,
    const float *inv_freq, __half *kc, __half *vc, float *out, float *scratch, const uint32_t *pos_p,
    uint32_t *status, uint32_t kv_heads, uint32_t n_rot, uint32_t cap, uint32_t window, float eps, float scale,
    const decode_seq_strides seqs) {
    TM_DECODE_SEQ_OFFSETS(seqs)
    constexpr int EPL = HD / 32;          // elements of a head vector per lane (strided by 32)
    constexpr int PAIRS = HD / 2;         // value dim pairs
    constexpr int KP = kFastThreads / PAIRS > 0 ? kFastThreads / PAIRS : 1;  // key parts in the value sum
    constexpr int PPT = PAIRS / kFastThreads > 0 ? PAIRS / kFastThreads : 1; // dim pairs per thread
    __shared__ __align__(16) float qs[G][HD];
    __shared__ __align__(16) __half kh[HD];
    __shared__ __align__(16) __half vh[HD];
    __shared__ float sc[G][kFastSplit];
    __shared__ float stat[G][2];
    __shared__ float opart[KP][G][HD];
    __shared__ uint32_t s_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t kvh = blockIdx.x, split = blockIdx.y;
    const uint32_t nsplit = (cap + kFastSplit - 1) / kFastSplit;
    const __half *kp = kc + (size_t)kvh * cap * HD, *vp = vc + (size_t)kvh * cap * HD;
    {   // value rows of this split: towards L2 (coherent; see the note on row pos - 1 below)
        const uint32_t j = min(split * kFastSplit + (tid >> 1), cap - 1u);
        const uint32_t half_bytes = HD;  // half a row of f16
        for (uint32_t off = 0; off < half_bytes; off += 128u)
            asm volatile("prefetch.global.L2 [%0];" ::"l"((const char *)(vp + (size_t)j * HD) + (tid & 1) * half_bytes + off));
    }
    // This thread's half of key row split*64 + tid/2: written by an earlier step's kernel (or is a row past
    // the sequence, masked below; or the current position's row, replaced below by the fresh one), so it
    // is read before the predecessor finishes.  One row is the exception: the attention call of the
    // PREVIOUS token (two kernels back in a chain of programmatic launches) may still be storing row
    // pos - 1; that row is read again after the wait.  Calls further back have finished, because an
    // attention kernel lets its successor start only after its own predecessor is complete.
    constexpr int NL0 = HD / 16;  // 16-byte loads per thread
    int4 kraw[NL0];
    {
        const uint32_t j = min(split * kFastSplit + ((uint32_t)tid >> 1), cap - 1u);
        const __half *kr = kp + (size_t)j * HD + (tid & 1) * (HD / 2);
#pragma unroll
        for (int c = 0; c < NL0; ++c) kraw[c] = *(const int4 *)(kr + c * 8);
    }
    // The same for this thread's value elements (one dim pair of up to 32 cached rows), when they fit.
    constexpr int KEYS0 = kFastSplit / KP;
    constexpr bool kHoistV = PPT == 1 && KEYS0 <= 32;
    __half2 vpre[kHoistV ? KEYS0 : 1];
    if constexpr (kHoistV) {
        const uint32_t kpart0 = tid / PAIRS < KP ? tid / PAIRS : 0, dp00 = tid % PAIRS;
#pragma unroll
        for (int c = 0; c < KEYS0; ++c) {
            const uint32_t j = min(split * kFastSplit + kpart0 * KEYS0 + (uint32_t)c, cap - 1u);
            vpre[c] = *(const __half2 *)(vp + (size_t)j * HD + 2 * dp00);
        }
    }
    tmdev::pdl_wait();
    // The successor may start only now, when this kernel's own predecessor has finished: a kernel that
    // let its successor start at once would let a whole chain of launches run ahead, and a later
    // attention call could read cache rows early that a call several places back is still storing.
    // This way only the call directly before can still be running: the row it stores is read again below.
    tmdev::pdl_trigger();
    // The first vector this warp will normalise (q_warp, or k for warp G) does not depend on the
    // position: its loads are issued together with the position's, one memory trip instead of two.
    constexpr int EPL0 = HD / 32;
    float x0[EPL0], w0[EPL0], v0[EPL0], f0[EPL0 / 2];
    {
        const bool pre_k = warp == G;
        const float *src = pre_k ? k + (size_t)blockIdx.x * HD : q + ((size_t)blockIdx.x * G + (warp < G ? warp : 0)) * HD;
        const float *nw = pre_k ? k_norm : q_norm;
#pragma unroll
        for (int r = 0; r < EPL0; ++r) {
            x0[r] = src[lane + 32 * r];
            w0[r] = nw[lane + 32 * r];
            v0[r] = pre_k ? v[(size_t)blockIdx.x * HD + lane + 32 * r] : 0.0f;
        }
#pragma unroll
        for (int r = 0; r < EPL0 / 2; ++r) f0[r] = inv_freq[lane + 32 * r];
    }
    const uint32_t pos = *pos_p;
    if (pos >= cap) {
        if (tid == 0 && split == 0 && kvh == 0) atomicOr(status, 1u);
        return;
    }
    const uint32_t seq = pos + 1u, start = attn_start(seq, window);
    const uint32_t first = start / kFastSplit, last = pos / kFastSplit;
    if (split < first || split > last) return;
    const bool owns_new = split == last;
    (void)n_rot;
    if (pos > 0u) {  // the previous token's row, now certainly complete (read past L1)
        const uint32_t prev = pos - 1u;
        if (split * kFastSplit + ((uint32_t)tid >> 1) == prev) {
            const int4 *kr = (const int4 *)(kp + (size_t)prev * HD + (tid & 1) * (HD / 2));
#pragma unroll
            for (int c = 0; c < NL0; ++c) kraw[c] = __ldcg(kr + c);
        }
        if constexpr (kHoistV) {
            const uint32_t kpart0 = tid / PAIRS < KP ? tid / PAIRS : 0, dp00 = tid % PAIRS;
#pragma unroll
            for (int c = 0; c < KEYS0; ++c)
                if (split * kFastSplit + kpart0 * KEYS0 + (uint32_t)c == prev) {
                    const uint32_t raw = __ldcg((const unsigned int *)(vp + (size_t)prev * HD + 2 * dp00));
                    vpre[c] = *(const __half2 *)&raw;
                }
        }
    }

    // ---- vectors q_0..q_{G-1} (and k for the owning split): RMS norm + RoPE, one warp each ----
    for (int vec = warp; vec < G + (owns_new ? 1 : 0); vec += kFastThreads / 32) {
        const bool is_k = vec == G;
        const float *src = is_k ? k + (size_t)kvh * HD : q + ((size_t)kvh * G + vec) * HD;
        const float *nw = is_k ? k_norm : q_norm;
        float x[EPL], w[EPL];
        const bool preloaded = vec == warp;  // the loop's first trip: the values are already here
#pragma unroll
        for (int r = 0; r < EPL; ++r) {
            x[r] = preloaded ? x0[r] : src[lane + 32 * r];
            w[r] = preloaded ? w0[r] : nw[lane + 32 * r];
        }
        float ss = 0.0f;
#pragma unroll
        for (int r = 0; r < EPL; ++r) ss = fmaf(x[r], x[r], ss);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int r = 0; r < EPL; ++r) x[r] = x[r] * inv * w[r];
        // full rotation (n_rot == HD, checked by the host): pair (i, i + HD/2), i = lane + 32 r,
        // has both members in this lane
#pragma unroll
        for (int r = 0; r < EPL / 2; ++r) {
            float sn, cs;
            sincosf((float)pos * f0[r], &sn, &cs);
            const float a0 = x[r], b0 = x[r + EPL / 2];
            x[r] = a0 * cs - b0 * sn;
            x[r + EPL / 2] = a0 * sn + b0 * cs;
        }
        if (is_k) {
            const float *vsrc = v + (size_t)kvh * HD;
#pragma unroll
            for (int r = 0; r < EPL; ++r) {
                const uint32_t e = lane + 32 * r;
                const __half hk = __float2half_rn(x[r]), hv = __float2half_rn(preloaded ? v0[r] : vsrc[e]);
                kh[e] = hk;
                vh[e] = hv;
                kc[((size_t)kvh * cap + pos) * HD + e] = hk;
                vc[((size_t)kvh * cap + pos) * HD + e] = hv;
            }
        } else {
#pragma unroll
            for (int r = 0; r < EPL; ++r) qs[vec][lane + 32 * r] = x[r];
        }
    }
    __syncthreads();
    // ---- scores: two threads per key, half the dims each ----
    {
        const uint32_t jj = tid >> 1, hsel = tid & 1, j = split * kFastSplit + jj;
        const bool valid = j >= start && j < seq;
        float dot[G][2];
#pragma unroll
        for (int g = 0; g < G; ++g) dot[g][0] = dot[g][1] = 0.0f;
        if (valid) {
            constexpr int NL = HD / 16;  // 16-byte loads per thread
            int4 raw[NL];
            const bool fresh = owns_new && j == pos;  // this step's own key: from shared memory
#pragma unroll
            for (int c = 0; c < NL; ++c) raw[c] = fresh ? *(const int4 *)(kh + hsel * (HD / 2) + c * 8) : kraw[c];
#pragma unroll
            for (int c = 0; c < NL; ++c) {
                const __half2 *h2 = (const __half2 *)&raw[c];
                float kf[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(h2[e]);
                    kf[2 * e] = f.x;
                    kf[2 * e + 1] = f.y;
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float *qp = &qs[g][hsel * (HD / 2) + c * 8];
                    const float4 q0 = *(const float4 *)qp, q1 = *(const float4 *)(qp + 4);
                    float t = dot[g][c & 1];
                    t = fmaf(q0.x, kf[0], t); t = fmaf(q0.y, kf[1], t); t = fmaf(q0.z, kf[2], t); t = fmaf(q0.w, kf[3], t);
                    t = fmaf(q1.x, kf[4], t); t = fmaf(q1.y, kf[5], t); t = fmaf(q1.z, kf[6], t); t = fmaf(q1.w, kf[7], t);
                    dot[g][c & 1] = t;
                }
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float d = dot[g][0] + dot[g][1];
            d += __shfl_xor_sync(0xffffffffu, d, 1);
            if (hsel == 0) sc[g][jj] = valid ? d * scale : -INFINITY;
        }
    }
    __syncthreads();
    // ---- split softmax: warp g owns head g ----
    for (int g = warp; g < G; g += kFastThreads / 32) {
        const float s0 = sc[g][lane], s1 = sc[g][lane + 32];
        float mx = fmaxf(s0, s1);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        const float p0 = s0 == -INFINITY ? 0.0f : expf(s0 - mx), p1 = s1 == -INFINITY ? 0.0f : expf(s1 - mx);
        float sum = p0 + p1;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        sc[g][lane] = p0;
        sc[g][lane + 32] = p1;
        if (lane == 0) {
            stat[g][0] = mx;
            stat[g][1] = sum;
        }
    }
    __syncthreads();
    // ---- values: thread = (dim pair(s), key part); keys of a part in order ----
    {
        const uint32_t kpart = tid / PAIRS < KP ? tid / PAIRS : 0, dp0 = tid % PAIRS;
        constexpr int KEYS = kFastSplit / KP;
        const uint32_t jbase = split * kFastSplit + kpart * KEYS;
        float acc[PPT][G][2];
#pragma unroll
        for (int pp = 0; pp < PPT; ++pp)
#pragma unroll
            for (int g = 0; g < G; ++g) acc[pp][g][0] = acc[pp][g][1] = 0.0f;
        if constexpr (kHoistV) {
#pragma unroll
            for (int c = 0; c < KEYS; ++c) {
                const uint32_t j = jbase + (uint32_t)c;
                __half2 hv = vpre[c];
                if (owns_new && j == pos) hv = *(const __half2 *)(vh + 2 * dp0);  // this step's own row
                if (j >= seq) hv = __float2half2_rn(0.0f);  // weight 0 there; never multiply stale bytes
                const float2 f = __half22float2(hv);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pj = sc[g][kpart * KEYS + c];
                    acc[0][g][0] = fmaf(pj, f.x, acc[0][g][0]);
                    acc[0][g][1] = fmaf(pj, f.y, acc[0][g][1]);
                }
            }
        }
        if constexpr (!kHoistV) {
#pragma unroll 1
        for (int kb = 0; kb < KEYS; kb += 8) {
            __half2 vv[8][PPT];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint32_t j = jbase + kb + c;
                const uint32_t jc = j < seq ? j : pos;  // rows past the sequence carry weight 0
                const __half *vr = owns_new && jc == pos ? vh : vp + (size_t)jc * HD;
#pragma unroll
                for (int pp = 0; pp < PPT; ++pp) vv[c][pp] = *(const __half2 *)(vr + 2 * (dp0 + pp * kFastThreads));
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pj = sc[g][kpart * KEYS + kb + c];
#pragma unroll
                    for (int pp = 0; pp < PPT; ++pp) {
                        const float2 f = __half22float2(vv[c][pp]);
                        acc[pp][g][0] = fmaf(pj, f.x, acc[pp][g][0]);
                        acc[pp][g][1] = fmaf(pj, f.y, acc[pp][g][1]);
                    }
                }
            }
        }
        }  // !kHoistV
#pragma unroll
        for (int pp = 0; pp < PPT; ++pp)
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const uint32_t d = 2 * (dp0 + pp * kFastThreads);
                opart[kpart][g][d] = acc[pp][g][0];
                opart[kpart][g][d + 1] = acc[pp][g][1];
            }
    }
    __syncthreads();
    // ---- this split's (m, l, o); finish here when it is the only one ----
    const bool single = first == last;
    constexpr uint32_t stride = HD + 2;
    float *part = scratch + ((size_t)kvh * nsplit + split) * G * stride;
    for (uint32_t i = tid; i < G * HD; i += kFastThreads) {
        const uint32_t g = i / HD, d = i % HD;
        float o = 0.0f;
#pragma unroll
        for (int kq = 0; kq < KP; ++kq) o += opart[kq][g][d];
        if (single) out[((size_t)kvh * G + g) * HD + d] = o / stat[g][1];
        else part[g * stride + 2 + d] = o;
    }
    if (single) return;
    if (tid < G) {
        part[tid * stride] = stat[tid][0];
        part[tid * stride + 1] = stat[tid][1];
    }
    __threadfence();
    __syncthreads();
    uint32_t *count = (uint32_t *)(scratch + (size_t)kv_heads * nsplit * G * stride) + kvh;
    if (tid == 0) s_last = atomicAdd(count, 1u) == last - first ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // ---- merge: warp w takes splits w, w + 4, ... with its own running (max, sum, output) per head, a
    // lane two value dims per 64; the loads of several splits and all heads are issued together, so the
    // loop costs one memory trip per 8 (16) splits of the CTA -- the merge is the serial tail of a
    // decode step at long contexts -- and the four warps' states meet in shared memory. ----
    {
        constexpr int DJ = HD / 64;            // float2 pieces of a head vector per lane
        constexpr int B = G > 2 ? 2 : 4;       // own splits fetched together
        __shared__ __align__(8) float mrg[kFastThreads / 32][G][HD + 2];
        const uint32_t nact = last - first + 1;
        const float *base0 = scratch + ((size_t)kvh * nsplit + first) * G * stride;
        float Mg[G], Lg[G], Og[G][2 * DJ];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            Mg[g] = -INFINITY;
            Lg[g] = 0.0f;
#pragma unroll
            for (int e = 0; e < 2 * DJ; ++e) Og[g][e] = 0.0f;
        }
        for (uint32_t s0 = (uint32_t)warp; s0 < nact; s0 += 4u * B) {
            float2 ml[B][G], ov[B][G][DJ];
#pragma unroll
            for (int c = 0; c < B; ++c) {
                const uint32_t s = s0 + 4u * c;
                const float *pb = base0 + (size_t)(s < nact ? s : nact - 1) * G * stride;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    ml[c][g] = __ldcg((const float2 *)(pb + g * stride));
#pragma unroll
                    for (int jj = 0; jj < DJ; ++jj)
                        ov[c][g][jj] = __ldcg((const float2 *)(pb + g * stride + 2 + 2 * lane + 64 * jj));
                }
            }
#pragma unroll
            for (int c = 0; c < B; ++c) {
                if (s0 + 4u * c >= nact) break;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float mx = fmaxf(Mg[g], ml[c][g].x);
                    const float a = expf(Mg[g] - mx), wgt = expf(ml[c][g].x - mx);
                    Lg[g] = fmaf(wgt, ml[c][g].y, Lg[g] * a);
#pragma unroll
                    for (int jj = 0; jj < DJ; ++jj) {
                        Og[g][2 * jj] = fmaf(wgt, ov[c][g][jj].x, Og[g][2 * jj] * a);
                        Og[g][2 * jj + 1] = fmaf(wgt, ov[c][g][jj].y, Og[g][2 * jj + 1] * a);
                    }
                    Mg[g] = mx;
                }
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            if (lane == 0) {
                mrg[warp][g][0] = Mg[g];
                mrg[warp][g][1] = Lg[g];
            }
#pragma unroll
            for (int jj = 0; jj < DJ; ++jj)
                *(float2 *)&mrg[warp][g][2 + 2 * lane + 64 * jj] = make_float2(Og[g][2 * jj], Og[g][2 * jj + 1]);
        }
        __syncthreads();
        for (uint32_t i = tid; i < G * HD; i += kFastThreads) {
            const uint32_t g = i / HD, d = i % HD;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < kFastThreads / 32; ++w) M = fmaxf(M, mrg[w][g][0]);
            float L = 0.0f, O = 0.0f;
#pragma unroll
            for (int w = 0; w < kFastThreads / 32; ++w) {
                const float f = expf(mrg[w][g][0] - M);  // a warp that took no split: exp(-inf) = 0
                L = fmaf(f, mrg[w][g][1], L);
                O = fmaf(f, mrg[w][g][2 + d], O);
            }
            out[((size_t)kvh * G + g) * HD + d] = O / L;
        }
    }
    if (tid == 0) *count = 0u;  // ready for the next launch on this stream
}

template <int G, int HD>
void launch_decode_fast(tm_cuda_ctx *ctx, const float *q, const float *k, const float *v, const float *qn,
                        const float *kn, const float *inv_freq, __half *kc, __half *vc, float *out, float *scratch,
                        const uint32_t *pos, uint32_t *status, uint32_t kvh, uint32_t n_rot, uint32_t cap,
                        uint32_t window, float eps, float scale, uint32_t n_seq = 1,
                        const decode_seq_strides seqs = decode_seq_strides()) {
    tm_launch_pdl(ctx, attention_decode_fast_kernel<G, HD>, dim3(kvh, (cap + kFastSplit - 1) / kFastSplit, n_seq),
                  dim3(kFastThreads), 0, q, k, v, qn, kn, inv_freq, kc, vc, out, scratch, pos, status, kvh, n_rot, cap,
                  window, eps, scale, seqs);
}

inline bool attn_fast_ok(uint32_t heads, uint32_t kv_heads, uint32_t hd, uint32_t n_rot) {
    const uint32_t g = heads / kv_heads;
    return (hd == 128 || hd == 256) && n_rot == hd && (g == 1 || g == 2 || g == 4);
}

// Launch helpers: G heads per warp (the group size, in chunks of at most 4) and
// DPL = head_dim / 32 value dims per lane are compile-time.
template <int G, int DPL>
void launch_chunk(cudaStream_t st, const float *q, const __half *kc, const __half *vc, float *out, uint32_t heads,
                  uint32_t kvh, uint32_t n, uint32_t pos0, uint32_t cap, uint32_t hd, uint32_t group0,
                  uint32_t group, float scale, uint32_t window) {
    attention_chunk_kernel<G, DPL><<<dim3(kvh, n), 32, 0, st>>>(q, kc, vc, out, heads, pos0, cap, hd, group0, group,
                                                                 scale, window);
}

template <int DPL>
void launch_decode(tm_cuda_ctx *ctx, const float *q, const float *k, const float *v, const float *qn, const float *kn,
                   const float *inv_freq, __half *kc, __half *vc, float *out, float *scratch, const uint32_t *pos,
                   uint32_t *status, uint32_t heads, uint32_t kvh, uint32_t hd, uint32_t n_rot, uint32_t cap,
                   uint32_t window, float eps, float scale, uint32_t n_seq = 1,
                   const decode_seq_strides seqs = decode_seq_strides()) {
    tm_launch_pdl(ctx, attention_decode_kernel<DPL>, dim3(heads, (cap + kAttnBlock - 1) / kAttnBlock, n_seq), dim3(32),
                  0, q, k, v, qn, kn, inv_freq, kc, vc, out, scratch, pos, status, heads, kvh, hd, n_rot, cap, window,
                  eps, scale, seqs);
}

#define TM_ATTN_DISPATCH(FN, G, DPL, ...)                                         \
    switch ((G) * 100 + (DPL)) {                                                   \
        case 101: FN<1, 1>(__VA_ARGS__); break; case 102: FN<1, 2>(__VA_ARGS__); break;  \
        case 103: FN<1, 3>(__VA_ARGS__); break; case 104: FN<1, 4>(__VA_ARGS__); break;  \
        case 108: FN<1, 8>(__VA_ARGS__); break;                                   \
        case 201: FN<2, 1>(__VA_ARGS__); break; case 202: FN<2, 2>(__VA_ARGS__); break;  \
        case 203: FN<2, 3>(__VA_ARGS__); break; case 204: FN<2, 4>(__VA_ARGS__); break;  \
        case 208: FN<2, 8>(__VA_ARGS__); break;                                   \
        case 301: FN<3, 1>(__VA_ARGS__); break; case 302: FN<3, 2>(__VA_ARGS__); break;  \
        case 303: FN<3, 3>(__VA_ARGS__); break; case 304: FN<3, 4>(__VA_ARGS__); break;  \
        case 308: FN<3, 8>(__VA_ARGS__); break;                                   \
        case 401: FN<4, 1>(__VA_ARGS__); break; case 402: FN<4, 2>(__VA_ARGS__); break;  \
        case 403: FN<4, 3>(__VA_ARGS__); break; case 404: FN<4, 4>(__VA_ARGS__); break;  \
        case 408: FN<4, 8>(__VA_ARGS__); break;                                   \
        default: break;                                                           \
    }

inline bool attn_shape_ok(uint32_t hd) { return hd % 32 == 0 && (hd / 32 <= 4 || hd / 32 == 8); }

}  // namespace

// Pass 1 of the greedy argmax alone (64 partial (value, index) pairs), for callers
// that finish the reduction themselves (the row-sharded head).
// The same for n_rows rows of n values: row r's 64 pairs at pv / pi + 64 r.
cudaError_t tm_argmax_rows_partial_launch(tm_cuda_ctx *ctx, const float *x, uint32_t n_rows, uint32_t n, float *pv,
                                          uint32_t *pi) {
    return tm_launch_pdl(ctx, argmax_rows_partial_kernel, dim3(kArgmaxGroups, n_rows), dim3(kThreads), 0, x, pv, pi, n);
}
cudaError_t tm_argmax_partial_launch(tm_cuda_ctx *ctx, const float *x, uint32_t n, float *pv, uint32_t *pi) {
    return tm_launch_pdl(ctx, argmax_partial_kernel, dim3(kArgmaxGroups), dim3(kThreads), 0, x, pv, pi, n);
}

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
    TM_CUDA_TRY(tm_launch_pdl(ctx, axpy_kernel, dim3(grid_for(n)), dim3(256), 0, (const float *)a->dev,
                              (float *)y->dev, alpha, n));
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
    if (ctx->program) return tm_step_record_pos_add(ctx, (uint32_t *)buf->dev + index, delta, err, err_cap);
    TM_OP_BEGIN("u32_add");
    TM_CUDA_TRY(tm_launch_pdl(ctx, u32_add_kernel, dim3(1), dim3(1), 0, (uint32_t *)buf->dev + index, delta));
    TM_OP_END(1);
}

int tm_cuda_reduce_ranks_add_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *slots, tm_cuda_buffer *x, tm_cuda_buffer *weight,
                                 uint32_t world, uint32_t n_rows, uint32_t cols, float eps, char *err, size_t err_cap) {
    TM_ENTER();
    if (world == 0 || n_rows == 0 || cols == 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "reduction geometry %u x %u x %u", world, n_rows, cols);
    TM_CHECK_BUF(slots, (size_t)world * n_rows * cols * 4, "rank slots");
    TM_CHECK_BUF(x, (size_t)n_rows * cols * 4, "x");
    if (weight) TM_CHECK_BUF(weight, (size_t)cols * 4, "norm weight");
    if (ctx->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "operator reduce_ranks_add cannot be recorded into a persistent program");
    TM_OP_BEGIN("reduce_ranks_add");
    // Without a norm the sum is elementwise: the columns of a row spread over several CTAs (a decode
    // step's single row would otherwise be one CTA walking 16 columns per thread).
    const uint32_t col_ctas = weight ? 1u : (cols + kThreads - 1) / kThreads;
    TM_CUDA_TRY(tm_launch_pdl(ctx, reduce_ranks_add_kernel, dim3(n_rows, col_ctas > 64u ? 64u : col_ctas), dim3(kThreads),
                              0, (float *)slots->dev, (float *)x->dev, weight ? (const float *)weight->dev : nullptr,
                              world, n_rows, cols, eps));
    TM_OP_END(1);
}

int tm_cuda_u32_add_sat(tm_cuda_ctx *ctx, tm_cuda_buffer *buf, uint32_t first, uint32_t count, uint32_t delta,
                        uint32_t limit, char *err, size_t err_cap) {
    TM_ENTER();
    if (count == 0) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "no counters");
    TM_CHECK_BUF(buf, ((size_t)first + count) * 4, "counters");
    if (ctx->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "operator u32_add_sat cannot be recorded into a persistent program");
    TM_OP_BEGIN("u32_add_sat");
    TM_CUDA_TRY(tm_launch_pdl(ctx, u32_add_sat_kernel, dim3((count + 127) / 128), dim3(128), 0,
                              (uint32_t *)buf->dev + first, count, delta, limit));
    TM_OP_END(1);
}

int tm_cuda_argmax_rows_f32_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *x, uint32_t n_rows, uint32_t n,
                                tm_cuda_buffer *partial, tm_cuda_buffer *out, uint32_t out_stride, uint32_t base,
                                tm_cuda_buffer *pos_buf, uint32_t out_cap, tm_cuda_buffer *mirror, char *err,
                                size_t err_cap) {
    TM_ENTER();
    if (n == 0 || n_rows == 0 || n_rows > 65535u)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "argmax over %u rows of %u elements", n_rows, n);
    if (out_cap == 0 || out_cap > out_stride)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "token log of %u slots in rows of %u", out_cap, out_stride);
    TM_CHECK_BUF(x, (size_t)n_rows * n * 4, "logits");
    TM_CHECK_BUF(partial, (size_t)n_rows * 512, "argmax partials");
    TM_CHECK_BUF(out, ((size_t)(n_rows - 1) * out_stride + out_cap) * 4, "token logs");
    if (mirror) TM_CHECK_BUF(mirror, ((size_t)(n_rows - 1) * out_stride + out_cap) * 4, "token log mirrors");
    TM_CHECK_BUF(pos_buf, (size_t)n_rows * 4, "positions");
    if (ctx->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "operator argmax_rows cannot be recorded into a persistent program");
    TM_OP_BEGIN("argmax_rows");
    float *pv = (float *)partial->dev;
    uint32_t *pi = (uint32_t *)(partial->dev + (size_t)n_rows * 256);
    TM_CUDA_TRY(tm_launch_pdl(ctx, argmax_rows_partial_kernel, dim3(kArgmaxGroups, n_rows), dim3(kThreads), 0,
                              (const float *)x->dev, pv, pi, n));
    TM_CUDA_TRY(tm_launch_pdl(ctx, argmax_rows_final_kernel, dim3(n_rows), dim3(kThreads), 0, (const float *)pv,
                              (const uint32_t *)pi, (uint32_t *)out->dev, out_stride, base,
                              (const uint32_t *)pos_buf->dev, out_cap, mirror ? (uint32_t *)mirror->dev : nullptr));
    TM_OP_END(2);
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
    TM_CUDA_TRY(tm_launch_pdl(ctx, rmsnorm_kernel, dim3(rows), dim3(kThreads), 0, (const float *)x->dev,
                              (const float *)weight->dev, (float *)y->dev, cols, eps));
    TM_OP_END(1);
}

int tm_cuda_rmsnorm_add_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *p, tm_cuda_buffer *weight, tm_cuda_buffer *x,
                            uint32_t rows, uint32_t cols, float eps, char *err, size_t err_cap) {
    TM_ENTER();
    if (rows == 0 || cols == 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "rmsnorm geometry %u x %u", rows, cols);
    TM_CHECK_BUF(p, (size_t)rows * cols * 4, "p");
    TM_CHECK_BUF(x, (size_t)rows * cols * 4, "x");
    TM_CHECK_BUF(weight, (size_t)cols * 4, "norm weight");
    if (p == x) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "rmsnorm_add in place");
    if (ctx->program)
        return tm_step_record_norm_add(ctx, (const float *)p->dev, (const float *)weight->dev, (float *)x->dev, rows,
                                       cols, eps, err, err_cap);
    TM_OP_BEGIN("rmsnorm_add");
    TM_CUDA_TRY(tm_launch_pdl(ctx, rmsnorm_add_kernel, dim3(rows), dim3(kThreads), 0, (const float *)p->dev,
                              (const float *)weight->dev, (float *)x->dev, cols, eps));
    TM_OP_END(1);
}

static int argmax_common(tm_cuda_ctx *ctx, tm_cuda_buffer *x, uint32_t n, tm_cuda_buffer *partial,
                         tm_cuda_buffer *out, uint32_t out_index, const uint32_t *pos,
                         uint32_t out_cap, uint32_t *mirror, char *err, size_t err_cap) {
    if (n == 0) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "argmax over zero elements");
    TM_CHECK_BUF(x, (size_t)n * 4, "logits");
    TM_CHECK_BUF(partial, 512, "argmax partials");
    if (ctx->program)
        return tm_step_record_argmax(ctx, (const float *)x->dev, n, (uint32_t *)out->dev, out_index, pos, out_cap, mirror,
                                     err, err_cap);
    TM_OP_BEGIN("argmax");
    float *pv = (float *)partial->dev;
    uint32_t *pi = (uint32_t *)(partial->dev + 256);
    TM_CUDA_TRY(tm_launch_pdl(ctx, argmax_partial_kernel, dim3(kArgmaxGroups), dim3(kThreads), 0,
                              (const float *)x->dev, pv, pi, n));
    TM_CUDA_TRY(tm_launch_pdl(ctx, argmax_final_kernel, dim3(1), dim3(kThreads), 0, (const float *)pv,
                              (const uint32_t *)pi, (uint32_t *)out->dev, out_index, pos, out_cap, mirror));
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
    if (n == 0 || n > 65535u || heads == 0 || group == 0 || heads % group != 0 || !attn_shape_ok(hd) || cap == 0 ||
        pos0 >= cap || n > cap - pos0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "attention geometry: heads %u, group %u, head_dim %u (32, 64, 96, 128 or 256), rows %u "
                       "at position %u, capacity %u", heads, group, hd, n, pos0, cap);
    const uint32_t kvh = heads / group;
    const size_t plane = (size_t)kvh * cap * hd * 2;
    TM_CHECK_BUF(q, (size_t)n * heads * hd * 4, "q");
    TM_CHECK_BUF(out, (size_t)n * heads * hd * 4, "attention output");
    TM_CHECK_BUF(k_cache, plane, "k cache");
    TM_CHECK_BUF(v_cache, plane, "v cache");
    // The reference sizes a score scratch of n*heads*cap f32; this kernel keeps
    // its state in registers and only checks that a buffer was passed.
    TM_CHECK_BUF(scratch, 4, "attention scratch");
    TM_OP_BEGIN("attention");
    uint64_t launches = 0;
    for (uint32_t g0 = 0; g0 < group; g0 += 4) {
        const uint32_t G = group - g0 < 4 ? group - g0 : 4;
        TM_ATTN_DISPATCH(launch_chunk, G, hd / 32, ctx->stream, (const float *)q->dev, (const __half *)k_cache->dev,
                         (const __half *)v_cache->dev, (float *)out->dev, heads, kvh, n, pos0, cap, hd, g0, group,
                         scale, window);
        ++launches;
    }
    TM_OP_END(launches);
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

size_t tm_cuda_attention_decode_scratch_bytes(uint32_t heads, uint32_t kv_heads, uint32_t head_dim,
                                              uint32_t cap) {
    if (heads == 0 || kv_heads == 0 || cap == 0) return 0;
    const size_t nblk = (cap + kAttnBlock - 1) / kAttnBlock;
    (void)kv_heads;
    return ((size_t)heads * nblk * (head_dim + 2) + (size_t)heads) * 4;
}

int tm_cuda_attention_decode_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k,
                                 tm_cuda_buffer *v, tm_cuda_buffer *q_norm, tm_cuda_buffer *k_norm,
                                 tm_cuda_buffer *inv_freq, tm_cuda_buffer *k_cache,
                                 tm_cuda_buffer *v_cache, tm_cuda_buffer *out,
                                 tm_cuda_buffer *scratch, tm_cuda_buffer *pos_buf,
                                 uint32_t pos_index, tm_cuda_buffer *status, uint32_t heads,
                                 uint32_t kv_heads, uint32_t head_dim, uint32_t n_rot,
                                 uint32_t cap, uint32_t window, float eps, float scale, int exact,
                                 char *err, size_t err_cap) {
    TM_ENTER();
    if (heads == 0 || kv_heads == 0 || heads % kv_heads != 0 || heads / kv_heads > 32 || !attn_shape_ok(head_dim) ||
        n_rot == 0 || n_rot > head_dim || n_rot % 2 != 0 || cap == 0 || cap > 65535u * kAttnBlock)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "decode attention geometry: heads %u/%u, head_dim %u (32, 64, 96, 128 or 256), n_rot %u, "
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
    TM_CHECK_BUF(scratch, tm_cuda_attention_decode_scratch_bytes(heads, kv_heads, head_dim, cap),
                 "decode attention scratch");
    TM_CHECK_BUF(pos_buf, ((size_t)pos_index + 1) * 4, "position");
    TM_CHECK_BUF(status, 4, "status");
    const float *qp = (const float *)q->dev, *kp = (const float *)k->dev, *vp = (const float *)v->dev;
    const float *qn = (const float *)q_norm->dev, *kn = (const float *)k_norm->dev, *fq = (const float *)inv_freq->dev;
    __half *kcp = (__half *)k_cache->dev, *vcp = (__half *)v_cache->dev;
    float *op = (float *)out->dev, *sp = (float *)scratch->dev;
    const uint32_t *pp = (const uint32_t *)pos_buf->dev + pos_index;
    uint32_t *stp = (uint32_t *)status->dev;
    if (ctx->program)
        return tm_step_record_attention(ctx, qp, kp, vp, qn, kn, fq, kcp, vcp, op, sp, pp, stp, heads, kv_heads, head_dim,
                                        n_rot, cap, window, eps, scale, exact, err, err_cap);
    TM_OP_BEGIN("attention_decode");
    if (!exact && attn_fast_ok(heads, kv_heads, head_dim, n_rot)) {
#define TM_FAST(G, HD)                                                                                       \
    launch_decode_fast<G, HD>(ctx, qp, kp, vp, qn, kn, fq, kcp, vcp, op, sp, pp, stp, kv_heads, n_rot, cap, window, \
                              eps, scale)
        switch ((heads / kv_heads) * 1000 + head_dim) {
            case 1128: TM_FAST(1, 128); break;
            case 2128: TM_FAST(2, 128); break;
            case 4128: TM_FAST(4, 128); break;
            case 1256: TM_FAST(1, 256); break;
            case 2256: TM_FAST(2, 256); break;
            default: TM_FAST(4, 256); break;
        }
#undef TM_FAST
        TM_OP_END(1);
    }
#define TM_DECODE(DPL)                                                                                        \
    launch_decode<DPL>(ctx, qp, kp, vp, qn, kn, fq, kcp, vcp, op, sp, pp, stp, heads, kv_heads, head_dim, n_rot, \
                       cap, window, eps, scale)
    switch (head_dim / 32) {
        case 1: TM_DECODE(1); break;
        case 2: TM_DECODE(2); break;
        case 3: TM_DECODE(3); break;
        case 4: TM_DECODE(4); break;
        default: TM_DECODE(8); break;
    }
#undef TM_DECODE
    const uint64_t launches = 1;
    TM_OP_END(launches);
}

int tm_cuda_attention_decode_batch_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k, tm_cuda_buffer *v,
                                       tm_cuda_buffer *q_norm, tm_cuda_buffer *k_norm, tm_cuda_buffer *inv_freq,
                                       tm_cuda_buffer *k_cache, tm_cuda_buffer *v_cache, tm_cuda_buffer *out,
                                       tm_cuda_buffer *scratch, tm_cuda_buffer *pos_buf, tm_cuda_buffer *status,
                                       uint32_t n_seq, uint32_t q_stride, uint32_t kv_stride, uint32_t heads,
                                       uint32_t kv_heads, uint32_t head_dim,
                                       uint32_t n_rot, uint32_t cap, uint32_t window, float eps, float scale,
                                       int exact, char *err, size_t err_cap) {
    TM_ENTER();
    if (heads == 0 || kv_heads == 0 || heads % kv_heads != 0 || heads / kv_heads > 32 || !attn_shape_ok(head_dim) ||
        n_rot == 0 || n_rot > head_dim || n_rot % 2 != 0 || cap == 0 || cap > 65535u * kAttnBlock)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "decode attention geometry: heads %u/%u, head_dim %u (32, 64, 96, 128 or 256), n_rot %u, "
                       "capacity %u", heads, kv_heads, head_dim, n_rot, cap);
    if (n_seq == 0 || n_seq > 65535u)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "sequence count %u outside 1..65535", n_seq);
    const size_t plane = (size_t)kv_heads * cap * head_dim * 2;
    const size_t per_seq = tm_cuda_attention_decode_scratch_bytes(heads, kv_heads, head_dim, cap);
    if (q_stride == 0) q_stride = heads * head_dim;
    if (kv_stride == 0) kv_stride = kv_heads * head_dim;
    if (q_stride < heads * head_dim || kv_stride < kv_heads * head_dim || q_stride % 4 != 0 || kv_stride % 4 != 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "row strides %u / %u below the row widths or not 16-byte multiples",
                       q_stride, kv_stride);
    TM_CHECK_BUF(q, ((size_t)(n_seq - 1) * q_stride + (size_t)heads * head_dim) * 4, "q");
    TM_CHECK_BUF(k, ((size_t)(n_seq - 1) * kv_stride + (size_t)kv_heads * head_dim) * 4, "k");
    TM_CHECK_BUF(v, ((size_t)(n_seq - 1) * kv_stride + (size_t)kv_heads * head_dim) * 4, "v");
    TM_CHECK_BUF(q_norm, (size_t)head_dim * 4, "q norm");
    TM_CHECK_BUF(k_norm, (size_t)head_dim * 4, "k norm");
    TM_CHECK_BUF(inv_freq, (size_t)(n_rot / 2) * 4, "inv_freq");
    TM_CHECK_BUF(k_cache, (size_t)n_seq * plane, "k caches");
    TM_CHECK_BUF(v_cache, (size_t)n_seq * plane, "v caches");
    TM_CHECK_BUF(out, (size_t)n_seq * heads * head_dim * 4, "attention output");
    TM_CHECK_BUF(scratch, (size_t)n_seq * per_seq, "decode attention scratch");
    TM_CHECK_BUF(pos_buf, (size_t)n_seq * 4, "positions");
    TM_CHECK_BUF(status, 4, "status");
    if (ctx->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "operator attention_decode_batch cannot be recorded into a persistent program");
    const float *qp = (const float *)q->dev, *kp = (const float *)k->dev, *vp = (const float *)v->dev;
    const float *qn = (const float *)q_norm->dev, *kn = (const float *)k_norm->dev, *fq = (const float *)inv_freq->dev;
    __half *kcp = (__half *)k_cache->dev, *vcp = (__half *)v_cache->dev;
    float *op = (float *)out->dev, *sp = (float *)scratch->dev;
    const uint32_t *pp = (const uint32_t *)pos_buf->dev;
    uint32_t *stp = (uint32_t *)status->dev;
    decode_seq_strides st;
    st.q = q_stride;
    st.out = (size_t)heads * head_dim;
    st.k = st.v = kv_stride;
    st.cache = plane / 2;
    st.scratch = per_seq / 4;
    TM_OP_BEGIN("attention_decode_batch");
    // Several sequences, tolerance mode: the throughput form on the tensor cores (a step of many
    // sequences is bound by the K/V bytes it reads).  TM_CUDA_DECODE_MMA=0 keeps the latency form.
    static const bool mma_off = [] { const char *e = getenv("TM_CUDA_DECODE_MMA"); return e && e[0] == '0'; }();
    if (!exact && n_seq > 1 && !mma_off && tm_attention_decode_mma_ok(heads, kv_heads, head_dim, n_rot)) {
        const size_t nsplit64 = (cap + kFastSplit - 1) / kFastSplit;
        const uint32_t count_off = (uint32_t)((size_t)kv_heads * nsplit64 * (heads / kv_heads) * (head_dim + 2));
        TM_CUDA_TRY(tm_attention_decode_mma_launch(ctx, qp, kp, vp, qn, kn, fq, kcp, vcp, op, sp, pp, stp, heads, kv_heads,
                                                   head_dim, cap, window, eps, scale, n_seq, st.q, st.k, st.out, st.cache,
                                                   st.scratch, count_off));
        TM_OP_END(1);
    }
    if (!exact && attn_fast_ok(heads, kv_heads, head_dim, n_rot)) {
#define TM_FAST(G, HD)                                                                                       \
    launch_decode_fast<G, HD>(ctx, qp, kp, vp, qn, kn, fq, kcp, vcp, op, sp, pp, stp, kv_heads, n_rot, cap, window, \
                              eps, scale, n_seq, st)
        switch ((heads / kv_heads) * 1000 + head_dim) {
            case 1128: TM_FAST(1, 128); break;
            case 2128: TM_FAST(2, 128); break;
            case 4128: TM_FAST(4, 128); break;
            case 1256: TM_FAST(1, 256); break;
            case 2256: TM_FAST(2, 256); break;
            default: TM_FAST(4, 256); break;
        }
#undef TM_FAST
        TM_OP_END(1);
    }
#define TM_DECODE(DPL)                                                                                        \
    launch_decode<DPL>(ctx, qp, kp, vp, qn, kn, fq, kcp, vcp, op, sp, pp, stp, heads, kv_heads, head_dim, n_rot, \
                       cap, window, eps, scale, n_seq, st)
    switch (head_dim / 32) {
        case 1: TM_DECODE(1); break;
        case 2: TM_DECODE(2); break;
        case 3: TM_DECODE(3); break;
        case 4: TM_DECODE(4); break;
        default: TM_DECODE(8); break;
    }
#undef TM_DECODE
    const uint64_t launches = 1;
    TM_OP_END(launches);
}

// ---- decode attention without any allocation ----------------------------------
// Scratch of the entry point below: lives in the library image, one copy per
// device that loads it, held until the process exits.
constexpr size_t kStaticDecodeScratchBytes = 9u << 20;
static __device__ __align__(256) unsigned char g_static_decode_scratch[kStaticDecodeScratchBytes];
// Device address of that array per device (the symbol's name is only a host-side
// stand-in; kernels must be handed the address cudaGetSymbolAddress returns).
// Contexts of one process share the table (each under its own lock), hence atomic slots; every
// writer stores the same address.
static std::atomic<unsigned char *> g_static_decode_scratch_ptr[64] = {};

size_t tm_cuda_attention_decode_static_max_scratch(void) { return kStaticDecodeScratchBytes; }

int tm_cuda_attention_decode_dev_static(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k,
                                        tm_cuda_buffer *v, tm_cuda_buffer *q_norm, tm_cuda_buffer *k_norm,
                                        tm_cuda_buffer *inv_freq, tm_cuda_buffer *k_cache,
                                        tm_cuda_buffer *v_cache, tm_cuda_buffer *out,
                                        tm_cuda_buffer *pos_buf, uint32_t pos_index, tm_cuda_buffer *status,
                                        uint32_t heads, uint32_t kv_heads, uint32_t head_dim, uint32_t n_rot,
                                        uint32_t cap, uint32_t window, float eps, float scale, int exact,
                                        char *err, size_t err_cap) {
    TM_ENTER();
    if (heads == 0 || kv_heads == 0 || heads % kv_heads != 0 || heads / kv_heads > 32 || !attn_shape_ok(head_dim) ||
        n_rot == 0 || n_rot > head_dim || n_rot % 2 != 0 || cap == 0 || cap > 65535u * kAttnBlock)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "decode attention geometry: heads %u/%u, head_dim %u (32, 64, 96, 128 or 256), n_rot %u, "
                       "capacity %u", heads, kv_heads, head_dim, n_rot, cap);
    const size_t need = tm_cuda_attention_decode_scratch_bytes(heads, kv_heads, head_dim, cap);
    if (need > kStaticDecodeScratchBytes)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "heads %u x capacity %u x head_dim %u needs %zu bytes of scratch; the built-in scratch of the "
                       "allocation-free entry point holds %zu (use tm_cuda_attention_decode_dev with a caller buffer)",
                       heads, cap, head_dim, need, (size_t)kStaticDecodeScratchBytes);
    if (ctx->device < 0 || ctx->device >= 64)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "device index %d outside 0..63", ctx->device);
    if (ctx->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "this entry point launches directly; it cannot be recorded");
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
    TM_CHECK_BUF(pos_buf, ((size_t)pos_index + 1) * 4, "position");
    TM_CHECK_BUF(status, 4, "status");
    // Set-up, once per device, with that device current (TM_ENTER made it so).
    if (!g_static_decode_scratch_ptr[ctx->device].load(std::memory_order_acquire)) {
        unsigned char *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void **)&p, g_static_decode_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "cudaGetSymbolAddress of the built-in scratch failed: %s",
                           cudaGetErrorString(e));
        }
        g_static_decode_scratch_ptr[ctx->device].store(p, std::memory_order_release);
    }
    float *sp = (float *)g_static_decode_scratch_ptr[ctx->device].load(std::memory_order_acquire);
    // The array keeps whatever the previous call left: the arrival counters (the
    // tail of the region this geometry uses) must start at zero.  Both kernels
    // keep their counters inside the last `heads` words of `need`.
    TM_CUDA_TRY(cudaMemsetAsync((unsigned char *)sp + need - (size_t)heads * 4, 0, (size_t)heads * 4, ctx->stream));
    const float *qp = (const float *)q->dev, *kp = (const float *)k->dev, *vp = (const float *)v->dev;
    const float *qn = (const float *)q_norm->dev, *kn = (const float *)k_norm->dev, *fq = (const float *)inv_freq->dev;
    __half *kcp = (__half *)k_cache->dev, *vcp = (__half *)v_cache->dev;
    float *op = (float *)out->dev;
    const uint32_t *pp = (const uint32_t *)pos_buf->dev + pos_index;
    uint32_t *stp = (uint32_t *)status->dev;
    if (!exact && attn_fast_ok(heads, kv_heads, head_dim, n_rot)) {
        // the fast kernel keeps kv_heads counters right after its partials; clear those too
        const size_t nsplit = (cap + kFastSplit - 1) / kFastSplit;
        const size_t off = (size_t)heads * nsplit * (head_dim + 2) * 4;
        TM_CUDA_TRY(cudaMemsetAsync((unsigned char *)sp + off, 0, (size_t)kv_heads * 4, ctx->stream));
#define TM_FAST(G, HD)                                                                                       \
    launch_decode_fast<G, HD>(ctx, qp, kp, vp, qn, kn, fq, kcp, vcp, op, sp, pp, stp, kv_heads, n_rot, cap, window, \
                              eps, scale)
        switch ((heads / kv_heads) * 1000 + head_dim) {
            case 1128: TM_FAST(1, 128); break;
            case 2128: TM_FAST(2, 128); break;
            case 4128: TM_FAST(4, 128); break;
            case 1256: TM_FAST(1, 256); break;
            case 2256: TM_FAST(2, 256); break;
            default: TM_FAST(4, 256); break;
        }
#undef TM_FAST
    } else {
#define TM_DECODE(DPL)                                                                                        \
    launch_decode<DPL>(ctx, qp, kp, vp, qn, kn, fq, kcp, vcp, op, sp, pp, stp, heads, kv_heads, head_dim, n_rot, \
                       cap, window, eps, scale)
        switch (head_dim / 32) {
            case 1: TM_DECODE(1); break;
            case 2: TM_DECODE(2); break;
            case 3: TM_DECODE(3); break;
            case 4: TM_DECODE(4); break;
            default: TM_DECODE(8); break;
        }
#undef TM_DECODE
    }
    const cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess)
        return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "launch failed: %s", cudaGetErrorString(le));
    ctx->launches.fetch_add(1);
    return TM_CUDA_OK;
}

}  // extern "C"
