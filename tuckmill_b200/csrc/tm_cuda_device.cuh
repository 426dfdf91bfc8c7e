// Device helpers shared by the kernel translation units.
#pragma once
#include <cuda_runtime.h>

namespace tmdev {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// Canonical sum of squares of a vector, shared by every kernel that computes an
// RMS norm so all of them produce the same bits:
//   * elements are taken in quads; quad Q belongs to thread Q % 256, which adds
//     its quads in increasing order, x*x folded in with one FMA per element;
//   * each warp adds its 32 partials with a xor butterfly (16, 8, 4, 2, 1);
//   * the 8 warp sums are added in order 0..7.
__device__ __forceinline__ float sumsq_quad(float s, const float4 v) {
    s = fmaf(v.x, v.x, s);
    s = fmaf(v.y, v.y, s);
    s = fmaf(v.z, v.z, s);
    s = fmaf(v.w, v.w, s);
    return s;
}

// Quad `quad` of x[0..n) (zeros past the end); vector load when `vec`.
__device__ __forceinline__ float4 load_quad(const float *x, uint32_t n, uint32_t quad, bool vec) {
    const uint32_t e = quad * 4u;
    if (vec) return *(const float4 *)(x + e);
    float4 v;
    v.x = e < n ? x[e] : 0.0f;
    v.y = e + 1 < n ? x[e + 1] : 0.0f;
    v.z = e + 2 < n ? x[e + 2] : 0.0f;
    v.w = e + 3 < n ? x[e + 3] : 0.0f;
    return v;
}

__device__ __forceinline__ bool quads_vectorizable(const float *x, uint32_t n) {
    return (((size_t)x) & 15u) == 0 && (n & 3u) == 0;
}

// Warp butterfly + ordered sum over the CTA's 8 warps of per-thread partials.
static __device__ float block_reduce_sumsq(float s, float *red /* [kWarps] */) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) t += red[w];
    return t;
}

static __device__ float block_sumsq(const float *x, uint32_t n, float *red /* [kWarps] */) {
    const bool vec = quads_vectorizable(x, n);
    const uint32_t quads = (n + 3u) / 4u;
    float s = 0.0f;
    for (uint32_t q = threadIdx.x; q < quads; q += kThreads) s = sumsq_quad(s, load_quad(x, n, q, vec));
    return block_reduce_sumsq(s, red);
}

// Programmatic dependent launch: a kernel launched with the stream-serialization
// attribute may start while its predecessor still runs.  `pdl_wait` blocks until
// the predecessor has completed and its writes are visible (a no-op for an
// ordinary launch); `pdl_trigger` lets the successor start launching.  Work that
// touches only constants (weights) goes before the wait.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + expf(-g)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
    const float inner = 0.7978845608028654f * x * (1.0f + 0.044715f * x * x);
    return 0.5f * x * (1.0f + tanhf(inner));
}


}  // namespace tmdev
