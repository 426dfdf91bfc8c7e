// Device helpers shared by the kernel translation units.
#pragma once
#include <cuda_runtime.h>

namespace tmdev {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// Sum of x[i]^2 over i < n with a fixed thread -> element mapping and a fixed
// tree, so every CTA (and the stand-alone RMS norm kernel) gets the same bits.
static __device__ float block_sumsq(const float *x, uint32_t n, float *red /* [kWarps] */) {
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < n; i += kThreads) s += x[i] * x[i];
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

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + expf(-g)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
    const float inner = 0.7978845608028654f * x * (1.0f + 0.044715f * x * x);
    return 0.5f * x * (1.0f + tanhf(inner));
}


}  // namespace tmdev
