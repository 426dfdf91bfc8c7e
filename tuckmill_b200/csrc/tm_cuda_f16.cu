// F16-weight matrices: y[r] = dot(f32(w_row_r), x) with f32 accumulation -- the reference's
// tm_f16_gemv / tm_f16_gemm / tm_f16_row_f32 (native/metal/kernels.metal:296-315, 638-668,
// native/metal/tm_metal.h:142,156,179), which serve F16-weight artifacts: the reference's own
// model fixtures (crates/manifest/src/testing.rs:241-256) and F16 twins of quantized models.
// A matrix is rows * cols binary16 values, row-major, uploaded verbatim.
//
// One kernel serves the GEMV, the batched form (any batch: a (row, token) result does not depend
// on how many tokens share the launch, so batch 1 is bit-identical to the GEMV, the contract of
// tm_metal.h:160-164) and the fused forms the decode step uses (the elementwise prologue of the
// Q8_0 GEMV: RMS norm with the same canonical sum of squares, silu/gelu * up; store or accumulate).
// A warp owns a row: lane l adds columns 2l, 2l+1, 2l+64, ... in that order, the lanes are added
// with a xor butterfly.  The hot path of this library is Q8_0; this kernel is sized for
// correctness on fixtures (coalesced 4-byte loads, activations staged once per CTA), not tuned.
#include "tm_cuda_internal.cuh"
#include "tm_cuda_device.cuh"

namespace {

constexpr int kThreads = tmdev::kThreads;
constexpr int kWarps = tmdev::kWarps;

struct f16_args {
    const __half *w;   // [rows][cols]
    const float *x;    // [M][cols]
    float *y;          // [M][rows]
    const float *pro;  // norm weight [cols] or the multiplicand [M][cols]
    uint32_t rows, cols;
    float eps;
    int prologue, epilogue;
};

template <int M>
__global__ void __launch_bounds__(kThreads) f16_gemv_kernel(const f16_args a) {
    extern __shared__ __align__(16) float xs[];  // [M][cols]
    __shared__ float red[kWarps];
    const uint32_t cols = a.cols, rows = a.rows;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
#pragma unroll 1
    for (int m = 0; m < M; ++m) {
        const float *xm = a.x + (size_t)m * cols;
        float inv_rms = 0.0f;
        if (a.prologue == TM_CUDA_PRO_RMSNORM) {
            const float ss = tmdev::block_sumsq(xm, cols, red);
            inv_rms = 1.0f / sqrtf(ss / (float)cols + a.eps);
        }
        for (uint32_t c = threadIdx.x; c < cols; c += kThreads) {
            float v = xm[c];
            if (a.prologue == TM_CUDA_PRO_RMSNORM) v = v * inv_rms * a.pro[c];
            else if (a.prologue == TM_CUDA_PRO_SILU_MUL) v = tmdev::silu_f(v) * a.pro[(size_t)m * cols + c];
            else if (a.prologue == TM_CUDA_PRO_GELU_MUL) v = tmdev::gelu_tanh_f(v) * a.pro[(size_t)m * cols + c];
            xs[(size_t)m * cols + c] = v;
        }
    }
    __syncthreads();
    for (uint32_t row = blockIdx.x * kWarps + warp; row < rows; row += gridDim.x * kWarps) {
        const __half *wr = a.w + (size_t)row * cols;
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.0f;
        if ((cols & 1u) == 0u && (((size_t)wr) & 3u) == 0u) {
            for (uint32_t c = 2u * lane; c < cols; c += 64u) {
                const float2 wv = __half22float2(*(const __half2 *)(wr + c));
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    acc[m] = fmaf(wv.x, xs[(size_t)m * cols + c], acc[m]);
                    acc[m] = fmaf(wv.y, xs[(size_t)m * cols + c + 1], acc[m]);
                }
            }
        } else {  // odd widths / unaligned rows: the same columns per lane, one value at a time
            for (uint32_t c = 2u * lane; c < cols; c += 64u) {
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    acc[m] = fmaf(__half2float(wr[c]), xs[(size_t)m * cols + c], acc[m]);
                    if (c + 1 < cols) acc[m] = fmaf(__half2float(wr[c + 1]), xs[(size_t)m * cols + c + 1], acc[m]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float v = acc[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) {
                float *yp = a.y + (size_t)m * rows + row;
                *yp = a.epilogue == TM_CUDA_EPI_ADD ? *yp + v : v;
            }
        }
    }
}

template <int M>
cudaError_t launch_f16(tm_cuda_ctx *ctx, const f16_args &a, size_t smem) {
    static std::atomic<bool> attr_set[64] = {};
    const int dev = ctx->device;
    if (smem > 48u * 1024u && (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire))) {
        cudaError_t e = cudaFuncSetAttribute(f16_gemv_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)ctx->smem_optin - 4096);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
    }
    uint32_t grid = (a.rows + kWarps - 1) / kWarps;
    const uint32_t cap = (uint32_t)ctx->sm_count * 8u;
    if (grid > cap) grid = cap;
    return tm_launch_pdl(ctx, f16_gemv_kernel<M>, dim3(grid), dim3(kThreads), smem, a);
}

// out[c] = f32(w[row][c]) (* scale when non-zero); row < 0 writes zeros.
__device__ __forceinline__ void f16_row(const __half *w, uint32_t cols, long row, float scale, float *out) {
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x) {
        float v = 0.0f;
        if (row >= 0) {
            v = __half2float(w[(size_t)row * cols + c]);
            if (scale != 0.0f) v *= scale;
        }
        out[c] = v;
    }
}
__global__ void f16_row_kernel(const __half *w, uint32_t cols, uint32_t row, float *out) {
    f16_row(w, cols, (long)row, 0.0f, out);
}
__global__ void f16_row_indirect_kernel(const __half *w, uint32_t rows, uint32_t cols, const uint32_t *ids, uint32_t slot,
                                        const uint32_t *pos, int bias, uint32_t ids_len, float scale, float *out) {
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    uint32_t s = slot;
    if (pos) s = slot + *pos + (uint32_t)bias;
    long row = -1;
    if (s < ids_len) {
        const uint32_t id = ids[s];
        if (id < rows) row = (long)id;
    }
    f16_row(w, cols, row, scale, out);
}
__global__ void f16_rows_gather_kernel(const __half *w, uint32_t rows, uint32_t cols, const uint32_t *ids,
                                       uint32_t first, float scale, float *out) {
    const uint32_t t = blockIdx.y, id = ids[first + t];
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x) {
        float v = 0.0f;
        if (id < rows) {
            v = __half2float(w[(size_t)id * cols + c]);
            if (scale != 0.0f) v *= scale;
        }
        out[(size_t)t * cols + c] = v;
    }
}

int f16_common(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t rows, uint32_t cols,
               uint32_t batch, uint32_t x_off, uint32_t y_off, int prologue, tm_cuda_buffer *pro, float eps, int epilogue,
               const char *label, char *err, size_t err_cap) {
    if (rows == 0 || cols == 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "F16 geometry %u x %u", rows, cols);
    if (batch == 0 || batch > TM_CUDA_GEMM_MAX_BATCH)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "batch %u outside 1..%u", batch, TM_CUDA_GEMM_MAX_BATCH);
    TM_CHECK_BUF(w, (size_t)rows * cols * 2, "F16 weights");
    TM_CHECK_BUF(x, ((size_t)x_off + (size_t)batch * cols) * 4, "activation");
    TM_CHECK_BUF(y, ((size_t)y_off + (size_t)batch * rows) * 4, "output");
    if (prologue < TM_CUDA_PRO_NONE || prologue > TM_CUDA_PRO_GELU_MUL ||
        (epilogue != TM_CUDA_EPI_STORE && epilogue != TM_CUDA_EPI_ADD))
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "unknown prologue/epilogue");
    if (prologue == TM_CUDA_PRO_RMSNORM) TM_CHECK_BUF(pro, (size_t)cols * 4, "norm weight");
    if (prologue == TM_CUDA_PRO_SILU_MUL || prologue == TM_CUDA_PRO_GELU_MUL)
        TM_CHECK_BUF(pro, (size_t)batch * cols * 4, "gate multiplicand");
    const size_t per_token = (size_t)cols * 4, budget = ctx->smem_optin - 4096;
    if (per_token > budget)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "cols %u exceeds the activation stage of one CTA", cols);
    if (ctx->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "operator %s cannot be recorded into a persistent program", label);
    TM_OP_BEGIN(label);
    uint64_t kernels = 0;
    uint32_t done = 0;
    while (done < batch) {
        int m = 8;
        while (m > 1 && ((uint32_t)m > batch - done || (size_t)m * per_token > budget)) m >>= 1;
        f16_args a;
        a.w = (const __half *)w->dev;
        a.x = (const float *)x->dev + x_off + (size_t)done * cols;
        a.y = (float *)y->dev + y_off + (size_t)done * rows;
        a.pro = pro ? (const float *)pro->dev : nullptr;
        if (pro && (prologue == TM_CUDA_PRO_SILU_MUL || prologue == TM_CUDA_PRO_GELU_MUL)) a.pro += (size_t)done * cols;
        a.rows = rows;
        a.cols = cols;
        a.eps = eps;
        a.prologue = prologue;
        a.epilogue = epilogue;
        const size_t smem = (size_t)m * per_token;
        cudaError_t e = m == 8   ? launch_f16<8>(ctx, a, smem)
                        : m == 4 ? launch_f16<4>(ctx, a, smem)
                        : m == 2 ? launch_f16<2>(ctx, a, smem)
                                 : launch_f16<1>(ctx, a, smem);
        if (e != cudaSuccess)
            return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "F16 GEMV launch failed: %s", cudaGetErrorString(e));
        kernels += 1;
        done += (uint32_t)m;
    }
    TM_OP_END(kernels);
}

}  // namespace

extern "C" {

int tm_cuda_f16_gemv(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t rows, uint32_t cols,
                     char *err, size_t err_cap) {
    TM_ENTER();
    return f16_common(ctx, w, x, y, rows, cols, 1, 0, 0, TM_CUDA_PRO_NONE, nullptr, 0.0f, TM_CUDA_EPI_STORE, "f16_gemv", err,
                      err_cap);
}

int tm_cuda_f16_gemm(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t rows, uint32_t cols,
                     uint32_t batch, uint32_t x_off, uint32_t y_off, char *err, size_t err_cap) {
    TM_ENTER();
    return f16_common(ctx, w, x, y, rows, cols, batch, x_off, y_off, TM_CUDA_PRO_NONE, nullptr, 0.0f, TM_CUDA_EPI_STORE,
                      "f16_gemm", err, err_cap);
}

int tm_cuda_f16_gemv_fused(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t rows,
                           uint32_t cols, int prologue, tm_cuda_buffer *pro, float eps, int epilogue, char *err,
                           size_t err_cap) {
    TM_ENTER();
    return f16_common(ctx, w, x, y, rows, cols, 1, 0, 0, prologue, pro, eps, epilogue, "f16_gemv_fused", err, err_cap);
}

int tm_cuda_f16_row_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *out, uint32_t row, uint32_t cols,
                        uint32_t out_off, char *err, size_t err_cap) {
    TM_ENTER();
    if (cols == 0) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "F16 row of zero columns");
    TM_CHECK_BUF(w, ((size_t)row + 1) * cols * 2, "F16 weights");
    TM_CHECK_BUF(out, ((size_t)out_off + cols) * 4, "row output");
    TM_OP_BEGIN("f16_row");
    f16_row_kernel<<<(cols + 255) / 256, 256, 0, ctx->stream>>>((const __half *)w->dev, cols, row,
                                                                 (float *)out->dev + out_off);
    TM_OP_END(1);
}

int tm_cuda_f16_row_indirect_f32_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows, uint32_t cols, tm_cuda_buffer *ids,
                                     uint32_t base, tm_cuda_buffer *pos_buf, uint32_t pos_index, int32_t bias, float scale,
                                     tm_cuda_buffer *out, char *err, size_t err_cap) {
    TM_ENTER();
    if (rows == 0 || cols == 0) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "F16 geometry %u x %u", rows, cols);
    TM_CHECK_BUF(w, (size_t)rows * cols * 2, "F16 weights");
    TM_CHECK_BUF(ids, ((size_t)base + 1) * 4, "token ids");
    TM_CHECK_BUF(out, (size_t)cols * 4, "row output");
    const uint32_t *pos = nullptr;
    if (pos_buf) {
        TM_CHECK_BUF(pos_buf, ((size_t)pos_index + 1) * 4, "position");
        pos = (const uint32_t *)pos_buf->dev + pos_index;
    }
    TM_OP_BEGIN("f16_row_indirect");
    TM_CUDA_TRY(tm_launch_pdl(ctx, f16_row_indirect_kernel, dim3((cols + 255) / 256), dim3(256), 0, (const __half *)w->dev,
                              rows, cols, (const uint32_t *)ids->dev, base, pos, (int)bias, (uint32_t)(ids->len / 4), scale,
                              (float *)out->dev));
    TM_OP_END(1);
}

int tm_cuda_f16_rows_indirect_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows, uint32_t cols, tm_cuda_buffer *ids,
                                  uint32_t first, uint32_t n, float scale, tm_cuda_buffer *out, char *err, size_t err_cap) {
    TM_ENTER();
    if (rows == 0 || cols == 0) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "F16 geometry %u x %u", rows, cols);
    if (n == 0 || n > 65535u) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "row count %u outside 1..65535", n);
    TM_CHECK_BUF(w, (size_t)rows * cols * 2, "F16 weights");
    TM_CHECK_BUF(ids, ((size_t)first + n) * 4, "token ids");
    TM_CHECK_BUF(out, (size_t)n * cols * 4, "rows output");
    TM_OP_BEGIN("f16_rows_indirect");
    f16_rows_gather_kernel<<<dim3((cols + 255) / 256, n), 256, 0, ctx->stream>>>(
        (const __half *)w->dev, rows, cols, (const uint32_t *)ids->dev, first, scale, (float *)out->dev);
    TM_OP_END(1);
}

}  // extern "C"
