// Q8_0 weights: plane repacking, the decode GEMV / exact batched GEMM, and the
// embedding-row dequantisers.
//
// Arithmetic contract (the reference's device GEMV, native/metal/kernels.metal:
// 72-118, and its batched twin :434-476): y[r] = sum over blocks of
// d_{r,b} * sum_l q_{r,b,l} * x[32b+l], f32 throughout, reduction order free
// (tolerance-registered against the scalar CPU order, crates/tuckcore/src/
// kernels.rs:186-204).  The design is not the Metal kernel's: weights sit in two
// planes so a lane fetches 16 quants with one 128-bit load, the activations are
// staged once per CTA in shared memory in a lane-major permutation (conflict
// free 128-bit reads), each warp owns whole rows, and row sums finish with a
// multi-value shuffle butterfly.  The lane -> column mapping and the butterfly
// order are the same for every tile shape and batch, so a (row, token) result
// is bit-identical whichever configuration computed it.
#include "tm_cuda_internal.cuh"
#include "tm_cuda_device.cuh"

namespace {

constexpr int kThreads = tmdev::kThreads;  // 8 warps per CTA
constexpr int kWarps = tmdev::kWarps;
using tmdev::block_sumsq;
using tmdev::silu_f;
using tmdev::gelu_tanh_f;
constexpr int kGroupCols = 512;  // one warp-wide 128-bit load of quants

__device__ __forceinline__ int4 ldg_stream(const int4 *p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Four signed bytes of `w` as floats (exact).
__device__ __forceinline__ void unpack4(int w, float &a, float &b, float &c, float &d) {
    a = (float)(signed char)(w);
    b = (float)(signed char)(w >> 8);
    c = (float)(signed char)(w >> 16);
    d = (float)(w >> 24);
}

// Shared-memory slot of column c of one token: group-major, then the four
// 4-float pieces of every lane interleaved so lanes read consecutive float4s.
__device__ __forceinline__ uint32_t x_slot(uint32_t c) {
    const uint32_t g = c / kGroupCols, w = c % kGroupCols;
    const uint32_t lane = w >> 4, piece = (w >> 2) & 3u, e = w & 3u;
    return g * kGroupCols + ((piece * 32u + lane) << 2) + e;
}

// Reduce R per-lane row partials across the warp.  Pairing order is lane bit
// 4,3,2,1,0 for every R; on return lane `row_lane(s)` holds row slot s.
template <int R>
__device__ __forceinline__ float reduce_rows(float (&a)[R], int lane) {
    float v;
    if (R == 4) {
        const bool hi = lane & 16;
        float k0 = hi ? a[2] : a[0], k1 = hi ? a[3] : a[1];
        const float s0 = hi ? a[0] : a[2], s1 = hi ? a[1] : a[3];
        k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
        k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
        const bool hi2 = lane & 8;
        v = hi2 ? k1 : k0;
        const float s = hi2 ? k0 : k1;
        v += __shfl_xor_sync(0xffffffffu, s, 8);
    } else if (R == 2) {
        const bool hi = lane & 16;
        v = hi ? a[1] : a[0];
        const float s = hi ? a[0] : a[1];
        v += __shfl_xor_sync(0xffffffffu, s, 16);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
    } else {
        v = a[0];
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
    }
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v;
}

struct gemv_args {
    const signed char *q;   // [rows][cols]
    const __half *d;        // [rows][cols/32]
    const float *x;         // [M][cols] (token stride = cols)
    float *y;               // [M][rows] (token stride = rows)
    const float *pro;       // norm weight [cols] or the `up` operand [M][cols]
    uint32_t rows, cols;
    float eps;
    int prologue, epilogue;
};

// M tokens, R rows per warp step.
template <int M, int R>
__global__ void __launch_bounds__(kThreads) q8_gemv_kernel(const gemv_args a) {
    extern __shared__ __align__(16) float xs[];  // [M][colsPad], permuted
    __shared__ float red[kWarps];
    const uint32_t cols = a.cols, rows = a.rows;
    const uint32_t cols_pad = (cols + kGroupCols - 1) / kGroupCols * kGroupCols;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // ---- stage the activations (with the folded elementwise operator) ----
#pragma unroll 1
    for (int m = 0; m < M; ++m) {
        const float *xm = a.x + (size_t)m * cols;
        float *dst = xs + (size_t)m * cols_pad;
        if (a.prologue == TM_CUDA_PRO_RMSNORM) {
            const float ss = block_sumsq(xm, cols, red);
            const float inv = 1.0f / sqrtf(ss / (float)cols + a.eps);
            for (uint32_t c = threadIdx.x; c < cols; c += kThreads)
                dst[x_slot(c)] = xm[c] * inv * a.pro[c];
        } else if (a.prologue == TM_CUDA_PRO_SILU_MUL) {
            const float *um = a.pro + (size_t)m * cols;
            for (uint32_t c = threadIdx.x; c < cols; c += kThreads)
                dst[x_slot(c)] = silu_f(xm[c]) * um[c];
        } else if (a.prologue == TM_CUDA_PRO_GELU_MUL) {
            const float *um = a.pro + (size_t)m * cols;
            for (uint32_t c = threadIdx.x; c < cols; c += kThreads)
                dst[x_slot(c)] = gelu_tanh_f(xm[c]) * um[c];
        } else {
            for (uint32_t c = threadIdx.x; c < cols; c += kThreads) dst[x_slot(c)] = xm[c];
        }
    }
    __syncthreads();

    const uint32_t nb = cols / 32u;
    const uint32_t groups = cols_pad / kGroupCols;
    const uint32_t steps = (rows + R - 1) / R;  // row tiles of R rows
    for (uint32_t t = blockIdx.x * kWarps + warp; t < steps; t += gridDim.x * kWarps) {
        const uint32_t r0 = t * R;
        float acc[M][R];
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
            for (int r = 0; r < R; ++r) acc[m][r] = 0.0f;

#pragma unroll 2
        for (uint32_t g = 0; g < groups; ++g) {
            const uint32_t c0 = g * kGroupCols + lane * 16u;
            if (c0 < cols) {
                int4 qv[R];
                float dv[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint32_t row = min(r0 + r, rows - 1u);
                    qv[r] = ldg_stream((const int4 *)(a.q + (size_t)row * cols + c0));
                    dv[r] = __half2float(__ldg(a.d + (size_t)row * nb + (c0 >> 5)));
                }
                float part[M][R];
#pragma unroll
                for (int m = 0; m < M; ++m)
#pragma unroll
                    for (int r = 0; r < R; ++r) part[m][r] = 0.0f;
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    float w[R][4];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const int word = p == 0 ? qv[r].x : p == 1 ? qv[r].y : p == 2 ? qv[r].z : qv[r].w;
                        unpack4(word, w[r][0], w[r][1], w[r][2], w[r][3]);
                    }
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        const float4 xv = *(const float4 *)(xs + (size_t)m * cols_pad +
                                                            g * kGroupCols + ((p * 32 + lane) << 2));
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            float s = part[m][r];
                            s = fmaf(w[r][0], xv.x, s);
                            s = fmaf(w[r][1], xv.y, s);
                            s = fmaf(w[r][2], xv.z, s);
                            s = fmaf(w[r][3], xv.w, s);
                            part[m][r] = s;
                        }
                    }
                }
#pragma unroll
                for (int m = 0; m < M; ++m)
#pragma unroll
                    for (int r = 0; r < R; ++r) acc[m][r] = fmaf(dv[r], part[m][r], acc[m][r]);
            }
        }
        // ---- finish the rows ----
        const int slot = R == 4 ? (((lane >> 4) & 1) * 2 + ((lane >> 3) & 1)) : R == 2 ? ((lane >> 4) & 1) : 0;
        const bool writer = R == 4 ? (lane & 7) == 0 : R == 2 ? (lane & 15) == 0 : lane == 0;
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const float v = reduce_rows<R>(acc[m], lane);
            const uint32_t row = r0 + slot;
            if (writer && row < rows) {
                float *yp = a.y + (size_t)m * rows + row;
                *yp = a.epilogue == TM_CUDA_EPI_ADD ? *yp + v : v;
            }
        }
    }
}

template <int M, int R>
cudaError_t launch_gemv(tm_cuda_ctx *ctx, const gemv_args &a, int grid, size_t smem) {
    static bool attr_set[16] = {};  // per device
    if (ctx->device < 16 && !attr_set[ctx->device]) {
        cudaError_t e = cudaFuncSetAttribute(q8_gemv_kernel<M, R>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)ctx->smem_optin - 1024);
        if (e != cudaSuccess) return e;
        attr_set[ctx->device] = true;
    }
    q8_gemv_kernel<M, R><<<grid, kThreads, smem, ctx->stream>>>(a);
    return cudaGetLastError();
}

template <int M>
cudaError_t launch_gemv_r(tm_cuda_ctx *ctx, const gemv_args &a, int R, int grid, size_t smem) {
    switch (R) {
        case 4: return launch_gemv<M, 4>(ctx, a, grid, smem);
        case 2: return launch_gemv<M, 2>(ctx, a, grid, smem);
        default: return launch_gemv<M, 1>(ctx, a, grid, smem);
    }
}

// One launch for `m` tokens (m in {1,2,4,8}); picks the row tile from the
// matrix height so small projections still fill the machine.
cudaError_t gemv_slice(tm_cuda_ctx *ctx, gemv_args a, int m) {
    const size_t cols_pad = tm_round_up(a.cols, kGroupCols);
    const size_t smem = (size_t)m * cols_pad * sizeof(float);
    const uint32_t target = (uint32_t)ctx->sm_count * 2u * kWarps;  // warps wanted in flight
    int R = 4;
    if (m >= 8) R = 2;
    while (R > 1 && (a.rows + R - 1) / R < target) R >>= 1;
    const uint32_t steps = (a.rows + R - 1) / R;
    uint32_t ctas = (steps + kWarps - 1) / kWarps;
    const uint32_t max_ctas = (uint32_t)ctx->sm_count * (smem > 48 * 1024 ? 2u : 8u);
    if (ctas > max_ctas) ctas = max_ctas;
    switch (m) {
        case 8: return launch_gemv_r<8>(ctx, a, R, (int)ctas, smem);
        case 4: return launch_gemv_r<4>(ctx, a, R, (int)ctas, smem);
        case 2: return launch_gemv_r<2>(ctx, a, R, (int)ctas, smem);
        default: return launch_gemv_r<1>(ctx, a, R, (int)ctas, smem);
    }
}

// Whole batch in slices of 8/4/2/1 tokens that fit shared memory.
int gemv_batch(tm_cuda_ctx *ctx, gemv_args a, uint32_t batch, uint64_t *kernels, char *err,
               size_t err_cap) {
    const size_t cols_pad = tm_round_up(a.cols, kGroupCols);
    const size_t budget = ctx->smem_optin - 2048;
    if (cols_pad * sizeof(float) > budget)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "cols %u exceeds the %zu-float activation stage of one CTA", a.cols,
                       budget / sizeof(float));
    uint32_t done = 0;
    while (done < batch) {
        int m = 8;
        while (m > 1 && ((uint32_t)m > batch - done || (size_t)m * cols_pad * sizeof(float) > budget))
            m >>= 1;
        gemv_args s = a;
        s.x = a.x + (size_t)done * a.cols;
        s.y = a.y + (size_t)done * a.rows;
        if (a.prologue == TM_CUDA_PRO_SILU_MUL || a.prologue == TM_CUDA_PRO_GELU_MUL)
            s.pro = a.pro + (size_t)done * a.cols;
        cudaError_t e = gemv_slice(ctx, s, m);
        if (e != cudaSuccess)
            return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "Q8_0 GEMV launch failed: %s",
                           cudaGetErrorString(e));
        *kernels += 1;
        done += (uint32_t)m;
    }
    return TM_CUDA_OK;
}

// ---- repacking --------------------------------------------------------------

// One thread per (row, block): 34 raw bytes -> 32 quants + 1 scale.
__global__ void q8_pack_kernel(const unsigned char *raw, signed char *q, __half *d, uint32_t cols,
                               uint32_t row0, uint32_t nrows) {
    const uint32_t nb = cols / 32u;
    const size_t total = (size_t)nrows * nb;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / nb), b = (uint32_t)(i % nb);
        const unsigned short *src = (const unsigned short *)(raw + i * 34);  // 2-byte aligned
        unsigned short h[17];
#pragma unroll
        for (int k = 0; k < 17; ++k) h[k] = src[k];
        ((unsigned short *)d)[(size_t)(row0 + r) * nb + b] = h[0];
        uint32_t *dst = (uint32_t *)(q + (size_t)(row0 + r) * cols + (size_t)b * 32);
#pragma unroll
        for (int k = 0; k < 8; ++k) dst[k] = (uint32_t)h[1 + 2 * k] | ((uint32_t)h[2 + 2 * k] << 16);
    }
}

__global__ void q8_unpack_kernel(unsigned char *raw, const signed char *q, const __half *d,
                                 uint32_t cols, uint32_t row0, uint32_t nrows) {
    const uint32_t nb = cols / 32u;
    const size_t total = (size_t)nrows * nb;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / nb), b = (uint32_t)(i % nb);
        unsigned short *dst = (unsigned short *)(raw + i * 34);
        dst[0] = ((const unsigned short *)d)[(size_t)(row0 + r) * nb + b];
        const unsigned short *src = (const unsigned short *)(q + (size_t)(row0 + r) * cols + (size_t)b * 32);
#pragma unroll
        for (int k = 0; k < 16; ++k) dst[1 + k] = src[k];
    }
}

// out[c] = d(row, c/32) * q(row, c), c < cols; row < 0 writes zeros.
__device__ __forceinline__ void dequant_row(const signed char *q, const __half *d, uint32_t cols,
                                            long row, float scale, float *out) {
    const uint32_t nb = cols / 32u;
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x) {
        float v = 0.0f;
        if (row >= 0) {
            v = __half2float(d[(size_t)row * nb + c / 32u]) * (float)q[(size_t)row * cols + c];
            if (scale != 0.0f) v *= scale;
        }
        out[c] = v;
    }
}

__global__ void q8_row_kernel(const signed char *q, const __half *d, uint32_t cols, uint32_t row,
                              float *out) {
    dequant_row(q, d, cols, (long)row, 0.0f, out);
}

__global__ void q8_row_indirect_kernel(const signed char *q, const __half *d, uint32_t rows,
                                       uint32_t cols, const uint32_t *ids, uint32_t slot,
                                       const uint32_t *pos, int bias, uint32_t ids_len, float scale,
                                       float *out) {
    uint32_t s = slot;
    if (pos) s = slot + *pos + (uint32_t)bias;
    long row = -1;
    if (s < ids_len) {
        const uint32_t id = ids[s];
        if (id < rows) row = (long)id;
    }
    dequant_row(q, d, cols, row, scale, out);
}

}  // namespace

extern "C" {

size_t tm_cuda_q8_0_packed_bytes(uint32_t rows, uint32_t cols) {
    if (rows == 0 || cols == 0 || cols % 32 != 0) return 0;
    return tm_q8_qplane_bytes(rows, cols) + (size_t)rows * (cols / 32) * 2;
}

int tm_cuda_q8_0_pack(tm_cuda_ctx *ctx, tm_cuda_buffer *dst, uint32_t rows, uint32_t cols,
                      tm_cuda_buffer *raw, size_t raw_off, uint32_t row0, uint32_t nrows,
                      char *err, size_t err_cap) {
    TM_ENTER();
    if (rows == 0 || cols == 0 || cols % 32 != 0 || nrows == 0 || row0 >= rows || nrows > rows - row0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "pack of rows [%u, +%u) of a %u x %u Q8_0 matrix is out of range", row0, nrows,
                       rows, cols);
    if (raw_off % 2 != 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "raw offset must be even");
    TM_CHECK_BUF(dst, tm_cuda_q8_0_packed_bytes(rows, cols), "packed matrix");
    TM_CHECK_BUF(raw, raw_off + (size_t)nrows * (cols / 32) * 34, "raw rows");
    if (dst->parent)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "a packed matrix must own its buffer");
    if (dst->layout == TM_LAYOUT_Q8_0_PACKED && (dst->rows != rows || dst->cols != cols))
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "buffer already holds a packed %u x %u matrix", dst->rows, dst->cols);
    TM_OP_BEGIN("q8_0_pack");
    const size_t total = (size_t)nrows * (cols / 32);
    const int grid = (int)((total + 255) / 256 > 65535 ? 65535 : (total + 255) / 256);
    q8_pack_kernel<<<grid, 256, 0, ctx->stream>>>(
        raw->dev + raw_off, (signed char *)dst->dev,
        (__half *)(dst->dev + tm_q8_qplane_bytes(rows, cols)), cols, row0, nrows);
    dst->layout = TM_LAYOUT_Q8_0_PACKED;
    dst->rows = rows;
    dst->cols = cols;
    TM_OP_END(1);
}

int tm_cuda_q8_0_unpack(tm_cuda_ctx *ctx, tm_cuda_buffer *src, uint32_t rows, uint32_t cols,
                        tm_cuda_buffer *raw, size_t raw_off, uint32_t row0, uint32_t nrows,
                        char *err, size_t err_cap) {
    TM_ENTER();
    int rc = tm_check_packed(ctx, src, rows, cols, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    if (nrows == 0 || row0 >= rows || nrows > rows - row0 || raw_off % 2 != 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "unpack row range out of bounds");
    TM_CHECK_BUF(raw, raw_off + (size_t)nrows * (cols / 32) * 34, "raw rows");
    TM_OP_BEGIN("q8_0_unpack");
    const size_t total = (size_t)nrows * (cols / 32);
    const int grid = (int)((total + 255) / 256 > 65535 ? 65535 : (total + 255) / 256);
    q8_unpack_kernel<<<grid, 256, 0, ctx->stream>>>(
        raw->dev + raw_off, (const signed char *)src->dev,
        (const __half *)(src->dev + tm_q8_qplane_bytes(rows, cols)), cols, row0, nrows);
    TM_OP_END(1);
}

static int gemv_common(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y,
                       uint32_t rows, uint32_t cols, uint32_t batch, uint32_t x_off, uint32_t y_off,
                       int prologue, tm_cuda_buffer *pro, float eps, int epilogue, const char *label,
                       char *err, size_t err_cap) {
    int rc = tm_check_packed(ctx, w, rows, cols, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    if (batch == 0 || batch > TM_CUDA_GEMM_MAX_BATCH)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "batch %u outside 1..%u", batch,
                       TM_CUDA_GEMM_MAX_BATCH);
    TM_CHECK_BUF(x, ((size_t)x_off + (size_t)batch * cols) * 4, "activation");
    TM_CHECK_BUF(y, ((size_t)y_off + (size_t)batch * rows) * 4, "output");
    if (prologue < TM_CUDA_PRO_NONE || prologue > TM_CUDA_PRO_GELU_MUL ||
        (epilogue != TM_CUDA_EPI_STORE && epilogue != TM_CUDA_EPI_ADD))
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "unknown prologue/epilogue");
    if (prologue == TM_CUDA_PRO_RMSNORM) TM_CHECK_BUF(pro, (size_t)cols * 4, "norm weight");
    if (prologue == TM_CUDA_PRO_SILU_MUL || prologue == TM_CUDA_PRO_GELU_MUL)
        TM_CHECK_BUF(pro, (size_t)batch * cols * 4, "gate multiplicand");
    gemv_args a;
    a.q = (const signed char *)w->dev;
    a.d = (const __half *)(w->dev + tm_q8_qplane_bytes(rows, cols));
    a.x = (const float *)x->dev + x_off;
    a.y = (float *)y->dev + y_off;
    a.pro = pro ? (const float *)pro->dev : nullptr;
    a.rows = rows;
    a.cols = cols;
    a.eps = eps;
    a.prologue = prologue;
    a.epilogue = epilogue;
    TM_OP_BEGIN(label);
    uint64_t kernels = 0;
    rc = gemv_batch(ctx, a, batch, &kernels, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    TM_OP_END(kernels);
}

int tm_cuda_q8_0_gemv(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y,
                      uint32_t rows, uint32_t cols, char *err, size_t err_cap) {
    TM_ENTER();
    return gemv_common(ctx, w, x, y, rows, cols, 1, 0, 0, TM_CUDA_PRO_NONE, nullptr, 0.0f,
                       TM_CUDA_EPI_STORE, "q8_0_gemv", err, err_cap);
}

int tm_cuda_q8_0_gemm(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y,
                      uint32_t rows, uint32_t cols, uint32_t batch, uint32_t x_off, uint32_t y_off,
                      char *err, size_t err_cap) {
    TM_ENTER();
    return gemv_common(ctx, w, x, y, rows, cols, batch, x_off, y_off, TM_CUDA_PRO_NONE, nullptr,
                       0.0f, TM_CUDA_EPI_STORE, "q8_0_gemm", err, err_cap);
}

int tm_cuda_q8_0_gemv_fused(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x,
                            tm_cuda_buffer *y, uint32_t rows, uint32_t cols, int prologue,
                            tm_cuda_buffer *pro, float eps, int epilogue, char *err,
                            size_t err_cap) {
    TM_ENTER();
    return gemv_common(ctx, w, x, y, rows, cols, 1, 0, 0, prologue, pro, eps, epilogue,
                       "q8_0_gemv_fused", err, err_cap);
}

int tm_cuda_q8_0_row_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *out, uint32_t row,
                         uint32_t cols, uint32_t out_off, char *err, size_t err_cap) {
    TM_ENTER();
    if (!w || ctx->live.find(w) == ctx->live.end() || w->layout != TM_LAYOUT_Q8_0_PACKED ||
        w->cols != cols)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "weight buffer is not a packed Q8_0 matrix of %u columns", cols);
    if (row >= w->rows)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "row %u outside the %u rows", row, w->rows);
    TM_CHECK_BUF(out, ((size_t)out_off + cols) * 4, "row output");
    TM_OP_BEGIN("q8_0_row");
    q8_row_kernel<<<(cols + 255) / 256, 256, 0, ctx->stream>>>(
        (const signed char *)w->dev, (const __half *)(w->dev + tm_q8_qplane_bytes(w->rows, cols)),
        cols, row, (float *)out->dev + out_off);
    TM_OP_END(1);
}

static int row_indirect(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows, uint32_t cols,
                        tm_cuda_buffer *ids, uint32_t slot, tm_cuda_buffer *pos_buf,
                        uint32_t pos_index, int32_t bias, float scale, tm_cuda_buffer *out,
                        char *err, size_t err_cap) {
    int rc = tm_check_packed(ctx, w, rows, cols, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    TM_CHECK_BUF(ids, ((size_t)slot + 1) * 4, "token ids");
    TM_CHECK_BUF(out, (size_t)cols * 4, "row output");
    const uint32_t *pos = nullptr;
    if (pos_buf) {
        TM_CHECK_BUF(pos_buf, ((size_t)pos_index + 1) * 4, "position");
        pos = (const uint32_t *)pos_buf->dev + pos_index;
    }
    TM_OP_BEGIN("row_indirect");
    q8_row_indirect_kernel<<<(cols + 255) / 256, 256, 0, ctx->stream>>>(
        (const signed char *)w->dev, (const __half *)(w->dev + tm_q8_qplane_bytes(rows, cols)), rows,
        cols, (const uint32_t *)ids->dev, slot, pos, bias, (uint32_t)(ids->len / 4), scale,
        (float *)out->dev);
    TM_OP_END(1);
}

int tm_cuda_row_indirect_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t type_id, uint32_t rows,
                             uint32_t cols, tm_cuda_buffer *ids, uint32_t slot,
                             tm_cuda_buffer *out, char *err, size_t err_cap) {
    TM_ENTER();
    if (type_id != 8)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "row_indirect supports Q8_0 (type 8) matrices; got type %u", type_id);
    return row_indirect(ctx, w, rows, cols, ids, slot, nullptr, 0, 0, 0.0f, out, err, err_cap);
}

int tm_cuda_row_indirect_f32_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows, uint32_t cols,
                                 tm_cuda_buffer *ids, uint32_t base, tm_cuda_buffer *pos_buf,
                                 uint32_t pos_index, int32_t bias, float scale,
                                 tm_cuda_buffer *out, char *err, size_t err_cap) {
    TM_ENTER();
    if (!pos_buf) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "null position buffer");
    return row_indirect(ctx, w, rows, cols, ids, base, pos_buf, pos_index, bias, scale, out, err,
                        err_cap);
}

}  // extern "C"
