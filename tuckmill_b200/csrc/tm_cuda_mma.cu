// Tensor-core prefill GEMM (placeholder body: exact slices until the tcgen05
// kernel lands in this file).
#include "tm_cuda_internal.cuh"

extern "C" int tm_cuda_q8_0_gemm_mma(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x,
                                     tm_cuda_buffer *y, uint32_t rows, uint32_t cols, uint32_t batch,
                                     uint32_t x_off, uint32_t y_off, char *err, size_t err_cap) {
    if (batch == 0 || batch > TM_CUDA_GEMM_MMA_MAX_BATCH)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "batch %u outside 1..%u", batch,
                       TM_CUDA_GEMM_MMA_MAX_BATCH);
    for (uint32_t t0 = 0; t0 < batch; t0 += TM_CUDA_GEMM_MAX_BATCH) {
        const uint32_t n = batch - t0 < TM_CUDA_GEMM_MAX_BATCH ? batch - t0 : TM_CUDA_GEMM_MAX_BATCH;
        int rc = tm_cuda_q8_0_gemm(ctx, w, x, y, rows, cols, n, x_off + t0 * cols, y_off + t0 * rows,
                                   err, err_cap);
        if (rc != TM_CUDA_OK) return rc;
    }
    return TM_CUDA_OK;
}
