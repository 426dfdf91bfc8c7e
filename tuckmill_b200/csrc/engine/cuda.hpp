// RAII wrapper over the tm_cuda C ABI: the C++ twin of the reference's device
// wrapper crate (crates/metal/src/lib.rs:695-2650 -- MetalContext with one method
// per operator, MetalBuffer handles freed on drop, ABI codes mapped to typed
// errors :732-747).  Header-only; calls nothing but the C ABI.
#pragma once
#include <initializer_list>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "error.hpp"
#include "tm_cuda.h"

namespace tuckmill {

inline void cuda_check(int rc, const char *err) {
    if (rc == TM_CUDA_OK) return;
    ErrorCode code = ErrorCode::Internal;
    if (rc == TM_CUDA_ERR_NO_DEVICE) code = ErrorCode::Unavailable;
    else if (rc == TM_CUDA_ERR_ALLOC) code = ErrorCode::ModelExceedsBudget;
    throw TuckmillError(code, std::string("cuda device call failed (") + std::to_string(rc) + "): " + err);
}

class CudaContext;

class CudaBuffer {
public:
    CudaBuffer() = default;
    CudaBuffer(tm_cuda_ctx *ctx, tm_cuda_buffer *h) : ctx_(ctx), h_(h) {}
    CudaBuffer(const CudaBuffer &) = delete;
    CudaBuffer &operator=(const CudaBuffer &) = delete;
    CudaBuffer(CudaBuffer &&o) noexcept : ctx_(o.ctx_), h_(o.h_) { o.h_ = nullptr; }
    CudaBuffer &operator=(CudaBuffer &&o) noexcept {
        if (this != &o) {
            reset();
            ctx_ = o.ctx_;
            h_ = o.h_;
            o.h_ = nullptr;
        }
        return *this;
    }
    ~CudaBuffer() { reset(); }
    void reset() {
        if (h_) tm_cuda_buffer_free(ctx_, h_);
        h_ = nullptr;
    }
    explicit operator bool() const { return h_ != nullptr; }
    tm_cuda_buffer *raw() const { return h_; }
    size_t len() const { return h_ ? tm_cuda_buffer_len(ctx_, h_) : 0; }
    void *contents() const { return tm_cuda_buffer_contents(ctx_, h_); }
    void zero(size_t off, size_t n) const {
        char e[256] = "";
        cuda_check(tm_cuda_buffer_zero(ctx_, h_, off, n, e, sizeof e), e);
    }
    void zero() const { zero(0, len()); }
    void upload(size_t off, const void *src, size_t n) const {
        char e[256] = "";
        cuda_check(tm_cuda_upload(ctx_, h_, off, src, n, e, sizeof e), e);
    }
    void download(size_t off, void *dst, size_t n) const {
        char e[256] = "";
        cuda_check(tm_cuda_download(ctx_, h_, off, dst, n, e, sizeof e), e);
    }
    void download_after(size_t off, void *dst, size_t n, uint64_t target) const {
        char e[256] = "";
        cuda_check(tm_cuda_download_after(ctx_, h_, off, dst, n, target, e, sizeof e), e);
    }
    CudaBuffer view(size_t off, size_t n) const {
        char e[256] = "";
        tm_cuda_buffer *v = tm_cuda_buffer_view(ctx_, h_, off, n, e, sizeof e);
        if (!v) throw TuckmillError(ErrorCode::Internal, std::string("buffer view failed: ") + e);
        return CudaBuffer(ctx_, v);
    }

private:
    tm_cuda_ctx *ctx_ = nullptr;
    tm_cuda_buffer *h_ = nullptr;
};

class CudaGraph {
public:
    CudaGraph() = default;
    CudaGraph(tm_cuda_ctx *ctx, tm_cuda_graph *g) : ctx_(ctx), g_(g) {}
    CudaGraph(const CudaGraph &) = delete;
    CudaGraph &operator=(const CudaGraph &) = delete;
    CudaGraph(CudaGraph &&o) noexcept : ctx_(o.ctx_), g_(o.g_) { o.g_ = nullptr; }
    CudaGraph &operator=(CudaGraph &&o) noexcept {
        if (this != &o) {
            reset();
            ctx_ = o.ctx_;
            g_ = o.g_;
            o.g_ = nullptr;
        }
        return *this;
    }
    ~CudaGraph() { reset(); }
    void reset() {
        if (g_) tm_cuda_graph_free(ctx_, g_);
        g_ = nullptr;
    }
    explicit operator bool() const { return g_ != nullptr; }
    tm_cuda_graph *raw() const { return g_; }
    void launch() const {
        char e[256] = "";
        cuda_check(tm_cuda_graph_launch(ctx_, g_, e, sizeof e), e);
    }

private:
    tm_cuda_ctx *ctx_ = nullptr;
    tm_cuda_graph *g_ = nullptr;
};

#define TM_CALL(fn, ...)                                          \
    do {                                                          \
        char e_[256] = "";                                        \
        cuda_check(fn(ctx_, __VA_ARGS__, e_, sizeof e_), e_);     \
    } while (0)

class CudaContext {
public:
    explicit CudaContext(int device) {
        char e[256] = "";
        ctx_ = tm_cuda_create(device, e, sizeof e);
        if (!ctx_)
            throw TuckmillError(ErrorCode::Unavailable,
                                std::string("the CUDA kernel implementation is unavailable: ") + e,
                                "Select --kernels auto, neon, or scalar on this machine.");
    }
    CudaContext(const CudaContext &) = delete;
    CudaContext &operator=(const CudaContext &) = delete;
    ~CudaContext() { tm_cuda_destroy(ctx_); }
    tm_cuda_ctx *raw() const { return ctx_; }

    CudaBuffer buffer(size_t bytes, bool shared = false) const {
        char e[256] = "";
        tm_cuda_buffer *b = tm_cuda_buffer_new(ctx_, bytes, shared ? 1 : 0, e, sizeof e);
        if (!b) throw TuckmillError(ErrorCode::ModelExceedsBudget, std::string("device allocation failed: ") + e);
        return CudaBuffer(ctx_, b);
    }
    CudaBuffer zeros(size_t bytes, bool shared = false) const {
        CudaBuffer b = buffer(bytes, shared);
        b.zero();
        return b;
    }
    // A zeroed exchange buffer mapped on every rank of the communicator (collective).
    CudaBuffer symm_zeros(size_t bytes) const {
        char e[256] = "";
        tm_cuda_buffer *b = tm_cuda_symm_alloc(ctx_, bytes, e, sizeof e);
        if (!b) throw TuckmillError(ErrorCode::Unavailable, std::string("peer-memory exchange buffer: ") + e,
                                    "The GPUs of a row split must be able to map one another's memory (CUDA IPC, peer access).");
        return CudaBuffer(ctx_, b);
    }
    CudaBuffer floats(const std::vector<float> &v) const {
        CudaBuffer b = buffer(v.size() * 4);
        b.upload(0, v.data(), v.size() * 4);
        return b;
    }
    CudaBuffer row_view(const CudaBuffer &w, uint32_t rows, uint32_t cols, uint32_t row0, uint32_t nrows) const {
        char e[256] = "";
        tm_cuda_buffer *v = tm_cuda_q8_0_row_view(ctx_, w.raw(), rows, cols, row0, nrows, e, sizeof e);
        if (!v) throw TuckmillError(ErrorCode::Internal, std::string("row view failed: ") + e);
        return CudaBuffer(ctx_, v);
    }

    // ---- operators: names and argument order of crates/metal/src/lib.rs ----
    void q8_0_pack(const CudaBuffer &dst, uint32_t rows, uint32_t cols, const CudaBuffer &raw, size_t raw_off,
                   uint32_t row0, uint32_t nrows) const {
        TM_CALL(tm_cuda_q8_0_pack, dst.raw(), rows, cols, raw.raw(), raw_off, row0, nrows);
    }
    void q8_0_gemv(const CudaBuffer &w, const CudaBuffer &x, const CudaBuffer &y, uint32_t rows, uint32_t cols) const {
        TM_CALL(tm_cuda_q8_0_gemv, w.raw(), x.raw(), y.raw(), rows, cols);
    }
    void q8_0_gemv_fused(const CudaBuffer &w, const CudaBuffer &x, const CudaBuffer &y, uint32_t rows,
                         uint32_t cols, int prologue, const CudaBuffer *pro, float eps, int epilogue) const {
        TM_CALL(tm_cuda_q8_0_gemv_fused, w.raw(), x.raw(), y.raw(), rows, cols, prologue,
                pro ? pro->raw() : nullptr, eps, epilogue);
    }
    // F16-weight forms (include/tm_cuda.h): matrices are rows * cols binary16 values, uploaded verbatim.
    void f16_gemv_fused(const CudaBuffer &w, const CudaBuffer &x, const CudaBuffer &y, uint32_t rows, uint32_t cols,
                        int prologue, const CudaBuffer *pro, float eps, int epilogue) const {
        TM_CALL(tm_cuda_f16_gemv_fused, w.raw(), x.raw(), y.raw(), rows, cols, prologue, pro ? pro->raw() : nullptr, eps,
                epilogue);
    }
    void f16_gemm(const CudaBuffer &w, const CudaBuffer &x, const CudaBuffer &y, uint32_t rows, uint32_t cols,
                  uint32_t batch, uint32_t x_off, uint32_t y_off) const {
        TM_CALL(tm_cuda_f16_gemm, w.raw(), x.raw(), y.raw(), rows, cols, batch, x_off, y_off);
    }
    void f16_row_indirect_dev(const CudaBuffer &w, uint32_t rows, uint32_t cols, const CudaBuffer &ids, uint32_t base,
                              const CudaBuffer &pos_buf, uint32_t pos_index, int32_t bias, float scale,
                              const CudaBuffer &out) const {
        TM_CALL(tm_cuda_f16_row_indirect_f32_dev, w.raw(), rows, cols, ids.raw(), base, pos_buf.raw(), pos_index, bias,
                scale, out.raw());
    }
    void f16_rows_indirect(const CudaBuffer &w, uint32_t rows, uint32_t cols, const CudaBuffer &ids, uint32_t first,
                           uint32_t n, float scale, const CudaBuffer &out) const {
        TM_CALL(tm_cuda_f16_rows_indirect_f32, w.raw(), rows, cols, ids.raw(), first, n, scale, out.raw());
    }
    void q8_0_gemm(const CudaBuffer &w, const CudaBuffer &x, const CudaBuffer &y, uint32_t rows, uint32_t cols,
                   uint32_t batch, uint32_t x_off, uint32_t y_off) const {
        TM_CALL(tm_cuda_q8_0_gemm, w.raw(), x.raw(), y.raw(), rows, cols, batch, x_off, y_off);
    }
    void q8_0_gemm_mma(const CudaBuffer &w, const CudaBuffer &x, const CudaBuffer &y, uint32_t rows,
                       uint32_t cols, uint32_t batch, uint32_t x_off, uint32_t y_off) const {
        TM_CALL(tm_cuda_q8_0_gemm_mma, w.raw(), x.raw(), y.raw(), rows, cols, batch, x_off, y_off);
    }
    // One prologue-fused f16 copy + one GEMM launch over up to three row parts (include/tm_cuda.h).
    void q8_0_gemm_mma_fused(const CudaBuffer &w, const CudaBuffer &x, uint32_t rows, uint32_t cols, uint32_t batch,
                             std::initializer_list<const CudaBuffer *> ys, std::initializer_list<uint32_t> part_rows,
                             int prologue, const CudaBuffer *pro, float eps, int epilogue) const {
        tm_cuda_buffer *yp[3] = {nullptr, nullptr, nullptr};
        uint32_t pr[3] = {0, 0, 0};
        uint32_t n = 0;
        for (const CudaBuffer *b : ys) yp[n++] = b->raw();
        n = 0;
        for (uint32_t r : part_rows) pr[n++] = r;
        TM_CALL(tm_cuda_q8_0_gemm_mma_fused, w.raw(), x.raw(), rows, cols, batch, n, yp, pr, prologue,
                pro ? pro->raw() : nullptr, eps, epilogue);
    }
    void qk_prep_chunk(const CudaBuffer &q, const CudaBuffer &k, const CudaBuffer &v, const CudaBuffer &qn,
                       const CudaBuffer &kn, const CudaBuffer &inv_freq, const CudaBuffer &kc, const CudaBuffer &vc,
                       uint32_t heads, uint32_t kvh, uint32_t hd, uint32_t n_rot, uint32_t pos0, uint32_t cap, uint32_t n,
                       float eps) const {
        TM_CALL(tm_cuda_qk_prep_chunk, q.raw(), k.raw(), v.raw(), qn.raw(), kn.raw(), inv_freq.raw(), kc.raw(), vc.raw(),
                heads, kvh, hd, n_rot, pos0, cap, n, eps);
    }
    void mma_workspace_reserve(size_t bytes) const {
        char e[256] = "";
        cuda_check(tm_cuda_mma_workspace_reserve(ctx_, bytes, e, sizeof e), e);
    }
    void q8_0_row(const CudaBuffer &w, const CudaBuffer &out, uint32_t row, uint32_t cols, uint32_t out_off) const {
        TM_CALL(tm_cuda_q8_0_row_f32, w.raw(), out.raw(), row, cols, out_off);
    }
    void rows_indirect(const CudaBuffer &w, uint32_t rows, uint32_t cols, const CudaBuffer &ids, uint32_t first,
                       uint32_t n, float scale, const CudaBuffer &out) const {
        TM_CALL(tm_cuda_rows_indirect_f32, w.raw(), rows, cols, ids.raw(), first, n, scale, out.raw());
    }
    void row_indirect_dev(const CudaBuffer &w, uint32_t rows, uint32_t cols, const CudaBuffer &ids, uint32_t base,
                          const CudaBuffer &pos, uint32_t pos_index, int32_t bias, float scale,
                          const CudaBuffer &out) const {
        TM_CALL(tm_cuda_row_indirect_f32_dev, w.raw(), rows, cols, ids.raw(), base, pos.raw(), pos_index, bias,
                scale, out.raw());
    }
    void rmsnorm_add(const CudaBuffer &p, const CudaBuffer &w, const CudaBuffer &x, uint32_t rows, uint32_t cols,
                     float eps) const {
        TM_CALL(tm_cuda_rmsnorm_add_f32, p.raw(), w.raw(), x.raw(), rows, cols, eps);
    }
    void rmsnorm(const CudaBuffer &x, const CudaBuffer &w, const CudaBuffer &y, uint32_t rows, uint32_t cols,
                 float eps) const {
        TM_CALL(tm_cuda_rmsnorm_f32, x.raw(), w.raw(), y.raw(), rows, cols, eps);
    }
    void silu_mul(const CudaBuffer &g, const CudaBuffer &u, const CudaBuffer &o, uint32_t n) const {
        TM_CALL(tm_cuda_silu_mul_f32, g.raw(), u.raw(), o.raw(), n);
    }
    void gelu_tanh_mul(const CudaBuffer &g, const CudaBuffer &u, const CudaBuffer &o, uint32_t n) const {
        TM_CALL(tm_cuda_gelu_tanh_mul_f32, g.raw(), u.raw(), o.raw(), n);
    }
    void f32_axpy(const CudaBuffer &a, const CudaBuffer &y, float alpha, uint32_t n) const {
        TM_CALL(tm_cuda_f32_axpy, a.raw(), y.raw(), alpha, n);
    }
    void f32_scale(const CudaBuffer &x, const CudaBuffer &y, float f, uint32_t n) const {
        TM_CALL(tm_cuda_f32_scale, x.raw(), y.raw(), f, n);
    }
    void copy_f32(const CudaBuffer &s, uint32_t so, const CudaBuffer &d, uint32_t d_off, uint32_t n) const {
        TM_CALL(tm_cuda_copy_f32, s.raw(), so, d.raw(), d_off, n);
    }
    void argmax_f32(const CudaBuffer &x, uint32_t n, const CudaBuffer &partial, const CudaBuffer &out,
                    uint32_t out_index) const {
        TM_CALL(tm_cuda_argmax_f32, x.raw(), n, partial.raw(), out.raw(), out_index);
    }
    void argmax_dev(const CudaBuffer &x, uint32_t n, const CudaBuffer &partial, const CudaBuffer &out, uint32_t base,
                    const CudaBuffer &pos, uint32_t pos_index, uint32_t out_cap, const CudaBuffer *mirror) const {
        TM_CALL(tm_cuda_argmax_f32_dev, x.raw(), n, partial.raw(), out.raw(), base, pos.raw(), pos_index, out_cap,
                mirror ? mirror->raw() : nullptr);
    }
    void u32_add(const CudaBuffer &b, uint32_t index, uint32_t delta) const {
        TM_CALL(tm_cuda_u32_add, b.raw(), index, delta);
    }
    void rope_partial_chunk(const CudaBuffer &q, const CudaBuffer &k, const CudaBuffer &inv_freq, uint32_t pos0,
                            uint32_t nq, uint32_t nkv, uint32_t hd, uint32_t n_rot, uint32_t n) const {
        TM_CALL(tm_cuda_qwen35_rope_partial_chunk, q.raw(), k.raw(), inv_freq.raw(), pos0, nq, nkv, hd, n_rot, n);
    }
    void kv_store_chunk(const CudaBuffer &ks, const CudaBuffer &vs, const CudaBuffer &kc, const CudaBuffer &vc,
                        uint32_t pos0, uint32_t cap, uint32_t hd, uint32_t kvh, uint32_t n) const {
        TM_CALL(tm_cuda_qwen35_kv_store_f16_chunk, ks.raw(), vs.raw(), kc.raw(), vc.raw(), pos0, cap, hd, kvh, n);
    }
    void attention_chunk(const CudaBuffer &q, const CudaBuffer &kc, const CudaBuffer &vc, const CudaBuffer &out,
                         const CudaBuffer &scratch, uint32_t heads, uint32_t pos0, uint32_t cap, uint32_t hd,
                         uint32_t group, float scale, uint32_t n, uint32_t window) const {
        TM_CALL(tm_cuda_qwen35_attention_f16_chunk, q.raw(), kc.raw(), vc.raw(), out.raw(), scratch.raw(), heads,
                pos0, cap, hd, group, scale, n, window);
    }
    void attention_chunk_mma(const CudaBuffer &q, const CudaBuffer &kc, const CudaBuffer &vc, const CudaBuffer &out,
                             uint32_t heads, uint32_t pos0, uint32_t cap, uint32_t hd, uint32_t group, float scale,
                             uint32_t n, uint32_t window) const {
        TM_CALL(tm_cuda_attention_chunk_mma, q.raw(), kc.raw(), vc.raw(), out.raw(), heads, pos0, cap, hd, group, scale,
                n, window);
    }
    void attention_decode_dev(const CudaBuffer &q, const CudaBuffer &k, const CudaBuffer &v, const CudaBuffer &qn,
                              const CudaBuffer &kn, const CudaBuffer &inv_freq, const CudaBuffer &kc,
                              const CudaBuffer &vc, const CudaBuffer &out, const CudaBuffer &scratch,
                              const CudaBuffer &pos, uint32_t pos_index, const CudaBuffer &status, uint32_t heads,
                              uint32_t kvh, uint32_t hd, uint32_t n_rot, uint32_t cap, uint32_t window, float eps,
                              float scale, bool exact) const {
        TM_CALL(tm_cuda_attention_decode_dev, q.raw(), k.raw(), v.raw(), qn.raw(), kn.raw(), inv_freq.raw(),
                kc.raw(), vc.raw(), out.raw(), scratch.raw(), pos.raw(), pos_index, status.raw(), heads, kvh, hd,
                n_rot, cap, window, eps, scale, exact ? 1 : 0);
    }

    // ---- decode steps of several sequences (include/tm_cuda.h) ----
    void attention_decode_batch(const CudaBuffer &q, const CudaBuffer &k, const CudaBuffer &v, const CudaBuffer &qn,
                                const CudaBuffer &kn, const CudaBuffer &inv_freq, const CudaBuffer &kc,
                                const CudaBuffer &vc, const CudaBuffer &out, const CudaBuffer &scratch,
                                const CudaBuffer &pos, const CudaBuffer &status, uint32_t n_seq, uint32_t q_stride,
                                uint32_t kv_stride, uint32_t heads, uint32_t kvh, uint32_t hd, uint32_t n_rot,
                                uint32_t cap, uint32_t window, float eps, float scale, bool exact) const {
        TM_CALL(tm_cuda_attention_decode_batch_dev, q.raw(), k.raw(), v.raw(), qn.raw(), kn.raw(), inv_freq.raw(),
                kc.raw(), vc.raw(), out.raw(), scratch.raw(), pos.raw(), status.raw(), n_seq, q_stride, kv_stride,
                heads, kvh, hd, n_rot, cap, window, eps, scale, exact ? 1 : 0);
    }
    void rows_indirect_seq(const CudaBuffer &w, uint32_t rows, uint32_t cols, const CudaBuffer &ids,
                           uint32_t ids_stride, const CudaBuffer &pos, uint32_t n_seq, int32_t bias, float scale,
                           const CudaBuffer &out) const {
        TM_CALL(tm_cuda_rows_indirect_seq_f32_dev, w.raw(), rows, cols, ids.raw(), ids_stride, pos.raw(), n_seq, bias,
                scale, out.raw());
    }
    void argmax_rows_dev(const CudaBuffer &x, uint32_t n_rows, uint32_t n, const CudaBuffer &partial,
                         const CudaBuffer &out, uint32_t out_stride, uint32_t base, const CudaBuffer &pos,
                         uint32_t out_cap, const CudaBuffer *mirror) const {
        TM_CALL(tm_cuda_argmax_rows_f32_dev, x.raw(), n_rows, n, partial.raw(), out.raw(), out_stride, base, pos.raw(),
                out_cap, mirror ? mirror->raw() : nullptr);
    }
    void u32_add_sat(const CudaBuffer &b, uint32_t first, uint32_t count, uint32_t delta, uint32_t limit) const {
        TM_CALL(tm_cuda_u32_add_sat, b.raw(), first, count, delta, limit);
    }
    // y = W rmsnorm(x + rmsnorm(add_p, add_w), norm_w); x + ... goes to x_out (include/tm_cuda.h).
    void q8_0_gemv_addnorm(const CudaBuffer &w, const CudaBuffer &x, const CudaBuffer &add_p, const CudaBuffer &add_w,
                           const CudaBuffer &x_out, const CudaBuffer &norm_w, const CudaBuffer &y, uint32_t rows,
                           uint32_t cols, float eps) const {
        TM_CALL(tm_cuda_q8_0_gemv_addnorm, w.raw(), x.raw(), add_p.raw(), add_w.raw(), x_out.raw(), norm_w.raw(), y.raw(),
                rows, cols, eps);
    }
    void q8_0_gemm_fused(const CudaBuffer &w, const CudaBuffer &x, const CudaBuffer &y, uint32_t rows, uint32_t cols,
                         uint32_t batch, int prologue, const CudaBuffer *pro, float eps, int epilogue) const {
        TM_CALL(tm_cuda_q8_0_gemm_fused, w.raw(), x.raw(), y.raw(), rows, cols, batch, prologue,
                pro ? pro->raw() : nullptr, eps, epilogue);
    }

    // ---- multi-GPU row split ----
    void comm_init(const void *id128, int rank, int world) const {
        char e[256] = "";
        cuda_check(tm_cuda_comm_init(ctx_, id128, rank, world, e, sizeof e), e);
    }
    void all_gather_rows(const CudaBuffer &src, const CudaBuffer &stage, const CudaBuffer &dst, uint32_t n_rows,
                         uint32_t width) const {
        TM_CALL(tm_cuda_all_gather_rows_f32, src.raw(), stage.raw(), dst.raw(), n_rows, width);
    }
    // The all-gather as a push into a symmetric buffer (include/tm_cuda.h): dst[t][rank*width + c] on every rank.
    void push_rows(const CudaBuffer &src, const CudaBuffer &dst, uint32_t n_rows, uint32_t width) const {
        TM_CALL(tm_cuda_push_rows_f32, src.raw(), dst.raw(), n_rows, width);
    }
    // GEMM whose epilogue writes this rank's rows into every rank's gathered output (include/tm_cuda.h).
    void q8_0_gemm_mma_push(const CudaBuffer &w, const CudaBuffer &x, const CudaBuffer &dst, uint32_t rows, uint32_t cols,
                            uint32_t batch) const {
        TM_CALL(tm_cuda_q8_0_gemm_mma_push, w.raw(), x.raw(), dst.raw(), rows, cols, batch);
    }
    void argmax_sharded(const CudaBuffer &x, uint32_t n, uint32_t index_offset, const CudaBuffer &partial,
                        const CudaBuffer &pairs, const CudaBuffer &out, uint32_t base, const CudaBuffer *pos,
                        uint32_t pos_index, uint32_t out_cap, const CudaBuffer *mirror) const {
        TM_CALL(tm_cuda_argmax_sharded_dev, x.raw(), n, index_offset, partial.raw(), pairs.raw(), out.raw(), base,
                pos ? pos->raw() : nullptr, pos_index, out_cap, mirror ? mirror->raw() : nullptr);
    }

    // x += sum of the ranks' partial products (then an optional output norm), include/tm_cuda.h.
    void reduce_ranks_add(const CudaBuffer &slots, const CudaBuffer &x, const CudaBuffer *weight, uint32_t world,
                          uint32_t n_rows, uint32_t cols, float eps) const {
        TM_CALL(tm_cuda_reduce_ranks_add_f32, slots.raw(), x.raw(), weight ? weight->raw() : nullptr, world, n_rows, cols,
                eps);
    }
    // y += sum over ranks of their `src` rows: push, reduction and add as one launch (one row).
    void exchange_add_ll(const CudaBuffer &src, const CudaBuffer &slots, const CudaBuffer &y, uint32_t width) const {
        TM_CALL(tm_cuda_exchange_add_ll_f32, src.raw(), slots.raw(), y.raw(), width);
    }
    void argmax_rows_sharded(const CudaBuffer &x, uint32_t n_rows, uint32_t n, uint32_t index_offset,
                             const CudaBuffer &partial, const CudaBuffer &pairs, const CudaBuffer &out,
                             uint32_t out_stride, uint32_t base, const CudaBuffer &pos, uint32_t out_cap,
                             const CudaBuffer *mirror) const {
        TM_CALL(tm_cuda_argmax_rows_sharded_dev, x.raw(), n_rows, n, index_offset, partial.raw(), pairs.raw(), out.raw(),
                out_stride, base, pos.raw(), out_cap, mirror ? mirror->raw() : nullptr);
    }

    void prefetch_l2(std::initializer_list<const CudaBuffer *> bufs) const {
        std::vector<tm_cuda_buffer *> raw;
        for (const CudaBuffer *b : bufs) raw.push_back(b->raw());
        TM_CALL(tm_cuda_prefetch_l2, raw.data(), (uint32_t)raw.size());
    }

    // ---- grouping / measurement (crates/tuckcore/src/qwen35_gpu.rs:62-86) ----
    void begin_group() const {
        char e[256] = "";
        cuda_check(tm_cuda_begin_group(ctx_, e, sizeof e), e);
    }
    void end_group() const {
        char e[256] = "";
        cuda_check(tm_cuda_end_group(ctx_, e, sizeof e), e);
    }
    void abort_group() const {
        char e[256] = "";
        tm_cuda_abort_group(ctx_, e, sizeof e);
    }
    CudaGraph end_group_retain() const {
        char e[256] = "";
        tm_cuda_graph *g = nullptr;
        cuda_check(tm_cuda_end_group_retain(ctx_, &g, e, sizeof e), e);
        return CudaGraph(ctx_, g);
    }
    // A decode step recorded as one persistent kernel (include/tm_cuda.h): the operators called
    // between begin_program and end_program are recorded, not launched.
    void begin_program(uint32_t max_ops, uint64_t vector_elems, uint64_t attention_elems) const {
        char e[256] = "";
        cuda_check(tm_cuda_begin_program(ctx_, max_ops, vector_elems, attention_elems, e, sizeof e), e);
    }
    void abort_program() const {
        char e[256] = "";
        tm_cuda_abort_program(ctx_, e, sizeof e);
    }
    CudaGraph end_program() const {
        char e[256] = "";
        tm_cuda_graph *g = nullptr;
        cuda_check(tm_cuda_end_program(ctx_, &g, e, sizeof e), e);
        return CudaGraph(ctx_, g);
    }
    // Status words of the bounded waits (each waits for the stream): non-zero = a wait ran out.
    uint32_t program_status(const CudaGraph &g) const {
        char e[256] = "";
        uint32_t st = 0;
        cuda_check(tm_cuda_program_status(ctx_, g.raw(), &st, e, sizeof e), e);
        return st;
    }
    bool mma_aborted() const { return tm_cuda_mma_aborted(ctx_) != 0; }
    uint32_t symm_status(const CudaBuffer &b) const {
        char e[256] = "";
        uint32_t st = 0;
        cuda_check(tm_cuda_symm_status(ctx_, b.raw(), &st, e, sizeof e), e);
        return st;
    }
    // One dispatch per step: a failure inside `encode` aborts the group so no
    // partial work reaches the device.
    template <class F>
    void grouped(F &&encode) const {
        begin_group();
        try {
            encode();
        } catch (...) {
            abort_group();
            throw;
        }
        end_group();
    }
    void fence() const {
        char e[256] = "";
        cuda_check(tm_cuda_fence(ctx_, e, sizeof e), e);
    }
    uint64_t committed() const { return tm_cuda_committed_dispatches(ctx_); }
    uint64_t completed() const { return tm_cuda_completed_dispatches(ctx_); }
    uint64_t allocated_bytes() const { return tm_cuda_allocated_bytes(ctx_); }
    uint64_t gpu_nanos_total() const { return tm_cuda_gpu_nanos_total(ctx_); }
    uint64_t kernel_launches() const { return tm_cuda_kernel_launches(ctx_); }

private:
    tm_cuda_ctx *ctx_ = nullptr;
};

#undef TM_CALL

}  // namespace tuckmill
