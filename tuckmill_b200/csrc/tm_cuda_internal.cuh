// Internal definitions shared by the translation units of libtm_cuda.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <deque>
#include <mutex>
#include <string>
#include <unordered_set>
#include <vector>

#include "tm_cuda.h"

// What a buffer is known to hold (set by the packing entry point, checked by
// the Q8_0 operators so a raw GGUF upload is never misread as packed planes).
enum tm_layout : uint32_t { TM_LAYOUT_OPAQUE = 0, TM_LAYOUT_Q8_0_PACKED = 1 };

struct tm_cuda_buffer {
    tm_cuda_ctx *owner = nullptr;
    tm_cuda_buffer *parent = nullptr;  // non-null for a view
    unsigned char *dev = nullptr;      // device-visible address
    size_t len = 0;
    int shared = 0;
    uint32_t views = 0;                // live views of this buffer
    tm_layout layout = TM_LAYOUT_OPAQUE;
    uint32_t rows = 0, cols = 0;       // geometry of a packed matrix
    const unsigned char *qp = nullptr; // packed: int8 quant plane of row 0
    const unsigned char *dp = nullptr; // packed: f16 scale plane of row 0
    void *symm = nullptr;              // peer mappings of a symmetric exchange buffer (tm_cuda_comm.cu)
};

// Closes the peer mappings of a symmetric buffer (no-op for ordinary buffers).
extern "C" void tm_cuda_symm_release(tm_cuda_buffer *b);

struct tm_step_program;  // a recorded decode step run by one persistent kernel (tm_cuda_step.cu)

struct tm_cuda_graph {
    tm_cuda_ctx *owner = nullptr;
    cudaGraphExec_t exec = nullptr;      // a captured group, or
    tm_step_program *program = nullptr;  // a persistent program
    uint64_t kernels = 0;
};

struct tm_commit {
    uint64_t seq = 0;
    cudaEvent_t begin = nullptr, end = nullptr;
    int label = -1;
};

struct tm_profile_row {
    std::string name;
    uint64_t nanos = 0, count = 0;
};

struct tm_cuda_ctx {
    int device = 0;
    int sm_count = 0;
    size_t smem_optin = 0;
    cudaStream_t stream = nullptr;
    // Side stream of tm_cuda_prefetch_l2: forks from `stream` at the call and joins it again before a
    // capture ends (or at once outside a group).
    cudaStream_t side = nullptr;
    cudaEvent_t side_fork = nullptr, side_join = nullptr;
    bool side_pending = false;
    std::mutex mu;
    std::unordered_set<const tm_cuda_buffer *> live;
    std::unordered_set<const tm_cuda_graph *> graphs;
    std::atomic<uint64_t> allocated{0};
    std::atomic<uint64_t> committed{0};
    std::atomic<uint64_t> completed{0};
    std::atomic<uint64_t> gpu_nanos{0};
    std::atomic<uint64_t> launches{0};
    std::atomic<uint64_t> last_gpu_ns{0};
    bool group_open = false;
    uint64_t group_kernels = 0;
    bool profiling = false;
    bool pdl = true;                     // chain kernels with programmatic dependent launch
    std::deque<tm_commit> pending;       // committed, completion not yet observed
    tm_commit open_commit;               // the ungrouped dispatch being encoded
    std::vector<cudaEvent_t> event_pool;
    std::vector<tm_profile_row> profile;
    // Scratch owned by the context for the tensor-core GEMM (f16 copy of X).
    unsigned char *mma_scratch = nullptr;
    size_t mma_scratch_bytes = 0;
    int mma_last_bn = 0;                 // token sub-tile width of the last tensor-core GEMM launch
    int mma_last_ksplit = 0;             // K parts per output tile of that launch
    void *comm = nullptr;  // multi-GPU communicator state (tm_cuda_comm.cu)
    void *program = nullptr;  // the persistent program being recorded (tm_step_program), if any
};

// ---- error plumbing -------------------------------------------------------

inline int tm_fail(char *err, size_t cap, int code, const char *fmt, ...) {
    if (err && cap) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, cap, fmt, ap);
        va_end(ap);
    }
    return code;
}

#define TM_CUDA_TRY(expr)                                                                   \
    do {                                                                                    \
        cudaError_t e_ = (expr);                                                            \
        if (e_ != cudaSuccess)                                                              \
            return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "%s failed: %s", #expr,      \
                           cudaGetErrorString(e_));                                         \
    } while (0)

// Owned-and-large-enough check, the CUDA twin of tm_check_buffer
// (native/metal/tm_metal.m:153-171).
inline int tm_check(tm_cuda_ctx *ctx, const tm_cuda_buffer *b, size_t need, const char *what,
                    char *err, size_t err_cap) {
    if (!b || ctx->live.find(b) == ctx->live.end())
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "%s buffer does not belong to this context", what);
    if (need == 0 || b->len < need)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "%s buffer holds %zu bytes, needs %zu",
                       what, b->len, need);
    return TM_CUDA_OK;
}

#define TM_CHECK_BUF(buf, need, what)                                        \
    do {                                                                     \
        int rc_ = tm_check(ctx, (buf), (need), (what), err, err_cap);        \
        if (rc_ != TM_CUDA_OK) return rc_;                                   \
    } while (0)

// Every operator entry point opens with this: context present, device current,
// dispatch serialised (crates/metal/src/lib.rs:695-707 holds a mutex the same way).
#define TM_ENTER()                                                                          \
    if (!ctx) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "null context");        \
    std::lock_guard<std::mutex> lock_(ctx->mu);                                             \
    TM_CUDA_TRY(cudaSetDevice(ctx->device))

// Book-keeping around one operator launch (ungrouped: one dispatch per op with
// its own timing events; grouped: counted into the open group).
int tm_op_begin(tm_cuda_ctx *ctx, const char *label, char *err, size_t err_cap);
int tm_op_end(tm_cuda_ctx *ctx, uint64_t kernels, char *err, size_t err_cap);

#define TM_OP_BEGIN(label)                                          \
    do {                                                            \
        int rc_ = tm_op_begin(ctx, (label), err, err_cap);          \
        if (rc_ != TM_CUDA_OK) return rc_;                          \
    } while (0)
#define TM_OP_END(kernels)                                                          \
    do {                                                                            \
        cudaError_t le_ = cudaGetLastError();                                       \
        if (le_ != cudaSuccess)                                                     \
            return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "launch failed: %s", \
                           cudaGetErrorString(le_));                                \
        return tm_op_end(ctx, (kernels), err, err_cap);                             \
    } while (0)

inline size_t tm_round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline size_t tm_q8_qplane_bytes(uint32_t rows, uint32_t cols) {
    return tm_round_up((size_t)rows * cols, 256);
}

// Checks `w` is a packed rows x cols Q8_0 matrix of this context.
int tm_check_packed(tm_cuda_ctx *ctx, const tm_cuda_buffer *w, uint32_t rows, uint32_t cols,
                    char *err, size_t err_cap);

// Launch on the context's stream, allowing the kernel to overlap the tail of
// its predecessor (the kernel itself orders its dependent reads with
// griddepcontrol.wait).
template <class... KArgs, class... Args>
inline cudaError_t tm_launch_pdl(tm_cuda_ctx *ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Tensor-core decode attention for several sequences in one launch (tm_cuda_attn_mma.cu).
bool tm_attention_decode_mma_ok(uint32_t heads, uint32_t kv_heads, uint32_t hd, uint32_t n_rot);
cudaError_t tm_attention_decode_mma_launch(tm_cuda_ctx *ctx, const float *q, const float *k, const float *v,
                                           const float *qn, const float *kn, const float *inv_freq, void *kc, void *vc,
                                           float *out, float *scratch, const uint32_t *pos, uint32_t *status,
                                           uint32_t heads, uint32_t kv_heads, uint32_t hd, uint32_t cap, uint32_t window,
                                           float eps, float scale, uint32_t n_seq, size_t sq, size_t skv, size_t so,
                                           size_t scache, size_t sscratch, uint32_t count_off);

cudaError_t tm_argmax_partial_launch(tm_cuda_ctx *ctx, const float *x, uint32_t n, float *pv, uint32_t *pi);
cudaError_t tm_argmax_rows_partial_launch(tm_cuda_ctx *ctx, const float *x, uint32_t n_rows, uint32_t n, float *pv,
                                          uint32_t *pi);

// ---- persistent decode program (tm_cuda_step.cu) ----
// While ctx->program is set, the operators a program can hold record themselves through these
// instead of launching; every other operator refuses (tm_op_begin).
int tm_step_record_gemv(tm_cuda_ctx *ctx, const void *q, const void *d, const float *x, float *y, const float *pro,
                        uint32_t rows, uint32_t cols, int prologue, int epilogue, float eps, uint32_t batch, char *err,
                        size_t err_cap);
int tm_step_record_embed(tm_cuda_ctx *ctx, const void *q, const void *d, uint32_t rows, uint32_t cols,
                         const uint32_t *ids, uint32_t slot, const uint32_t *pos, int bias, uint32_t ids_len,
                         float scale, float *out, char *err, size_t err_cap);
int tm_step_record_attention(tm_cuda_ctx *ctx, const float *q, const float *k, const float *v, const float *qn,
                             const float *kn, const float *inv_freq, void *kc, void *vc, float *out, float *scratch,
                             const uint32_t *pos, uint32_t *status, uint32_t heads, uint32_t kv_heads, uint32_t hd,
                             uint32_t n_rot, uint32_t cap, uint32_t window, float eps, float scale, int exact,
                             char *err, size_t err_cap);
int tm_step_record_argmax(tm_cuda_ctx *ctx, const float *x, uint32_t n, uint32_t *out, uint32_t base,
                          const uint32_t *pos, uint32_t out_cap, uint32_t *mirror, char *err, size_t err_cap);
int tm_step_record_norm_add(tm_cuda_ctx *ctx, const float *p, const float *w, float *x, uint32_t rows, uint32_t cols,
                            float eps, char *err, size_t err_cap);
int tm_step_record_pos_add(tm_cuda_ctx *ctx, uint32_t *counter, uint32_t delta, char *err, size_t err_cap);
int tm_step_launch(tm_cuda_ctx *ctx, tm_step_program *p, char *err, size_t err_cap);
void tm_step_free(tm_cuda_ctx *ctx, tm_step_program *p);
