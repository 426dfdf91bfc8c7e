/*
 * tm_cuda.h -- TuckCore <-> CUDA narrow C ABI for NVIDIA B200 (sm_100a).
 *
 * The CUDA counterpart of the reference's device interface
 * native/metal/tm_metal.h: one context owns one device, one in-order stream
 * and the kernels for the operations declared here; buffers are opaque
 * handles with explicit lifetime; every operation is asynchronous, ordered on
 * the context's stream, and returns 0 or a TM_CUDA_ERR_* code with a
 * NUL-terminated message in the caller-owned `err` (may be NULL).  A context
 * is used from one thread at a time; counters may be read from any thread.
 *
 * Each declaration cites the reference declaration it replaces
 * (native/metal/tm_metal.h:<line>).  Declarations marked "no counterpart"
 * exist because CUDA needs them (weight repacking, retained graphs, device
 * positions, multi-GPU row split); a host that only knows the reference
 * surface can ignore them and still run every operator.
 *
 * There is no CPU fallback anywhere behind this interface: without a usable
 * CUDA device tm_cuda_create fails with TM_CUDA_ERR_NO_DEVICE.
 */
#ifndef TM_CUDA_H
#define TM_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tm_cuda_ctx tm_cuda_ctx;
typedef struct tm_cuda_buffer tm_cuda_buffer;
typedef struct tm_cuda_graph tm_cuda_graph;

/* Error codes: the values of tm_metal.h:32-40. */
enum {
    TM_CUDA_OK = 0,
    TM_CUDA_ERR_NO_DEVICE = -1,   /* no CUDA device / wrong architecture */
    TM_CUDA_ERR_SOURCE = -2,      /* kernel image failed to load */
    TM_CUDA_ERR_ALLOC = -3,       /* buffer allocation failed */
    TM_CUDA_ERR_BOUNDS = -4,      /* size/range mismatch, zero length */
    TM_CUDA_ERR_UNSUPPORTED = -5, /* invalid arguments / mode */
    TM_CUDA_ERR_INTERNAL = -6     /* CUDA runtime failure */
};

/* tm_metal.h:43 tm_metal_available -- number of usable sm_100 devices. */
int tm_cuda_available(void);
/* tm_metal.h:47 tm_metal_runtime_info -- one-line description, static. */
const char *tm_cuda_runtime_info(void);
/* tm_metal.h:52 tm_metal_create -- device `device` (0-based) and its stream.
 * NULL on failure, `err` filled. */
tm_cuda_ctx *tm_cuda_create(int device, char *err, size_t err_cap);
/* tm_metal.h:56 tm_metal_destroy -- buffers must have been freed first. */
void tm_cuda_destroy(tm_cuda_ctx *ctx);

/* tm_metal.h:61 tm_metal_buffer_new -- `shared` buffers are pinned host
 * memory mapped into the device (CPU-readable through
 * tm_cuda_buffer_contents); private buffers live in HBM. */
tm_cuda_buffer *tm_cuda_buffer_new(tm_cuda_ctx *ctx, size_t bytes, int shared, char *err,
                                   size_t err_cap);
/* tm_metal.h:66 tm_metal_buffer_free -- waits for the device to finish the
 * work already committed, so storage is never reused under a running kernel. */
void tm_cuda_buffer_free(tm_cuda_ctx *ctx, tm_cuda_buffer *buffer);
/* tm_metal.h:70 tm_metal_buffer_contents. */
void *tm_cuda_buffer_contents(tm_cuda_ctx *ctx, tm_cuda_buffer *buffer);
/* tm_metal.h:73 tm_metal_buffer_len. */
size_t tm_cuda_buffer_len(const tm_cuda_ctx *ctx, const tm_cuda_buffer *buffer);
/* tm_metal.h:78 tm_metal_buffer_zero. */
int tm_cuda_buffer_zero(tm_cuda_ctx *ctx, tm_cuda_buffer *buffer, size_t off, size_t len,
                        char *err, size_t err_cap);
/* tm_metal.h:82,84 tm_metal_upload / tm_metal_download -- ordered after all
 * committed work; return when the copy is complete.  No open group. */
int tm_cuda_upload(tm_cuda_ctx *ctx, tm_cuda_buffer *dst, size_t off, const void *src, size_t len,
                   char *err, size_t err_cap);
int tm_cuda_download(tm_cuda_ctx *ctx, tm_cuda_buffer *src, size_t off, void *dst, size_t len,
                     char *err, size_t err_cap);
/* No counterpart: a handle aliasing `len` bytes of `parent` at byte offset
 * `off` (16-byte aligned), so operators without offset arguments can work
 * on a slice of a fused output.  Counts 0 bytes in the ledger; must be freed
 * before its parent. */
tm_cuda_buffer *tm_cuda_buffer_view(tm_cuda_ctx *ctx, tm_cuda_buffer *parent, size_t off,
                                    size_t len, char *err, size_t err_cap);
/* No counterpart: raw device address of a buffer (for a host that shares the
 * CUDA primary context, e.g. to hand a buffer to NCCL or torch). */
void *tm_cuda_buffer_device_ptr(tm_cuda_ctx *ctx, tm_cuda_buffer *buffer);

/* ---------------- elementwise utilities ---------------- */
/* tm_metal.h:88 tm_metal_f32_scale: y[i] = x[i] * factor. */
int tm_cuda_f32_scale(tm_cuda_ctx *ctx, tm_cuda_buffer *x, tm_cuda_buffer *y, float factor,
                      uint32_t n, char *err, size_t err_cap);
/* tm_metal.h:115 tm_metal_f32_axpy: y[i] += alpha * a[i]. */
int tm_cuda_f32_axpy(tm_cuda_ctx *ctx, tm_cuda_buffer *a, tm_cuda_buffer *y, float alpha,
                     uint32_t n, char *err, size_t err_cap);
/* tm_metal.h:111 tm_metal_copy_f32: dst[dst_off+i] = src[src_off+i]. */
int tm_cuda_copy_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *src, uint32_t src_off, tm_cuda_buffer *dst,
                     uint32_t dst_off, uint32_t n, char *err, size_t err_cap);
/* tm_metal.h:119,123 casts between binary16 and f32 (encode rounds to
 * nearest even and saturates to infinity). */
int tm_cuda_cast_f16_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t n,
                         char *err, size_t err_cap);
int tm_cuda_cast_f32_f16(tm_cuda_ctx *ctx, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t n,
                         char *err, size_t err_cap);
/* tm_metal.h:96 tm_metal_argmax_f32 -- NaN skipped, largest wins, ties to the
 * lowest index, 0xFFFFFFFF when every entry is NaN; `partial` is 512 bytes. */
int tm_cuda_argmax_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *x, uint32_t n, tm_cuda_buffer *partial,
                       tm_cuda_buffer *out, uint32_t out_index, char *err, size_t err_cap);
/* tm_metal.h:147 tm_metal_rmsnorm_f32. */
int tm_cuda_rmsnorm_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *x, tm_cuda_buffer *weight,
                        tm_cuda_buffer *y, uint32_t rows, uint32_t cols, float eps, char *err,
                        size_t err_cap);
/* No counterpart: x[row] += rmsnorm(p[row]) * weight, i.e. tm_cuda_rmsnorm_f32 followed by
 * tm_cuda_f32_axpy(alpha = 1) as one launch, bit for bit (the output norm plus residual add of
 * Gemma-style layers). */
int tm_cuda_rmsnorm_add_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *p, tm_cuda_buffer *weight, tm_cuda_buffer *x,
                            uint32_t rows, uint32_t cols, float eps, char *err, size_t err_cap);
/* tm_metal.h:189 tm_metal_silu_mul_f32 / :193 tm_metal_gelu_tanh_mul_f32. */
int tm_cuda_silu_mul_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *gate, tm_cuda_buffer *up,
                         tm_cuda_buffer *out, uint32_t n, char *err, size_t err_cap);
int tm_cuda_gelu_tanh_mul_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *gate, tm_cuda_buffer *up,
                              tm_cuda_buffer *out, uint32_t n, char *err, size_t err_cap);

/* ---------------- Q8_0 weights ---------------- */
/*
 * Weight layout.  The reference keeps a Q8_0 matrix as the GGUF bytes
 * verbatim (tm_metal.h:196-199: rows * cols/32 blocks of 34 bytes).  A 34-byte
 * stride leaves quants 2-byte aligned, which rules out 128-bit loads, so this
 * library keeps the SAME values in two planes inside one buffer:
 *   int8  q[rows][cols]      at byte 0
 *   f16   d[rows][cols/32]   at byte tm_cuda_q8_0_packed_bytes' q-plane size
 *                            rounded up to 256
 * Repacking moves bytes; no value changes (1.0625 bytes per weight either
 * way).  Every Q8_0 operator below takes a PACKED buffer produced by
 * tm_cuda_q8_0_pack and refuses anything else with TM_CUDA_ERR_UNSUPPORTED.
 */
/* No counterpart: bytes of the packed form of a rows x cols matrix
 * (0 when cols is not a positive multiple of 32 or rows is 0). */
size_t tm_cuda_q8_0_packed_bytes(uint32_t rows, uint32_t cols);
/* No counterpart: repack `nrows` raw GGUF rows held in `raw` (device buffer,
 * nrows * cols/32 * 34 bytes at byte offset raw_off) into rows
 * [row0, row0+nrows) of the packed matrix `dst` (rows x cols).  A matrix is
 * usable by the operators once every row has been packed. */
int tm_cuda_q8_0_pack(tm_cuda_ctx *ctx, tm_cuda_buffer *dst, uint32_t rows, uint32_t cols,
                      tm_cuda_buffer *raw, size_t raw_off, uint32_t row0, uint32_t nrows,
                      char *err, size_t err_cap);
/* No counterpart: a handle on rows [row0, row0+nrows) of a packed matrix, usable
 * wherever a packed nrows x cols matrix is (so projections stored as one fused
 * matrix can also be multiplied one at a time).  Freed like a buffer view. */
tm_cuda_buffer *tm_cuda_q8_0_row_view(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows,
                                      uint32_t cols, uint32_t row0, uint32_t nrows, char *err,
                                      size_t err_cap);
/* No counterpart: the inverse, for round-trip checks: write rows
 * [row0,row0+nrows) of packed `src` as raw GGUF bytes into `raw`. */
int tm_cuda_q8_0_unpack(tm_cuda_ctx *ctx, tm_cuda_buffer *src, uint32_t rows, uint32_t cols,
                        tm_cuda_buffer *raw, size_t raw_off, uint32_t row0, uint32_t nrows,
                        char *err, size_t err_cap);

/* tm_metal.h:200 tm_metal_q8_0_gemv: y[r] = dot(dequant(w_row_r), x), f32. */
int tm_cuda_q8_0_gemv(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y,
                      uint32_t rows, uint32_t cols, char *err, size_t err_cap);
/* tm_metal.h:165 tm_metal_q8_0_gemm: Y[b,:] = W X[b,:], b < batch (1..32), X
 * at f32 offset x_off, Y at y_off; per-token arithmetic is that of the GEMV,
 * so any batch is bit-identical to `batch` GEMV calls. */
#define TM_CUDA_GEMM_MAX_BATCH 32u
int tm_cuda_q8_0_gemm(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y,
                      uint32_t rows, uint32_t cols, uint32_t batch, uint32_t x_off, uint32_t y_off,
                      char *err, size_t err_cap);
/* tm_metal.h:176 tm_metal_q8_0_gemm_mma: the same contract on the tensor
 * cores (tcgen05, f16 operands: x and d*q are rounded to binary16, f32
 * accumulation in tensor memory); tolerance-qualified, not bit-identical.
 * The batch limit is the reference's 512 raised to what one launch tiles.  One or two tokens (up to
 * eight when cols < 2048) are handed to tm_cuda_q8_0_gemm, which is exact and as fast there. */
#define TM_CUDA_GEMM_MMA_MAX_BATCH 8192u
int tm_cuda_q8_0_gemm_mma(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x,
                          tm_cuda_buffer *y, uint32_t rows, uint32_t cols, uint32_t batch,
                          uint32_t x_off, uint32_t y_off, char *err, size_t err_cap);
/* No counterpart: the tensor-core GEMM reads an f16 copy of X through TMA; the
 * copy lives in a workspace owned by the context (cols * batch * 2 bytes plus a
 * fixed 20 MB of split-K slots, counted in tm_cuda_allocated_bytes).  It grows on
 * demand, except inside an open dispatch group, where it must have been reserved
 * beforehand with the size tm_cuda_mma_workspace_bytes gives. */
size_t tm_cuda_mma_workspace_bytes(uint32_t cols, uint32_t batch);
int tm_cuda_mma_workspace_reserve(tm_cuda_ctx *ctx, size_t bytes, char *err, size_t err_cap);
/* No counterpart: 1 when a tensor-core GEMM of this context gave up one of its
 * bounded pipeline waits (its output is then undefined); waits for the stream. */
int tm_cuda_mma_aborted(tm_cuda_ctx *ctx);
/* No counterpart: which instantiation of the tensor-core kernel the context's last GEMM
 * launch used, as its token sub-tile width (64, 128 or 192; 0 before the first launch).
 * The launcher picks it from the shape; tests use this to prove each one is covered. */
int tm_cuda_mma_last_tile(tm_cuda_ctx *ctx);
/* No counterpart: how many parts the last GEMM launch cut the K range of every output tile into
 * (1: none; 0 before the first launch).  A call with fewer output tiles than half the SMs (a batch of
 * decode rows, a narrow projection) is split so that the whole machine streams its weights; the
 * parts' sums are added in part order by whichever part finishes last, so the result does not depend
 * on timing. */
int tm_cuda_mma_last_split(tm_cuda_ctx *ctx);
/* tm_metal.h:138 tm_metal_q8_0_row_f32: dequantise one row to out[out_off..]. */
int tm_cuda_q8_0_row_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *out, uint32_t row,
                         uint32_t cols, uint32_t out_off, char *err, size_t err_cap);
/* ---------------- F16 weights ----------------
 * tm_metal.h:142 tm_metal_f16_gemv: y[r] = dot(f32(w_row_r), x); `w` holds rows * cols binary16
 * values, row-major, uploaded verbatim (no packing).  Serves F16-weight artifacts: the
 * reference's own model fixtures and F16 twins of quantized models. */
int tm_cuda_f16_gemv(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t rows,
                     uint32_t cols, char *err, size_t err_cap);
/* tm_metal.h:179 tm_metal_f16_gemm: the contract of tm_cuda_q8_0_gemm (batch 1..32, x_off / y_off,
 * batch 1 bit-identical to the GEMV). */
int tm_cuda_f16_gemm(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t rows,
                     uint32_t cols, uint32_t batch, uint32_t x_off, uint32_t y_off, char *err, size_t err_cap);
/* tm_metal.h:156 tm_metal_f16_row_f32: row `row` as f32 to out[out_off..]. */
int tm_cuda_f16_row_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *out, uint32_t row, uint32_t cols,
                        uint32_t out_off, char *err, size_t err_cap);
/* No counterpart: the F16 forms of tm_cuda_q8_0_gemv_fused, tm_cuda_row_indirect_f32_dev (pos_buf may
 * be NULL: slot = base) and tm_cuda_rows_indirect_f32, so the engine's decode and prefill loops run
 * F16-weight artifacts with the same launches per layer. */
int tm_cuda_f16_gemv_fused(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t rows,
                           uint32_t cols, int prologue, tm_cuda_buffer *pro, float eps, int epilogue, char *err,
                           size_t err_cap);
int tm_cuda_f16_row_indirect_f32_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows, uint32_t cols,
                                     tm_cuda_buffer *ids, uint32_t base, tm_cuda_buffer *pos_buf, uint32_t pos_index,
                                     int32_t bias, float scale, tm_cuda_buffer *out, char *err, size_t err_cap);
int tm_cuda_f16_rows_indirect_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows, uint32_t cols, tm_cuda_buffer *ids,
                                  uint32_t first, uint32_t n, float scale, tm_cuda_buffer *out, char *err,
                                  size_t err_cap);

/* tm_metal.h:104 tm_metal_row_indirect_f32: row ids[slot] (type 8 only); an
 * id >= rows writes zeros. */
int tm_cuda_row_indirect_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t type_id, uint32_t rows,
                             uint32_t cols, tm_cuda_buffer *ids, uint32_t slot,
                             tm_cuda_buffer *out, char *err, size_t err_cap);

/* No counterpart: the batched embedding lookup of a prefill chunk, one launch:
 * out[t] = row ids[first + t] (times `scale` when non-zero), t < n; an id
 * >= rows writes zeros.  Replaces n calls of tm_cuda_q8_0_row_f32. */
int tm_cuda_rows_indirect_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows, uint32_t cols,
                              tm_cuda_buffer *ids, uint32_t first, uint32_t n, float scale,
                              tm_cuda_buffer *out, char *err, size_t err_cap);

/* No counterpart: the GEMV with the neighbouring elementwise operators folded
 * into its activation load and its store, so a decode layer is a handful of
 * launches.  Per-row arithmetic is that of tm_cuda_q8_0_gemv on the same
 * activation values.
 *   prologue: 0 x as is | 1 x = rmsnorm(x, pw, eps) | 2 x = silu(x) * px
 *             | 3 x = gelu_tanh(x) * px            (pw/px: `pro` buffer)
 *   epilogue: 0 y = Wx  | 1 y += Wx */
enum { TM_CUDA_PRO_NONE = 0, TM_CUDA_PRO_RMSNORM = 1, TM_CUDA_PRO_SILU_MUL = 2,
       TM_CUDA_PRO_GELU_MUL = 3 };
enum { TM_CUDA_EPI_STORE = 0, TM_CUDA_EPI_ADD = 1 };
int tm_cuda_q8_0_gemv_fused(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x,
                            tm_cuda_buffer *y, uint32_t rows, uint32_t cols, int prologue,
                            tm_cuda_buffer *pro, float eps, int epilogue, char *err,
                            size_t err_cap);
/* No counterpart: a layer's output norm and residual add folded into the projection that consumes
 * the result (layers with output norms, e.g. Gemma's): x' = x + rmsnorm(add_p, add_w, eps) rounded
 * exactly as tm_cuda_rmsnorm_add_f32 rounds it, y = W rmsnorm(x', norm_w, eps) as
 * tm_cuda_q8_0_gemv_fused(prologue 1) computes it, and x' written to x_out -- a buffer OTHER than x,
 * because every CTA of the launch reads x.  One launch instead of two; cols <= 4096.  When the row
 * cut of a tall matrix makes it two launches, both write the same x'. */
int tm_cuda_q8_0_gemv_addnorm(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *add_p,
                              tm_cuda_buffer *add_w, tm_cuda_buffer *x_out, tm_cuda_buffer *norm_w, tm_cuda_buffer *y,
                              uint32_t rows, uint32_t cols, float eps, char *err, size_t err_cap);
/* No counterpart: the same fused forms for `batch` tokens (1..TM_CUDA_GEMM_MAX_BATCH), token-major x
 * [batch][cols] and y [batch][rows]; the activation prologues take `pro` as [batch][cols], the norm
 * weight as [cols].  Row t of the result is bit-identical to the one-token call on row t (the
 * contract of tm_cuda_q8_0_gemm).  A decode step of several sequences uses it. */
int tm_cuda_q8_0_gemm_fused(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t rows,
                            uint32_t cols, uint32_t batch, int prologue, tm_cuda_buffer *pro, float eps, int epilogue,
                            char *err, size_t err_cap);

/* ---------------- grouped encoding ---------------- */
/* tm_metal.h:133-135 begin/end/abort_group: operations between begin and end
 * are captured into one CUDA graph launched at end_group; abort discards
 * them without running anything.  Copies and fence need no open group. */
int tm_cuda_begin_group(tm_cuda_ctx *ctx, char *err, size_t err_cap);
int tm_cuda_end_group(tm_cuda_ctx *ctx, char *err, size_t err_cap);
int tm_cuda_abort_group(tm_cuda_ctx *ctx, char *err, size_t err_cap);
/* No counterpart: end the open group WITHOUT running it and keep it as a
 * replayable graph; each launch is one committed dispatch.  A decode step
 * whose position lives on the device (below) is recorded once and replayed
 * per token. */
int tm_cuda_end_group_retain(tm_cuda_ctx *ctx, tm_cuda_graph **out, char *err, size_t err_cap);
int tm_cuda_graph_launch(tm_cuda_ctx *ctx, tm_cuda_graph *graph, char *err, size_t err_cap);
void tm_cuda_graph_free(tm_cuda_ctx *ctx, tm_cuda_graph *graph);

/* No counterpart: ask for the bytes of up to 64 buffers to be brought into the L2 cache, on a side
 * stream that forks from the context's stream at this call and runs beside whatever is dispatched
 * next; it joins the stream again when the open dispatch group ends (at once outside a group).  A
 * decode step whose per-layer weights fit the cache calls it a layer or two ahead, so that a
 * projection finds its weights in L2 instead of paying a DRAM round trip per launch.  A hint only:
 * results never depend on it.  The first call of a context must be made outside a dispatch group. */
int tm_cuda_prefetch_l2(tm_cuda_ctx *ctx, tm_cuda_buffer *const *bufs, uint32_t n, char *err, size_t err_cap);

/* No counterpart: a decode step as ONE persistent kernel.  Between begin_program and
 * end_program the operators a step is made of do not launch; they are recorded, in
 * order, into a program: tm_cuda_q8_0_gemv / _gemv_fused (one token),
 * tm_cuda_row_indirect_f32(_dev), tm_cuda_attention_decode_dev (exact = 0, a geometry
 * tm_cuda_program_supports_attention accepts), tm_cuda_rmsnorm_add_f32 (one row),
 * tm_cuda_argmax_f32(_dev) and tm_cuda_u32_add; any other operator fails with
 * TM_CUDA_ERR_UNSUPPORTED and the caller falls back to a dispatch group.  The result is
 * launched and freed like a retained group (tm_cuda_graph_launch / _free; one committed
 * dispatch, one kernel per launch) and computes what the recorded operators would have
 * computed one after the other -- same arithmetic per operator, the GEMV's partial sums
 * added in a different (fixed) order, hence tolerance-qualified like the decode
 * attention it contains.  A buffer that several operators of the program write (the
 * residual stream) holds, after a launch, what the last of them wrote.
 * One CTA per SM walks the program: a producer warp streams the Q8_0 weights of ALL
 * operators through a shared-memory ring without stopping at operator boundaries, the
 * other warps multiply; vectors travel between operators as {value, sequence number}
 * words that consumers poll (no grid barrier), every poll bounded.
 * Device memory: tm_cuda_program_bytes(max_ops, vector_elems, attention_elems), counted in
 * tm_cuda_allocated_bytes until the program is freed.  vector_elems >= the sum of the
 * output lengths of the recorded operators (GEMV rows, embedding columns, attention
 * heads x head_dim, normed columns); attention_elems >= the largest
 * tm_cuda_program_attention_elems(heads, head_dim, capacity) of its attention operators.
 * Bits of tm_cuda_program_status (waits for the stream): 1 a wait for activations ran
 * out, 2 a weight-stage wait ran out.  A program whose status is non-zero computes
 * nothing further; free it and record a new one. */
size_t tm_cuda_program_bytes(uint32_t max_ops, uint64_t vector_elems, uint64_t attention_elems);
uint64_t tm_cuda_program_attention_elems(uint32_t heads, uint32_t head_dim, uint32_t cap);
int tm_cuda_program_supports_gemv(uint32_t cols);
int tm_cuda_program_supports_attention(uint32_t heads, uint32_t kv_heads, uint32_t head_dim, uint32_t n_rot);
int tm_cuda_begin_program(tm_cuda_ctx *ctx, uint32_t max_ops, uint64_t vector_elems, uint64_t attention_elems,
                          char *err, size_t err_cap);
int tm_cuda_end_program(tm_cuda_ctx *ctx, tm_cuda_graph **out, char *err, size_t err_cap);
int tm_cuda_abort_program(tm_cuda_ctx *ctx, char *err, size_t err_cap);
int tm_cuda_program_status(tm_cuda_ctx *ctx, tm_cuda_graph *program, uint32_t *status, char *err, size_t err_cap);
/* No counterpart, a profiling aid: time stamps (device global timer, ns) that CTA 0 took in the
 * program's last launch: out[8*i + 0] = operator i started, [1] = its activations were staged
 * (GEMV), [2] = its work on this CTA was done, [7] = the weight producer reached it; kinds[i]
 * (optional) = the operator's kind (1 embedding, 2 GEMV, 3 attention, 4 argmax, 5 norm + add,
 * 6 position).  The first call switches the stamps on and returns zeros.  `out` holds
 * 8 * max_ops words. */
int tm_cuda_program_trace(tm_cuda_ctx *ctx, tm_cuda_graph *program, uint64_t *out, uint32_t max_ops, uint32_t *kinds,
                          char *err, size_t err_cap);
/* No counterpart, for tests of the bounded waits: consumers expect sequence numbers
 * `sequence_skew` higher than producers write (0 = normal), and poll at most `spin_limit`
 * times (0 = unchanged).  With a skew no wait for activations can be satisfied: the kernel must
 * raise status bit 1 and return. */
int tm_cuda_program_debug(tm_cuda_ctx *ctx, tm_cuda_graph *program, uint32_t sequence_skew, uint32_t spin_limit,
                          char *err, size_t err_cap);

/* tm_metal.h:291 tm_metal_fence. */
int tm_cuda_fence(tm_cuda_ctx *ctx, char *err, size_t err_cap);
/* tm_metal.h:294,301 committed / completed dispatch counters. */
uint64_t tm_cuda_committed_dispatches(const tm_cuda_ctx *ctx);
uint64_t tm_cuda_completed_dispatches(const tm_cuda_ctx *ctx);
/* tm_metal.h:299 tm_metal_download_after: copy from a SHARED buffer once the
 * first `completed_target` committed dispatches have completed. */
int tm_cuda_download_after(tm_cuda_ctx *ctx, tm_cuda_buffer *src, size_t off, void *dst,
                           size_t len, uint64_t completed_target, char *err, size_t err_cap);
/* tm_metal.h:304,307 GPU time of the last completed dispatch / cumulative. */
double tm_cuda_last_gpu_ms(const tm_cuda_ctx *ctx);
uint64_t tm_cuda_gpu_nanos_total(const tm_cuda_ctx *ctx);
/* tm_metal.h:312,315 per-operator attribution (CUDA events per dispatch). */
int tm_cuda_profile_set(tm_cuda_ctx *ctx, int enabled);
int tm_cuda_profile_read(tm_cuda_ctx *ctx, uint32_t index, char *name, size_t name_cap,
                         uint64_t *nanos, uint64_t *count);
/* tm_metal.h:318 live bytes in buffers; :325 bytes leased by pending work
 * (always 0 here: tm_cuda_buffer_free waits instead of leasing). */
uint64_t tm_cuda_allocated_bytes(const tm_cuda_ctx *ctx);
uint64_t tm_cuda_in_flight_bytes(const tm_cuda_ctx *ctx);
/* No counterpart: kernels launched by this context so far (each operator
 * launch and each graph node counts one). */
uint64_t tm_cuda_kernel_launches(const tm_cuda_ctx *ctx);
/* No counterpart: free and total bytes of the context's device (the budget B
 * the planner admits against when the caller names none). */
int tm_cuda_device_memory(tm_cuda_ctx *ctx, uint64_t *free_bytes, uint64_t *total_bytes);
/* No counterpart: the context's cudaStream_t, so a host that shares the CUDA
 * primary context can record its own events on the stream the kernels run on. */
void *tm_cuda_stream(tm_cuda_ctx *ctx);

/* ---------------- attention operators ---------------- */
/* tm_metal.h:257 tm_metal_qwen35_rope_partial: split-half RoPE on the first
 * n_rot dims of every q/k head row, angle (float)pos * inv_freq[i]. */
int tm_cuda_qwen35_rope_partial(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k,
                                tm_cuda_buffer *inv_freq, uint32_t pos, uint32_t n_q_heads,
                                uint32_t n_kv_heads, uint32_t head_dim, uint32_t n_rot, char *err,
                                size_t err_cap);
/* tm_metal.h:368 ..._rope_partial_chunk: token t rotates at pos0 + t. */
int tm_cuda_qwen35_rope_partial_chunk(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k,
                                      tm_cuda_buffer *inv_freq, uint32_t pos0, uint32_t n_q_heads,
                                      uint32_t n_kv_heads, uint32_t head_dim, uint32_t n_rot,
                                      uint32_t n, char *err, size_t err_cap);
/* tm_metal.h:264 ..._kv_store_f16 / :373 ..._kv_store_f16_chunk:
 * cache[h][pos0+t][d] = (half) src[t][h][d], planes [kv_head][cap][head_dim]. */
int tm_cuda_qwen35_kv_store_f16(tm_cuda_ctx *ctx, tm_cuda_buffer *k_src, tm_cuda_buffer *v_src,
                                tm_cuda_buffer *k_cache, tm_cuda_buffer *v_cache, uint32_t pos,
                                uint32_t cap, uint32_t head_dim, uint32_t kv_heads, char *err,
                                size_t err_cap);
int tm_cuda_qwen35_kv_store_f16_chunk(tm_cuda_ctx *ctx, tm_cuda_buffer *k_src,
                                      tm_cuda_buffer *v_src, tm_cuda_buffer *k_cache,
                                      tm_cuda_buffer *v_cache, uint32_t pos0, uint32_t cap,
                                      uint32_t head_dim, uint32_t kv_heads, uint32_t n, char *err,
                                      size_t err_cap);
/* tm_metal.h:270 ..._attention_f16: causal GQA attention of one query row
 * over keys 0..=pos of a packed f16 cache (`scratch`: see the chunk form). */
int tm_cuda_qwen35_attention_f16(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k_cache,
                                 tm_cuda_buffer *v_cache, tm_cuda_buffer *out,
                                 tm_cuda_buffer *scratch, uint32_t heads, uint32_t pos,
                                 uint32_t cap, uint32_t head_dim, uint32_t group, float scale,
                                 char *err, size_t err_cap);
/* tm_metal.h:378 ..._attention_f16_chunk: query row t attends keys
 * [start, pos0+t] where start = seq > window ? seq - window : 0 (window 0 =
 * full causal).  The reference's scratch is n*heads*cap f32 of scores; this
 * implementation streams key blocks through registers and only requires
 * `scratch` to be a valid buffer (>= 4 bytes). */
int tm_cuda_qwen35_attention_f16_chunk(tm_cuda_ctx *ctx, tm_cuda_buffer *q,
                                       tm_cuda_buffer *k_cache, tm_cuda_buffer *v_cache,
                                       tm_cuda_buffer *out, tm_cuda_buffer *scratch,
                                       uint32_t heads, uint32_t pos0, uint32_t cap,
                                       uint32_t head_dim, uint32_t group, float scale, uint32_t n,
                                       uint32_t window, char *err, size_t err_cap);

/* No counterpart: the batched-prefill forms that fold the surrounding elementwise
 * launches into the tensor-core GEMM (tolerance-qualified like tm_cuda_q8_0_gemm_mma).
 * One call = the f16 copy of X with `prologue` applied (TM_CUDA_PRO_NONE; _RMSNORM:
 * x * rsqrt(mean x^2 + eps) * pro[cols]; _SILU_MUL / _GELU_MUL: act(x) * pro[batch][cols])
 * + ONE GEMM launch over the whole matrix whose rows are cut into n_parts (1..3)
 * consecutive parts -- q | k | v, gate | up -- each written densely to its own
 * y_parts[p][t * part_rows[p] + r]; every part but the last must be a multiple of 128
 * rows.  epilogue TM_CUDA_EPI_ADD accumulates into y (the residual add). */
int tm_cuda_q8_0_gemm_mma_fused(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, uint32_t rows,
                                uint32_t cols, uint32_t batch, uint32_t n_parts,
                                tm_cuda_buffer *const *y_parts, const uint32_t *part_rows, int prologue,
                                tm_cuda_buffer *pro, float eps, int epilogue, char *err, size_t err_cap);
/* No counterpart: tm_cuda_rmsnorm_f32 (q heads), tm_cuda_rmsnorm_f32 (k heads),
 * tm_cuda_qwen35_rope_partial_chunk and tm_cuda_qwen35_kv_store_f16_chunk as one
 * launch for a chunk of n token rows at pos0: q [n][heads][head_dim] is normed and
 * rotated in place; k is normed, rotated and stored to the f16 cache with v (k and v
 * themselves are not modified).  Warp-level sums: tolerance-qualified. */
int tm_cuda_qk_prep_chunk(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k, tm_cuda_buffer *v,
                          tm_cuda_buffer *q_norm, tm_cuda_buffer *k_norm, tm_cuda_buffer *inv_freq,
                          tm_cuda_buffer *k_cache, tm_cuda_buffer *v_cache, uint32_t heads,
                          uint32_t kv_heads, uint32_t head_dim, uint32_t n_rot, uint32_t pos0, uint32_t cap,
                          uint32_t n, float eps, char *err, size_t err_cap);

/* No counterpart: the same operator as tm_cuda_qwen35_attention_f16_chunk on the
 * tensor cores (mma.sync m16n8k16: Q and the softmax weights rounded to binary16,
 * f32 accumulation, keys visited in tiles of 64 with a running maximum), hence
 * tolerance-qualified (about 1e-3 of the output scale) instead of bit-identical
 * to the per-token form.  The engine uses it for batched prefill unless `exact`
 * is asked.  head_dim 32, 64, 128 or 256; buffers 16-byte aligned; no scratch. */
int tm_cuda_attention_chunk_mma_supported(uint32_t head_dim);
int tm_cuda_attention_chunk_mma(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k_cache,
                                tm_cuda_buffer *v_cache, tm_cuda_buffer *out, uint32_t heads,
                                uint32_t pos0, uint32_t cap, uint32_t head_dim, uint32_t group,
                                float scale, uint32_t n, uint32_t window, char *err, size_t err_cap);

/* No counterpart: the per-token attention core with the position read from
 * device memory (u32 pos_buf[pos_index]), so one recorded decode graph serves
 * every step: per-head q/k RMS norm, RoPE, f16 KV store and (windowed) causal
 * attention for ONE token -- the sequence of tm_cuda_rmsnorm_f32 x2,
 * tm_cuda_qwen35_rope_partial, tm_cuda_qwen35_kv_store_f16 and
 * tm_cuda_qwen35_attention_f16_chunk(n = 1): bit for bit with `exact` = 1;
 * with `exact` = 0 a latency-optimised kernel with the same mathematics and a
 * different summation order (tolerance-qualified) runs where it applies.  A
 * position >= cap writes nothing and sets bit 0 of status[0] (u32, shared).
 * `scratch` holds the per-key-block partial results and arrival counters
 * (tm_cuda_attention_decode_scratch_bytes, zero-filled once by the caller;
 * the kernel leaves the counters at zero).  Calls sharing one scratch buffer
 * must be ordered on the stream.
 * Cache contract: the kernel reads cache rows below `pos` while kernels
 * launched before it on the stream may still be running (programmatic
 * dependent launch).  Row pos - 1 is read again once they have finished, and
 * an attention kernel lets its successor start only after its own predecessor
 * is complete, so any sequence of decode calls at pos, pos + 1, pos + 2, ... on
 * one cache is safe however close together the calls are issued (one dispatch
 * group included).  Rows that something OTHER than this operator wrote (a
 * prefill chunk, a host upload) must be complete when the call is made, which
 * every earlier dispatch group, graph launch or upload is. */
size_t tm_cuda_attention_decode_scratch_bytes(uint32_t heads, uint32_t kv_heads, uint32_t head_dim,
                                              uint32_t cap);
int tm_cuda_attention_decode_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k,
                                 tm_cuda_buffer *v, tm_cuda_buffer *q_norm, tm_cuda_buffer *k_norm,
                                 tm_cuda_buffer *inv_freq, tm_cuda_buffer *k_cache,
                                 tm_cuda_buffer *v_cache, tm_cuda_buffer *out,
                                 tm_cuda_buffer *scratch, tm_cuda_buffer *pos_buf,
                                 uint32_t pos_index, tm_cuda_buffer *status, uint32_t heads,
                                 uint32_t kv_heads, uint32_t head_dim, uint32_t n_rot,
                                 uint32_t cap, uint32_t window, float eps, float scale, int exact,
                                 char *err, size_t err_cap);
/* No counterpart in the reference.  tm_cuda_attention_decode_dev for callers that
 * must not allocate: a serving process that has handed every byte of HBM to its
 * own arena at start-up, so that a later cudaMalloc fails or forces the driver
 * to synchronise the whole device in the middle of a token; or a host that is
 * only allowed to touch memory it was given (a sandboxed plug-in, a worker
 * whose ledger must equal its plan to the byte).  Such a caller has no buffer
 * to pass as `scratch`, so this variant takes none: the per-key-block partials
 * and the arrival counters live in an array built into the library image (one
 * copy on every device that loads the library, kept until the process exits).
 * Limit: tm_cuda_attention_decode_scratch_bytes(heads, kv_heads, head_dim, cap)
 * must not exceed tm_cuda_attention_decode_static_max_scratch() (9 MiB: e.g. 16
 * heads x 128 dims up to a capacity of ~36000, 64 heads x 128 up to ~9000); a
 * larger geometry is refused with TM_CUDA_ERR_BOUNDS and a message naming both
 * sizes.  The first call on a device looks the array's device address up
 * (cudaGetSymbolAddress); make that first call before any stream capture
 * begins.  Every call on a device shares the one array and each call clears
 * the counters it is about to use, so two calls whose kernels overlap on the
 * GPU (different streams or contexts of one device) race: keep them ordered.
 * Inputs, outputs and results are those of tm_cuda_attention_decode_dev.  The
 * call launches directly on the context's stream and is not entered in the
 * committed / completed dispatch counters or the profile table. */
size_t tm_cuda_attention_decode_static_max_scratch(void);
int tm_cuda_attention_decode_dev_static(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k,
                                        tm_cuda_buffer *v, tm_cuda_buffer *q_norm, tm_cuda_buffer *k_norm,
                                        tm_cuda_buffer *inv_freq, tm_cuda_buffer *k_cache,
                                        tm_cuda_buffer *v_cache, tm_cuda_buffer *out,
                                        tm_cuda_buffer *pos_buf, uint32_t pos_index, tm_cuda_buffer *status,
                                        uint32_t heads, uint32_t kv_heads, uint32_t head_dim, uint32_t n_rot,
                                        uint32_t cap, uint32_t window, float eps, float scale, int exact,
                                        char *err, size_t err_cap);
/* No counterpart: decode steps of SEVERAL sequences in one recorded graph (the reference serves one
 * request at a time, crates/supervisor/src/queue.rs:1-4).  A step of n_seq sequences is a batch of
 * n_seq rows through the batched projections (tm_cuda_q8_0_gemm / _gemm_mma), with these operators
 * around them; sequence s owns position pos_buf[s] (consecutive u32), the s-th row of every
 * activation matrix, the s-th cache plane pair and the s-th token log.
 * tm_cuda_attention_decode_batch_dev: tm_cuda_attention_decode_dev for every sequence in ONE launch.
 * Row s of q starts at element s * q_stride (0 = dense, heads * head_dim), rows of k and v at
 * s * kv_stride (0 = kv_heads * head_dim) -- so the three may be views into one [n_seq][q|k|v]
 * projection output; the caches are [n_seq][kv_heads][cap][head_dim] f16, out is dense
 * [n_seq][heads * head_dim], scratch n_seq regions of
 * tm_cuda_attention_decode_scratch_bytes (zero-filled once).  Results per sequence are those of the
 * single call, bit for bit (same kernels, one more grid dimension); a sequence whose position is
 * >= cap writes nothing and sets bit 0 of status[0]. */
int tm_cuda_attention_decode_batch_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k, tm_cuda_buffer *v,
                                       tm_cuda_buffer *q_norm, tm_cuda_buffer *k_norm, tm_cuda_buffer *inv_freq,
                                       tm_cuda_buffer *k_cache, tm_cuda_buffer *v_cache, tm_cuda_buffer *out,
                                       tm_cuda_buffer *scratch, tm_cuda_buffer *pos_buf, tm_cuda_buffer *status,
                                       uint32_t n_seq, uint32_t q_stride, uint32_t kv_stride, uint32_t heads,
                                       uint32_t kv_heads, uint32_t head_dim,
                                       uint32_t n_rot, uint32_t cap, uint32_t window, float eps, float scale,
                                       int exact, char *err, size_t err_cap);
/* out[s] = row ids[s * ids_stride + pos_buf[s] + bias] of the packed Q8_0 matrix (times `scale` when
 * non-zero), s < n_seq: the embedding rows of a batched step, each sequence reading its own token
 * log at its own position.  A slot outside the log or an id >= rows writes zeros. */
int tm_cuda_rows_indirect_seq_f32_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows, uint32_t cols,
                                      tm_cuda_buffer *ids, uint32_t ids_stride, tm_cuda_buffer *pos_buf,
                                      uint32_t n_seq, int32_t bias, float scale, tm_cuda_buffer *out, char *err,
                                      size_t err_cap);
/* Greedy choice of n_rows rows of n logits in two launches: row r's winner (the rule of
 * tm_cuda_argmax_f32) goes to out[r * out_stride + base + pos_buf[r]] (and to `mirror`, when given)
 * if base + pos_buf[r] < out_cap <= out_stride.  `partial` holds n_rows * 512 bytes. */
int tm_cuda_argmax_rows_f32_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *x, uint32_t n_rows, uint32_t n,
                                tm_cuda_buffer *partial, tm_cuda_buffer *out, uint32_t out_stride, uint32_t base,
                                tm_cuda_buffer *pos_buf, uint32_t out_cap, tm_cuda_buffer *mirror, char *err,
                                size_t err_cap);
/* buf[first + i] = min(buf[first + i] + delta, limit), i < count: advances every sequence's position;
 * a sequence that has filled its cache stays on its last row instead of running past it. */
int tm_cuda_u32_add_sat(tm_cuda_ctx *ctx, tm_cuda_buffer *buf, uint32_t first, uint32_t count, uint32_t delta,
                        uint32_t limit, char *err, size_t err_cap);
/* No counterpart: buf[index] += delta (u32), to advance a device position
 * inside a recorded graph. */
int tm_cuda_u32_add(tm_cuda_ctx *ctx, tm_cuda_buffer *buf, uint32_t index, uint32_t delta,
                    char *err, size_t err_cap);
/* No counterpart: argmax whose output index is taken from the device,
 * out[base + pos_buf[pos_index]], so a replayed graph appends each step's
 * token to a device-side token log; `mirror` (optional, same length, shared)
 * receives the same value for the host to read with download_after. */
int tm_cuda_argmax_f32_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *x, uint32_t n,
                           tm_cuda_buffer *partial, tm_cuda_buffer *out, uint32_t base,
                           tm_cuda_buffer *pos_buf, uint32_t pos_index, uint32_t out_cap,
                           tm_cuda_buffer *mirror, char *err, size_t err_cap);
/* No counterpart: tm_cuda_row_indirect_f32 whose slot is base +
 * pos_buf[pos_index] + bias (bias may be negative: "the previous token"),
 * followed by an optional scale (0 = none). */
int tm_cuda_row_indirect_f32_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows, uint32_t cols,
                                 tm_cuda_buffer *ids, uint32_t base, tm_cuda_buffer *pos_buf,
                                 uint32_t pos_index, int32_t bias, float scale,
                                 tm_cuda_buffer *out, char *err, size_t err_cap);

/* ---------------- multi-GPU output-row split (no counterpart: the reference is
 * single-device) ----------------
 * Rank r of `world` GPUs of one box owns rows [r*N/world, (r+1)*N/world) of every
 * projection and of the lm_head, runs the operators above on its slice, and an
 * all-gather over NVLink reassembles each output vector.  NCCL is loaded at run
 * time; a process that never calls these needs no NCCL. */
/* 128-byte rendezvous id, created on one rank and handed to the others by the host. */
int tm_cuda_comm_unique_id(void *out128, char *err, size_t err_cap);
/* Join the communicator (collective over all ranks; one per context). */
int tm_cuda_comm_init(tm_cuda_ctx *ctx, const void *id128, int rank, int world, char *err, size_t err_cap);
int tm_cuda_comm_rank(const tm_cuda_ctx *ctx, int *rank, int *world);
/* dst[dst_off + r*count + i] = rank r's src[src_off + i]; on the context's stream,
 * recordable in a dispatch group. */
int tm_cuda_all_gather_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *src, uint32_t src_off, tm_cuda_buffer *dst,
                           uint32_t dst_off, uint32_t count, char *err, size_t err_cap);
/* Row-wise form for a chunk of n_rows token rows: dst[t][r*width + c] = rank r's
 * src[t][c].  `stage` (world*n_rows*width f32) receives NCCL's rank-major result
 * before the interleave; unused when n_rows == 1. */
int tm_cuda_all_gather_rows_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *src, tm_cuda_buffer *stage, tm_cuda_buffer *dst,
                                uint32_t n_rows, uint32_t width, char *err, size_t err_cap);
/* The same exchange through PEER MEMORY instead of a library collective.  A
 * symmetric buffer is the same allocation on every rank, each mapped into every
 * other rank's address space (CUDA IPC; collective call, outside dispatch groups,
 * after tm_cuda_comm_init).  tm_cuda_push_rows_f32 is then the all-gather as a
 * push: one kernel stores this rank's n_rows x width slice straight into every
 * rank's copy at dst[t][rank*width + c] (plain stores over NVLink), raises a
 * per-sender sequence flag on every rank and waits, with an iteration limit, until
 * every sender's flag on this rank has reached the same number -- when the kernel
 * ends, dst holds all ranks' slices.  Recordable in a dispatch group.  The same
 * symmetric buffer must not be the target of two consecutive pushes (a peer may
 * still be reading the previous contents); alternate between at least two.  Bit 0
 * of tm_cuda_symm_status: a wait ran out (the consumer read stale rows). */
tm_cuda_buffer *tm_cuda_symm_alloc(tm_cuda_ctx *ctx, size_t bytes, char *err, size_t err_cap);
/* The tensor-core GEMM and the exchange as ONE kernel: the epilogue of
 * tm_cuda_q8_0_gemm_mma stores each finished tile of this rank's `rows` output rows
 * straight into every rank's gathered Y (dst[t][rank*rows + r], dst a symmetric buffer
 * or a view of one), so the transfer of a tile overlaps the MMAs of the next; the
 * last CTA ends the exchange like tm_cuda_push_rows_f32 does.  STORE only. */
int tm_cuda_q8_0_gemm_mma_push(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *dst,
                               uint32_t rows, uint32_t cols, uint32_t batch, char *err, size_t err_cap);

int tm_cuda_push_rows_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *src, tm_cuda_buffer *dst, uint32_t n_rows, uint32_t width,
                          char *err, size_t err_cap);
int tm_cuda_symm_status(tm_cuda_ctx *ctx, tm_cuda_buffer *buf, uint32_t *status, char *err, size_t err_cap);
/* Greedy token of a row-sharded head: argmax of the local logits slice (global
 * index = local + index_offset), all-gather of the (value, index) pairs (8 bytes
 * per rank instead of the logits), then the single-device rule over the pairs
 * (larger value, ties to the lower GLOBAL index), so every rank writes the token
 * one device would have chosen to out[base + pos_buf[pos_index]] (pos_buf may be
 * NULL: out[base]).  `pairs` holds (world + 1) * 8 bytes. */
int tm_cuda_argmax_sharded_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *x, uint32_t n, uint32_t index_offset,
                               tm_cuda_buffer *partial, tm_cuda_buffer *pairs, tm_cuda_buffer *out, uint32_t base,
                               tm_cuda_buffer *pos_buf, uint32_t pos_index, uint32_t out_cap,
                               tm_cuda_buffer *mirror, char *err, size_t err_cap);
/* The reduction of a projection split by COLUMNS over the ranks (each rank multiplies its column
 * range by its own slice of the input and holds a full-width partial product): `slots` is
 * [world][n_rows][cols] f32 with rank r's partial in slot r (tm_cuda_push_rows_f32 with one row of
 * n_rows * cols values puts it there on every rank); x[t][c] += slots[0][t][c] + slots[1][t][c] + ...
 * added in rank order, so every rank computes the same bits.  With `weight` (may be NULL) the sum is
 * RMS-normed with that weight before it is added (a layer's output norm; slot 0 is overwritten). */
int tm_cuda_reduce_ranks_add_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *slots, tm_cuda_buffer *x, tm_cuda_buffer *weight,
                                 uint32_t world, uint32_t n_rows, uint32_t cols, float eps, char *err, size_t err_cap);
/* No counterpart.  The push and the reduction above as ONE launch for one row (a decode step of one
 * sequence): y[c] += src_0[c] + src_1[c] + ... over the ranks' `src` rows, added in rank order (the
 * bits of tm_cuda_push_rows_f32 + tm_cuda_reduce_ranks_add_f32 without a weight).  `slots` is a
 * view of a symmetric buffer of world * width 8-byte words: every value travels as a (value,
 * exchange number) pair written with one store, and a reader polls the pair it needs until it carries
 * this exchange's number -- no fence, no flag, no second kernel.  The polls are bounded; one that runs
 * out sets bit 0 of tm_cuda_symm_status and the sum takes what the slot holds.  Every rank must issue
 * the same sequence of these calls on the buffer, and two CONSECUTIVE calls must not use the same
 * view (a fast rank would overwrite a pair a slow rank has not read yet); a view may be reused
 * once another exchange lies between. */
int tm_cuda_exchange_add_ll_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *src, tm_cuda_buffer *slots, tm_cuda_buffer *y,
                                uint32_t width, char *err, size_t err_cap);
/* The same for n_rows rows in one exchange (a decode step of several sequences on a split model):
 * row r of the local [n_rows][n] logits slice; its winner over all ranks goes to
 * out[r * out_stride + base + pos_buf[r]] when that slot is below out_cap <= out_stride.
 * `partial` holds n_rows * 512 bytes, `pairs` (world + 1) * n_rows * 8. */
int tm_cuda_argmax_rows_sharded_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *x, uint32_t n_rows, uint32_t n,
                                    uint32_t index_offset, tm_cuda_buffer *partial, tm_cuda_buffer *pairs,
                                    tm_cuda_buffer *out, uint32_t out_stride, uint32_t base, tm_cuda_buffer *pos_buf,
                                    uint32_t out_cap, tm_cuda_buffer *mirror, char *err, size_t err_cap);

#ifdef __cplusplus
}
#endif

#endif /* TM_CUDA_H */
