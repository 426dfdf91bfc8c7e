#include "engine.hpp"

#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>

namespace tuckmill {

namespace {

uint64_t f32_bytes(size_t elems) { return 4ull * (elems ? elems : 1); }

// Allocation accumulator mirroring every buffer a block creates
// (crates/tuckcore/src/engine/metal.rs:254-272).
inline size_t gather_bytes(size_t n) { return (f32_bytes(n) + 255) / 256 * 256; }

struct Plan {
    uint64_t weights = 0, state = 0, scratch = 0, gather = 0;
    // A buffer other ranks store into when the model is split, an ordinary one otherwise.
    void target_f32(size_t n, uint32_t world) {
        if (world > 1) {
            scratch += gather_bytes(n);
            gather += gather_bytes(n);
        } else {
            scratch += f32_bytes(n);
        }
    }
    void weights_f32(size_t n) { weights += f32_bytes(n); }
    void scratch_f32(size_t n) { scratch += f32_bytes(n); }
    void scratch_bytes(size_t n) { scratch += n ? n : 4; }
};

size_t vector_len(const WeightSource &src, Tensor t) {
    auto d = src.tensor_dims(t.index);
    return (size_t)(d.first * (d.second ? d.second : 1));
}

// With a row split the gather targets of every exchange live in ONE buffer that all ranks map
// (peer memory); blocks take 256-byte aligned views of it in plan order.
struct GatherArena {
    CudaBuffer buf;
    size_t off = 0;
};

struct Shard {
    uint32_t rank = 0, world = 1;
    GatherArena *arena = nullptr;  // set while loading a split model
    // One-row exchanges as a single launch of (value, number) pairs (tm_cuda_exchange_add_ll_f32)
    // instead of push + reduction; the one-row targets are sized for the pairs either way.
    bool pair_exchange = false;
};

// Gather targets of a row split are exchange buffers every rank can store into.
CudaBuffer gather_target_f32(const CudaContext &ctx, size_t n, const Shard &sh) {
    if (sh.world <= 1) return ctx.zeros(f32_bytes(n));
    if (!sh.arena || sh.arena->off + gather_bytes(n) > sh.arena->buf.len())
        throw TuckmillError(ErrorCode::Internal, "exchange arena smaller than the plan");
    CudaBuffer v = sh.arena->buf.view(sh.arena->off, f32_bytes(n));
    sh.arena->off += gather_bytes(n);
    return v;
}

CudaBuffer vector(const CudaContext &ctx, const WeightSource &src, Tensor t) {
    std::vector<float> v = src.read_vector(t.index);
    return ctx.floats(v);
}

CudaBuffer zeros_f32(const CudaContext &ctx, size_t elems) { return ctx.zeros(f32_bytes(elems)); }

// RoPE inverse-frequency table, f64 pow then f32 (crates/tuckcore/src/qwen35_ops.rs:265-272).
std::vector<float> rope_inv_freq(size_t rope_dims, float base) {
    std::vector<float> out(rope_dims / 2);
    for (size_t i = 0; i < out.size(); ++i) {
        const double exponent = 2.0 * (double)i / (double)rope_dims;
        out[i] = (float)(1.0 / std::pow((double)base, exponent));
    }
    return out;
}

// The split over `world` devices: q|k|v, gate|up and the head are cut by OUTPUT ROWS (rank r owns rows
// [r*N/world, (r+1)*N/world): whole attention heads, a slice of the FFN width, a slice of the
// vocabulary), so attention and the gated activation stay on the rank; o and down are cut by INPUT
// COLUMNS (Matrix::load_cols: the columns that multiply this rank's heads / FFN slice), each rank
// produces a full-width partial product and one exchange per projection adds the partials in rank
// order -- two exchanges per layer, none between a rank's q|k|v and its o, or its gate|up and its down.
// A device matrix: one or more Q8_0 tensors of equal width, rows concatenated,
// repacked into the two-plane form at upload (crates/tuckcore/src/engine/
// metal.rs:107-226 uploads the GGUF bytes verbatim; the row concatenation and
// the repack are this engine's).
struct Matrix {
    CudaBuffer buf;
    std::vector<CudaBuffer> parts;  // row views, one per source tensor (empty when single)
    std::vector<uint32_t> part_rows;
    uint32_t rows = 0, cols = 0;
    uint32_t type = 8;  // GGML type of the source tensors: 8 = Q8_0 (repacked), 1 = F16 (verbatim)

    static void geometry(const WeightSource &src, const std::vector<Tensor> &ts, Shard sh, uint32_t *rows,
                         uint32_t *cols, uint32_t *type = nullptr) {
        *rows = 0;
        *cols = 0;
        uint32_t seen = 0;
        for (Tensor t : ts) {
            const uint32_t ty = src.tensor_type_id(t.index);
            auto d = src.tensor_dims(t.index);
            if (d.second <= 1)
                throw TuckmillError(ErrorCode::Internal,
                                    "tensor " + std::to_string(t.index) + " is 1-D; vectors use the f32 path");
            // F16 or Q8_0, like the reference's Matrix::load (engine/metal.rs:129-137)
            if (ty != 8 && ty != 1)
                throw TuckmillError(ErrorCode::UnsupportedQuantization,
                                    "CUDA engine matrices must be Q8_0 or F16; tensor " + std::to_string(t.index) +
                                        " is type " + std::to_string(ty));
            if (seen != 0 && seen != ty)
                throw TuckmillError(ErrorCode::UnsupportedQuantization, "fused projections differ in type");
            seen = ty;
            if ((ty == 8 && d.first % 32 != 0) || d.first > UINT32_MAX || d.second > UINT32_MAX)
                throw TuckmillError(ErrorCode::InvalidArtifact, "Q8_0 tensor rows are not block aligned");
            if (*cols != 0 && *cols != (uint32_t)d.first)
                throw TuckmillError(ErrorCode::Internal, "fused projections differ in input width");
            if (d.second % sh.world != 0)
                throw TuckmillError(ErrorCode::InvalidRequest,
                                    "tensor " + std::to_string(t.index) + " has " + std::to_string(d.second) +
                                        " rows, not divisible by the " + std::to_string(sh.world) + " devices of the split");
            *cols = (uint32_t)d.first;
            *rows += (uint32_t)(d.second / sh.world);
        }
        if (type) *type = seen;
    }

    static uint64_t bytes_of(uint32_t type, uint32_t rows, uint32_t cols) {
        return type == 1 ? (uint64_t)rows * cols * 2 : tm_cuda_q8_0_packed_bytes(rows, cols);
    }

    static uint64_t plan(const WeightSource &src, const std::vector<Tensor> &ts, Shard sh = Shard()) {
        uint32_t rows, cols, type;
        geometry(src, ts, sh, &rows, &cols, &type);
        return bytes_of(type, rows, cols);
    }

    // Column shard of ONE tensor: every row, this rank's cols/world columns of it (whole Q8_0 blocks).
    static void geometry_cols(const WeightSource &src, Tensor t, Shard sh, uint32_t *rows, uint32_t *cols,
                              uint32_t *type) {
        Shard whole;
        geometry(src, {t}, whole, rows, cols, type);
        if (*cols % sh.world != 0 || (*type == 8 && (*cols / sh.world) % 32 != 0) || (*type == 1 && (*cols / sh.world) % 8 != 0))
            throw TuckmillError(ErrorCode::InvalidRequest, "tensor " + std::to_string(t.index) + " has " +
                                                               std::to_string(*cols) + " columns, which do not divide into " +
                                                               std::to_string(sh.world) + " block-aligned ranges");
        *cols /= sh.world;
    }
    static uint64_t plan_cols(const WeightSource &src, Tensor t, Shard sh) {
        uint32_t rows, cols, type;
        geometry_cols(src, t, sh, &rows, &cols, &type);
        return bytes_of(type, rows, cols);
    }
    static Matrix load_cols(const CudaContext &ctx, const WeightSource &src, Tensor t, Shard sh) {
        Matrix m;
        geometry_cols(src, t, sh, &m.rows, &m.cols, &m.type);
        const bool q8 = m.type == 8;
        const size_t full_row = q8 ? (size_t)m.cols * sh.world / 32 * 34 : (size_t)m.cols * sh.world * 2;
        const size_t row_bytes = q8 ? (size_t)m.cols / 32 * 34 : (size_t)m.cols * 2;
        const size_t col0 = (size_t)sh.rank * row_bytes;  // this rank's bytes inside a source row
        m.buf = ctx.buffer(bytes_of(m.type, m.rows, m.cols));
        const size_t step = std::max<size_t>(1, kStagingChunkBytes / row_bytes);
        std::vector<unsigned char> host(step * row_bytes);
        CudaBuffer stage;
        if (q8) stage = ctx.buffer(step * row_bytes);  // transient: freed before the ledger is checked
        for (uint32_t r = 0; r < m.rows; r += (uint32_t)step) {
            const uint32_t k = std::min<uint32_t>((uint32_t)step, m.rows - r);
            for (uint32_t i = 0; i < k; ++i)
                src.read_tensor_into(t.index, (size_t)(r + i) * full_row + col0, host.data() + (size_t)i * row_bytes,
                                     row_bytes);
            if (q8) {
                stage.upload(0, host.data(), (size_t)k * row_bytes);
                ctx.q8_0_pack(m.buf, m.rows, m.cols, stage, 0, r, k);
            } else {
                m.buf.upload((size_t)r * row_bytes, host.data(), (size_t)k * row_bytes);
            }
        }
        ctx.fence();
        m.part_rows.push_back(m.rows);
        return m;
    }

    // F16: the tensor bytes verbatim, row ranges uploaded straight into place.
    static Matrix load_f16(const CudaContext &ctx, const WeightSource &src, const std::vector<Tensor> &ts, Shard sh,
                           Matrix m) {
        m.buf = ctx.buffer(bytes_of(1, m.rows, m.cols));
        const size_t row_bytes = (size_t)m.cols * 2;
        const size_t step = std::max<size_t>(1, kStagingChunkBytes / row_bytes);
        std::vector<unsigned char> host(step * row_bytes);
        uint32_t row0 = 0;
        for (Tensor t : ts) {
            const uint32_t n = (uint32_t)(src.tensor_dims(t.index).second / sh.world);
            const uint64_t first = (uint64_t)sh.rank * n;
            for (uint32_t r = 0; r < n; r += (uint32_t)step) {
                const uint32_t k = std::min<uint32_t>((uint32_t)step, n - r);
                src.read_tensor_into(t.index, (first + r) * row_bytes, host.data(), (size_t)k * row_bytes);
                m.buf.upload((size_t)(row0 + r) * row_bytes, host.data(), (size_t)k * row_bytes);
            }
            m.part_rows.push_back(n);
            row0 += n;
        }
        if (ts.size() > 1) {
            uint32_t r = 0;
            for (uint32_t n : m.part_rows) {
                if (((size_t)r * row_bytes) % 16 != 0)
                    throw TuckmillError(ErrorCode::UnsupportedArchitecture, "a fused F16 projection does not start on a 16-byte boundary");
                m.parts.push_back(m.buf.view((size_t)r * row_bytes, (size_t)n * row_bytes));
                r += n;
            }
        }
        return m;
    }

    static Matrix load(const CudaContext &ctx, const WeightSource &src, const std::vector<Tensor> &ts,
                       Shard sh = Shard()) {
        Matrix m;
        geometry(src, ts, sh, &m.rows, &m.cols, &m.type);
        if (m.type == 1) return load_f16(ctx, src, ts, sh, std::move(m));
        m.buf = ctx.buffer(tm_cuda_q8_0_packed_bytes(m.rows, m.cols));
        const size_t row_bytes = (size_t)m.cols / 32 * 34;
        const size_t step = std::max<size_t>(1, kStagingChunkBytes / row_bytes);
        CudaBuffer stage = ctx.buffer(step * row_bytes);  // transient: freed before the ledger is checked
        std::vector<unsigned char> host(step * row_bytes);
        uint32_t row0 = 0;
        for (Tensor t : ts) {
            const uint32_t n = (uint32_t)(src.tensor_dims(t.index).second / sh.world);
            const uint64_t first = (uint64_t)sh.rank * n;  // this rank's first row of the tensor
            for (uint32_t r = 0; r < n; r += (uint32_t)step) {
                const uint32_t k = std::min<uint32_t>((uint32_t)step, n - r);
                src.read_tensor_into(t.index, (first + r) * row_bytes, host.data(), (size_t)k * row_bytes);
                stage.upload(0, host.data(), (size_t)k * row_bytes);
                ctx.q8_0_pack(m.buf, m.rows, m.cols, stage, 0, row0 + r, k);
            }
            m.part_rows.push_back(n);
            row0 += n;
        }
        ctx.fence();
        if (ts.size() > 1) {
            uint32_t r = 0;
            for (uint32_t n : m.part_rows) {
                m.parts.push_back(ctx.row_view(m.buf, m.rows, m.cols, r, n));
                r += n;
            }
        }
        return m;
    }

    // Y[b] = W X[b].  Batch 1 and `exact` keep the GEMV's per-row arithmetic in
    // slices of at most 32 tokens; other batches use the tensor cores in one
    // launch (the dispatch rule of engine/metal.rs:167-196).
    static void gemm(const CudaContext &ctx, const CudaBuffer &w, uint32_t rows, uint32_t cols, const CudaBuffer &x,
                     const CudaBuffer &y, uint32_t batch, bool exact, uint32_t type = 8) {
        if (type == 1) {  // F16: the per-row kernel in slices (engine/metal.rs:181-195 keeps F16 off the matrix units too)
            for (uint32_t t0 = 0; t0 < batch; t0 += TM_CUDA_GEMM_MAX_BATCH) {
                const uint32_t n = std::min<uint32_t>(batch - t0, TM_CUDA_GEMM_MAX_BATCH);
                ctx.f16_gemm(w, x, y, rows, cols, n, t0 * cols, t0 * rows);
            }
            return;
        }
        if (!exact && batch >= 2 && batch <= TM_CUDA_GEMM_MMA_MAX_BATCH) {
            ctx.q8_0_gemm_mma(w, x, y, rows, cols, batch, 0, 0);
            return;
        }
        for (uint32_t t0 = 0; t0 < batch; t0 += TM_CUDA_GEMM_MAX_BATCH) {
            const uint32_t n = std::min<uint32_t>(batch - t0, TM_CUDA_GEMM_MAX_BATCH);
            ctx.q8_0_gemm(w, x, y, rows, cols, n, t0 * cols, t0 * rows);
        }
    }
    void gemm_part(const CudaContext &ctx, size_t part, const CudaBuffer &x, const CudaBuffer &y, uint32_t batch,
                   bool exact) const {
        gemm(ctx, parts[part], part_rows[part], cols, x, y, batch, exact, type);
    }
    void gemm_all(const CudaContext &ctx, const CudaBuffer &x, const CudaBuffer &y, uint32_t batch, bool exact) const {
        gemm(ctx, buf, rows, cols, x, y, batch, exact, type);
    }
    // One token, with the neighbouring elementwise operators folded in (include/tm_cuda.h).
    void gemv_fused(const CudaContext &ctx, const CudaBuffer &x, const CudaBuffer &y, int prologue, const CudaBuffer *pro,
                    float eps, int epilogue) const {
        if (type == 1) ctx.f16_gemv_fused(buf, x, y, rows, cols, prologue, pro, eps, epilogue);
        else ctx.q8_0_gemv_fused(buf, x, y, rows, cols, prologue, pro, eps, epilogue);
    }
    void gemv(const CudaContext &ctx, const CudaBuffer &x, const CudaBuffer &y) const {
        gemv_fused(ctx, x, y, TM_CUDA_PRO_NONE, nullptr, 0.0f, TM_CUDA_EPI_STORE);
    }
};

// Chunk-wide scratch shared by every layer (engine/metal.rs:334-425): rows are
// token-major, `n` = prefill batch.
struct PrefillScratch {
    CudaBuffer x, h, a, b, c, e, proj, h2, g, u, d2, ascr;
    CudaBuffer loc, loc2;  // split only: a rank's local GEMM outputs
    static size_t widest(const ModelGraph &g) {
        size_t w = g.hidden;
        for (const LayerSpec &l : g.layers) w = std::max(w, std::max(l.mixer.heads * l.mixer.head_dim, l.ffn.width));
        return w;
    }
    // f16 copy of the widest GEMM input of a chunk (the tensor-core GEMM's TMA source).
    static size_t mma_workspace(const ModelGraph &g, size_t n) {
        size_t widest = g.hidden;
        for (const LayerSpec &l : g.layers)
            widest = std::max(widest, std::max(l.mixer.heads * l.mixer.head_dim, l.ffn.width));
        return tm_cuda_mma_workspace_bytes((uint32_t)widest, (uint32_t)n);
    }
    static void plan(const ModelGraph &g, size_t cap, size_t n, Shard sh, Plan &p) {
        if (sh.world > 1)
            for (int i = 0; i < 2; ++i) p.scratch_f32(n * widest(g));  // loc, loc2
        size_t aw = 0, kvw = 0, ffn = 0, heads = 0;
        for (const LayerSpec &l : g.layers) {
            aw = std::max(aw, l.mixer.heads * l.mixer.head_dim);
            kvw = std::max(kvw, l.mixer.kv_heads * l.mixer.head_dim);
            ffn = std::max(ffn, l.ffn.width);
            heads = std::max(heads, l.mixer.heads);
        }
        for (size_t e : {g.hidden, g.hidden, aw, kvw, kvw, aw, g.hidden, ffn})  // x h a b c e h2 u
            p.scratch_f32(n * e);
        // proj, d2: every rank's full-width partial product lands here when the model is split
        for (int i = 0; i < 2; ++i) p.target_f32(n * g.hidden * sh.world, sh.world);
        p.scratch_f32(sh.world > 1 ? 1 : n * ffn);  // g (a split rank keeps its gate slice in loc)
        (void)heads;
        (void)cap;
        p.scratch_f32(1);  // the chunk attention streams key blocks; its scratch argument is a placeholder
    }
    static PrefillScratch alloc(const CudaContext &ctx, const ModelGraph &g, size_t cap, size_t n, Shard sh) {
        size_t aw = 0, kvw = 0, ffn = 0, heads = 0;
        for (const LayerSpec &l : g.layers) {
            aw = std::max(aw, l.mixer.heads * l.mixer.head_dim);
            kvw = std::max(kvw, l.mixer.kv_heads * l.mixer.head_dim);
            ffn = std::max(ffn, l.ffn.width);
            heads = std::max(heads, l.mixer.heads);
        }
        PrefillScratch s;
        s.x = zeros_f32(ctx, n * g.hidden);
        s.h = zeros_f32(ctx, n * g.hidden);
        s.a = zeros_f32(ctx, n * aw);
        s.b = zeros_f32(ctx, n * kvw);
        s.c = zeros_f32(ctx, n * kvw);
        s.e = zeros_f32(ctx, n * aw);
        s.proj = gather_target_f32(ctx, n * g.hidden * sh.world, sh);
        s.h2 = zeros_f32(ctx, n * g.hidden);
        s.g = zeros_f32(ctx, sh.world > 1 ? 1 : n * ffn);
        s.u = zeros_f32(ctx, n * ffn);
        s.d2 = gather_target_f32(ctx, n * g.hidden * sh.world, sh);
        (void)heads;
        (void)cap;
        s.ascr = zeros_f32(ctx, 1);
        if (sh.world > 1) {
            s.loc = zeros_f32(ctx, n * widest(g));
            s.loc2 = zeros_f32(ctx, n * widest(g));
        }
        return s;
    }
};

// The residual stream of a one-token step on a model whose layers end in output norms: the vector that
// is still to be normed and added (`pend_p` with weight `pend_w`) rides along until the next projection
// consumes it (tm_cuda_q8_0_gemv_addnorm), which writes the updated stream to the other of two buffers.
struct Residual {
    const CudaBuffer *cur = nullptr, *alt = nullptr;
    const CudaBuffer *pend_p = nullptr, *pend_w = nullptr;
    // y = W rmsnorm(stream, norm_w) with whatever is pending folded in first.
    void project(const CudaContext &ctx, const CudaBuffer &w, uint32_t rows, uint32_t cols, const CudaBuffer &norm_w,
                 const CudaBuffer &y, float eps) {
        if (pend_p) {
            ctx.q8_0_gemv_addnorm(w, *cur, *pend_p, *pend_w, *alt, norm_w, y, rows, cols, eps);
            std::swap(cur, alt);
            pend_p = pend_w = nullptr;
        } else {
            ctx.q8_0_gemv_fused(w, *cur, y, rows, cols, TM_CUDA_PRO_RMSNORM, &norm_w, eps, TM_CUDA_EPI_STORE);
        }
    }
};

// What the n rows of a batched pass are: n consecutive positions of sequence `seq` (a prefill chunk),
// or -- with `pos_buf` set -- one decode row per sequence, sequence s at the device position pos_buf[s].
struct RowsAre {
    size_t seq = 0;
    const CudaBuffer *pos_buf = nullptr, *status = nullptr;
};

// Gated FFN: down(act(gate x) * up x), optional RMS norm on the output before
// the residual add (engine/metal.rs:431-535).  gate|up are one matrix.  On a split
// model every rank owns width/world gate and up rows and the matching width/world
// COLUMNS of down: its activated slice feeds its own down columns, and the ranks'
// full-width partial products are added in one exchange (with the residual).
struct SwiGluBlock {
    Matrix gate_up, down;
    GluActivation act = GluActivation::Silu;
    CudaBuffer out_norm;  // empty unless the artifact has it
    float eps = 0;
    CudaBuffer gu, g_view, u_view, out;
    CudaBuffer out_local;  // split only: this rank's partial product
    size_t width = 0, wl = 0;      // full and per-rank FFN width
    Shard sh;

    static void plan(const FfnSpec &f, bool has_norm, Tensor norm, size_t hidden, const WeightSource &src, Shard sh,
                     Plan &p) {
        p.weights += Matrix::plan(src, {f.gate, f.up}, sh) +
                     (sh.world > 1 ? Matrix::plan_cols(src, f.down, sh) : Matrix::plan(src, {f.down}));
        if (has_norm) p.weights_f32(vector_len(src, norm));
        p.scratch_f32(2 * f.width / sh.world);
        p.target_f32(hidden * sh.world * (sh.world > 1 ? 2 : 1), sh.world);  // out: one slot per rank when split (8-byte pairs)
        if (sh.world > 1) p.scratch_f32(hidden);    // out_local
    }
    static SwiGluBlock load(const CudaContext &ctx, const WeightSource &src, const FfnSpec &f, bool has_norm,
                            Tensor norm, size_t hidden, float eps, Shard sh) {
        SwiGluBlock b;
        b.sh = sh;
        b.gate_up = Matrix::load(ctx, src, {f.gate, f.up}, sh);
        b.down = sh.world > 1 ? Matrix::load_cols(ctx, src, f.down, sh) : Matrix::load(ctx, src, {f.down});
        b.act = f.act;
        if (has_norm) b.out_norm = vector(ctx, src, norm);
        b.eps = eps;
        b.width = f.width;
        b.wl = f.width / sh.world;
        if (f.width % sh.world != 0 || hidden % sh.world != 0 || (b.wl * 4) % 16 != 0)
            throw TuckmillError(ErrorCode::InvalidRequest, "FFN width does not divide over the devices of the split");
        b.gu = zeros_f32(ctx, 2 * b.wl);
        b.g_view = b.gu.view(0, b.wl * 4);
        b.u_view = b.gu.view(b.wl * 4, b.wl * 4);
        b.out = gather_target_f32(ctx, hidden * sh.world * (sh.world > 1 ? 2 : 1), sh);
        if (sh.world > 1) b.out_local = zeros_f32(ctx, hidden);
        if (b.down.rows != hidden || b.down.cols != b.wl)
            throw TuckmillError(ErrorCode::UnsupportedArchitecture, "down projection shape does not match the FFN width");
        return b;
    }
    void act_mul(const CudaContext &ctx, const CudaBuffer &g, const CudaBuffer &u, uint32_t n) const {
        if (act == GluActivation::Silu) ctx.silu_mul(g, u, g, n);
        else ctx.gelu_tanh_mul(g, u, g, n);
    }
    // x += ffn(norm(x, post_norm)) for one token: 2 launches (3 more with an output norm).
    void decode(const CudaContext &ctx, const CudaBuffer &x, const CudaBuffer &post_norm, size_t hidden) const {
        gate_up.gemv_fused(ctx, x, gu, TM_CUDA_PRO_RMSNORM, &post_norm, eps, TM_CUDA_EPI_STORE);
        const int pro = act == GluActivation::Silu ? TM_CUDA_PRO_SILU_MUL : TM_CUDA_PRO_GELU_MUL;
        if (sh.world > 1) {  // this rank's columns of down, then the ranks' partial products added (4 launches)
            down.gemv_fused(ctx, g_view, out_local, pro, &u_view, 0.0f, TM_CUDA_EPI_STORE);
            if (sh.pair_exchange && !out_norm) {
                ctx.exchange_add_ll(out_local, out, x, (uint32_t)hidden);
                return;
            }
            ctx.push_rows(out_local, out, 1, (uint32_t)hidden);
            ctx.reduce_ranks_add(out, x, out_norm ? &out_norm : nullptr, sh.world, 1, (uint32_t)hidden, eps);
            return;
        }
        if (out_norm) {
            down.gemv_fused(ctx, g_view, out, pro, &u_view, 0.0f, TM_CUDA_EPI_STORE);
            ctx.rmsnorm_add(out, out_norm, x, 1, (uint32_t)hidden, eps);
        } else {
            down.gemv_fused(ctx, g_view, x, pro, &u_view, 0.0f, TM_CUDA_EPI_ADD);
        }
    }
    // The tolerance-qualified batched form: norm and activation folded into the GEMMs' f16 copies,
    // gate|up as one launch, the residual add in the down projection's epilogue (5 launches -> 4).
    bool fusable() const { return sh.world == 1 && width % 128 == 0 && gate_up.type == 8 && down.type == 8; }
    bool fusable_rows() const { return wl % 128 == 0 && gate_up.type == 8 && down.type == 8; }
    // A rank's share of the tolerance-qualified batched form: norm folded into ONE gate|up launch over
    // the rank's rows, the activation into the rank's columns of down, then the one exchange.
    void prefill_split_fused(const CudaContext &ctx, const PrefillScratch &s, size_t n, const CudaBuffer &post_norm,
                             size_t hidden) const {
        const uint32_t nn = (uint32_t)n;
        ctx.q8_0_gemm_mma_fused(gate_up.buf, s.x, gate_up.rows, gate_up.cols, nn, {&s.loc, &s.loc2},
                                {(uint32_t)wl, (uint32_t)wl}, TM_CUDA_PRO_RMSNORM, &post_norm, eps, TM_CUDA_EPI_STORE);
        const int pro = act == GluActivation::Silu ? TM_CUDA_PRO_SILU_MUL : TM_CUDA_PRO_GELU_MUL;
        ctx.q8_0_gemm_mma_fused(down.buf, s.loc, down.rows, down.cols, nn, {&s.h}, {down.rows}, pro, &s.loc2, 0.0f,
                                TM_CUDA_EPI_STORE);
        ctx.push_rows(s.h, s.d2, 1, (uint32_t)(n * hidden));
        ctx.reduce_ranks_add(s.d2, s.x, out_norm ? &out_norm : nullptr, sh.world, nn, (uint32_t)hidden, eps);
    }
    void prefill_fused(const CudaContext &ctx, const PrefillScratch &s, size_t n, const CudaBuffer &post_norm,
                       size_t hidden) const {
        const uint32_t nn = (uint32_t)n;
        ctx.q8_0_gemm_mma_fused(gate_up.buf, s.x, gate_up.rows, gate_up.cols, nn, {&s.g, &s.u},
                                {(uint32_t)width, (uint32_t)width}, TM_CUDA_PRO_RMSNORM, &post_norm, eps,
                                TM_CUDA_EPI_STORE);
        const int pro = act == GluActivation::Silu ? TM_CUDA_PRO_SILU_MUL : TM_CUDA_PRO_GELU_MUL;
        if (out_norm) {
            ctx.q8_0_gemm_mma_fused(down.buf, s.g, down.rows, down.cols, nn, {&s.d2}, {down.rows}, pro, &s.u, 0.0f,
                                    TM_CUDA_EPI_STORE);
            ctx.rmsnorm_add(s.d2, out_norm, s.x, nn, (uint32_t)hidden, eps);
        } else {
            ctx.q8_0_gemm_mma_fused(down.buf, s.g, down.rows, down.cols, nn, {&s.x}, {down.rows}, pro, &s.u, 0.0f,
                                    TM_CUDA_EPI_ADD);
        }
    }
    // x += ffn(h2) for the n chunk rows of s.h2 / s.x (engine/metal.rs:514-534).
    void prefill(const CudaContext &ctx, const PrefillScratch &s, size_t n, size_t hidden, bool exact) const {
        const uint32_t nn = (uint32_t)n;
        if (sh.world > 1) {
            gate_up.gemm_part(ctx, 0, s.h2, s.loc, nn, exact);
            gate_up.gemm_part(ctx, 1, s.h2, s.loc2, nn, exact);
            act_mul(ctx, s.loc, s.loc2, (uint32_t)(n * wl));
            down.gemm_all(ctx, s.loc, s.loc2, nn, exact);  // this rank's partial product [n][hidden]
            ctx.push_rows(s.loc2, s.d2, 1, (uint32_t)(n * hidden));
            ctx.reduce_ranks_add(s.d2, s.x, out_norm ? &out_norm : nullptr, sh.world, nn, (uint32_t)hidden, eps);
            return;
        } else {
            gate_up.gemm_part(ctx, 0, s.h2, s.g, nn, exact);
            gate_up.gemm_part(ctx, 1, s.h2, s.u, nn, exact);
            act_mul(ctx, s.g, s.u, (uint32_t)(n * width));
            down.gemm_all(ctx, s.g, s.d2, nn, exact);
        }
        if (out_norm) ctx.rmsnorm_add(s.d2, out_norm, s.x, nn, (uint32_t)hidden, eps);
        else ctx.f32_axpy(s.d2, s.x, 1.0f, (uint32_t)(n * hidden));
    }
};

// Grouped-query attention with per-head Q/K RMS norms, RoPE, packed f16 KV and
// an optional sliding window (engine/metal.rs:989-1364).  q|k|v are one matrix.
// On a split model every rank owns heads/world query heads and kv_heads/world
// KV heads (and only their cache planes) and the COLUMNS of o that multiply them:
// attention is local to the rank and feeds its own o columns; the ranks' partial
// products are added in one exchange.
struct AttentionBlock {
    AttentionSpec spec;
    float eps = 0;
    Matrix qkv, o;
    CudaBuffer q_norm, k_norm, inv_freq, k_cache, v_cache;
    CudaBuffer qkv_out, q_view, k_view, v_view, attn, kv_scratch;
    CudaBuffer proj_local;  // split only: this rank's partial product of the o projection
    size_t cap = 0, heads_l = 0, kv_l = 0;
    Shard sh;
    // Several sequences: the caches are [seqs] plane pairs (sequence 0 first, so the one-sequence
    // operators work on the whole buffers), the views below are the single planes a prefill writes.
    size_t seqs = 1;
    std::vector<CudaBuffer> k_seq, v_seq;
    CudaBuffer q_rows, k_rows, v_rows;  // q | k | v columns of the [seqs][q|k|v] projection output
    const CudaBuffer &kc(size_t seq) const { return seqs > 1 ? k_seq[seq] : k_cache; }
    const CudaBuffer &vc(size_t seq) const { return seqs > 1 ? v_seq[seq] : v_cache; }

    static uint64_t kv_plane_bytes(const AttentionSpec &s, size_t cap, Shard sh) {
        return (uint64_t)(s.kv_heads / sh.world) * cap * s.head_dim * 2;
    }
    static void plan(const AttentionSpec &s, const WeightSource &src, size_t cap, size_t hidden, Shard sh, Plan &p,
                     size_t seqs) {
        p.weights += Matrix::plan(src, {s.q, s.k, s.v}, sh) +
                     (sh.world > 1 ? Matrix::plan_cols(src, s.o, sh) : Matrix::plan(src, {s.o}));
        p.weights_f32(vector_len(src, s.q_norm));
        p.weights_f32(vector_len(src, s.k_norm));
        // The RoPE table is derived by the engine, not artifact bytes: scratch.
        p.scratch_f32(s.rope_dims / 2);
        p.state += 2 * kv_plane_bytes(s, cap, sh) * seqs;
        const size_t hl = s.heads / sh.world, kl = s.kv_heads / sh.world;
        p.scratch_f32((hl + 2 * kl) * s.head_dim * seqs);
        p.scratch_f32(hl * s.head_dim);
        p.scratch_bytes(seqs * tm_cuda_attention_decode_scratch_bytes((uint32_t)hl, (uint32_t)kl, (uint32_t)s.head_dim,
                                                                      (uint32_t)cap));
        if (sh.world > 1) p.scratch_f32(hidden);  // proj_local
    }
    static AttentionBlock load(const CudaContext &ctx, const WeightSource &src, const AttentionSpec &s, float eps,
                               size_t cap, size_t hidden, Shard sh, size_t seqs) {
        if (s.head_dim % 32 != 0 || (s.head_dim / 32 > 4 && s.head_dim != 256) || s.rope_dims % 2 != 0)
            throw TuckmillError(ErrorCode::UnsupportedArchitecture,
                                "attention head size " + std::to_string(s.head_dim) + " has no CUDA block");
        if (s.heads % sh.world != 0 || s.kv_heads % sh.world != 0 || hidden % sh.world != 0)
            throw TuckmillError(ErrorCode::InvalidRequest,
                                std::to_string(s.heads) + " query / " + std::to_string(s.kv_heads) +
                                    " KV heads do not divide over " + std::to_string(sh.world) + " devices");
        AttentionBlock b;
        b.spec = s;
        b.eps = eps;
        b.cap = cap;
        b.sh = sh;
        b.heads_l = s.heads / sh.world;
        b.kv_l = s.kv_heads / sh.world;
        b.qkv = Matrix::load(ctx, src, {s.q, s.k, s.v}, sh);
        b.o = sh.world > 1 ? Matrix::load_cols(ctx, src, s.o, sh) : Matrix::load(ctx, src, {s.o});
        const size_t hd = b.heads_l * s.head_dim, kv = b.kv_l * s.head_dim;
        if (b.qkv.part_rows[0] != hd || b.qkv.part_rows[1] != kv || b.qkv.part_rows[2] != kv || b.o.cols != hd ||
            b.o.rows != hidden)
            throw TuckmillError(ErrorCode::UnsupportedArchitecture, "attention projection shapes do not match the head geometry");
        b.q_norm = vector(ctx, src, s.q_norm);
        b.k_norm = vector(ctx, src, s.k_norm);
        b.inv_freq = ctx.floats(rope_inv_freq(s.rope_dims, s.rope_base));
        b.seqs = seqs;
        const size_t plane = kv_plane_bytes(s, cap, sh);
        b.k_cache = ctx.buffer(plane * seqs);
        b.v_cache = ctx.buffer(plane * seqs);
        if (seqs > 1) {
            if (plane % 16 != 0)
                throw TuckmillError(ErrorCode::InvalidRequest, "KV plane of one sequence is not a 16-byte multiple");
            for (size_t i = 0; i < seqs; ++i) {
                b.k_seq.push_back(b.k_cache.view(i * plane, plane));
                b.v_seq.push_back(b.v_cache.view(i * plane, plane));
            }
        }
        b.qkv_out = zeros_f32(ctx, (hd + 2 * kv) * seqs);
        {
            const size_t all = (hd + 2 * kv) * seqs * 4;
            b.q_rows = b.qkv_out.view(0, all);
            b.k_rows = b.qkv_out.view(hd * 4, all - hd * 4);
            b.v_rows = b.qkv_out.view((hd + kv) * 4, all - (hd + kv) * 4);
        }
        b.q_view = b.qkv_out.view(0, hd * 4);
        b.k_view = b.qkv_out.view(hd * 4, kv * 4);
        b.v_view = b.qkv_out.view((hd + kv) * 4, kv * 4);
        b.attn = zeros_f32(ctx, hd);
        b.kv_scratch = ctx.zeros(seqs * tm_cuda_attention_decode_scratch_bytes((uint32_t)b.heads_l, (uint32_t)b.kv_l,
                                                                               (uint32_t)s.head_dim, (uint32_t)cap));
        if (sh.world > 1) b.proj_local = zeros_f32(ctx, hidden);
        return b;
    }
    void reset() const {
        k_cache.zero();
        v_cache.zero();
    }
    float scale() const { return 1.0f / std::sqrt((float)spec.head_dim); }

    // attn = attention(norm(x, pre_norm)) at the device-held position: 2 launches.
    void decode(const CudaContext &ctx, const CudaBuffer &x, const CudaBuffer &pre_norm, const CudaBuffer &pos_buf,
                const CudaBuffer &status, bool exact) const {
        qkv.gemv_fused(ctx, x, qkv_out, TM_CUDA_PRO_RMSNORM, &pre_norm, eps, TM_CUDA_EPI_STORE);
        ctx.attention_decode_dev(q_view, k_view, v_view, q_norm, k_norm, inv_freq, k_cache, v_cache, attn, kv_scratch,
                                 pos_buf, 0, status, (uint32_t)heads_l, (uint32_t)kv_l, (uint32_t)spec.head_dim,
                                 (uint32_t)spec.rope_dims, (uint32_t)cap, (uint32_t)spec.window, eps, scale(), exact);
    }
    // The per-token core for one row per sequence: row s of q / k / v (strides in elements, 0 = dense) is
    // sequence s at its own position pos_buf[s], attending to its own cache planes.
    void attend_batch(const CudaContext &ctx, const CudaBuffer &q, const CudaBuffer &k, const CudaBuffer &v,
                      uint32_t q_stride, uint32_t kv_stride, const CudaBuffer &out, size_t n_seq,
                      const CudaBuffer &pos_buf, const CudaBuffer &status, bool exact) const {
        ctx.attention_decode_batch(q, k, v, q_norm, k_norm, inv_freq, k_cache, v_cache, out, kv_scratch, pos_buf, status,
                                   (uint32_t)n_seq, q_stride, kv_stride, (uint32_t)heads_l, (uint32_t)kv_l,
                                   (uint32_t)spec.head_dim, (uint32_t)spec.rope_dims, (uint32_t)cap,
                                   (uint32_t)spec.window, eps, scale(), exact);
    }
    // Split model, one token: this rank's columns of o times its own heads' output, pushed into this
    // rank's slot of `proj` on every rank (the caller adds the slots).
    void project_sharded(const CudaContext &ctx, const CudaBuffer &proj, size_t hidden) const {
        o.gemv(ctx, attn, proj_local);
        ctx.push_rows(proj_local, proj, 1, (uint32_t)hidden);
    }
    // The tolerance-qualified batched form: input norm folded into the f16 copy, q|k|v as one GEMM
    // launch, the four launches before attention as one, tensor-core attention (9 launches -> 4).
    // (the q|k|v part of it applies to a rank's rows of a split model as well: fusable_rows)
    bool fusable_rows() const {
        return qkv.type == 8 && o.type == 8 && qkv.part_rows.size() == 3 && qkv.part_rows[0] % 128 == 0 &&
               qkv.part_rows[1] % 128 == 0 && tm_cuda_attention_chunk_mma_supported((uint32_t)spec.head_dim);
    }
    bool fusable() const { return sh.world == 1 && fusable_rows(); }
    void prefill_fused(const CudaContext &ctx, const PrefillScratch &s, size_t n, uint32_t pos0,
                       const CudaBuffer &pre_norm, const RowsAre &rows) const {
        const uint32_t nn = (uint32_t)n, heads = (uint32_t)heads_l, kv = (uint32_t)kv_l, hd = (uint32_t)spec.head_dim;
        ctx.q8_0_gemm_mma_fused(qkv.buf, s.x, qkv.rows, qkv.cols, nn, {&s.a, &s.b, &s.c},
                                {qkv.part_rows[0], qkv.part_rows[1], qkv.part_rows[2]}, TM_CUDA_PRO_RMSNORM, &pre_norm,
                                eps, TM_CUDA_EPI_STORE);
        if (rows.pos_buf) {  // one row per sequence
            attend_batch(ctx, s.a, s.b, s.c, 0, 0, s.e, n, *rows.pos_buf, *rows.status, false);
            return;
        }
        ctx.qk_prep_chunk(s.a, s.b, s.c, q_norm, k_norm, inv_freq, kc(rows.seq), vc(rows.seq), heads, kv, hd,
                          (uint32_t)spec.rope_dims, pos0, (uint32_t)cap, nn, eps);
        ctx.attention_chunk_mma(s.a, kc(rows.seq), vc(rows.seq), s.e, heads, pos0, (uint32_t)cap, hd, heads / kv,
                                scale(), nn, (uint32_t)spec.window);
    }
    // Chunk core over n queries at pos0.. (engine/metal.rs:1170-1233): every
    // chunk K/V row is stored before any chunk query attends.
    void prefill(const CudaContext &ctx, const PrefillScratch &s, size_t n, uint32_t pos0, size_t hidden,
                 bool exact, const RowsAre &rows) const {
        const uint32_t nn = (uint32_t)n, heads = (uint32_t)heads_l, kv = (uint32_t)kv_l, hd = (uint32_t)spec.head_dim;
        qkv.gemm_part(ctx, 0, s.h, s.a, nn, exact);
        qkv.gemm_part(ctx, 1, s.h, s.b, nn, exact);
        qkv.gemm_part(ctx, 2, s.h, s.c, nn, exact);
        if (rows.pos_buf) {  // one row per sequence
            attend_batch(ctx, s.a, s.b, s.c, 0, 0, s.e, n, *rows.pos_buf, *rows.status, exact);
        } else {
            const CudaBuffer &kcs = kc(rows.seq), &vcs = vc(rows.seq);
            ctx.rmsnorm(s.a, q_norm, s.a, nn * heads, hd, eps);
            ctx.rmsnorm(s.b, k_norm, s.b, nn * kv, hd, eps);
            ctx.rope_partial_chunk(s.a, s.b, inv_freq, pos0, heads, kv, hd, (uint32_t)spec.rope_dims, nn);
            ctx.kv_store_chunk(s.b, s.c, kcs, vcs, pos0, (uint32_t)cap, hd, kv, nn);
            // Tolerance-qualified tensor-core form unless bit identity with the per-token path is asked.
            if (!exact && tm_cuda_attention_chunk_mma_supported(hd))
                ctx.attention_chunk_mma(s.a, kcs, vcs, s.e, heads, pos0, (uint32_t)cap, hd, heads / kv, scale(), nn,
                                        (uint32_t)spec.window);
            else
                ctx.attention_chunk(s.a, kcs, vcs, s.e, s.ascr, heads, pos0, (uint32_t)cap, hd, heads / kv, scale(),
                                    nn, (uint32_t)spec.window);
        }
        if (sh.world > 1) {  // this rank's partial product into its slot of s.proj on every rank
            o.gemm_all(ctx, s.e, s.loc, nn, exact);
            ctx.push_rows(s.loc, s.proj, 1, (uint32_t)(n * hidden));
        } else {
            o.gemm_all(ctx, s.e, s.proj, nn, exact);
        }
    }
};

// One layer: x += [norm](mixer(norm(x))); x += [norm](ffn(norm(x))) (engine/metal.rs:1379-1525).
struct Layer {
    CudaBuffer pre_norm, mixer_out_norm, post_norm, proj;
    AttentionBlock mixer;
    SwiGluBlock ffn;

    static void plan(const LayerSpec &l, const ModelGraph &g, const WeightSource &src, size_t cap, Shard sh, Plan &p,
                     size_t seqs) {
        p.weights_f32(vector_len(src, l.pre_norm));
        p.weights_f32(vector_len(src, l.post_norm));
        if (l.has_mixer_out_norm) p.weights_f32(vector_len(src, l.mixer_out_norm));
        p.target_f32(g.hidden * sh.world * (sh.world > 1 ? 2 : 1), sh.world);  // proj: one slot per rank when split (8-byte pairs)
        AttentionBlock::plan(l.mixer, src, cap, g.hidden, sh, p, seqs);
        SwiGluBlock::plan(l.ffn, l.has_ffn_out_norm, l.ffn_out_norm, g.hidden, src, sh, p);
    }
    static Layer load(const CudaContext &ctx, const WeightSource &src, const LayerSpec &l, const ModelGraph &g,
                      size_t cap, Shard sh, size_t seqs) {
        Layer L;
        L.pre_norm = vector(ctx, src, l.pre_norm);
        if (l.has_mixer_out_norm) L.mixer_out_norm = vector(ctx, src, l.mixer_out_norm);
        L.post_norm = vector(ctx, src, l.post_norm);
        L.proj = gather_target_f32(ctx, g.hidden * sh.world * (sh.world > 1 ? 2 : 1), sh);
        L.mixer = AttentionBlock::load(ctx, src, l.mixer, g.eps, cap, g.hidden, sh, seqs);
        L.ffn = SwiGluBlock::load(ctx, src, l.ffn, l.has_ffn_out_norm, l.ffn_out_norm, g.hidden, g.eps, sh);
        return L;
    }
    void decode(const CudaContext &ctx, const CudaBuffer &x, const CudaBuffer &pos_buf, const CudaBuffer &status,
                size_t hidden, float eps, bool exact) const {
        mixer.decode(ctx, x, pre_norm, pos_buf, status, exact);
        if (mixer.sh.world > 1 && mixer.sh.pair_exchange && !mixer_out_norm) {
            mixer.o.gemv(ctx, mixer.attn, mixer.proj_local);
            ctx.exchange_add_ll(mixer.proj_local, proj, x, (uint32_t)hidden);
        } else if (mixer.sh.world > 1) {
            mixer.project_sharded(ctx, proj, hidden);
            ctx.reduce_ranks_add(proj, x, mixer_out_norm ? &mixer_out_norm : nullptr, mixer.sh.world, 1, (uint32_t)hidden,
                                 eps);
        } else if (mixer_out_norm) {
            mixer.o.gemv(ctx, mixer.attn, proj);
            ctx.rmsnorm_add(proj, mixer_out_norm, x, 1, (uint32_t)hidden, eps);
        } else {
            mixer.o.gemv_fused(ctx, mixer.attn, x, TM_CUDA_PRO_NONE, nullptr, 0.0f, TM_CUDA_EPI_ADD);
        }
        ffn.decode(ctx, x, post_norm, hidden);
    }
    // A one-token step of a layer that ends both halves in an output norm (Gemma): the norm-and-add of
    // each half is folded into the projection that follows it -- 5 launches instead of 7, the same
    // arithmetic (tm_cuda_q8_0_gemv_addnorm).
    bool norms_fold(size_t hidden) const {
        return slices_apply() && mixer_out_norm && ffn.out_norm && hidden <= 4096;
    }
    void decode_folded(const CudaContext &ctx, Residual &R, const CudaBuffer &pos_buf, const CudaBuffer &status,
                       size_t hidden, float eps, bool exact) const {
        (void)hidden;
        R.project(ctx, mixer.qkv.buf, mixer.qkv.rows, mixer.qkv.cols, pre_norm, mixer.qkv_out, eps);
        ctx.attention_decode_dev(mixer.q_view, mixer.k_view, mixer.v_view, mixer.q_norm, mixer.k_norm, mixer.inv_freq,
                                 mixer.k_cache, mixer.v_cache, mixer.attn, mixer.kv_scratch, pos_buf, 0, status,
                                 (uint32_t)mixer.heads_l, (uint32_t)mixer.kv_l, (uint32_t)mixer.spec.head_dim,
                                 (uint32_t)mixer.spec.rope_dims, (uint32_t)mixer.cap, (uint32_t)mixer.spec.window, eps,
                                 mixer.scale(), exact);
        mixer.o.gemv(ctx, mixer.attn, proj);
        R.pend_p = &proj;
        R.pend_w = &mixer_out_norm;
        R.project(ctx, ffn.gate_up.buf, ffn.gate_up.rows, ffn.gate_up.cols, post_norm, ffn.gu, eps);
        const int pro = ffn.act == GluActivation::Silu ? TM_CUDA_PRO_SILU_MUL : TM_CUDA_PRO_GELU_MUL;
        ffn.down.gemv_fused(ctx, ffn.g_view, ffn.out, pro, &ffn.u_view, 0.0f, TM_CUDA_EPI_STORE);
        R.pend_p = &ffn.out;
        R.pend_w = &ffn.out_norm;
    }
    // Every matrix Q8_0 on one device: the batched fused GEMV forms apply.
    bool slices_apply() const {
        return mixer.sh.world == 1 && mixer.qkv.type == 8 && mixer.o.type == 8 && ffn.gate_up.type == 8 &&
               ffn.down.type == 8;
    }
    // One decode row per sequence with the decode step's own launches (q|k|v as one fused-norm multiply,
    // activation and residual folded into the projections), `n` rows per launch in slices of 8: row s
    // is bit-identical to the one-sequence step.  Serves `exact` mode and small batches.
    void decode_rows(const CudaContext &ctx, const PrefillScratch &s, size_t n, const CudaBuffer &pos_buf,
                     const CudaBuffer &status, size_t hidden, float eps, bool exact) const {
        const uint32_t nn = (uint32_t)n, stride = mixer.qkv.rows;
        ctx.q8_0_gemm_fused(mixer.qkv.buf, s.x, mixer.qkv_out, mixer.qkv.rows, mixer.qkv.cols, nn, TM_CUDA_PRO_RMSNORM,
                            &pre_norm, eps, TM_CUDA_EPI_STORE);
        mixer.attend_batch(ctx, mixer.q_rows, mixer.k_rows, mixer.v_rows, stride, stride, s.e, n, pos_buf, status, exact);
        if (mixer_out_norm) {
            ctx.q8_0_gemm_fused(mixer.o.buf, s.e, s.proj, mixer.o.rows, mixer.o.cols, nn, TM_CUDA_PRO_NONE, nullptr, 0.0f,
                                TM_CUDA_EPI_STORE);
            ctx.rmsnorm_add(s.proj, mixer_out_norm, s.x, nn, (uint32_t)hidden, eps);
        } else {
            ctx.q8_0_gemm_fused(mixer.o.buf, s.e, s.x, mixer.o.rows, mixer.o.cols, nn, TM_CUDA_PRO_NONE, nullptr, 0.0f,
                                TM_CUDA_EPI_ADD);
        }
        // gate and up as two launches into dense [n][width] matrices (the activation prologue of the
        // down projection wants dense operands); each part takes the whole matrix's column split.
        const Matrix &gu = ffn.gate_up;
        ctx.q8_0_gemm_fused(gu.parts[0], s.x, s.g, gu.part_rows[0], gu.cols, nn, TM_CUDA_PRO_RMSNORM, &post_norm, eps,
                            TM_CUDA_EPI_STORE);
        ctx.q8_0_gemm_fused(gu.parts[1], s.x, s.u, gu.part_rows[1], gu.cols, nn, TM_CUDA_PRO_RMSNORM, &post_norm, eps,
                            TM_CUDA_EPI_STORE);
        const int pro = ffn.act == GluActivation::Silu ? TM_CUDA_PRO_SILU_MUL : TM_CUDA_PRO_GELU_MUL;
        if (ffn.out_norm) {
            ctx.q8_0_gemm_fused(ffn.down.buf, s.g, s.d2, ffn.down.rows, ffn.down.cols, nn, pro, &s.u, 0.0f,
                                TM_CUDA_EPI_STORE);
            ctx.rmsnorm_add(s.d2, ffn.out_norm, s.x, nn, (uint32_t)hidden, eps);
        } else {
            ctx.q8_0_gemm_fused(ffn.down.buf, s.g, s.x, ffn.down.rows, ffn.down.cols, nn, pro, &s.u, 0.0f,
                                TM_CUDA_EPI_ADD);
        }
    }
    void prefill(const CudaContext &ctx, const PrefillScratch &s, size_t n, uint32_t pos0, size_t hidden, float eps,
                 bool exact, const RowsAre &rows = RowsAre()) const {
        const uint32_t nn = (uint32_t)n;
        if (!exact && mixer.fusable() && ffn.fusable()) {
            mixer.prefill_fused(ctx, s, n, pos0, pre_norm, rows);
            if (mixer_out_norm) {
                mixer.o.gemm_all(ctx, s.e, s.proj, nn, false);
                ctx.rmsnorm_add(s.proj, mixer_out_norm, s.x, nn, (uint32_t)hidden, eps);
            } else {
                ctx.q8_0_gemm_mma_fused(mixer.o.buf, s.e, mixer.o.rows, mixer.o.cols, nn, {&s.x}, {mixer.o.rows},
                                        TM_CUDA_PRO_NONE, nullptr, 0.0f, TM_CUDA_EPI_ADD);
            }
            ffn.prefill_fused(ctx, s, n, post_norm, hidden);
            return;
        }
        if (!exact && mixer.sh.world > 1 && mixer.fusable_rows() && ffn.fusable_rows()) {
            // Split model, tolerance mode: q|k|v and gate|up as one fused launch each over this rank's
            // rows, attention on the rank's heads, o and down over this rank's columns (4 GEMM calls and
            // 2 exchanges per layer).
            mixer.prefill_fused(ctx, s, n, pos0, pre_norm, rows);
            ctx.q8_0_gemm_mma_fused(mixer.o.buf, s.e, mixer.o.rows, mixer.o.cols, nn, {&s.h}, {mixer.o.rows},
                                    TM_CUDA_PRO_NONE, nullptr, 0.0f, TM_CUDA_EPI_STORE);
            ctx.push_rows(s.h, s.proj, 1, (uint32_t)(n * hidden));
            ctx.reduce_ranks_add(s.proj, s.x, mixer_out_norm ? &mixer_out_norm : nullptr, mixer.sh.world, nn,
                                 (uint32_t)hidden, eps);
            ffn.prefill_split_fused(ctx, s, n, post_norm, hidden);
            return;
        }
        ctx.rmsnorm(s.x, pre_norm, s.h, nn, (uint32_t)hidden, eps);
        mixer.prefill(ctx, s, n, pos0, hidden, exact, rows);
        if (mixer.sh.world > 1)
            ctx.reduce_ranks_add(s.proj, s.x, mixer_out_norm ? &mixer_out_norm : nullptr, mixer.sh.world, nn,
                                 (uint32_t)hidden, eps);
        else if (mixer_out_norm) ctx.rmsnorm_add(s.proj, mixer_out_norm, s.x, nn, (uint32_t)hidden, eps);
        else ctx.f32_axpy(s.proj, s.x, 1.0f, (uint32_t)(n * hidden));
        ctx.rmsnorm(s.x, post_norm, s.h2, nn, (uint32_t)hidden, eps);
        ffn.prefill(ctx, s, n, hidden, exact);
    }
};

uint64_t now_ns() {
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
               std::chrono::steady_clock::now().time_since_epoch())
        .count();
}

}  // namespace

struct EngineModel::Impl {
    Matrix embedding, head_own;
    bool tied = false;
    Shard sh;
    GatherArena arena;  // declared before the blocks that hold views of it (views are released first)
    CudaBuffer tied_view;  // row split of a tied head: this rank's rows of the (replicated) embedding
    uint32_t head_rows = 0;  // rows of the head this rank multiplies (vocab / world)
    CudaBuffer final_norm, x, x2, logits, partial, tokens, tokens_mirror, pos_buf, status;
    bool fold_norms = false;  // every layer's output norms ride into the next projection (Residual)
    CudaBuffer logits_full, pairs;  // row split only
    std::vector<Layer> layers;
    PrefillScratch scratch;
    CudaGraph decode_graph;
    bool persistent = false;  // decode_graph is a persistent program
    // Several sequences: positions pos_buf[s], token logs tokens[s * log_stride ..], logits [s][head_rows];
    // one recorded step advances all of them.
    size_t seqs = 1, log_stride = 0;
    size_t l2_ahead = 0;  // layers whose weights the decode step asks into L2 ahead of use (0: off)
    CudaGraph batch_graph;
    std::vector<size_t> pos_b;  // host copy of every sequence's position
    const CudaBuffer &head_buf() const { return tied ? (sh.world > 1 ? tied_view : embedding.buf) : head_own.buf; }
    uint32_t head_cols() const { return embedding.cols; }
    uint32_t head_type() const { return tied ? embedding.type : head_own.type; }
    // Final norm folded into the vocabulary projection of the one row in `x`.
    void project_head(const CudaContext &c, float eps) const {
        if (head_type() == 1)
            c.f16_gemv_fused(head_buf(), x, logits, head_rows, head_cols(), TM_CUDA_PRO_RMSNORM, &final_norm, eps,
                             TM_CUDA_EPI_STORE);
        else
            c.q8_0_gemv_fused(head_buf(), x, logits, head_rows, head_cols(), TM_CUDA_PRO_RMSNORM, &final_norm, eps,
                              TM_CUDA_EPI_STORE);
    }
};

DecodeProgramSize decode_program_size(const ModelGraph &graph, size_t capacity) {
    DecodeProgramSize s;
    s.max_ops = (uint32_t)graph.layers.size() * 8u + 8u;
    s.vector_elems = graph.hidden + graph.vocab;  // embedding row, logits
    for (const LayerSpec &l : graph.layers) {
        const AttentionSpec &m = l.mixer;
        // q|k|v, attention output, o projection (+ its normed residual form), gate|up, down (+ normed form)
        s.vector_elems += (m.heads + 2 * m.kv_heads) * m.head_dim + m.heads * m.head_dim + 2 * graph.hidden +
                          2 * l.ffn.width + 2 * graph.hidden;
        s.attention_elems = std::max<uint64_t>(
            s.attention_elems, tm_cuda_program_attention_elems((uint32_t)m.heads, (uint32_t)m.head_dim, (uint32_t)capacity));
    }
    return s;
}

bool persistent_decode_applies(const ModelGraph &graph, const WeightSource &src, const EngineOptions &opts) {
    // the program's weight ring streams the repacked Q8_0 planes only
    auto q8 = [&](Tensor t) { return src.tensor_type_id(t.index) == 8; };
    if (!q8(graph.embedding) || !q8(graph.head)) return false;
    for (const LayerSpec &l : graph.layers)
        if (!q8(l.mixer.q) || !q8(l.mixer.k) || !q8(l.mixer.v) || !q8(l.mixer.o) || !q8(l.ffn.gate) || !q8(l.ffn.up) ||
            !q8(l.ffn.down))
            return false;
    return persistent_decode_applies(graph, opts);
}

bool persistent_decode_applies(const ModelGraph &graph, const EngineOptions &opts) {
    bool want = opts.persistent;
    if (const char *e = std::getenv("TM_ENGINE_PERSISTENT")) want = e[0] != '0';  // experiments: overrides the option
    if (!want || opts.exact || opts.shard_world > 1) return false;
    if (!tm_cuda_program_supports_gemv((uint32_t)graph.hidden)) return false;
    for (const LayerSpec &l : graph.layers) {
        const AttentionSpec &m = l.mixer;
        if (!tm_cuda_program_supports_attention((uint32_t)m.heads, (uint32_t)m.kv_heads, (uint32_t)m.head_dim,
                                                (uint32_t)m.rope_dims) ||
            !tm_cuda_program_supports_gemv((uint32_t)(m.heads * m.head_dim)) ||
            !tm_cuda_program_supports_gemv((uint32_t)l.ffn.width))
            return false;
    }
    return true;
}

// Slots of one sequence's token log: capacity + 1, rounded so that every sequence's log starts on a
// 16-byte boundary when there are several.
static size_t token_log_stride(size_t capacity, size_t seqs) {
    return seqs > 1 ? (capacity + 1 + 3) & ~(size_t)3 : capacity + 1;
}
// Rows of the chunk-wide scratch: a prefill chunk, or one decode row per sequence.
static size_t chunk_rows(const EngineOptions &opts, size_t capacity) {
    return std::max<size_t>(std::min<size_t>(opts.prefill_batch, capacity), opts.sequences);
}

GpuAllocPlan alloc_plan_with(const ModelGraph &graph, const WeightSource &src, size_t capacity,
                             const EngineOptions &opts) {
    if (opts.shard_world == 0 || opts.shard_rank >= opts.shard_world)
        throw TuckmillError(ErrorCode::InvalidRequest, "shard rank outside the split");
    if (opts.sequences == 0 || opts.sequences > kMaxSequences)
        throw TuckmillError(ErrorCode::InvalidRequest, "sequences must be 1.." + std::to_string(kMaxSequences));
    const Shard sh{opts.shard_rank, opts.shard_world};
    // Whole attention heads stay on one rank, and every row range is N/world.
    auto divides = [&](size_t v, const char *what) {
        if (v % sh.world != 0)
            throw TuckmillError(ErrorCode::InvalidRequest,
                                std::string(what) + " = " + std::to_string(v) + " does not divide over " +
                                    std::to_string(sh.world) + " devices",
                                "Choose a device count that divides the head counts, the FFN width and the vocabulary.");
    };
    divides(graph.vocab, "vocabulary");
    divides(graph.hidden, "hidden size");
    for (const LayerSpec &l : graph.layers) {
        divides(l.mixer.heads, "query heads");
        divides(l.mixer.kv_heads, "KV heads");
        divides(l.ffn.width, "FFN width");
    }
    Plan p;
    const size_t seqs = opts.sequences;
    for (const LayerSpec &l : graph.layers) Layer::plan(l, graph, src, capacity, sh, p, seqs);
    p.weights += Matrix::plan(src, {graph.embedding});  // the embedding table is replicated
    if (graph.head != graph.embedding) p.weights += Matrix::plan(src, {graph.head}, sh);
    p.weights_f32(vector_len(src, graph.final_norm));
    p.scratch_f32(graph.hidden);              // x
    p.scratch_f32(graph.hidden);              // x2: the other buffer of a residual stream that alternates
    p.scratch_f32(graph.vocab / sh.world * seqs);  // logits (this rank's slice), a row per sequence
    p.scratch_bytes(kArgmaxPartialBytes * seqs);   // argmax partials
    p.scratch_bytes(token_log_stride(capacity, seqs) * seqs * 4);  // device token logs
    p.scratch_bytes(token_log_stride(capacity, seqs) * seqs * 4);  // their host-visible mirror
    p.scratch_bytes(std::max<size_t>(16, seqs * 4));  // device positions
    p.scratch_bytes(16);                      // status word
    if (sh.world > 1) {
        p.scratch_f32(graph.vocab);           // gathered logits (only when a caller asks for them)
        p.scratch_bytes((sh.world + 1) * 8 * seqs);  // (value, index) pairs of the sharded argmax, per sequence
    }
    const size_t n = chunk_rows(opts, capacity);
    PrefillScratch::plan(graph, capacity, n, sh, p);
    if (!opts.exact) p.scratch_bytes(PrefillScratch::mma_workspace(graph, n));
    if (persistent_decode_applies(graph, src, opts)) p.scratch_bytes(decode_program_size(graph, capacity).bytes());
    GpuAllocPlan out;
    out.weights = p.weights;
    out.state = p.state;
    out.scratch = p.scratch;
    out.gather = p.gather;
    return out;
}

std::unique_ptr<EngineModel> EngineModel::load_with(std::shared_ptr<CudaContext> ctx, ModelGraph graph,
                                                    const WeightSource &src, size_t capacity,
                                                    uint64_t expected_total, const EngineOptions &opts) {
    if (capacity == 0 || capacity > (1u << 24))
        throw TuckmillError(ErrorCode::InvalidRequest, "context capacity " + std::to_string(capacity) + " is out of range");
    if (opts.prefill_batch == 0 || opts.prefill_batch > TM_CUDA_GEMM_MMA_MAX_BATCH)
        throw TuckmillError(ErrorCode::InvalidRequest, "prefill batch must be 1.." + std::to_string(TM_CUDA_GEMM_MMA_MAX_BATCH));
    std::unique_ptr<EngineModel> m(new EngineModel());
    m->ctx_ = ctx;
    m->opts_ = opts;
    m->capacity_ = capacity;
    m->plan_ = alloc_plan_with(graph, src, capacity, opts);
    if (m->plan_.total() != expected_total)
        throw TuckmillError(ErrorCode::Internal, "engine preflight " + std::to_string(m->plan_.total()) +
                                                     " differs from the admitted total " + std::to_string(expected_total));
    const uint64_t base = ctx->allocated_bytes();
    m->impl_.reset(new Impl());
    Impl &I = *m->impl_;
    const CudaContext &c = *ctx;
    I.layers.reserve(graph.layers.size());
    // Split model: the exchange arena first (one collective allocation every rank maps), then the
    // blocks take their gather targets from it in plan order.
    if (opts.shard_world > 1) I.arena.buf = c.symm_zeros(m->plan_.gather);
    Shard sh{opts.shard_rank, opts.shard_world, opts.shard_world > 1 ? &I.arena : nullptr};
    // The single-launch pair exchange of a one-sequence decode step (TM_ENGINE_PAIR_EXCHANGE=0 in
    // every rank's environment goes back to push + reduction).
    sh.pair_exchange = opts.shard_world > 1;
    if (const char *e = std::getenv("TM_ENGINE_PAIR_EXCHANGE")) sh.pair_exchange = opts.shard_world > 1 && e[0] != '0';
    I.sh = sh;
    I.seqs = opts.sequences;
    I.log_stride = token_log_stride(capacity, I.seqs);
    I.pos_b.assign(I.seqs, 0);
    for (const LayerSpec &l : graph.layers) I.layers.push_back(Layer::load(c, src, l, graph, capacity, sh, I.seqs));
    I.embedding = Matrix::load(c, src, {graph.embedding});
    I.tied = graph.head == graph.embedding;
    I.head_rows = (uint32_t)(graph.vocab / sh.world);
    if (!I.tied) I.head_own = Matrix::load(c, src, {graph.head}, sh);
    else if (sh.world > 1)
        I.tied_view = I.embedding.type == 1
                          ? I.embedding.buf.view((size_t)sh.rank * I.head_rows * I.embedding.cols * 2,
                                                 (size_t)I.head_rows * I.embedding.cols * 2)
                          : c.row_view(I.embedding.buf, I.embedding.rows, I.embedding.cols, sh.rank * I.head_rows,
                                       I.head_rows);
    if (I.embedding.cols != graph.hidden || I.embedding.rows != graph.vocab ||
        (!I.tied && (I.head_own.cols != graph.hidden || I.head_own.rows != I.head_rows)))
        throw TuckmillError(ErrorCode::UnsupportedArchitecture, "embedding / head shapes do not match the graph");
    I.final_norm = vector(c, src, graph.final_norm);
    I.x = zeros_f32(c, graph.hidden);
    I.x2 = zeros_f32(c, graph.hidden);
    I.logits = zeros_f32(c, (size_t)I.head_rows * I.seqs);
    if (sh.world > 1) {
        I.logits_full = zeros_f32(c, graph.vocab);
        I.pairs = c.zeros((sh.world + 1) * 8 * I.seqs);
    }
    I.partial = c.zeros(kArgmaxPartialBytes * I.seqs);
    I.tokens = c.zeros(I.log_stride * I.seqs * 4);
    I.tokens_mirror = c.zeros(I.log_stride * I.seqs * 4, true);
    I.pos_buf = c.zeros(std::max<size_t>(16, I.seqs * 4));
    I.status = c.zeros(16, true);
    I.scratch = PrefillScratch::alloc(c, graph, capacity, chunk_rows(opts, capacity), sh);
    if (!opts.exact) c.mma_workspace_reserve(PrefillScratch::mma_workspace(graph, chunk_rows(opts, capacity)));

    m->graph_ = std::move(graph);
    const ModelGraph &g = m->graph_;

    // Record the decode step once: embedding of the logged token at the device
    // position, every layer, last norm + head, greedy token appended to the log,
    // position advanced.  (One command buffer per step in the reference:
    // crates/tuckcore/src/qwen35_gpu.rs:66-86, engine/metal.rs:2381-2449.)  Where the
    // model allows it the step becomes one persistent kernel, else a graph of kernels.
    I.persistent = persistent_decode_applies(g, src, opts);
    {
        // Bytes of one layer's four matrices.  Measured on this part: a decoder whose projections are
        // 2-6 MB (17 MB per layer) gains nothing -- its launches are bound by the dependency chain, not by
        // the DRAM round trip, and the side branch costs a microsecond per layer (827 -> 857 us per token) --
        // while 20-40 MB layers (the 1B-class shape, 7-15 MB projections) gain 2 % with one layer ahead;
        // wider models stream long enough per launch to be bandwidth-bound and do not fit anyway.
        uint64_t per_layer = 0;
        if (!I.layers.empty())
            for (const Matrix *mx : {&I.layers[0].mixer.qkv, &I.layers[0].mixer.o, &I.layers[0].ffn.gate_up,
                                     &I.layers[0].ffn.down})
                per_layer += Matrix::bytes_of(mx->type, mx->rows, mx->cols);
        size_t ahead = per_layer > (20u << 20) && per_layer <= (40u << 20) ? 1 : 0;
        if (const char *e = std::getenv("TM_ENGINE_L2_AHEAD")) ahead = (size_t)std::max(0, std::min(8, std::atoi(e)));
        if (opts.shard_world > 1 || I.persistent) ahead = 0;
        I.l2_ahead = ahead;
        // Folding the output norms into the next projection (Layer::decode_folded) saves two launches per
        // layer and is bit-identical, but measured slower on the Gemma-3-1B shape (1344 against 1299 us per
        // token: every CTA of the wide gate|up projection repeats a second reduction and two more vector
        // loads, which costs more than the small kernel it replaces): off unless TM_ENGINE_FOLD_NORMS=1.
        const char *fold = std::getenv("TM_ENGINE_FOLD_NORMS");
        I.fold_norms = fold && fold[0] == '1' && !I.persistent && opts.shard_world == 1 && I.head_type() == 8 &&
                       !I.layers.empty();
        for (const Layer &L : I.layers) I.fold_norms = I.fold_norms && L.norms_fold(g.hidden);
        if (ahead) c.prefetch_l2({&I.final_norm});  // the context's side stream comes into being outside a group
    }
    if (I.persistent) {
        const DecodeProgramSize ps = decode_program_size(g, capacity);
        c.begin_program(ps.max_ops, ps.vector_elems, ps.attention_elems);
        try {
            m->encode_decode_step();
        } catch (...) {
            c.abort_program();
            throw;
        }
        I.decode_graph = c.end_program();
    } else {
        c.begin_group();
        try {
            m->encode_decode_step();
        } catch (...) {
            c.abort_group();
            throw;
        }
        I.decode_graph = c.end_group_retain();
    }
    if (I.seqs > 1) {  // the step of all sequences, recorded once too
        c.begin_group();
        try {
            m->encode_batch_step();
        } catch (...) {
            c.abort_group();
            throw;
        }
        I.batch_graph = c.end_group_retain();
    }

    // The ledger must equal the preflight (crates/tuckcore/src/executor.rs:1571-1580).
    const uint64_t held = ctx->allocated_bytes() - base;
    if (held != m->plan_.total())
        throw TuckmillError(ErrorCode::Internal, g.architecture + " GPU ledger holds " + std::to_string(held) +
                                                     " but the preflight priced " + std::to_string(m->plan_.total()) +
                                                     "; refusing an unaccounted allocation");
    m->reset();
    return m;
}

void EngineModel::encode_decode_step() {
    Impl &I = *impl_;
    const CudaContext &c = *ctx_;
    const ModelGraph &g = graph_;
    if (I.embedding.type == 1)
        c.f16_row_indirect_dev(I.embedding.buf, I.embedding.rows, I.embedding.cols, I.tokens, 0, I.pos_buf, 0, 0,
                               g.embedding_scale, I.x);
    else
        c.row_indirect_dev(I.embedding.buf, I.embedding.rows, I.embedding.cols, I.tokens, 0, I.pos_buf, 0, 0,
                           g.embedding_scale, I.x);
    // Where it pays (see load_with), the weights of the layer(s) ahead are asked into L2 on a side
    // branch of the recorded graph.
    const size_t ahead = I.l2_ahead;
    auto prefetch = [&](size_t l) {
        if (ahead == 0 || l >= I.layers.size()) return;
        const Layer &P = I.layers[l];
        c.prefetch_l2({&P.mixer.qkv.buf, &P.mixer.o.buf, &P.ffn.gate_up.buf, &P.ffn.down.buf});
    };
    for (size_t l = 0; l < ahead; ++l) prefetch(l);
    if (I.fold_norms) {
        Residual R;
        R.cur = &I.x;
        R.alt = &I.x2;
        for (size_t l = 0; l < I.layers.size(); ++l) {
            prefetch(l + ahead);
            I.layers[l].decode_folded(c, R, I.pos_buf, I.status, g.hidden, g.eps, opts_.exact);
        }
        R.project(c, I.head_buf(), I.head_rows, I.head_cols(), I.final_norm, I.logits, g.eps);
    } else {
        for (size_t l = 0; l < I.layers.size(); ++l) {
            prefetch(l + ahead);
            I.layers[l].decode(c, I.x, I.pos_buf, I.status, g.hidden, g.eps, opts_.exact);
        }
        I.project_head(c, g.eps);
    }
    if (I.sh.world > 1)
        c.argmax_sharded(I.logits, I.head_rows, I.sh.rank * I.head_rows, I.partial, I.pairs, I.tokens, 1, &I.pos_buf, 0,
                         (uint32_t)capacity_ + 1, &I.tokens_mirror);
    else
        c.argmax_dev(I.logits, (uint32_t)g.vocab, I.partial, I.tokens, 1, I.pos_buf, 0, (uint32_t)capacity_ + 1,
                     &I.tokens_mirror);
    c.u32_add(I.pos_buf, 0, 1);
}

// One decode row per sequence: sequence s reads its logged token at pos_buf[s], attends to its own
// cache planes, appends its greedy token to its own log; every position advances (and stays on the
// last cache row once a sequence is full -- the host has stopped reading that sequence by then).
void EngineModel::encode_batch_step() {
    Impl &I = *impl_;
    const CudaContext &c = *ctx_;
    const ModelGraph &g = graph_;
    const size_t S = I.seqs;
    const uint32_t cap1 = (uint32_t)capacity_ + 1, stride = (uint32_t)I.log_stride;
    if (I.embedding.type != 8)
        throw TuckmillError(ErrorCode::UnsupportedQuantization, "several sequences need a Q8_0 embedding table");
    c.rows_indirect_seq(I.embedding.buf, I.embedding.rows, I.embedding.cols, I.tokens, stride, I.pos_buf, (uint32_t)S, 0,
                        g.embedding_scale, I.scratch.x);
    // The batched fused GEMV (rows bit-identical to the one-sequence step) serves `exact` mode and the
    // small cases; from three sequences on a wide model, and from nine on any, the tensor-core GEMM
    // streams the weights once for all rows and wins (measured on the 0.6B and 8B shapes).
    const size_t slice_limit = g.hidden >= 2048 ? 2 : 8;
    bool slices = S <= TM_CUDA_GEMM_MAX_BATCH && (opts_.exact || S <= slice_limit) && I.head_type() == 8;
    for (const Layer &L : I.layers) slices = slices && L.slices_apply();
    RowsAre rows;
    rows.pos_buf = &I.pos_buf;
    rows.status = &I.status;
    for (const Layer &L : I.layers) {
        if (slices) L.decode_rows(c, I.scratch, S, I.pos_buf, I.status, g.hidden, g.eps, opts_.exact);
        else L.prefill(c, I.scratch, S, 0, g.hidden, g.eps, opts_.exact, rows);
    }
    if (slices) {
        c.q8_0_gemm_fused(I.head_buf(), I.scratch.x, I.logits, I.head_rows, I.head_cols(), (uint32_t)S,
                          TM_CUDA_PRO_RMSNORM, &I.final_norm, g.eps, TM_CUDA_EPI_STORE);
    } else {
        c.rmsnorm(I.scratch.x, I.final_norm, I.scratch.h, (uint32_t)S, (uint32_t)g.hidden, g.eps);
        Matrix::gemm(c, I.head_buf(), I.head_rows, I.head_cols(), I.scratch.h, I.logits, (uint32_t)S, opts_.exact,
                     I.head_type());
    }
    if (I.sh.world > 1) {
        c.argmax_rows_sharded(I.logits, (uint32_t)S, I.head_rows, I.sh.rank * I.head_rows, I.partial, I.pairs, I.tokens,
                              stride, 1, I.pos_buf, cap1, &I.tokens_mirror);
    } else {
        c.argmax_rows_dev(I.logits, (uint32_t)S, (uint32_t)g.vocab, I.partial, I.tokens, stride, 1, I.pos_buf, cap1,
                          &I.tokens_mirror);
    }
    c.u32_add_sat(I.pos_buf, 0, (uint32_t)S, 1, (uint32_t)capacity_ - 1);
}

void EngineModel::step_ungrouped() {
    if (pos_ >= capacity_)
        throw TuckmillError(ErrorCode::ContextExceedsBudget,
                            "position " + std::to_string(pos_) + " exceeds KV capacity " + std::to_string(capacity_));
    encode_decode_step();
    pos_ += 1;
}

void EngineModel::check_device_status() {
    Impl &I = *impl_;
    ctx_->fence();
    uint32_t st = 0;
    I.status.download(0, &st, 4);
    if (st != 0) throw TuckmillError(ErrorCode::Internal, "a decode step ran past the KV capacity on the device");
    if (!opts_.exact && ctx_->mma_aborted())
        throw TuckmillError(ErrorCode::Internal,
                            "a pipeline wait of the tensor-core GEMM ran out; the prefill results are undefined");
    if (I.sh.world > 1 && ctx_->symm_status(I.arena.buf) != 0)
        throw TuckmillError(ErrorCode::Internal,
                            "a peer-memory exchange wait ran out; gathered activations of a step are stale");
    if (I.persistent) {
        const uint32_t ps = ctx_->program_status(I.decode_graph);
        if (ps != 0)
            throw TuckmillError(ErrorCode::Internal,
                                std::string("a bounded wait of the persistent decode kernel ran out (") +
                                    ((ps & 1u) ? "activations" : "weight stage") + "); the step's results are undefined");
    }
}

tm_cuda_graph *EngineModel::decode_program() const {
    return impl_->persistent ? impl_->decode_graph.raw() : nullptr;
}

EngineModel::~EngineModel() {
    if (ctx_) {
        try {
            ctx_->fence();
        } catch (...) {
        }
    }
}

void EngineModel::reset() {
    for (const Layer &L : impl_->layers) L.mixer.reset();
    impl_->pos_buf.zero();
    impl_->status.zero();
    ctx_->fence();
    pos_ = 0;
    std::fill(impl_->pos_b.begin(), impl_->pos_b.end(), 0);
}

size_t EngineModel::sequences() const { return impl_->seqs; }
size_t EngineModel::position_of(size_t seq) const { return seq < impl_->seqs ? impl_->pos_b[seq] : 0; }

void EngineModel::prefill(const uint32_t *tokens, size_t n, bool want_token) { prefill_seq(0, tokens, n, want_token); }

void EngineModel::prefill_seq(size_t seq, const uint32_t *tokens, size_t n, bool want_token) {
    if (seq >= impl_->seqs)
        throw TuckmillError(ErrorCode::InvalidRequest, "sequence " + std::to_string(seq) + " outside the " +
                                                           std::to_string(impl_->seqs) + " the engine holds");
    const size_t pos_ = impl_->pos_b[seq];  // this sequence's position (shadows the member: sequence 0's)
    if (n == 0) throw TuckmillError(ErrorCode::InvalidRequest, "prefill of zero tokens");
    if (pos_ + n > capacity_)
        throw TuckmillError(ErrorCode::ContextExceedsBudget, "position " + std::to_string(pos_ + n - 1) +
                                                                 " exceeds KV capacity " + std::to_string(capacity_));
    for (size_t i = 0; i < n; ++i)
        if (tokens[i] >= graph_.vocab)
            throw TuckmillError(ErrorCode::InvalidRequest, "token id " + std::to_string(tokens[i]) +
                                                               " is outside the vocabulary (0.." +
                                                               std::to_string(graph_.vocab) + ")");
    Impl &I = *impl_;
    const CudaContext &c = *ctx_;
    const size_t log0 = seq * I.log_stride;  // this sequence's token log
    I.tokens.upload((log0 + pos_) * 4, tokens, n * 4);
    const size_t batch = std::min<size_t>(opts_.prefill_batch, capacity_);
    RowsAre rows;
    rows.seq = seq;
    for (size_t t0 = 0; t0 < n; t0 += batch) {
        const size_t k = std::min(batch, n - t0);
        const bool last = t0 + k == n;
        const uint32_t pos0 = (uint32_t)(pos_ + t0), slot0 = (uint32_t)(log0 + pos_ + t0);
        c.grouped([&] {
            if (I.embedding.type == 1)
                c.f16_rows_indirect(I.embedding.buf, I.embedding.rows, I.embedding.cols, I.tokens, slot0, (uint32_t)k,
                                    graph_.embedding_scale, I.scratch.x);
            else
                c.rows_indirect(I.embedding.buf, I.embedding.rows, I.embedding.cols, I.tokens, slot0, (uint32_t)k,
                                graph_.embedding_scale, I.scratch.x);
            for (const Layer &L : I.layers)
                L.prefill(c, I.scratch, k, pos0, graph_.hidden, graph_.eps, opts_.exact, rows);
            if (last && want_token) {
                // Vocabulary projection for the last row only (engine/metal.rs:2610-2617).
                c.copy_f32(I.scratch.x, (uint32_t)((k - 1) * graph_.hidden), I.x, 0, (uint32_t)graph_.hidden);
                I.project_head(c, graph_.eps);
                if (I.sh.world > 1)
                    c.argmax_sharded(I.logits, I.head_rows, I.sh.rank * I.head_rows, I.partial, I.pairs, I.tokens,
                                     slot0 + (uint32_t)k, nullptr, 0, (uint32_t)(I.log_stride * I.seqs), nullptr);
                else
                    c.argmax_f32(I.logits, (uint32_t)graph_.vocab, I.partial, I.tokens, slot0 + (uint32_t)k);
            }
        });
    }
    I.pos_b[seq] = pos_ + n;
    if (seq == 0) this->pos_ = I.pos_b[0];
    const uint32_t p32 = (uint32_t)I.pos_b[seq];
    I.pos_buf.upload(seq * 4, &p32, 4);
}

uint32_t EngineModel::prefill_token() { return prefill_token_of(0); }

uint32_t EngineModel::prefill_token_of(size_t seq) {
    if (seq >= impl_->seqs) throw TuckmillError(ErrorCode::InvalidRequest, "sequence outside the engine's");
    uint32_t t = 0;
    impl_->tokens.download((seq * impl_->log_stride + impl_->pos_b[seq]) * 4, &t, 4);
    return t;
}

void EngineModel::step_batch(const uint32_t *tokens) {
    Impl &I = *impl_;
    if (I.seqs < 2) throw TuckmillError(ErrorCode::InvalidRequest, "the engine was loaded for one sequence");
    for (size_t s = 0; s < I.seqs; ++s) {
        if (tokens[s] >= graph_.vocab)
            throw TuckmillError(ErrorCode::InvalidRequest, "token id " + std::to_string(tokens[s]) +
                                                               " is outside the vocabulary (0.." +
                                                               std::to_string(graph_.vocab) + ")");
        if (I.pos_b[s] >= capacity_)
            throw TuckmillError(ErrorCode::ContextExceedsBudget, "sequence " + std::to_string(s) + " at position " +
                                                                     std::to_string(I.pos_b[s]) + " exceeds KV capacity " +
                                                                     std::to_string(capacity_));
    }
    for (size_t s = 0; s < I.seqs; ++s) I.tokens.upload((s * I.log_stride + I.pos_b[s]) * 4, &tokens[s], 4);
    I.batch_graph.launch();
    for (size_t s = 0; s < I.seqs; ++s) I.pos_b[s] += 1;
    pos_ = I.pos_b[0];
}

void EngineModel::submit_batch_greedy() {
    Impl &I = *impl_;
    if (I.seqs < 2) throw TuckmillError(ErrorCode::InvalidRequest, "the engine was loaded for one sequence");
    for (size_t s = 0; s < I.seqs; ++s)
        if (I.pos_b[s] >= capacity_)
            throw TuckmillError(ErrorCode::ContextExceedsBudget, "sequence " + std::to_string(s) + " is at capacity");
    I.batch_graph.launch();
    for (size_t s = 0; s < I.seqs; ++s) I.pos_b[s] += 1;
    pos_ = I.pos_b[0];
}

void EngineModel::logits_batch(float *out) {
    Impl &I = *impl_;
    check_device_status();
    if (I.sh.world > 1)
        throw TuckmillError(ErrorCode::InvalidRequest, "per-sequence logits are not gathered across a row split");
    I.logits.download(0, out, (size_t)I.seqs * graph_.vocab * 4);
}

std::vector<std::vector<uint32_t>> EngineModel::generate_batch(const std::vector<std::vector<uint32_t>> &prompts,
                                                               size_t max_new, bool ignore_eos, GenerateStats *stats) {
    Impl &I = *impl_;
    const size_t S = I.seqs, R = prompts.size();
    if (S < 2) throw TuckmillError(ErrorCode::InvalidRequest, "the engine was loaded for one sequence");
    if (R == 0 || R > S)
        throw TuckmillError(ErrorCode::InvalidRequest, std::to_string(R) + " requests for " + std::to_string(S) + " sequences");
    std::vector<std::vector<uint32_t>> out(R);
    if (max_new == 0) return out;
    const uint64_t l0 = ctx_->kernel_launches(), d0 = ctx_->committed();
    const uint64_t t_start = now_ns();
    reset();
    uint64_t n_prompt = 0;
    for (size_t s = 0; s < R; ++s) {
        prefill_seq(s, prompts[s].data(), prompts[s].size(), true);
        n_prompt += prompts[s].size();
    }
    auto is_stop = [&](uint32_t t) {
        return t == 0xFFFFFFFFu || (!ignore_eos && graph_.has_eos && t == graph_.eos_token_id);
    };
    std::vector<char> done(R, 0);
    for (size_t s = 0; s < R; ++s) {
        const uint32_t tok = prefill_token_of(s);
        if (tok == 0xFFFFFFFFu)
            throw TuckmillError(ErrorCode::Internal, "every logit was NaN; refusing to guess a token");
        out[s].push_back(tok);
        done[s] = is_stop(tok);
    }
    const uint64_t t_first = now_ns();
    uint64_t t_last = t_first;
    // A step advances every sequence on the device; the host follows the ones still wanted.  Step
    // i + 1 is submitted before step i is read (executor.rs:1080-1087), so a sequence that stops runs
    // one step too many, whose token is dropped.
    constexpr size_t kNone = (size_t)-1;
    struct Flight { uint64_t dispatch; std::vector<size_t> slot; };
    std::vector<size_t> submitted(R, 0), host_pos(I.pos_b.begin(), I.pos_b.begin() + R);
    auto wants = [&](size_t s) { return !done[s] && submitted[s] + 1 < max_new && host_pos[s] < capacity_; };
    auto any_wants = [&] {
        for (size_t s = 0; s < R; ++s)
            if (wants(s)) return true;
        return false;
    };
    auto submit = [&] {
        Flight f;
        f.slot.assign(R, kNone);
        for (size_t s = 0; s < R; ++s)
            if (wants(s)) {
                f.slot[s] = s * I.log_stride + host_pos[s] + 1;
                host_pos[s] += 1;
                submitted[s] += 1;
            }
        I.batch_graph.launch();
        f.dispatch = ctx_->committed();
        return f;
    };
    std::vector<Flight> inflight;
    if (any_wants()) inflight.push_back(submit());
    while (!inflight.empty()) {
        if (any_wants()) inflight.push_back(submit());
        const Flight f = inflight.front();
        inflight.erase(inflight.begin());
        for (size_t s = 0; s < R; ++s) {
            if (f.slot[s] == kNone || done[s]) continue;
            uint32_t tok = 0;
            I.tokens_mirror.download_after(f.slot[s] * 4, &tok, 4, f.dispatch);
            if (tok == 0xFFFFFFFFu)
                throw TuckmillError(ErrorCode::Internal, "every logit was NaN; refusing to guess a token");
            out[s].push_back(tok);
            if (is_stop(tok)) done[s] = 1;
        }
        t_last = now_ns();
    }
    ctx_->fence();
    check_device_status();
    // The device went on stepping the sequences the host had stopped following: the engine's state is
    // spent until the next reset().
    for (size_t s = 0; s < S; ++s) I.pos_b[s] = capacity_;
    pos_ = capacity_;
    if (stats) {
        uint64_t gen = 0;
        for (const auto &o : out) gen += o.size();
        stats->ttft_ns = t_first - t_start;
        stats->decode_span_ns = t_last - t_first;
        stats->prompt_tokens = n_prompt;
        stats->generated = gen;
        stats->kernel_launches = ctx_->kernel_launches() - l0;
        stats->dispatches = ctx_->committed() - d0;
        stats->h2d_bytes = n_prompt * 4 + 4 * R;
        stats->d2h_bytes = gen * 4 + 4 * R;
    }
    return out;
}

void EngineModel::step(uint32_t token) {
    if (token >= graph_.vocab)
        throw TuckmillError(ErrorCode::InvalidRequest, "token id " + std::to_string(token) +
                                                           " is outside the vocabulary (0.." +
                                                           std::to_string(graph_.vocab) + ")");
    if (pos_ >= capacity_)
        throw TuckmillError(ErrorCode::ContextExceedsBudget,
                            "position " + std::to_string(pos_) + " exceeds KV capacity " + std::to_string(capacity_));
    impl_->tokens.upload(pos_ * 4, &token, 4);
    impl_->decode_graph.launch();
    pos_ += 1;
    impl_->pos_b[0] = pos_;
}

// With a row split this is a collective: every rank must call it.
void EngineModel::logits(float *out) {
    Impl &I = *impl_;
    check_device_status();
    if (I.sh.world > 1) {
        ctx_->all_gather_rows(I.logits, I.logits_full, I.logits_full, 1, I.head_rows);
        I.logits_full.download(0, out, graph_.vocab * 4);
    } else {
        I.logits.download(0, out, graph_.vocab * 4);
    }
}

EngineModel::Ticket EngineModel::submit_greedy() {
    if (pos_ >= capacity_)
        throw TuckmillError(ErrorCode::ContextExceedsBudget,
                            "position " + std::to_string(pos_) + " exceeds KV capacity " + std::to_string(capacity_));
    impl_->decode_graph.launch();
    Ticket t;
    t.dispatch = ctx_->committed();
    t.slot = pos_ + 1;
    pos_ += 1;
    impl_->pos_b[0] = pos_;
    return t;
}

uint32_t EngineModel::collect_greedy(const Ticket &t) {
    uint32_t tok = 0;
    impl_->tokens_mirror.download_after(t.slot * 4, &tok, 4, t.dispatch);
    return tok;
}

std::vector<uint32_t> EngineModel::generate(const uint32_t *prompt, size_t n_prompt, size_t max_new, bool ignore_eos,
                                            GenerateStats *stats) {
    std::vector<uint32_t> out;
    if (max_new == 0) return out;
    const uint64_t l0 = ctx_->kernel_launches(), d0 = ctx_->committed();
    const uint64_t t_start = now_ns();
    reset();
    prefill(prompt, n_prompt, true);
    uint32_t tok = prefill_token();
    const uint64_t t_first = now_ns();
    uint64_t t_last = t_first;
    auto is_stop = [&](uint32_t t) {
        return t == 0xFFFFFFFFu || (!ignore_eos && graph_.has_eos && t == graph_.eos_token_id);
    };
    out.push_back(tok);
    if (tok == 0xFFFFFFFFu)
        throw TuckmillError(ErrorCode::Internal, "every logit was NaN; refusing to guess a token");
    if (!is_stop(tok)) {
        // Step i+1 is submitted before step i is collected (executor.rs:1080-1087):
        // the device already has token i in its log.
        std::vector<Ticket> inflight;
        size_t submitted = 0;
        const size_t want = max_new - 1;
        auto can_submit = [&] { return submitted < want && pos_ < capacity_; };
        if (can_submit()) { inflight.push_back(submit_greedy()); ++submitted; }
        while (!inflight.empty()) {
            if (can_submit()) { inflight.push_back(submit_greedy()); ++submitted; }
            const Ticket t = inflight.front();
            inflight.erase(inflight.begin());
            tok = collect_greedy(t);
            t_last = now_ns();
            if (tok == 0xFFFFFFFFu)
                throw TuckmillError(ErrorCode::Internal, "every logit was NaN; refusing to guess a token");
            out.push_back(tok);
            if (is_stop(tok)) break;
        }
        ctx_->fence();
    }
    check_device_status();
    if (stats) {
        stats->ttft_ns = t_first - t_start;
        stats->decode_span_ns = t_last - t_first;
        stats->prompt_tokens = n_prompt;
        stats->generated = out.size();
        stats->kernel_launches = ctx_->kernel_launches() - l0;
        stats->dispatches = ctx_->committed() - d0;
        stats->h2d_bytes = n_prompt * 4 + 4;
        stats->d2h_bytes = out.size() * 4 + 4;
    }
    return out;
}

}  // namespace tuckmill
