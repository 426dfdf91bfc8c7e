// Multi-GPU output-row split: the exchange step.  Every projection is split by
// output rows across the GPUs of one box (each output element needs one weight
// row and the whole input vector: crates/tuckcore/src/kernels.rs:186-204), each
// rank runs the single-GPU kernels on its slice, and one all-gather over
// NVLink/NVSwitch reassembles the vector.  The reference is single-device; this
// file has no counterpart there.
//
// NCCL is loaded at run time (dlopen of libnccl.so.2: the copy a host process
// such as torch already mapped, else the system one), so single-GPU users of
// the library need no NCCL at all.  Collectives are enqueued on the context's
// stream and can be recorded in a dispatch group like any operator.
#include <dlfcn.h>

#include <vector>

#include "tm_cuda_internal.cuh"
#include "tm_cuda_symm.cuh"
#include "tm_cuda_device.cuh"

namespace {

// The slice of the NCCL ABI this file uses (nccl.h: stable since 2.x).
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;  // ncclSuccess == 0
enum { ncclChar = 0, ncclFloat32 = 7 };

struct nccl_api {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

nccl_api *nccl() {
    static nccl_api api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        // TM_CUDA_NCCL_LIB names a specific copy; otherwise the loader's search order decides.
        const char *named = getenv("TM_CUDA_NCCL_LIB");
        void *h = named && *named ? dlopen(named, RTLD_NOW | RTLD_GLOBAL) : nullptr;
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h) {
            api.lib = h;
            api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
            api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
            api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
            api.AllGather = (decltype(api.AllGather))dlsym(h, "ncclAllGather");
            api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
            if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllGather) api.lib = nullptr;
        }
    }
    return api.lib ? &api : nullptr;
}

struct comm_state {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
};

// dst[t][r * w + c] = src[r][t][c]: NCCL concatenates whole per-rank buffers, a
// chunk of n token rows wants the ranks' slices side by side inside each row.
__global__ void interleave_kernel(const float *src, float *dst, uint32_t world, uint32_t n, uint32_t w) {
    const size_t total = (size_t)world * n * w;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = (uint32_t)(i % w);
        const uint32_t t = (uint32_t)((i / w) % n);
        const uint32_t r = (uint32_t)(i / ((size_t)w * n));
        dst[((size_t)t * world + r) * w + c] = src[i];
    }
}

constexpr uint32_t kNone = 0xFFFFFFFFu;

// One CTA: greedy choice among `world` (value, global index) pairs with the
// single-device rule -- larger value wins, equal values go to the lower global
// index, an index of 0xFFFFFFFF (all-NaN slice) never wins
// (crates/backend/src/sampling.rs:68-82).
__global__ void argmax_pairs_final_kernel(const float *pairs, uint32_t world, uint32_t *out, uint32_t base,
                                          const uint32_t *pos, uint32_t out_cap, uint32_t *mirror) {
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    if (threadIdx.x != 0) return;
    float bv = 0.0f;
    uint32_t bi = kNone;
    for (uint32_t r = 0; r < world; ++r) {
        const float v = pairs[2 * r];
        const uint32_t i = __float_as_uint(pairs[2 * r + 1]);
        if (i == kNone) continue;
        if (bi == kNone || v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
    const uint32_t slot = pos ? base + *pos : base;
    if (slot < out_cap) {
        out[slot] = bi;
        if (mirror) mirror[slot] = bi;
    }
}

// (value, global index) of this rank's slice from the 64 partials of argmax_partial.
__global__ void argmax_pair_kernel(const float *pv, const uint32_t *pi, float *pair, uint32_t index_offset) {
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    if (threadIdx.x != 0) return;
    float bv = 0.0f;
    uint32_t bi = kNone;
    for (int g = 0; g < 64; ++g) {
        const uint32_t i = pi[g];
        const float v = pv[g];
        if (i == kNone) continue;
        if (bi == kNone || v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
    pair[0] = bv;
    pair[1] = __uint_as_float(bi == kNone ? kNone : bi + index_offset);
}


// The two kernels above for n_rows rows: thread r handles row r.
__global__ void argmax_pair_rows_kernel(const float *pv, const uint32_t *pi, float *pair, uint32_t index_offset,
                                        uint32_t n_rows) {
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    float bv = 0.0f;
    uint32_t bi = kNone;
    for (int g = 0; g < 64; ++g) {
        const uint32_t i = pi[r * 64u + g];
        const float v = pv[r * 64u + g];
        if (i == kNone) continue;
        if (bi == kNone || v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
    pair[2 * r] = bv;
    pair[2 * r + 1] = __uint_as_float(bi == kNone ? kNone : bi + index_offset);
}
// pairs: [world][n_rows] (value, index); row r's winner goes to out[r * out_stride + base + pos[r]].
__global__ void argmax_pairs_final_rows_kernel(const float *pairs, uint32_t world, uint32_t n_rows, uint32_t *out,
                                               uint32_t out_stride, uint32_t base, const uint32_t *pos,
                                               uint32_t out_cap, uint32_t *mirror) {
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    float bv = 0.0f;
    uint32_t bi = kNone;
    for (uint32_t w = 0; w < world; ++w) {
        const float v = pairs[2 * ((size_t)w * n_rows + r)];
        const uint32_t i = __float_as_uint(pairs[2 * ((size_t)w * n_rows + r) + 1]);
        if (i == kNone) continue;
        if (bi == kNone || v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
    const uint32_t slot = base + pos[r];
    if (slot < out_cap) {
        out[(size_t)r * out_stride + slot] = bi;
        if (mirror) mirror[(size_t)r * out_stride + slot] = bi;
    }
}

// ---- exchange through peer memory --------------------------------------------
// A symmetric buffer is the same allocation on every rank, each mapped into every
// other rank's address space (CUDA IPC).  An all-gather is then a PUSH: the producer
// stores its slice straight into every rank's copy (plain stores over NVLink, no
// multicast, no library kernel touching peer memory), the last block of the push
// raises a per-sender sequence flag on every rank and waits -- bounded -- until
// every sender's flag on THIS rank has reached the same sequence number.
using symm_state = tm_symm_state;

struct push_args {
    const float *src;        // [n_rows][width] local slice
    float *const *peer;      // device table: the target buffer on every rank
    uint32_t world, rank, n_rows, width;
    uint32_t tail_off;       // float offset of the flag tail inside the buffer
    uint32_t dst_off;        // float offset of the target view inside the buffer
};

__global__ void __launch_bounds__(256) push_rows_kernel(const push_args a) {
    __shared__ uint32_t s_flag[2];
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    const size_t total = (size_t)a.n_rows * a.width;
    const bool vec = (a.width & 3u) == 0u;
    if (vec) {
        const size_t quads = total / 4;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (size_t)gridDim.x * blockDim.x) {
            const float4 v = *(const float4 *)(a.src + i * 4);
            const size_t t = (i * 4) / a.width, c = (i * 4) % a.width;
            const size_t dst = a.dst_off + (t * a.world + a.rank) * a.width + c;
            for (uint32_t r = 0; r < a.world; ++r) *(float4 *)(a.peer[r] + dst) = v;
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
            const size_t t = i / a.width, c = i % a.width;
            const size_t dst = a.dst_off + (t * a.world + a.rank) * a.width + c;
            const float v = a.src[i];
            for (uint32_t r = 0; r < a.world; ++r) a.peer[r][dst] = v;
        }
    }
    // Every block's stores are fenced to system scope before it counts itself in; the block that
    // counts last therefore signals after ALL of this launch's stores.
    __threadfence_system();
    __syncthreads();
    tm_symm_finish(a.peer, a.tail_off, a.world, a.rank, s_flag);
}

// One-row exchange with the sum folded in, for a decode step's partial products: every word on the
// wire is an 8-byte (value, sequence number) pair, written with ONE store into this rank's slot on
// every peer, so a reader needs no fence and no flag -- it polls the word it wants until the pair
// carries this exchange's number.  Each thread sends its column of the rank's partial row, collects
// the same column from every other rank's slot (all loads issued together, re-polled only where the
// number is old), adds the ranks' values in rank order and adds the sum to y: the exchange, the
// reduction and the residual add are one launch.  Every poll loop is bounded; one that runs out sets
// the buffer's status bit 0 and goes on with whatever the slot holds.
struct ll_args {
    const float *src;        // [width] this rank's partial row
    float *y;                // [width] += sum over ranks
    float *const *peer;      // device table: the arena on every rank
    uint32_t world, rank, width;
    uint32_t tail_off;       // float offset of the flag tail inside the arena
    uint32_t dst_off;        // float offset of the slot view [world][width] of 8-byte pairs
};
constexpr uint32_t kLlSpinLimit = 1u << 23;  // re-polls of ~0.5 us: a few seconds (ranks start a step from their own hosts)

__device__ __forceinline__ unsigned long long ll_load(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256) exchange_add_ll_kernel(const ll_args a) {
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    uint32_t *tail = (uint32_t *)(a.peer[a.rank] + a.tail_off);
    const uint32_t seq = *(volatile uint32_t *)(tail + 80) + 1u;  // the same number on every rank
    const uint32_t i = blockIdx.x * 256u + threadIdx.x;
    if (i < a.width) {
        const float own = a.src[i];
        const unsigned long long word = ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(own);
        for (uint32_t r = 0; r < a.world; ++r) {
            if (r == a.rank) continue;
            unsigned long long *q = (unsigned long long *)(a.peer[r] + a.dst_off) + (size_t)a.rank * a.width + i;
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(q), "l"(word) : "memory");
        }
        const unsigned long long *mine = (const unsigned long long *)(a.peer[a.rank] + a.dst_off) + i;
        float p = 0.0f;
        for (uint32_t r0 = 0; r0 < a.world; r0 += 8) {
            unsigned long long w[8];
#pragma unroll
            for (uint32_t k = 0; k < 8; ++k)
                w[k] = r0 + k < a.world && r0 + k != a.rank ? ll_load(mine + (size_t)(r0 + k) * a.width) : 0ull;
#pragma unroll
            for (uint32_t k = 0; k < 8; ++k) {
                const uint32_t r = r0 + k;
                if (r >= a.world) break;
                float v = own;
                if (r != a.rank) {
                    uint32_t spin = 0;
                    while ((uint32_t)(w[k] >> 32) != seq) {
                        if (++spin > kLlSpinLimit) {
                            atomicOr(tail + 72, 1u);
                            break;
                        }
                        w[k] = ll_load(mine + (size_t)r * a.width);
                    }
                    v = __uint_as_float((uint32_t)w[k]);
                }
                p = r == 0 ? v : __fadd_rn(p, v);
            }
        }
        a.y[i] = __fadd_rn(a.y[i], p);
    }
    // The block that finishes last publishes the number: the next exchange on this rank reads it.
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(tail + 84, 1u) == gridDim.x - 1u) {
            tail[84] = 0u;
            *(volatile uint32_t *)(tail + 80) = seq;
        }
    }
}

}  // namespace

extern "C" {

void tm_cuda_comm_release(tm_cuda_ctx *ctx) {
    if (!ctx || !ctx->comm) return;
    comm_state *c = (comm_state *)ctx->comm;
    nccl_api *n = nccl();
    if (n && c->comm) n->CommDestroy(c->comm);
    delete c;
    ctx->comm = nullptr;
}

int tm_cuda_comm_unique_id(void *out128, char *err, size_t err_cap) {
    nccl_api *n = nccl();
    if (!n) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded: %s", dlerror());
    if (!out128) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "null id buffer");
    ncclUniqueId id;
    const ncclResult_t r = n->GetUniqueId(&id);
    if (r != 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "ncclGetUniqueId failed: %s",
                       n->GetErrorString ? n->GetErrorString(r) : "?");
    memcpy(out128, &id, sizeof id);
    return TM_CUDA_OK;
}

int tm_cuda_comm_init(tm_cuda_ctx *ctx, const void *id128, int rank, int world, char *err, size_t err_cap) {
    TM_ENTER();
    nccl_api *n = nccl();
    if (!n) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded");
    if (!id128 || world < 1 || world > 64 || rank < 0 || rank >= world)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "rank %d of %d", rank, world);
    if (ctx->comm) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "the context already has a communicator");
    ncclUniqueId id;
    memcpy(&id, id128, sizeof id);
    comm_state *c = new comm_state();
    c->rank = rank;
    c->world = world;
    const ncclResult_t r = n->CommInitRank(&c->comm, world, id, rank);
    if (r != 0) {
        delete c;
        return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "ncclCommInitRank failed: %s",
                       n->GetErrorString ? n->GetErrorString(r) : "?");
    }
    ctx->comm = c;
    return TM_CUDA_OK;
}

int tm_cuda_comm_rank(const tm_cuda_ctx *ctx, int *rank, int *world) {
    if (!ctx || !ctx->comm) return TM_CUDA_ERR_UNSUPPORTED;
    const comm_state *c = (const comm_state *)ctx->comm;
    if (rank) *rank = c->rank;
    if (world) *world = c->world;
    return TM_CUDA_OK;
}

int tm_cuda_all_gather_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *src, uint32_t src_off, tm_cuda_buffer *dst,
                           uint32_t dst_off, uint32_t count, char *err, size_t err_cap) {
    TM_ENTER();
    comm_state *c = (comm_state *)ctx->comm;
    nccl_api *n = nccl();
    if (!c || !n) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "the context has no communicator");
    if (count == 0) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "empty all-gather");
    TM_CHECK_BUF(src, ((size_t)src_off + count) * 4, "all-gather source");
    TM_CHECK_BUF(dst, ((size_t)dst_off + (size_t)count * c->world) * 4, "all-gather target");
    TM_OP_BEGIN("all_gather");
    const ncclResult_t r = n->AllGather((const float *)src->dev + src_off, (float *)dst->dev + dst_off, count,
                                        ncclFloat32, c->comm, ctx->stream);
    if (r != 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "ncclAllGather failed: %s",
                       n->GetErrorString ? n->GetErrorString(r) : "?");
    TM_OP_END(1);
}

int tm_cuda_all_gather_rows_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *src, tm_cuda_buffer *stage, tm_cuda_buffer *dst,
                                uint32_t n_rows, uint32_t width, char *err, size_t err_cap) {
    TM_ENTER();
    comm_state *c = (comm_state *)ctx->comm;
    nccl_api *n = nccl();
    if (!c || !n) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "the context has no communicator");
    if (n_rows == 0 || width == 0) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "empty all-gather");
    const size_t per = (size_t)n_rows * width;
    TM_CHECK_BUF(src, per * 4, "all-gather source");
    TM_CHECK_BUF(stage, per * c->world * 4, "all-gather staging");
    TM_CHECK_BUF(dst, per * c->world * 4, "all-gather target");
    TM_OP_BEGIN("all_gather_rows");
    const ncclResult_t r = n->AllGather(src->dev, n_rows == 1 ? dst->dev : stage->dev, per, ncclFloat32, c->comm,
                                        ctx->stream);
    if (r != 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "ncclAllGather failed: %s",
                       n->GetErrorString ? n->GetErrorString(r) : "?");
    uint64_t kernels = 1;
    if (n_rows > 1) {
        const size_t total = per * c->world;
        const int grid = (int)((total + 255) / 256 > 148 * 8 ? 148 * 8 : (total + 255) / 256);
        interleave_kernel<<<grid, 256, 0, ctx->stream>>>((const float *)stage->dev, (float *)dst->dev,
                                                          (uint32_t)c->world, n_rows, width);
        kernels = 2;
    }
    TM_OP_END(kernels);
}

int tm_cuda_argmax_sharded_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *x, uint32_t n, uint32_t index_offset,
                               tm_cuda_buffer *partial, tm_cuda_buffer *pairs, tm_cuda_buffer *out, uint32_t base,
                               tm_cuda_buffer *pos_buf, uint32_t pos_index, uint32_t out_cap,
                               tm_cuda_buffer *mirror, char *err, size_t err_cap) {
    // local slice -> (value, global index); all-gather of the pairs; the single-device rule over them
    TM_ENTER();
    if (n == 0) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "argmax over zero elements");
    TM_CHECK_BUF(x, (size_t)n * 4, "logits");
    TM_CHECK_BUF(partial, 512, "argmax partials");
    comm_state *c = (comm_state *)ctx->comm;
    nccl_api *nc = nccl();
    if (!c || !nc) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "the context has no communicator");
    TM_CHECK_BUF(pairs, (size_t)(c->world + 1) * 8, "argmax pairs");
    TM_CHECK_BUF(out, (size_t)out_cap * 4, "token log");
    if (mirror) TM_CHECK_BUF(mirror, (size_t)out_cap * 4, "token log mirror");
    const uint32_t *pos = nullptr;
    if (pos_buf) {
        TM_CHECK_BUF(pos_buf, ((size_t)pos_index + 1) * 4, "position");
        pos = (const uint32_t *)pos_buf->dev + pos_index;
    }
    TM_OP_BEGIN("argmax_sharded");
    float *mine = (float *)pairs->dev + 2 * c->world;  // own pair after the gathered block
    TM_CUDA_TRY(tm_argmax_partial_launch(ctx, (const float *)x->dev, n, (float *)partial->dev,
                                         (uint32_t *)(partial->dev + 256)));
    TM_CUDA_TRY(tm_launch_pdl(ctx, argmax_pair_kernel, dim3(1), dim3(32), 0, (const float *)partial->dev,
                              (const uint32_t *)(partial->dev + 256), mine, index_offset));
    const ncclResult_t r = nc->AllGather(mine, pairs->dev, 2, ncclFloat32, c->comm, ctx->stream);
    if (r != 0) return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "ncclAllGather failed");
    argmax_pairs_final_kernel<<<1, 32, 0, ctx->stream>>>((const float *)pairs->dev, (uint32_t)c->world,
                                                         (uint32_t *)out->dev, base, pos, out_cap,
                                                         mirror ? (uint32_t *)mirror->dev : nullptr);
    TM_OP_END(4);
}

int tm_cuda_argmax_rows_sharded_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *x, uint32_t n_rows, uint32_t n,
                                    uint32_t index_offset, tm_cuda_buffer *partial, tm_cuda_buffer *pairs,
                                    tm_cuda_buffer *out, uint32_t out_stride, uint32_t base, tm_cuda_buffer *pos_buf,
                                    uint32_t out_cap, tm_cuda_buffer *mirror, char *err, size_t err_cap) {
    TM_ENTER();
    if (n == 0 || n_rows == 0 || n_rows > 65535u)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "argmax over %u rows of %u elements", n_rows, n);
    if (out_cap == 0 || out_cap > out_stride)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "token log of %u slots in rows of %u", out_cap, out_stride);
    comm_state *c = (comm_state *)ctx->comm;
    nccl_api *nc = nccl();
    if (!c || !nc) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "the context has no communicator");
    TM_CHECK_BUF(x, (size_t)n_rows * n * 4, "logits");
    TM_CHECK_BUF(partial, (size_t)n_rows * 512, "argmax partials");
    TM_CHECK_BUF(pairs, (size_t)(c->world + 1) * n_rows * 8, "argmax pairs");
    TM_CHECK_BUF(out, ((size_t)(n_rows - 1) * out_stride + out_cap) * 4, "token logs");
    if (mirror) TM_CHECK_BUF(mirror, ((size_t)(n_rows - 1) * out_stride + out_cap) * 4, "token log mirrors");
    TM_CHECK_BUF(pos_buf, (size_t)n_rows * 4, "positions");
    TM_OP_BEGIN("argmax_rows_sharded");
    float *pv = (float *)partial->dev;
    uint32_t *pi = (uint32_t *)(partial->dev + (size_t)n_rows * 256);
    float *mine = (float *)pairs->dev + 2 * (size_t)c->world * n_rows;  // own pairs after the gathered block
    TM_CUDA_TRY(tm_argmax_rows_partial_launch(ctx, (const float *)x->dev, n_rows, n, pv, pi));
    TM_CUDA_TRY(tm_launch_pdl(ctx, argmax_pair_rows_kernel, dim3((n_rows + 63) / 64), dim3(64), 0, (const float *)pv,
                              (const uint32_t *)pi, mine, index_offset, n_rows));
    const ncclResult_t r = nc->AllGather(mine, pairs->dev, 2 * (size_t)n_rows, ncclFloat32, c->comm, ctx->stream);
    if (r != 0) return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "ncclAllGather failed");
    argmax_pairs_final_rows_kernel<<<(n_rows + 63) / 64, 64, 0, ctx->stream>>>(
        (const float *)pairs->dev, (uint32_t)c->world, n_rows, (uint32_t *)out->dev, out_stride, base,
        (const uint32_t *)pos_buf->dev, out_cap, mirror ? (uint32_t *)mirror->dev : nullptr);
    TM_OP_END(4);
}

void tm_cuda_symm_release(tm_cuda_buffer *b) {
    if (!b || !b->symm) return;
    symm_state *st = (symm_state *)b->symm;
    for (int r = 0; r < st->world; ++r)
        if (r != st->rank && st->peer[r]) cudaIpcCloseMemHandle(st->peer[r]);
    if (st->d_peer) cudaFree(st->d_peer);
    delete st;
    b->symm = nullptr;
}

tm_cuda_buffer *tm_cuda_symm_alloc(tm_cuda_ctx *ctx, size_t bytes, char *err, size_t err_cap) {
    if (!ctx) {
        tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "null context");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(ctx->mu);
    comm_state *c = (comm_state *)ctx->comm;
    nccl_api *n = nccl();
    if (!c || !n || c->world < 2 || c->world > kSymmMaxWorld || bytes == 0) {
        tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "a symmetric buffer needs a communicator of 2..%d ranks", kSymmMaxWorld);
        return nullptr;
    }
    if (ctx->group_open) {
        tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "symmetric buffers are allocated outside dispatch groups");
        return nullptr;
    }
    cudaSetDevice(ctx->device);
    const size_t payload = tm_round_up(bytes, 256), total = payload + kSymmTail;
    unsigned char *dev = nullptr, *hbuf = nullptr;
    symm_state *st = new symm_state();
    st->world = c->world;
    st->rank = c->rank;
    st->payload = payload;
    cudaIpcMemHandle_t mine;
    std::vector<cudaIpcMemHandle_t> all((size_t)c->world);
    bool ok = cudaMalloc(&dev, total) == cudaSuccess && cudaMemset(dev, 0, total) == cudaSuccess &&
              cudaIpcGetMemHandle(&mine, dev) == cudaSuccess &&
              cudaMalloc(&hbuf, sizeof(mine) * (size_t)(c->world + 1)) == cudaSuccess;
    if (ok) {
        // every rank's handle, gathered through the communicator
        ok = cudaMemcpy(hbuf + sizeof(mine) * (size_t)c->world, &mine, sizeof(mine), cudaMemcpyHostToDevice) == cudaSuccess &&
             n->AllGather(hbuf + sizeof(mine) * (size_t)c->world, hbuf, sizeof(mine), ncclChar, c->comm, ctx->stream) == 0 &&
             cudaStreamSynchronize(ctx->stream) == cudaSuccess &&
             cudaMemcpy(all.data(), hbuf, sizeof(mine) * (size_t)c->world, cudaMemcpyDeviceToHost) == cudaSuccess;
    }
    for (int r = 0; ok && r < c->world; ++r) {
        if (r == c->rank) st->peer[r] = dev;
        else ok = cudaIpcOpenMemHandle(&st->peer[r], all[(size_t)r], cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
    }
    if (ok)
        ok = cudaMalloc(&st->d_peer, sizeof(void *) * kSymmMaxWorld) == cudaSuccess &&
             cudaMemcpy(st->d_peer, st->peer, sizeof(void *) * kSymmMaxWorld, cudaMemcpyHostToDevice) == cudaSuccess;
    if (hbuf) cudaFree(hbuf);
    if (!ok) {
        const cudaError_t e = cudaGetLastError();
        tm_fail(err, err_cap, TM_CUDA_ERR_ALLOC, "symmetric buffer of %zu bytes could not be set up: %s", bytes,
                cudaGetErrorString(e));
        tm_cuda_buffer tmp;
        tmp.symm = st;
        tm_cuda_symm_release(&tmp);
        if (dev) cudaFree(dev);
        return nullptr;
    }
    tm_cuda_buffer *b = new tm_cuda_buffer();
    b->owner = ctx;
    b->dev = dev;
    b->len = bytes;  // the ledger counts what was asked for; rounding and the flag tail are bookkeeping
    b->symm = st;
    ctx->live.insert(b);
    ctx->allocated.fetch_add(bytes);
    return b;
}

int tm_cuda_push_rows_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *src, tm_cuda_buffer *dst, uint32_t n_rows, uint32_t width,
                          char *err, size_t err_cap) {
    TM_ENTER();
    if (n_rows == 0 || width == 0) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "empty push");
    // The target is a symmetric buffer or a view into one (same offset on every rank).
    tm_cuda_buffer *root = dst && dst->parent ? dst->parent : dst;
    if (!dst || ctx->live.find(dst) == ctx->live.end() || !root || !root->symm)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "the push target is not (a view of) a symmetric buffer of this context");
    symm_state *st = (symm_state *)root->symm;
    const size_t dst_off = (size_t)(dst->dev - root->dev);
    if (dst_off % 16 != 0) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "push target view is not 16-byte aligned");
    const size_t per = (size_t)n_rows * width;
    TM_CHECK_BUF(src, per * 4, "push source");
    TM_CHECK_BUF(dst, per * (size_t)st->world * 4, "push target");
    if (src == dst) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "push in place");
    TM_OP_BEGIN("push_rows");
    push_args a;
    a.src = (const float *)src->dev;
    a.peer = (float *const *)st->d_peer;
    a.world = (uint32_t)st->world;
    a.rank = (uint32_t)st->rank;
    a.n_rows = n_rows;
    a.width = width;
    a.tail_off = (uint32_t)(st->payload / 4);
    a.dst_off = (uint32_t)(dst_off / 4);
    const size_t work = (width & 3u) == 0u ? per / 4 : per;
    int grid = (int)((work + 255) / 256);
    grid = grid < 1 ? 1 : grid > ctx->sm_count * 2 ? ctx->sm_count * 2 : grid;
    TM_CUDA_TRY(tm_launch_pdl(ctx, push_rows_kernel, dim3(grid), dim3(256), 0, a));
    TM_OP_END(1);
}

int tm_cuda_exchange_add_ll_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *src, tm_cuda_buffer *slots, tm_cuda_buffer *y,
                                uint32_t width, char *err, size_t err_cap) {
    TM_ENTER();
    if (width == 0) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "empty exchange");
    tm_cuda_buffer *root = slots && slots->parent ? slots->parent : slots;
    if (!slots || ctx->live.find(slots) == ctx->live.end() || !root || !root->symm)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "the slots are not (a view of) a symmetric buffer of this context");
    symm_state *st = (symm_state *)root->symm;
    const size_t dst_off = (size_t)(slots->dev - root->dev);
    if (dst_off % 16 != 0) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "slot view is not 16-byte aligned");
    TM_CHECK_BUF(src, (size_t)width * 4, "partial row");
    TM_CHECK_BUF(y, (size_t)width * 4, "accumulated row");
    TM_CHECK_BUF(slots, (size_t)width * (size_t)st->world * 8, "exchange slots");
    if (src == slots || y == slots) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "exchange in place");
    if (ctx->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "operator exchange_add_ll cannot be recorded into a persistent program");
    TM_OP_BEGIN("exchange_add_ll");
    ll_args a;
    a.src = (const float *)src->dev;
    a.y = (float *)y->dev;
    a.peer = (float *const *)st->d_peer;
    a.world = (uint32_t)st->world;
    a.rank = (uint32_t)st->rank;
    a.width = width;
    a.tail_off = (uint32_t)(st->payload / 4);
    a.dst_off = (uint32_t)(dst_off / 4);
    TM_CUDA_TRY(tm_launch_pdl(ctx, exchange_add_ll_kernel, dim3((width + 255) / 256), dim3(256), 0, a));
    TM_OP_END(1);
}

// Bit 0 set: a push on this buffer gave up waiting for a peer (its consumer read stale rows).
int tm_cuda_symm_status(tm_cuda_ctx *ctx, tm_cuda_buffer *buf, uint32_t *status, char *err, size_t err_cap) {
    TM_ENTER();
    if (!buf || ctx->live.find(buf) == ctx->live.end() || !buf->symm || !status)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "not a symmetric buffer of this context");
    symm_state *st = (symm_state *)buf->symm;
    TM_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    TM_CUDA_TRY(cudaMemcpy(status, buf->dev + st->payload + 72 * 4, 4, cudaMemcpyDeviceToHost));
    return TM_CUDA_OK;
}

}  // extern "C"
