// Context, buffers, copies, grouped encoding (CUDA graphs) and the measurement
// surface of the C ABI.  The Metal original is native/metal/tm_metal.m:226-760,
// 1346-1420 (one device + one queue, typed handles, command-buffer groups,
// completion counters); this is the CUDA design of the same contract: one
// device + one in-order stream, stream capture for groups, events for
// completion and GPU time.
#include <cstdlib>

#include "tm_cuda_internal.cuh"

namespace {

char g_info[256] = "";
std::once_flag g_info_once;

cudaEvent_t take_event(tm_cuda_ctx *ctx) {
    if (!ctx->event_pool.empty()) {
        cudaEvent_t e = ctx->event_pool.back();
        ctx->event_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
    return e;
}

int label_index(tm_cuda_ctx *ctx, const char *label) {
    if (!ctx->profiling) return -1;
    for (size_t i = 0; i < ctx->profile.size(); ++i)
        if (ctx->profile[i].name == label) return (int)i;
    ctx->profile.push_back({label, 0, 0});
    return (int)ctx->profile.size() - 1;
}

// Retire every pending dispatch whose end event has fired (in order).
void poll_locked(tm_cuda_ctx *ctx, bool wait_all) {
    while (!ctx->pending.empty()) {
        tm_commit &c = ctx->pending.front();
        cudaError_t q = wait_all ? cudaEventSynchronize(c.end) : cudaEventQuery(c.end);
        if (q != cudaSuccess) {
            if (q != cudaErrorNotReady) cudaGetLastError();
            break;
        }
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, c.begin, c.end) == cudaSuccess) {
            const uint64_t ns = (uint64_t)((double)ms * 1e6);
            ctx->gpu_nanos.fetch_add(ns);
            ctx->last_gpu_ns.store(ns);
            if (c.label >= 0 && (size_t)c.label < ctx->profile.size()) {
                ctx->profile[c.label].nanos += ns;
                ctx->profile[c.label].count += 1;
            }
        }
        ctx->event_pool.push_back(c.begin);
        ctx->event_pool.push_back(c.end);
        ctx->completed.store(c.seq);
        ctx->pending.pop_front();
    }
}

int commit_begin(tm_cuda_ctx *ctx, tm_commit *c, const char *label, char *err, size_t err_cap) {
    c->begin = take_event(ctx);
    c->end = take_event(ctx);
    if (!c->begin || !c->end)
        return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "cannot create CUDA events");
    c->label = label_index(ctx, label);
    TM_CUDA_TRY(cudaEventRecord(c->begin, ctx->stream));
    return TM_CUDA_OK;
}

int commit_end(tm_cuda_ctx *ctx, tm_commit *c, char *err, size_t err_cap) {
    TM_CUDA_TRY(cudaEventRecord(c->end, ctx->stream));
    c->seq = ctx->committed.fetch_add(1) + 1;
    ctx->pending.push_back(*c);
    if (ctx->pending.size() > 256) poll_locked(ctx, false);
    return TM_CUDA_OK;
}

}  // namespace

int tm_op_begin(tm_cuda_ctx *ctx, const char *label, char *err, size_t err_cap) {
    if (ctx->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "operator %s cannot be recorded into a persistent program", label);
    if (ctx->group_open) return TM_CUDA_OK;
    return commit_begin(ctx, &ctx->open_commit, label, err, err_cap);
}

int tm_op_end(tm_cuda_ctx *ctx, uint64_t kernels, char *err, size_t err_cap) {
    if (ctx->group_open) {
        ctx->group_kernels += kernels;
        return TM_CUDA_OK;
    }
    ctx->launches.fetch_add(kernels);
    return commit_end(ctx, &ctx->open_commit, err, err_cap);
}

int tm_check_packed(tm_cuda_ctx *ctx, const tm_cuda_buffer *w, uint32_t rows, uint32_t cols,
                    char *err, size_t err_cap) {
    if (rows == 0 || cols == 0 || cols % 32 != 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "Q8_0 geometry %u x %u: rows and cols must be positive, cols a multiple of 32",
                       rows, cols);
    if (!w || ctx->live.find(w) == ctx->live.end())
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "weight buffer does not belong to this context");
    if (!w->parent && w->len < tm_cuda_q8_0_packed_bytes(rows, cols))
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "weight buffer holds %zu bytes, needs %zu",
                       w->len, tm_cuda_q8_0_packed_bytes(rows, cols));
    if (w->layout != TM_LAYOUT_Q8_0_PACKED || w->rows != rows || w->cols != cols)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "weight buffer is not a packed %u x %u Q8_0 matrix (pack it with "
                       "tm_cuda_q8_0_pack first)", rows, cols);
    return TM_CUDA_OK;
}

extern "C" {

int tm_cuda_available(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int usable = 0;
    for (int d = 0; d < n; ++d) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d) == cudaSuccess &&
            major == 10)
            ++usable;
    }
    return usable;
}

const char *tm_cuda_runtime_info(void) {
    std::call_once(g_info_once, [] {
        int n = 0;
        cudaDeviceProp p;
        if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0 ||
            cudaGetDeviceProperties(&p, 0) != cudaSuccess) {
            cudaGetLastError();
            snprintf(g_info, sizeof g_info, "no CUDA device");
            return;
        }
        snprintf(g_info, sizeof g_info, "%s sm_%d%d, %d SMs, %.1f GiB, %d device(s)", p.name,
                 p.major, p.minor, p.multiProcessorCount,
                 (double)p.totalGlobalMem / (1024.0 * 1024.0 * 1024.0), n);
    });
    return g_info;
}

tm_cuda_ctx *tm_cuda_create(int device, char *err, size_t err_cap) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        cudaGetLastError();
        tm_fail(err, err_cap, TM_CUDA_ERR_NO_DEVICE, "no CUDA device is available");
        return nullptr;
    }
    if (device < 0 || device >= n) {
        tm_fail(err, err_cap, TM_CUDA_ERR_NO_DEVICE, "device %d out of range (%d present)", device, n);
        return nullptr;
    }
    int major = 0, minor = 0, sms = 0, optin = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    if (major != 10) {
        tm_fail(err, err_cap, TM_CUDA_ERR_NO_DEVICE,
                "device %d is sm_%d%d; this library carries sm_100a code only", device, major, minor);
        return nullptr;
    }
    if (cudaSetDevice(device) != cudaSuccess) {
        tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "cudaSetDevice(%d) failed", device);
        return nullptr;
    }
    tm_cuda_ctx *ctx = new tm_cuda_ctx();
    ctx->device = device;
    ctx->sm_count = sms;
    ctx->smem_optin = (size_t)optin;
    if (const char *e = getenv("TM_CUDA_PDL")) ctx->pdl = e[0] != '0';
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
        tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "cannot create a stream: %s",
                cudaGetErrorString(cudaGetLastError()));
        delete ctx;
        return nullptr;
    }
    return ctx;
}

void tm_cuda_comm_release(tm_cuda_ctx *ctx);  // tm_cuda_comm.cu

void tm_cuda_destroy(tm_cuda_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    tm_cuda_comm_release(ctx);
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        poll_locked(ctx, true);
        for (cudaEvent_t e : ctx->event_pool) cudaEventDestroy(e);
        if (ctx->mma_scratch) cudaFree(ctx->mma_scratch);
    }
    if (ctx->side) {
        cudaStreamSynchronize(ctx->side);
        cudaEventDestroy(ctx->side_fork);
        cudaEventDestroy(ctx->side_join);
        cudaStreamDestroy(ctx->side);
    }
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

tm_cuda_buffer *tm_cuda_buffer_new(tm_cuda_ctx *ctx, size_t bytes, int shared, char *err,
                                   size_t err_cap) {
    if (!ctx || bytes == 0) {
        tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "buffer size must be positive");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaSetDevice(ctx->device);
    void *p = nullptr;
    cudaError_t e = shared ? cudaHostAlloc(&p, bytes, cudaHostAllocMapped | cudaHostAllocPortable)
                           : cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        tm_fail(err, err_cap, TM_CUDA_ERR_ALLOC, "allocating %zu %s bytes failed: %s", bytes,
                shared ? "shared" : "device", cudaGetErrorString(e));
        return nullptr;
    }
    tm_cuda_buffer *b = new tm_cuda_buffer();
    b->owner = ctx;
    b->dev = (unsigned char *)p;
    b->len = bytes;
    b->shared = shared ? 1 : 0;
    ctx->live.insert(b);
    ctx->allocated.fetch_add(bytes);
    return b;
}

tm_cuda_buffer *tm_cuda_buffer_view(tm_cuda_ctx *ctx, tm_cuda_buffer *parent, size_t off,
                                    size_t len, char *err, size_t err_cap) {
    if (!ctx) {
        tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "null context");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (!parent || ctx->live.find(parent) == ctx->live.end()) {
        tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "parent buffer does not belong to this context");
        return nullptr;
    }
    if (len == 0 || off % 16 != 0 || off > parent->len || len > parent->len - off) {
        tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                "view [%zu, +%zu) of a %zu-byte buffer (offset must be 16-byte aligned)", off, len,
                parent->len);
        return nullptr;
    }
    tm_cuda_buffer *b = new tm_cuda_buffer();
    b->owner = ctx;
    b->parent = parent;
    b->dev = parent->dev + off;
    b->len = len;
    b->shared = parent->shared;
    parent->views += 1;
    ctx->live.insert(b);
    return b;
}

void tm_cuda_buffer_free(tm_cuda_ctx *ctx, tm_cuda_buffer *buffer) {
    if (!ctx || !buffer) return;
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (ctx->live.find(buffer) == ctx->live.end() || buffer->views != 0) return;
    ctx->live.erase(buffer);
    if (buffer->parent) {
        buffer->parent->views -= 1;
    } else {
        cudaSetDevice(ctx->device);
        // Committed work may still read the storage: wait for it (the Metal
        // original leases the storage to its pending command buffers instead).
        cudaStreamSynchronize(ctx->stream);
        if (buffer->symm) tm_cuda_symm_release(buffer);
        if (buffer->shared) cudaFreeHost(buffer->dev); else cudaFree(buffer->dev);
        ctx->allocated.fetch_sub(buffer->len);
    }
    delete buffer;
}

void *tm_cuda_buffer_contents(tm_cuda_ctx *ctx, tm_cuda_buffer *buffer) {
    if (!ctx || !buffer) return nullptr;
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (ctx->live.find(buffer) == ctx->live.end() || !buffer->shared) return nullptr;
    return buffer->dev;
}

void *tm_cuda_buffer_device_ptr(tm_cuda_ctx *ctx, tm_cuda_buffer *buffer) {
    if (!ctx || !buffer) return nullptr;
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (ctx->live.find(buffer) == ctx->live.end()) return nullptr;
    return buffer->dev;
}

size_t tm_cuda_buffer_len(const tm_cuda_ctx *ctx, const tm_cuda_buffer *buffer) {
    if (!ctx || !buffer) return 0;
    tm_cuda_ctx *c = const_cast<tm_cuda_ctx *>(ctx);
    std::lock_guard<std::mutex> lock(c->mu);
    return c->live.find(buffer) == c->live.end() ? 0 : buffer->len;
}

int tm_cuda_buffer_zero(tm_cuda_ctx *ctx, tm_cuda_buffer *buffer, size_t off, size_t len,
                        char *err, size_t err_cap) {
    TM_ENTER();
    if (len == 0 || off > SIZE_MAX - len)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "zero range is empty or overflows");
    TM_CHECK_BUF(buffer, off + len, "zero target");
    TM_OP_BEGIN("buffer_zero");
    TM_CUDA_TRY(cudaMemsetAsync(buffer->dev + off, 0, len, ctx->stream));
    TM_OP_END(1);
}

int tm_cuda_upload(tm_cuda_ctx *ctx, tm_cuda_buffer *dst, size_t off, const void *src, size_t len,
                   char *err, size_t err_cap) {
    TM_ENTER();
    if (ctx->group_open)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "upload with a dispatch group open");
    if (!src || len == 0 || off > SIZE_MAX - len)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "upload range is empty or overflows");
    TM_CHECK_BUF(dst, off + len, "upload target");
    TM_CUDA_TRY(cudaMemcpyAsync(dst->dev + off, src, len, cudaMemcpyDefault, ctx->stream));
    TM_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    poll_locked(ctx, false);
    return TM_CUDA_OK;
}

int tm_cuda_download(tm_cuda_ctx *ctx, tm_cuda_buffer *src, size_t off, void *dst, size_t len,
                     char *err, size_t err_cap) {
    TM_ENTER();
    if (ctx->group_open)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "download with a dispatch group open");
    if (!dst || len == 0 || off > SIZE_MAX - len)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "download range is empty or overflows");
    TM_CHECK_BUF(src, off + len, "download source");
    TM_CUDA_TRY(cudaMemcpyAsync(dst, src->dev + off, len, cudaMemcpyDefault, ctx->stream));
    TM_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    poll_locked(ctx, false);
    return TM_CUDA_OK;
}

int tm_cuda_download_after(tm_cuda_ctx *ctx, tm_cuda_buffer *src, size_t off, void *dst,
                           size_t len, uint64_t completed_target, char *err, size_t err_cap) {
    TM_ENTER();
    if (!dst || len == 0 || off > SIZE_MAX - len)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "download range is empty or overflows");
    TM_CHECK_BUF(src, off + len, "download source");
    if (!src->shared)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "download_after reads a shared buffer; this one is device-private");
    if (completed_target > ctx->committed.load())
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "completion target %llu is beyond the %llu committed dispatches",
                       (unsigned long long)completed_target,
                       (unsigned long long)ctx->committed.load());
    poll_locked(ctx, false);
    if (ctx->completed.load() < completed_target) {
        for (const tm_commit &c : ctx->pending) {
            if (c.seq == completed_target) {
                TM_CUDA_TRY(cudaEventSynchronize(c.end));
                break;
            }
        }
        poll_locked(ctx, false);
    }
    memcpy(dst, src->dev + off, len);
    return TM_CUDA_OK;
}

static void join_side(tm_cuda_ctx *ctx);

__global__ void l2_prefetch_kernel(const char *p, size_t bytes) {
    const size_t stride = (size_t)gridDim.x * blockDim.x * 128u;
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 128u; i < bytes; i += stride)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p + i));
}

int tm_cuda_prefetch_l2(tm_cuda_ctx *ctx, tm_cuda_buffer *const *bufs, uint32_t n, char *err, size_t err_cap) {
    TM_ENTER();
    if (!bufs || n == 0 || n > 64) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "1 to 64 buffers, got %u", n);
    for (uint32_t i = 0; i < n; ++i)
        if (!bufs[i] || ctx->live.find(bufs[i]) == ctx->live.end())
            return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "buffer %u does not belong to this context", i);
    if (ctx->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "operator prefetch_l2 cannot be recorded into a persistent program");
    if (!ctx->side) {
        if (ctx->group_open)
            return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "the first prefetch of a context must come outside a dispatch group");
        TM_CUDA_TRY(cudaStreamCreateWithFlags(&ctx->side, cudaStreamNonBlocking));
        TM_CUDA_TRY(cudaEventCreateWithFlags(&ctx->side_fork, cudaEventDisableTiming));
        TM_CUDA_TRY(cudaEventCreateWithFlags(&ctx->side_join, cudaEventDisableTiming));
    }
    TM_CUDA_TRY(cudaEventRecord(ctx->side_fork, ctx->stream));
    TM_CUDA_TRY(cudaStreamWaitEvent(ctx->side, ctx->side_fork, 0));
    for (uint32_t i = 0; i < n; ++i)
        l2_prefetch_kernel<<<8, 256, 0, ctx->side>>>((const char *)bufs[i]->dev, bufs[i]->len);
    TM_CUDA_TRY(cudaGetLastError());
    ctx->side_pending = true;
    if (ctx->group_open) ctx->group_kernels += n;
    else {
        ctx->launches.fetch_add(n);
        join_side(ctx);
    }
    return TM_CUDA_OK;
}

int tm_cuda_begin_group(tm_cuda_ctx *ctx, char *err, size_t err_cap) {
    TM_ENTER();
    if (ctx->group_open || ctx->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "a dispatch group is already open");
    TM_CUDA_TRY(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
    ctx->group_open = true;
    ctx->group_kernels = 0;
    return TM_CUDA_OK;
}

// The side stream's work rejoins the main stream (inside a capture: before the capture can end).
static void join_side(tm_cuda_ctx *ctx) {
    if (!ctx->side_pending) return;
    ctx->side_pending = false;
    if (cudaEventRecord(ctx->side_join, ctx->side) == cudaSuccess) cudaStreamWaitEvent(ctx->stream, ctx->side_join, 0);
}

static int end_capture(tm_cuda_ctx *ctx, cudaGraphExec_t *exec, char *err, size_t err_cap) {
    cudaGraph_t graph = nullptr;
    join_side(ctx);
    ctx->group_open = false;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    if (e != cudaSuccess || !graph) {
        cudaGetLastError();
        return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "ending the group capture failed: %s",
                       cudaGetErrorString(e));
    }
    if (!exec) {
        cudaGraphDestroy(graph);
        return TM_CUDA_OK;
    }
    e = cudaGraphInstantiate(exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "graph instantiation failed: %s",
                       cudaGetErrorString(e));
    }
    return TM_CUDA_OK;
}

static int launch_exec(tm_cuda_ctx *ctx, cudaGraphExec_t exec, uint64_t kernels, const char *label,
                       char *err, size_t err_cap) {
    tm_commit c;
    int rc = commit_begin(ctx, &c, label, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    TM_CUDA_TRY(cudaGraphLaunch(exec, ctx->stream));
    ctx->launches.fetch_add(kernels);
    return commit_end(ctx, &c, err, err_cap);
}

int tm_cuda_end_group(tm_cuda_ctx *ctx, char *err, size_t err_cap) {
    TM_ENTER();
    if (!ctx->group_open)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "no dispatch group is open");
    cudaGraphExec_t exec = nullptr;
    int rc = end_capture(ctx, &exec, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    rc = launch_exec(ctx, exec, ctx->group_kernels, "group", err, err_cap);
    cudaGraphExecDestroy(exec);  // released by the runtime once the launch has completed
    return rc;
}

int tm_cuda_abort_group(tm_cuda_ctx *ctx, char *err, size_t err_cap) {
    TM_ENTER();
    if (!ctx->group_open)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "no dispatch group is open");
    return end_capture(ctx, nullptr, err, err_cap);
}

int tm_cuda_end_group_retain(tm_cuda_ctx *ctx, tm_cuda_graph **out, char *err, size_t err_cap) {
    TM_ENTER();
    if (!out) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "null graph output");
    if (!ctx->group_open)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "no dispatch group is open");
    cudaGraphExec_t exec = nullptr;
    int rc = end_capture(ctx, &exec, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    tm_cuda_graph *g = new tm_cuda_graph();
    g->owner = ctx;
    g->exec = exec;
    g->kernels = ctx->group_kernels;
    ctx->graphs.insert(g);
    *out = g;
    return TM_CUDA_OK;
}

int tm_cuda_graph_launch(tm_cuda_ctx *ctx, tm_cuda_graph *graph, char *err, size_t err_cap) {
    TM_ENTER();
    if (ctx->group_open)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "graph launch with a dispatch group open");
    if (!graph || ctx->graphs.find(graph) == ctx->graphs.end())
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "graph does not belong to this context");
    if (graph->program) {  // a persistent program: one kernel launch is the whole dispatch
        if (ctx->program)
            return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "program launch with a program open");
        tm_commit c;
        int rc = commit_begin(ctx, &c, "program", err, err_cap);
        if (rc != TM_CUDA_OK) return rc;
        rc = tm_step_launch(ctx, graph->program, err, err_cap);
        if (rc != TM_CUDA_OK) return rc;
        ctx->launches.fetch_add(1);
        return commit_end(ctx, &c, err, err_cap);
    }
    return launch_exec(ctx, graph->exec, graph->kernels, "graph", err, err_cap);
}

void tm_cuda_graph_free(tm_cuda_ctx *ctx, tm_cuda_graph *graph) {
    if (!ctx || !graph) return;
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (ctx->graphs.find(graph) == ctx->graphs.end()) return;
    ctx->graphs.erase(graph);
    cudaSetDevice(ctx->device);
    if (graph->program) {
        cudaStreamSynchronize(ctx->stream);  // a launch may still be reading the operator table
        tm_step_free(ctx, graph->program);
    } else {
        cudaGraphExecDestroy(graph->exec);
    }
    delete graph;
}

int tm_cuda_fence(tm_cuda_ctx *ctx, char *err, size_t err_cap) {
    TM_ENTER();
    if (ctx->group_open)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "fence with a dispatch group open");
    TM_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    poll_locked(ctx, true);
    return TM_CUDA_OK;
}

uint64_t tm_cuda_committed_dispatches(const tm_cuda_ctx *ctx) {
    return ctx ? ctx->committed.load() : 0;
}

uint64_t tm_cuda_completed_dispatches(const tm_cuda_ctx *ctx) {
    if (!ctx) return 0;
    tm_cuda_ctx *c = const_cast<tm_cuda_ctx *>(ctx);
    std::lock_guard<std::mutex> lock(c->mu);
    cudaSetDevice(c->device);
    poll_locked(c, false);
    return c->completed.load();
}

double tm_cuda_last_gpu_ms(const tm_cuda_ctx *ctx) {
    return ctx ? (double)ctx->last_gpu_ns.load() / 1e6 : 0.0;
}

uint64_t tm_cuda_gpu_nanos_total(const tm_cuda_ctx *ctx) { return ctx ? ctx->gpu_nanos.load() : 0; }

int tm_cuda_profile_set(tm_cuda_ctx *ctx, int enabled) {
    if (!ctx) return TM_CUDA_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    poll_locked(ctx, true);
    ctx->profiling = enabled != 0;
    ctx->profile.clear();
    return TM_CUDA_OK;
}

int tm_cuda_profile_read(tm_cuda_ctx *ctx, uint32_t index, char *name, size_t name_cap,
                         uint64_t *nanos, uint64_t *count) {
    if (!ctx) return 0;
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaSetDevice(ctx->device);
    poll_locked(ctx, false);
    if (index >= ctx->profile.size()) return 0;
    const tm_profile_row &r = ctx->profile[index];
    if (name && name_cap) snprintf(name, name_cap, "%s", r.name.c_str());
    if (nanos) *nanos = r.nanos;
    if (count) *count = r.count;
    return 1;
}

uint64_t tm_cuda_allocated_bytes(const tm_cuda_ctx *ctx) { return ctx ? ctx->allocated.load() : 0; }
uint64_t tm_cuda_in_flight_bytes(const tm_cuda_ctx *) { return 0; }
uint64_t tm_cuda_kernel_launches(const tm_cuda_ctx *ctx) { return ctx ? ctx->launches.load() : 0; }
int tm_cuda_device_memory(tm_cuda_ctx *ctx, uint64_t *free_bytes, uint64_t *total_bytes) {
    if (!ctx) return TM_CUDA_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(ctx->mu);
    size_t f = 0, t = 0;
    if (cudaSetDevice(ctx->device) != cudaSuccess || cudaMemGetInfo(&f, &t) != cudaSuccess) {
        cudaGetLastError();
        return TM_CUDA_ERR_INTERNAL;
    }
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return TM_CUDA_OK;
}
void *tm_cuda_stream(tm_cuda_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

}  // extern "C"
