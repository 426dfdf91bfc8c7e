// C entry points of the engine host layer (include/tm_engine.h) and the load
// path: options, adapter, admission, exact preflight, per-class check, load.
#include <cstdio>
#include <cstring>
#include <memory>

#include "adapters.hpp"
#include "engine.hpp"
#include "kernels.hpp"
#include "planner.hpp"
#include "tm_engine.h"

using namespace tuckmill;

struct tm_engine {
    std::unique_ptr<GgufInspection> insp;
    std::unique_ptr<GgufWeights> weights;
    std::shared_ptr<CudaContext> ctx;
    std::unique_ptr<EngineModel> model;
    PlanBudget budget;
    uint32_t prefill_batch = 0;
};

namespace {

int fail(const TuckmillError &e, char *err, size_t cap) {
    if (err && cap) snprintf(err, cap, "%s", e.what());
    return 1 + (int)e.code;
}
int fail_std(const std::exception &e, char *err, size_t cap) {
    if (err && cap) snprintf(err, cap, "INTERNAL: %s", e.what());
    return TM_ENGINE_INTERNAL;
}

#define GUARD(...)                                                   \
    try {                                                            \
        __VA_ARGS__;                                                 \
        return TM_ENGINE_OK;                                         \
    } catch (const TuckmillError &e_) {                              \
        return fail(e_, err, err_cap);                               \
    } catch (const std::exception &e_) {                             \
        return fail_std(e_, err, err_cap);                           \
    }

// Weight bytes of the artifact as the planner prices them: every matrix the
// graph binds (tied heads once) plus the f32 norm vectors.
uint64_t artifact_weight_bytes(const ModelGraph &g, const WeightSource &src) {
    EngineOptions o;
    return alloc_plan_with(g, src, 1, o).weights;
}

PlanBudget admit(const ModelGraph &g, const WeightSource &src, uint32_t context, uint64_t budget,
                 uint32_t sequences = 1) {
    KvGeometry kv;
    kv.layers = g.layers.size();
    kv.kv_head_count = g.layers.empty() ? 0 : g.layers[0].mixer.kv_heads;
    kv.key_length = kv.value_length = g.layers.empty() ? 0 : g.layers[0].mixer.head_dim;
    PlannerPolicy policy;
    uint64_t kv_total = 0, per_token = 0;
    // every sequence holds `context` positions of KV
    if (!estimate_kv_bytes(kv, (uint64_t)context * sequences, policy.kv_bytes_per_element, &kv_total, &per_token))
        throw TuckmillError(ErrorCode::ContextExceedsBudget, "KV payload overflows at context " + std::to_string(context));
    PlanBudget b = make_resident_plan(budget, artifact_weight_bytes(g, src), kv_total, policy);
    require_admitted(b, context);
    return b;
}

void fill_budget(const PlanBudget &b, tm_engine_info *out) {
    out->budget = b.requested_budget;
    out->reservation = b.reservation();
    out->overhead = b.overhead_estimate;
    out->safety_reserve = b.safety_reserve;
}

}  // namespace

extern "C" {

int tm_engine_load(const tm_engine_options *o, tm_engine **out, char *err, size_t err_cap) {
    GUARD({
        if (!o || !out || !o->gguf_path)
            throw TuckmillError(ErrorCode::InvalidRequest, "null engine options");
        KernelSelection sel;
        if (!parse_kernel_selection(o->kernels ? o->kernels : "auto", &sel))
            throw TuckmillError(ErrorCode::InvalidRequest, std::string("unknown --kernels value \"") +
                                                               (o->kernels ? o->kernels : "") + "\"");
        // A forced selection never falls back (crates/tuckcore/src/kernels.rs:60-86).
        if (resolve_kernel_selection(sel) != ResolvedKernels::Cuda)
            throw TuckmillError(ErrorCode::InvalidRequest,
                                "this engine serves --kernels cuda only; other selections belong to the CPU executor");
        if (o->context == 0) throw TuckmillError(ErrorCode::InvalidRequest, "context must be positive");
        std::unique_ptr<tm_engine> e(new tm_engine());
        e->insp.reset(new GgufInspection(GgufInspection::open(o->gguf_path)));
        e->weights.reset(new GgufWeights(*e->insp));
        ModelGraph graph = adapt(*e->insp);
        e->ctx = std::make_shared<CudaContext>(o->device);
        uint64_t budget = o->budget_bytes;
        if (budget == 0) {
            uint64_t free_b = 0, total_b = 0;
            if (tm_cuda_device_memory(e->ctx->raw(), &free_b, &total_b) != TM_CUDA_OK)
                throw TuckmillError(ErrorCode::Internal, "cannot query device memory");
            budget = total_b;
        }
        EngineOptions eo;
        eo.sequences = o->sequences ? o->sequences : 1;
        if (eo.sequences > kMaxSequences)
            throw TuckmillError(ErrorCode::InvalidRequest, "sequences must be 1.." + std::to_string(kMaxSequences));
        e->budget = admit(graph, *e->weights, o->context, budget, eo.sequences);
        eo.prefill_batch = o->prefill_batch ? o->prefill_batch : kPrefillBatchDefault;
        eo.exact = o->exact != 0;
        eo.persistent = o->persistent_step != 0;
        eo.shard_world = o->shard_world ? o->shard_world : 1;
        eo.shard_rank = o->shard_rank;
        if (eo.shard_world > 1) {
            if (!o->comm_id) throw TuckmillError(ErrorCode::InvalidRequest, "a row split needs a communicator id");
            if (eo.shard_rank >= eo.shard_world)
                throw TuckmillError(ErrorCode::InvalidRequest, "shard rank outside the split");
            e->ctx->comm_init(o->comm_id, (int)eo.shard_rank, (int)eo.shard_world);
        }
        e->prefill_batch = eo.prefill_batch;
        // Exact preflight, then every class against its reservation BEFORE any
        // allocation (crates/tuckcore/src/executor.rs:1543-1562).
        const GpuAllocPlan alloc = alloc_plan_with(graph, *e->weights, o->context, eo);
        const ReservationBreakdown &r = e->budget.reservation_breakdown;
        const struct { const char *cls; uint64_t need, have; } checks[] = {
            {"weights", alloc.weights, r.weights}, {"kv_state", alloc.state, r.kv_state},
            {"workspaces", alloc.scratch, r.workspaces}};
        for (const auto &c : checks)
            if (c.need > c.have)
                throw TuckmillError(ErrorCode::InvalidRequest,
                                    std::string("the plan reserves ") + std::to_string(c.have) + " for " + c.cls +
                                        " but the " + graph.architecture + " GPU model needs " + std::to_string(c.need) +
                                        " at context " + std::to_string(o->context) +
                                        "; refusing before any GPU allocation",
                                    "Rebuild the plan for this executor; understated reservations are never loaded.");
        e->model = EngineModel::load_with(e->ctx, std::move(graph), *e->weights, o->context, alloc.total(), eo);
        *out = e.release();
    })
}

int tm_engine_comm_id(void *out128, char *err, size_t err_cap) {
    GUARD({
        char e[256] = {0};
        if (tm_cuda_comm_unique_id(out128, e, sizeof e) != TM_CUDA_OK) throw TuckmillError(ErrorCode::Unavailable, e);
    })
}

void tm_engine_free(tm_engine *e) { delete e; }

int tm_engine_get_info(tm_engine *e, tm_engine_info *out) {
    if (!e || !out) return TM_ENGINE_INVALID_REQUEST;
    memset(out, 0, sizeof *out);
    const ModelGraph &g = e->model->graph();
    out->vocab = (uint32_t)g.vocab;
    out->hidden = (uint32_t)g.hidden;
    out->layers = (uint32_t)g.layers.size();
    out->context = (uint32_t)e->model->capacity();
    out->prefill_batch = e->prefill_batch;
    out->plan_weights = e->model->plan().weights;
    out->plan_state = e->model->plan().state;
    out->plan_scratch = e->model->plan().scratch;
    out->allocated_bytes = e->model->allocated_bytes();
    fill_budget(e->budget, out);
    snprintf(out->kernel_impl, sizeof out->kernel_impl, "%s", resolved_kernels_str(ResolvedKernels::Cuda));
    snprintf(out->kernel_id, sizeof out->kernel_id, "%s", engine_kernel_id(g.architecture).c_str());
    snprintf(out->architecture, sizeof out->architecture, "%s", g.architecture.c_str());
    return TM_ENGINE_OK;
}

void *tm_engine_cuda_ctx(tm_engine *e) { return e ? (void *)e->ctx->raw() : nullptr; }
void *tm_engine_decode_program(tm_engine *e) { return e && e->model ? (void *)e->model->decode_program() : nullptr; }

int tm_engine_reset(tm_engine *e, char *err, size_t err_cap) { GUARD(e->model->reset()) }

int tm_engine_prefill(tm_engine *e, const uint32_t *tokens, uint32_t n, int want_token, char *err,
                      size_t err_cap) {
    GUARD(e->model->prefill(tokens, n, want_token != 0))
}

int tm_engine_prefill_token(tm_engine *e, uint32_t *token, char *err, size_t err_cap) {
    GUARD(*token = e->model->prefill_token())
}

int tm_engine_step(tm_engine *e, uint32_t token, float *logits, char *err, size_t err_cap) {
    GUARD({
        e->model->step(token);
        if (logits) e->model->logits(logits);
    })
}

int tm_engine_logits(tm_engine *e, float *logits, char *err, size_t err_cap) { GUARD(e->model->logits(logits)) }

int tm_engine_generate(tm_engine *e, const uint32_t *prompt, uint32_t n_prompt, uint32_t max_new,
                       int ignore_eos, uint32_t *out_tokens, uint32_t *n_out, tm_engine_stats *stats,
                       char *err, size_t err_cap) {
    GUARD({
        GenerateStats s;
        std::vector<uint32_t> toks = e->model->generate(prompt, n_prompt, max_new, ignore_eos != 0, &s);
        for (size_t i = 0; i < toks.size(); ++i) out_tokens[i] = toks[i];
        *n_out = (uint32_t)toks.size();
        if (stats) {
            stats->ttft_ns = s.ttft_ns;
            stats->decode_span_ns = s.decode_span_ns;
            stats->prompt_tokens = s.prompt_tokens;
            stats->generated = s.generated;
            stats->kernel_launches = s.kernel_launches;
            stats->dispatches = s.dispatches;
            stats->h2d_bytes = s.h2d_bytes;
            stats->d2h_bytes = s.d2h_bytes;
        }
    })
}

int tm_engine_prefill_seq(tm_engine *e, uint32_t seq, const uint32_t *tokens, uint32_t n, int want_token, char *err,
                          size_t err_cap) {
    GUARD(e->model->prefill_seq(seq, tokens, n, want_token != 0))
}

int tm_engine_prefill_token_of(tm_engine *e, uint32_t seq, uint32_t *token, char *err, size_t err_cap) {
    GUARD(*token = e->model->prefill_token_of(seq))
}

int tm_engine_step_batch(tm_engine *e, const uint32_t *tokens, float *logits, char *err, size_t err_cap) {
    GUARD({
        e->model->step_batch(tokens);
        if (logits) e->model->logits_batch(logits);
    })
}

int tm_engine_decode_steps_batch(tm_engine *e, uint32_t steps, char *err, size_t err_cap) {
    GUARD({
        for (uint32_t i = 0; i < steps; ++i) e->model->submit_batch_greedy();
    })
}

int tm_engine_generate_batch(tm_engine *e, const uint32_t *prompts, const uint32_t *prompt_lens, uint32_t n_requests,
                             uint32_t max_new, int ignore_eos, uint32_t *out_tokens, uint32_t *out_counts,
                             tm_engine_stats *stats, char *err, size_t err_cap) {
    GUARD({
        if (!prompts || !prompt_lens || !out_tokens || !out_counts)
            throw TuckmillError(ErrorCode::InvalidRequest, "null batch arguments");
        std::vector<std::vector<uint32_t>> ps(n_requests);
        size_t off = 0;
        for (uint32_t r = 0; r < n_requests; ++r) {
            ps[r].assign(prompts + off, prompts + off + prompt_lens[r]);
            off += prompt_lens[r];
        }
        GenerateStats s;
        const auto toks = e->model->generate_batch(ps, max_new, ignore_eos != 0, &s);
        for (uint32_t r = 0; r < n_requests; ++r) {
            for (size_t i = 0; i < toks[r].size(); ++i) out_tokens[(size_t)r * max_new + i] = toks[r][i];
            out_counts[r] = (uint32_t)toks[r].size();
        }
        if (stats) {
            stats->ttft_ns = s.ttft_ns;
            stats->decode_span_ns = s.decode_span_ns;
            stats->prompt_tokens = s.prompt_tokens;
            stats->generated = s.generated;
            stats->kernel_launches = s.kernel_launches;
            stats->dispatches = s.dispatches;
            stats->h2d_bytes = s.h2d_bytes;
            stats->d2h_bytes = s.d2h_bytes;
        }
    })
}

int tm_engine_decode_steps(tm_engine *e, uint32_t steps, char *err, size_t err_cap) {
    GUARD({
        for (uint32_t i = 0; i < steps; ++i) e->model->submit_greedy();
    })
}

int tm_engine_decode_ungrouped(tm_engine *e, uint32_t steps, char *err, size_t err_cap) {
    GUARD({
        for (uint32_t i = 0; i < steps; ++i) e->model->step_ungrouped();
    })
}

int tm_engine_plan(const char *gguf_path, uint32_t context, uint64_t budget_bytes, tm_engine_info *out,
                   char *err, size_t err_cap) {
    return tm_engine_plan_shard(gguf_path, context, budget_bytes, 0, 1, out, err, err_cap);
}

int tm_engine_plan_shard(const char *gguf_path, uint32_t context, uint64_t budget_bytes, uint32_t shard_rank,
                         uint32_t shard_world, tm_engine_info *out, char *err, size_t err_cap) {
    GUARD({
        if (!gguf_path || !out) throw TuckmillError(ErrorCode::InvalidRequest, "null plan arguments");
        GgufInspection insp = GgufInspection::open(gguf_path);
        GgufWeights w(insp);
        ModelGraph g = adapt(insp);
        memset(out, 0, sizeof *out);
        out->vocab = (uint32_t)g.vocab;
        out->hidden = (uint32_t)g.hidden;
        out->layers = (uint32_t)g.layers.size();
        out->context = context;
        EngineOptions eo;
        eo.shard_rank = shard_rank;
        eo.shard_world = shard_world ? shard_world : 1;
        const GpuAllocPlan alloc = alloc_plan_with(g, w, context, eo);
        out->plan_weights = alloc.weights;
        out->plan_state = alloc.state;
        out->plan_scratch = alloc.scratch;
        snprintf(out->architecture, sizeof out->architecture, "%s", g.architecture.c_str());
        KvGeometry kv;
        kv.layers = g.layers.size();
        kv.kv_head_count = g.layers[0].mixer.kv_heads;
        kv.key_length = kv.value_length = g.layers[0].mixer.head_dim;
        PlannerPolicy policy;
        uint64_t kv_total = 0, per_token = 0;
        if (!estimate_kv_bytes(kv, context, policy.kv_bytes_per_element, &kv_total, &per_token))
            throw TuckmillError(ErrorCode::ContextExceedsBudget, "KV payload overflows");
        PlanBudget b = make_resident_plan(budget_bytes, alloc.weights, kv_total, policy);
        fill_budget(b, out);
        require_admitted(b, context);
    })
}

}  // extern "C"
