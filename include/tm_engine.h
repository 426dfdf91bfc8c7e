/*
 * tm_engine.h -- C entry points of the CUDA engine host layer (C++), for hosts
 * and test harnesses that cannot link C++ directly.
 *
 * The engine is the CUDA counterpart of TuckCore's unified layer engine and of
 * the executor's load / prefill / decode loops, above the tm_cuda.h device ABI:
 *   load      crates/tuckcore/src/executor.rs:245-602 (options, architecture
 *             branch), :1518-1633 load_engine (exact preflight, per-class check
 *             against the plan BEFORE any allocation, ledger == plan after)
 *   generate  crates/tuckcore/src/executor.rs:870-1125 run_session (chunked
 *             prefill, pipelined device-greedy decode)
 *   step      crates/tuckcore/src/engine/metal.rs:2475-2507 EngineModel::step
 * Every function returns 0 or 1 + the index of the typed error code below and
 * writes a NUL-terminated message into `err` (may be NULL).
 */
#ifndef TM_ENGINE_H
#define TM_ENGINE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tm_engine tm_engine;

enum {
    TM_ENGINE_OK = 0,
    TM_ENGINE_INVALID_REQUEST = 1,
    TM_ENGINE_INVALID_ARTIFACT = 2,
    TM_ENGINE_UNSUPPORTED_ARCHITECTURE = 3,
    TM_ENGINE_UNSUPPORTED_QUANTIZATION = 4,
    TM_ENGINE_CONTEXT_EXCEEDS_BUDGET = 5,
    TM_ENGINE_MODEL_EXCEEDS_BUDGET = 6,
    TM_ENGINE_UNAVAILABLE = 7,
    TM_ENGINE_CANCELLED = 8,
    TM_ENGINE_INTERNAL = 9
};

typedef struct {
    const char *gguf_path;
    const char *kernels;      /* the --kernels string; only "cuda" loads this engine */
    int device;               /* CUDA device index */
    uint32_t context;         /* admitted total positions (prompt + output) */
    uint32_t prefill_batch;   /* 0 = default (512) */
    int exact;                /* 1: batched projections keep the GEMV arithmetic */
    uint64_t budget_bytes;    /* B of R + U + H <= B; 0 = the device's total memory */
    /* Output-row split over the devices of one node, one process per device.
     * shard_world 0 or 1 = single device.  Otherwise every process loads the same
     * artifact with its own shard_rank and the SAME comm_id (128 bytes from
     * tm_engine_comm_id on rank 0, handed to the others by the launcher); rank r
     * keeps rows [r*N/world, (r+1)*N/world) of each projection and of the head,
     * whole attention heads stay on one rank, and every call below becomes a
     * collective that all ranks make in the same order. */
    uint32_t shard_rank, shard_world;
    const void *comm_id;
    /* 0 (default): a decode step replays the recorded graph of per-operator kernels; 1: it runs
     * as ONE persistent kernel (tm_cuda_begin_program) where the model allows it (single device,
     * not exact, attention shapes the program kernel serves), the graph otherwise. */
    int persistent_step;
    /* Concurrent sequences the engine holds state for and decodes together, one row each, in one
     * recorded step (0 or 1 = one sequence: the reference's engine, which serves one request at a
     * time, crates/supervisor/src/queue.rs:1-4).  KV state and admission scale with it. */
    uint32_t sequences;
} tm_engine_options;

/* 128 opaque bytes naming a new communicator (tm_cuda_comm_unique_id). */
int tm_engine_comm_id(void *out128, char *err, size_t err_cap);

typedef struct {
    uint32_t vocab, hidden, layers, context, prefill_batch;
    uint64_t plan_weights, plan_state, plan_scratch; /* exact preflight by class */
    uint64_t allocated_bytes;                        /* device ledger after load */
    uint64_t budget, reservation, overhead, safety_reserve;
    char kernel_impl[16];   /* "cuda": what the supervisor's acknowledgement check compares */
    char kernel_id[64];     /* "ADR011:<arch>-q8_0+f16:cuda" */
    char architecture[32];
} tm_engine_info;

typedef struct {
    uint64_t ttft_ns, decode_span_ns, prompt_tokens, generated, kernel_launches, dispatches;
    uint64_t h2d_bytes, d2h_bytes;
} tm_engine_stats;

int tm_engine_load(const tm_engine_options *opts, tm_engine **out, char *err, size_t err_cap);
void tm_engine_free(tm_engine *e);
int tm_engine_get_info(tm_engine *e, tm_engine_info *out);
/* The tm_cuda_ctx the engine runs on (for event timing on its stream). */
void *tm_engine_cuda_ctx(tm_engine *e);
/* The tm_cuda_graph of the persistent decode program (tm_cuda_program_status / _trace), or
 * NULL when a decode step is a graph of per-operator kernels. */
void *tm_engine_decode_program(tm_engine *e);
int tm_engine_reset(tm_engine *e, char *err, size_t err_cap);
int tm_engine_prefill(tm_engine *e, const uint32_t *tokens, uint32_t n, int want_token, char *err,
                      size_t err_cap);
/* Greedy token chosen by the last prefill(want_token = 1). */
int tm_engine_prefill_token(tm_engine *e, uint32_t *token, char *err, size_t err_cap);
/* One decode step for `token`; `logits` (vocab f32, may be NULL) receives the
 * step's logits. */
int tm_engine_step(tm_engine *e, uint32_t token, float *logits, char *err, size_t err_cap);
int tm_engine_logits(tm_engine *e, float *logits, char *err, size_t err_cap);
/* Greedy generation of up to max_new tokens into out_tokens; *n_out receives the
 * count.  ignore_eos = 1 keeps going past the artifact's EOS id. */
int tm_engine_generate(tm_engine *e, const uint32_t *prompt, uint32_t n_prompt, uint32_t max_new,
                       int ignore_eos, uint32_t *out_tokens, uint32_t *n_out, tm_engine_stats *stats,
                       char *err, size_t err_cap);
/* ---- several sequences (tm_engine_options.sequences > 1); no counterpart in the reference ---- */
/* Prompt tokens of sequence `seq` at its own position; the other sequences are untouched. */
int tm_engine_prefill_seq(tm_engine *e, uint32_t seq, const uint32_t *tokens, uint32_t n, int want_token, char *err,
                          size_t err_cap);
int tm_engine_prefill_token_of(tm_engine *e, uint32_t seq, uint32_t *token, char *err, size_t err_cap);
/* One decode step of every sequence: tokens[s] goes to sequence s at its position; `logits` (NULL or
 * sequences * vocab floats) receives every row.  Row s equals the one-sequence step on the same state
 * bit for bit in `exact` mode; otherwise within the bars of the tolerance-qualified kernels. */
int tm_engine_step_batch(tm_engine *e, const uint32_t *tokens, float *logits, char *err, size_t err_cap);
/* `steps` device-greedy steps of all sequences with no host read in between (kernel-only timing). */
int tm_engine_decode_steps_batch(tm_engine *e, uint32_t steps, char *err, size_t err_cap);
/* Greedy generation for n_requests <= sequences prompts at once (prompts concatenated in `prompts`,
 * lengths in prompt_lens): request r's tokens go to out_tokens[r * max_new ..], its count to
 * out_counts[r].  A request stops at max_new tokens, at EOS unless ignore_eos, or at capacity; the
 * others go on.  `stats` counts all requests. */
int tm_engine_generate_batch(tm_engine *e, const uint32_t *prompts, const uint32_t *prompt_lens, uint32_t n_requests,
                             uint32_t max_new, int ignore_eos, uint32_t *out_tokens, uint32_t *out_counts,
                             tm_engine_stats *stats, char *err, size_t err_cap);

/* `steps` decode-graph replays with no host read in between (device-greedy),
 * for kernel-only timing; the caller brackets it with events on the stream. */
int tm_engine_decode_steps(tm_engine *e, uint32_t steps, char *err, size_t err_cap);

/* The same steps encoded operator by operator (one dispatch per operator), so
 * the device context's profile table (tm_cuda_profile_set / _read) attributes
 * GPU time per operator: crates/tuckcore/src/engine/metal.rs:1964-1968. */
int tm_engine_decode_ungrouped(tm_engine *e, uint32_t steps, char *err, size_t err_cap);

/* Stand-alone admission arithmetic (R + U + H <= B) for a GGUF at a context,
 * without touching a device: fills the budget fields of `out`; returns
 * TM_ENGINE_*_EXCEEDS_BUDGET when the plan does not fit. */
int tm_engine_plan(const char *gguf_path, uint32_t context, uint64_t budget_bytes, tm_engine_info *out,
                   char *err, size_t err_cap);
/* The same for one rank of an output-row split: plan_weights / plan_state /
 * plan_scratch are that rank's exact device bytes (the embedding table is
 * replicated, every projection and the KV cache are divided). */
int tm_engine_plan_shard(const char *gguf_path, uint32_t context, uint64_t budget_bytes, uint32_t shard_rank,
                         uint32_t shard_world, tm_engine_info *out, char *err, size_t err_cap);

#ifdef __cplusplus
}
#endif

#endif /* TM_ENGINE_H */
