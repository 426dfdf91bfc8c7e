// The unified layer engine on CUDA: executes a typed ModelGraph with the
// operators of the tm_cuda C ABI.  Host-side counterpart of
// crates/tuckcore/src/engine/metal.rs (Matrix :107-226, Plan :254-272,
// PrefillScratch :365-425, SwiGluBlock :431-535, AttentionBlock :989-1364,
// Layer :1379-1525, alloc_plan_with :1729-1758, EngineModel :1774-2677), keeping
// its contracts -- exact byte ledger priced before any allocation, one dispatch
// per step, last-position-only vocabulary projection, device-side greedy with
// a pipelined host read -- re-designed for a B200:
//   * q|k|v and gate|up are stored as one row-concatenated matrix each, so a
//     decode layer is 5 launches (fused norm / activation / residual around the
//     GEMVs) instead of ~17;
//   * the position and the token log live on the device, so ONE recorded CUDA
//     graph is replayed for every decode step;
//   * prefill chunks are 512 tokens through the tensor-core GEMM.
#pragma once
#include <memory>
#include <vector>

#include "cuda.hpp"
#include "gguf.hpp"
#include "graph.hpp"

namespace tuckmill {

constexpr uint32_t kPrefillBatchDefault = 512;  // reference PREFILL_BATCH is 128 (engine/metal.rs:25)
constexpr uint32_t kArgmaxPartialBytes = 512;
constexpr size_t kStagingChunkBytes = 4u << 20;  // crates/tuckcore/src/qwen35_gpu.rs:1176
constexpr uint32_t kMaxSequences = 256;

struct EngineOptions {
    uint32_t prefill_batch = kPrefillBatchDefault;
    bool exact = false;  // batched projections keep the GEMV's per-row arithmetic (no tensor cores)
    // Output-row split of every projection across `world` devices (rank owns
    // rows [rank*N/world, (rank+1)*N/world)); 1 = single device.
    uint32_t shard_rank = 0, shard_world = 1;
    // true: decode steps run as ONE persistent kernel (a recorded program, include/tm_cuda.h) where
    // the model allows it: single device, not `exact`, attention geometries and widths the program
    // kernel serves.  Off by default: on the decoders measured so far the recorded graph of
    // per-operator kernels is the faster of the two.
    bool persistent = false;
    // Concurrent sequences the engine holds state for (KV planes, position and token log per
    // sequence) and decodes together, one row each, in ONE recorded step.  The reference serves one
    // request at a time (crates/supervisor/src/queue.rs:1-4); 1 keeps exactly that engine.
    uint32_t sequences = 1;
};

// Whether load_with will record the decode step as a persistent program for this graph and options
// (the plan prices the program's device memory exactly when this holds).
bool persistent_decode_applies(const ModelGraph &graph, const EngineOptions &opts);
// The same, also requiring every matrix of `src` to be Q8_0 (what load_with and the plan ask).
bool persistent_decode_applies(const ModelGraph &graph, const WeightSource &src, const EngineOptions &opts);
// What the decode program of `graph` at `capacity` positions is opened for: operators at most,
// elements of all the vectors its operators produce, elements of its largest attention's partials
// (the arguments of tm_cuda_begin_program / tm_cuda_program_bytes).
struct DecodeProgramSize {
    uint32_t max_ops = 0;
    uint64_t vector_elems = 0, attention_elems = 0;
    uint64_t bytes() const { return tm_cuda_program_bytes(max_ops, vector_elems, attention_elems); }
};
DecodeProgramSize decode_program_size(const ModelGraph &graph, size_t capacity);

// Exact device bytes by class (crates/tuckcore/src/qwen35_gpu.rs:1181-1193).
struct GpuAllocPlan {
    uint64_t weights = 0, state = 0, scratch = 0;
    uint64_t gather = 0;  // part of `scratch`: the peer-mapped exchange arena of a row split
    uint64_t total() const { return weights + state + scratch; }
};

GpuAllocPlan alloc_plan_with(const ModelGraph &graph, const WeightSource &src, size_t capacity,
                             const EngineOptions &opts);

struct GenerateStats {
    uint64_t ttft_ns = 0;         // request start -> first generated token on the host
    uint64_t decode_span_ns = 0;  // first -> last generated token (reference tok/s span)
    uint64_t prompt_tokens = 0, generated = 0;
    uint64_t kernel_launches = 0, dispatches = 0;
    uint64_t h2d_bytes = 0, d2h_bytes = 0;
};

class EngineModel {
public:
    // Prices the model (alloc_plan_with), allocates exactly that, uploads and
    // repacks every matrix, records the decode graph.  `expected_total` is the
    // preflight total the caller admitted; a ledger that differs is refused.
    static std::unique_ptr<EngineModel> load_with(std::shared_ptr<CudaContext> ctx, ModelGraph graph,
                                                  const WeightSource &src, size_t capacity,
                                                  uint64_t expected_total, const EngineOptions &opts);
    ~EngineModel();

    const ModelGraph &graph() const { return graph_; }
    size_t capacity() const { return capacity_; }
    size_t position() const { return pos_; }
    uint64_t allocated_bytes() const { return ctx_->allocated_bytes(); }
    const GpuAllocPlan &plan() const { return plan_; }
    CudaContext &context() { return *ctx_; }

    // Start a new sequence at position 0 (KV planes zero-filled on the device).
    void reset();
    // Feed `n` prompt tokens at the current position in chunks; with
    // `want_token` the last chunk also projects the last row onto the
    // vocabulary and writes its greedy token into the token log.
    void prefill(const uint32_t *tokens, size_t n, bool want_token);
    // One decode step for `token` at the current position; returns after the
    // logits are on the device (download with `logits`).
    void step(uint32_t token);
    void logits(float *out);
    // Device-greedy pipeline: `submit_greedy` replays the decode graph (the
    // token comes from the device-side log), `collect_greedy` reads the token
    // produced by the submit that returned `ticket`, without waiting for later
    // submits.
    struct Ticket { uint64_t dispatch = 0; size_t slot = 0; };
    Ticket submit_greedy();
    uint32_t collect_greedy(const Ticket &t);
    // ---- several sequences (EngineOptions::sequences > 1) ----
    size_t sequences() const;
    size_t position_of(size_t seq) const;
    // `n` prompt tokens of sequence `seq` at its current position (chunked like prefill; the other
    // sequences are untouched); with `want_token` its greedy token goes to that sequence's log.
    void prefill_seq(size_t seq, const uint32_t *tokens, size_t n, bool want_token);
    uint32_t prefill_token_of(size_t seq);
    // One decode step of EVERY sequence: tokens[s] is fed to sequence s at its position.  Every
    // sequence must have room.  Row s of the result equals the one-sequence step on the same state
    // bit for bit in `exact` mode; otherwise within the bars of the tolerance-qualified kernels.
    void step_batch(const uint32_t *tokens);
    void logits_batch(float *out);  // [sequences][vocab]; single device only
    // Device-greedy steps of all sequences with no host read in between (kernel-only timing).
    void submit_batch_greedy();
    // Greedy generation for prompts.size() <= sequences() requests at once: each prompt is
    // prefilled into its own sequence, then all decode together, step i + 1 submitted before step i
    // is read.  Sequence s stops at max_new tokens, at EOS unless ignore_eos, or at capacity, the
    // others go on.  `stats` counts all sequences (ttft = until every first token is on the host).
    std::vector<std::vector<uint32_t>> generate_batch(const std::vector<std::vector<uint32_t>> &prompts, size_t max_new,
                                                      bool ignore_eos, GenerateStats *stats);
    // The same decode step encoded operator by operator (one dispatch each, no
    // graph): the attribution mode of engine/metal.rs:1964-1968, used with the
    // context's per-operator profile table.
    void step_ungrouped();
    // Throws Internal naming the wait when a bounded device-side wait ran out (tensor-core GEMM
    // pipeline, peer-memory exchange, persistent decode program) or a step ran past the KV capacity:
    // the results of such a dispatch are undefined and must not be returned as tokens.  Waits for
    // the stream.
    void check_device_status();
    // The persistent decode program (for tm_cuda_program_status / _trace), or null when a decode step
    // is a graph of kernels.
    tm_cuda_graph *decode_program() const;
    // Token the last prefill(want_token) chose (blocking read).
    uint32_t prefill_token();
    // The reference's run_session loop (crates/tuckcore/src/executor.rs:870-1125)
    // for a greedy request: chunked prefill, then decode with step i+1 submitted
    // before step i is collected.  Stops at `max_new` tokens, at EOS unless
    // `ignore_eos`, or at capacity.
    std::vector<uint32_t> generate(const uint32_t *prompt, size_t n_prompt, size_t max_new, bool ignore_eos,
                                   GenerateStats *stats);

private:
    struct Impl;
    EngineModel() = default;
    void encode_decode_step();
    void encode_batch_step();
    std::shared_ptr<CudaContext> ctx_;
    ModelGraph graph_;
    EngineOptions opts_;
    GpuAllocPlan plan_;
    size_t capacity_ = 0, pos_ = 0;
    std::unique_ptr<Impl> impl_;
};

}  // namespace tuckmill
