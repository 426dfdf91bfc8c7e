// The typed model graph every adapter produces and the engine executes -- the
// structures of crates/tuckcore/src/engine/graph.rs:7-170 restricted to the
// dense-attention decoders (the Gated-DeltaNet mixer and the MTP head belong to
// the Qwen3.5 hybrid, which this path does not serve).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace tuckmill {

struct Tensor {
    size_t index = 0;
    bool operator==(const Tensor &o) const { return index == o.index; }
    bool operator!=(const Tensor &o) const { return index != o.index; }
};

struct AttentionSpec {
    Tensor q, k, v, o;
    Tensor q_norm, k_norm;  // per-head RMS norms of Q and K (weighted, before RoPE)
    size_t heads = 0, kv_heads = 0, head_dim = 0;
    size_t rope_dims = 0;   // rotated dims per head (== head_dim for full rotation)
    float rope_base = 10000.0f;
    size_t window = 0;      // 0 = full causal attention
};

enum class GluActivation { Silu, GeluTanh };

struct FfnSpec {
    Tensor gate, up, down;
    size_t width = 0;
    GluActivation act = GluActivation::Silu;  // SwiGlu | GeGlu
};

// x += out_norm(mixer(norm(x))); x += out_norm(ffn(norm(x))); each output norm
// only when the artifact has it (Gemma's post-attention / post-FFN norms).
struct LayerSpec {
    Tensor pre_norm;
    AttentionSpec mixer;
    bool has_mixer_out_norm = false;
    Tensor mixer_out_norm;
    Tensor post_norm;
    FfnSpec ffn;
    bool has_ffn_out_norm = false;
    Tensor ffn_out_norm;
};

struct ModelGraph {
    std::string architecture;
    size_t hidden = 0, vocab = 0;
    float eps = 1e-6f;
    Tensor embedding;
    float embedding_scale = 0.0f;  // 0 = none (Gemma: sqrt(hidden))
    std::vector<LayerSpec> layers;
    Tensor final_norm;
    Tensor head;  // the embedding itself when the artifact ties them
    bool has_eos = false;
    uint32_t eos_token_id = 0;
};

}  // namespace tuckmill
