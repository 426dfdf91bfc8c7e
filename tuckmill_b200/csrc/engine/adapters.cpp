// Family adapters: GGUF metadata + tensor names -> ModelGraph.  Follows
// crates/tuckcore/src/engine/adapters.rs:130-200 (dense Qwen3; config
// resolution crates/tuckcore/src/model.rs:125-237) and :202-336 (Gemma 3).
// Variants a graph does not express exactly are refused, never approximated.
#include <cmath>

#include "adapters.hpp"

namespace tuckmill {

namespace {

Tensor need(const GgufInspection &insp, const std::string &name, const char *family) {
    const long i = insp.find(name);
    if (i < 0)
        throw TuckmillError(ErrorCode::UnsupportedArchitecture,
                            "artifact is missing required tensor \"" + name + "\" for " + family);
    return Tensor{(size_t)i};
}

uint64_t need_u64(const GgufInspection &insp, const std::string &key) {
    uint64_t v = 0;
    if (!insp.get_u64(key, &v) || v == 0)
        throw TuckmillError(ErrorCode::UnsupportedArchitecture, key + " is required");
    return v;
}

}  // namespace

ModelGraph adapt_qwen3(const GgufInspection &insp) {
    const uint64_t layers = need_u64(insp, "qwen3.block_count");
    const uint64_t hidden = need_u64(insp, "qwen3.embedding_length");
    const uint64_t ffn = need_u64(insp, "qwen3.feed_forward_length");
    const uint64_t heads = need_u64(insp, "qwen3.attention.head_count");
    const uint64_t kv_heads = need_u64(insp, "qwen3.attention.head_count_kv");
    uint64_t key_len = 0, value_len = 0;
    if (!insp.get_u64("qwen3.attention.key_length", &key_len)) key_len = hidden / heads;
    if (!insp.get_u64("qwen3.attention.value_length", &value_len)) value_len = key_len;
    if (key_len != value_len)
        throw TuckmillError(ErrorCode::UnsupportedArchitecture,
                            "dense Qwen3 with key length " + std::to_string(key_len) + " != value length " +
                                std::to_string(value_len) + " has no engine block; attention heads are square",
                            "Use an artifact with equal key and value head sizes; shapes are never approximated.");
    if (heads % kv_heads != 0)
        throw TuckmillError(ErrorCode::UnsupportedArchitecture, "head count is not a multiple of the KV head count");
    float rope_base = 10000.0f, eps = 1e-6f;
    insp.get_f32("qwen3.rope.freq_base", &rope_base);
    insp.get_f32("qwen3.attention.layer_norm_rms_epsilon", &eps);

    ModelGraph g;
    g.architecture = "qwen3";
    g.hidden = hidden;
    g.eps = eps;
    g.embedding = need(insp, "token_embd.weight", "dense Qwen3");
    const GgufTensor &emb = insp.tensors[g.embedding.index];
    if (emb.dims.size() != 2 || emb.dims[0] != hidden)
        throw TuckmillError(ErrorCode::UnsupportedArchitecture,
                            "token_embd.weight dims do not match embedding_length " + std::to_string(hidden));
    g.vocab = emb.dims[1];
    for (uint64_t l = 0; l < layers; ++l) {
        const std::string p = "blk." + std::to_string(l) + ".";
        LayerSpec L;
        L.pre_norm = need(insp, p + "attn_norm.weight", "dense Qwen3");
        L.mixer.q = need(insp, p + "attn_q.weight", "dense Qwen3");
        L.mixer.k = need(insp, p + "attn_k.weight", "dense Qwen3");
        L.mixer.v = need(insp, p + "attn_v.weight", "dense Qwen3");
        L.mixer.o = need(insp, p + "attn_output.weight", "dense Qwen3");
        L.mixer.q_norm = need(insp, p + "attn_q_norm.weight", "dense Qwen3");
        L.mixer.k_norm = need(insp, p + "attn_k_norm.weight", "dense Qwen3");
        L.mixer.heads = heads;
        L.mixer.kv_heads = kv_heads;
        L.mixer.head_dim = key_len;
        L.mixer.rope_dims = key_len;
        L.mixer.rope_base = rope_base;
        L.mixer.window = 0;
        L.post_norm = need(insp, p + "ffn_norm.weight", "dense Qwen3");
        L.ffn.gate = need(insp, p + "ffn_gate.weight", "dense Qwen3");
        L.ffn.up = need(insp, p + "ffn_up.weight", "dense Qwen3");
        L.ffn.down = need(insp, p + "ffn_down.weight", "dense Qwen3");
        L.ffn.width = ffn;
        L.ffn.act = GluActivation::Silu;
        g.layers.push_back(L);
    }
    g.final_norm = need(insp, "output_norm.weight", "dense Qwen3");
    // Absence of output.weight means tied embeddings by the format's convention.
    const long out = insp.find("output.weight");
    g.head = out >= 0 ? Tensor{(size_t)out} : g.embedding;
    uint64_t eos = 0;
    if (insp.get_u64("tokenizer.ggml.eos_token_id", &eos)) {
        g.has_eos = true;
        g.eos_token_id = (uint32_t)eos;
    }
    return g;
}

// Every 6th layer (1-based) attends globally; the others use the sliding window
// with RoPE base 10000 (fixed by the architecture).
static constexpr size_t kGemma3SwaPattern = 6;
static constexpr float kGemma3SwaRopeBase = 10000.0f;

ModelGraph adapt_gemma3(const GgufInspection &insp) {
    auto refuse = [](const std::string &what) {
        return TuckmillError(ErrorCode::UnsupportedArchitecture, what,
                             "Use a Gemma 3 text artifact this graph expresses exactly; variants are never approximated.");
    };
    for (const char *key : {"gemma3.rope.scaling.factor", "gemma3.final_logit_softcapping",
                            "gemma3.attn_logit_softcapping"})
        if (insp.get(key)) throw refuse(std::string("gemma3 artifact declares ") + key + ", which this graph does not implement");
    uint64_t pattern = 0;
    if (insp.get_u64("gemma3.attention.sliding_window_pattern", &pattern) && pattern != kGemma3SwaPattern)
        throw refuse("gemma3 sliding-window pattern is not every 6th layer");
    auto num = [&](const std::string &key) {
        uint64_t v = 0;
        if (!insp.get_u64("gemma3." + key, &v)) throw refuse("gemma3 artifact lacks gemma3." + key);
        return (size_t)v;
    };
    const size_t layers = num("block_count"), hidden = num("embedding_length"), ffn = num("feed_forward_length");
    const size_t heads = num("attention.head_count"), kv_heads = num("attention.head_count_kv");
    const size_t key_len = num("attention.key_length"), value_len = num("attention.value_length");
    const size_t window = num("attention.sliding_window");
    if (key_len != value_len || heads == 0 || kv_heads == 0 || heads % kv_heads != 0 || window == 0)
        throw refuse("gemma3 attention geometry has no engine block");
    float eps = 0.0f, global_base = 0.0f;
    if (!insp.get_f32("gemma3.attention.layer_norm_rms_epsilon", &eps)) throw refuse("gemma3 artifact lacks its RMS norm epsilon");
    if (!insp.get_f32("gemma3.rope.freq_base", &global_base)) throw refuse("gemma3 artifact lacks gemma3.rope.freq_base");
    if (insp.find("output.weight") >= 0) throw refuse("gemma3 artifact carries an untied output head; this graph ties it");

    ModelGraph g;
    g.architecture = "gemma3";
    g.hidden = hidden;
    g.eps = eps;
    g.embedding = need(insp, "token_embd.weight", "gemma3");
    const GgufTensor &emb = insp.tensors[g.embedding.index];
    if (emb.dims.size() != 2) throw refuse("token embedding is not 2-D");
    g.vocab = emb.dims[1];
    for (size_t l = 0; l < layers; ++l) {
        const std::string p = "blk." + std::to_string(l) + ".";
        const bool global = (l + 1) % kGemma3SwaPattern == 0;
        LayerSpec L;
        L.pre_norm = need(insp, p + "attn_norm.weight", "gemma3");
        L.mixer.q = need(insp, p + "attn_q.weight", "gemma3");
        L.mixer.k = need(insp, p + "attn_k.weight", "gemma3");
        L.mixer.v = need(insp, p + "attn_v.weight", "gemma3");
        L.mixer.o = need(insp, p + "attn_output.weight", "gemma3");
        L.mixer.q_norm = need(insp, p + "attn_q_norm.weight", "gemma3");
        L.mixer.k_norm = need(insp, p + "attn_k_norm.weight", "gemma3");
        L.mixer.heads = heads;
        L.mixer.kv_heads = kv_heads;
        L.mixer.head_dim = key_len;
        L.mixer.rope_dims = key_len;
        L.mixer.rope_base = global ? global_base : kGemma3SwaRopeBase;
        L.mixer.window = global ? 0 : window;
        L.has_mixer_out_norm = true;
        L.mixer_out_norm = need(insp, p + "post_attention_norm.weight", "gemma3");
        L.post_norm = need(insp, p + "ffn_norm.weight", "gemma3");
        L.ffn.gate = need(insp, p + "ffn_gate.weight", "gemma3");
        L.ffn.up = need(insp, p + "ffn_up.weight", "gemma3");
        L.ffn.down = need(insp, p + "ffn_down.weight", "gemma3");
        L.ffn.width = ffn;
        L.ffn.act = GluActivation::GeluTanh;
        L.has_ffn_out_norm = true;
        L.ffn_out_norm = need(insp, p + "post_ffw_norm.weight", "gemma3");
        g.layers.push_back(L);
    }
    g.embedding_scale = std::sqrt((float)hidden);
    g.final_norm = need(insp, "output_norm.weight", "gemma3");
    g.head = g.embedding;
    uint64_t eos = 0;
    if (insp.get_u64("tokenizer.ggml.eos_token_id", &eos)) {
        g.has_eos = true;
        g.eos_token_id = (uint32_t)eos;
    }
    return g;
}

ModelGraph adapt(const GgufInspection &insp) {
    const std::string arch = insp.arch_id();
    if (arch.empty()) throw TuckmillError(ErrorCode::UnsupportedArchitecture, "artifact declares no architecture");
    if (arch == "qwen3") return adapt_qwen3(insp);
    if (arch == "gemma3") return adapt_gemma3(insp);
    throw TuckmillError(ErrorCode::UnsupportedArchitecture,
                        "the CUDA engine executes dense qwen3 and gemma3 artifacts; this artifact is \"" + arch + "\"",
                        "Hybrid (qwen35) and MoE graphs have no CUDA blocks; architectures are never substituted.");
}

}  // namespace tuckmill
