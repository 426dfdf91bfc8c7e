#pragma once
#include "gguf.hpp"
#include "graph.hpp"

namespace tuckmill {
ModelGraph adapt_qwen3(const GgufInspection &insp);
ModelGraph adapt_gemma3(const GgufInspection &insp);
// Dispatch on general.architecture; anything else is a typed refusal.
ModelGraph adapt(const GgufInspection &insp);
}  // namespace tuckmill
