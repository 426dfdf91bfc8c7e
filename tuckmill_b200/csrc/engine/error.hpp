// Typed errors of the host layer.  The codes are the subset of the reference's
// ErrorCode list (crates/manifest/src/error.rs:15-43) this path can raise; every
// refusal carries a message and, where the reference gives one, an action.
#pragma once
#include <stdexcept>
#include <string>

namespace tuckmill {

enum class ErrorCode {
    InvalidRequest,
    InvalidArtifact,
    UnsupportedArchitecture,
    UnsupportedQuantization,
    ContextExceedsBudget,
    ModelExceedsBudget,
    Unavailable,
    Cancelled,
    Internal,
};

inline const char *error_code_name(ErrorCode c) {
    switch (c) {
        case ErrorCode::InvalidRequest: return "INVALID_REQUEST";
        case ErrorCode::InvalidArtifact: return "INVALID_ARTIFACT";
        case ErrorCode::UnsupportedArchitecture: return "UNSUPPORTED_ARCHITECTURE";
        case ErrorCode::UnsupportedQuantization: return "UNSUPPORTED_QUANTIZATION";
        case ErrorCode::ContextExceedsBudget: return "CONTEXT_EXCEEDS_BUDGET";
        case ErrorCode::ModelExceedsBudget: return "MODEL_EXCEEDS_BUDGET";
        case ErrorCode::Unavailable: return "UNAVAILABLE";
        case ErrorCode::Cancelled: return "CANCELLED";
        default: return "INTERNAL";
    }
}

class TuckmillError : public std::runtime_error {
public:
    TuckmillError(ErrorCode code, const std::string &message, const std::string &action = "")
        : std::runtime_error(std::string(error_code_name(code)) + ": " + message +
                             (action.empty() ? "" : " (" + action + ")")),
          code(code), message(message), action(action) {}
    ErrorCode code;
    std::string message, action;
};

}  // namespace tuckmill
