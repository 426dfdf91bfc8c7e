// Kernel implementation selection: the reference's `--kernels` surface
// (crates/tuckcore/src/kernels.rs:36-113) with the `cuda` variant joined to it.
// Forced selections never fall back: a machine without a usable sm_100 device
// gets a typed Unavailable refusal at load, exactly as `metal` does off macOS.
#pragma once
#include <string>

#include "error.hpp"
#include "tm_cuda.h"

namespace tuckmill {

enum class KernelSelection { Auto, Scalar, Neon, Metal, Cuda };
enum class ResolvedKernels { Scalar, Neon, Metal, Cuda };

inline bool parse_kernel_selection(const std::string &s, KernelSelection *out) {
    if (s == "auto") *out = KernelSelection::Auto;
    else if (s == "scalar") *out = KernelSelection::Scalar;
    else if (s == "neon") *out = KernelSelection::Neon;
    else if (s == "metal") *out = KernelSelection::Metal;
    else if (s == "cuda") *out = KernelSelection::Cuda;
    else return false;
    return true;
}

inline const char *resolved_kernels_str(ResolvedKernels k) {
    switch (k) {
        case ResolvedKernels::Scalar: return "scalar";
        case ResolvedKernels::Neon: return "neon";
        case ResolvedKernels::Metal: return "metal";
        default: return "cuda";
    }
}

// `auto` keeps the reference's meaning (the CPU kernels of the target); only an
// explicit `cuda` selects this library.  The CPU implementations themselves
// are the reference's and are not part of this library: resolving to them here
// reports which implementation the caller must route to.
inline ResolvedKernels resolve_kernel_selection(KernelSelection s) {
    switch (s) {
        case KernelSelection::Scalar:
        case KernelSelection::Auto:
            return ResolvedKernels::Scalar;
        case KernelSelection::Neon:
            throw TuckmillError(ErrorCode::InvalidRequest,
                                "the NEON kernel implementation requires an aarch64 target",
                                "Select --kernels auto or --kernels scalar on this machine.");
        case KernelSelection::Metal:
            throw TuckmillError(ErrorCode::Unavailable, "the Metal kernel implementation requires macOS",
                                "Select --kernels auto, neon, scalar or cuda on this machine.");
        case KernelSelection::Cuda:
            if (tm_cuda_available() <= 0)
                throw TuckmillError(ErrorCode::Unavailable,
                                    "the CUDA kernel implementation requires an NVIDIA sm_100 device",
                                    "Select --kernels auto or scalar on this machine.");
            return ResolvedKernels::Cuda;
    }
    return ResolvedKernels::Scalar;
}

// Kernel id strings reported in stats (crates/tuckcore/src/executor.rs:1296-1302,
// 1705-1710): "ADR011:<arch>-q8_0+f16:cuda" and "K01:q8_0+f16:cuda".
inline std::string engine_kernel_id(const std::string &arch) { return "ADR011:" + arch + "-q8_0+f16:cuda"; }
inline std::string k01_kernel_id() { return "K01:q8_0+f16:cuda"; }

}  // namespace tuckmill
