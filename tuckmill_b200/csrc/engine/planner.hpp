// Admission arithmetic re-used against HBM: R + U + H <= B
// (crates/planner/src/budget.rs:78-150, crates/manifest/src/plan.rs:68-96,
// policy defaults crates/planner/src/lib.rs:75-110, KV payload
// crates/planner/src/kv.rs:19-35).  Integers only; nothing here touches a device.
#pragma once
#include <cmath>
#include <cstdint>
#include <string>

#include "error.hpp"

namespace tuckmill {

inline uint64_t sat_add(uint64_t a, uint64_t b) { return a > UINT64_MAX - b ? UINT64_MAX : a + b; }

struct PlannerPolicy {
    double safety_reserve_ratio = 0.125;
    uint64_t safety_reserve_floor_bytes = 192ull << 20;
    uint64_t overhead_estimate_bytes = 192ull << 20;
    // The reference reserves 192 MiB of workspaces for a 128-token prefill chunk
    // on an 8 GB machine; the B200 path runs 512-token chunks, so the resident
    // workspace class is sized for those (the exact preflight still has to fit).
    uint64_t workspaces_resident_bytes = 2048ull << 20;
    uint64_t io_buffers_resident_bytes = 16ull << 20;
    uint32_t kv_bytes_per_element = 2;
    uint64_t safety_reserve(uint64_t budget) const {
        const uint64_t by_ratio = (uint64_t)std::llround((double)budget * safety_reserve_ratio);
        return by_ratio > safety_reserve_floor_bytes ? by_ratio : safety_reserve_floor_bytes;
    }
};

struct KvGeometry {
    uint64_t layers = 0, kv_head_count = 0, key_length = 0, value_length = 0;
};

// layers * kv_heads * (k + v) * bytes * tokens; false on overflow (never wraps).
inline bool estimate_kv_bytes(const KvGeometry &kv, uint64_t total_tokens, uint32_t bytes_per_element,
                              uint64_t *total, uint64_t *per_token) {
    auto mul = [](uint64_t a, uint64_t b, uint64_t *o) {
        if (b != 0 && a > UINT64_MAX / b) return false;
        *o = a * b;
        return true;
    };
    uint64_t pt = 0;
    if (kv.key_length > UINT64_MAX - kv.value_length) return false;
    if (!mul(kv.layers, kv.kv_head_count, &pt) || !mul(pt, kv.key_length + kv.value_length, &pt) ||
        !mul(pt, bytes_per_element, &pt))
        return false;
    uint64_t t = 0;
    if (!mul(pt, total_tokens, &t)) return false;
    *total = t;
    *per_token = pt;
    return true;
}

struct ReservationBreakdown {
    uint64_t weights = 0, kv_state = 0, workspaces = 0, io_buffers = 0;
    uint64_t total() const { return sat_add(sat_add(weights, kv_state), sat_add(workspaces, io_buffers)); }
};

struct PlanBudget {
    uint64_t requested_budget = 0;   // B
    uint64_t overhead_estimate = 0;  // U
    uint64_t safety_reserve = 0;     // H
    ReservationBreakdown reservation_breakdown;  // R by class
    uint64_t reservation() const { return reservation_breakdown.total(); }
    uint64_t admitted_total() const { return sat_add(sat_add(reservation(), overhead_estimate), safety_reserve); }
    bool fits() const { return admitted_total() <= requested_budget; }
    uint64_t headroom() const { return fits() ? requested_budget - admitted_total() : 0; }
};

// Resident-mode reservation for one device (reserve_resident + make_plan_budget).
inline PlanBudget make_resident_plan(uint64_t budget, uint64_t weight_bytes, uint64_t kv_bytes,
                                     const PlannerPolicy &policy = PlannerPolicy()) {
    PlanBudget b;
    b.requested_budget = budget;
    b.overhead_estimate = policy.overhead_estimate_bytes;
    b.safety_reserve = policy.safety_reserve(budget);
    b.reservation_breakdown.weights = weight_bytes;
    b.reservation_breakdown.kv_state = kv_bytes;
    b.reservation_breakdown.workspaces = policy.workspaces_resident_bytes;
    b.reservation_breakdown.io_buffers = policy.io_buffers_resident_bytes;
    return b;
}

// Refuse a plan that does not fit, naming the class that broke it.
inline void require_admitted(const PlanBudget &b, uint64_t context_tokens) {
    if (b.fits()) return;
    const bool model_alone = sat_add(sat_add(b.reservation_breakdown.weights, b.reservation_breakdown.workspaces),
                                     sat_add(b.overhead_estimate, b.safety_reserve)) > b.requested_budget;
    throw TuckmillError(model_alone ? ErrorCode::ModelExceedsBudget : ErrorCode::ContextExceedsBudget,
                        "reservation " + std::to_string(b.reservation()) + " + overhead " +
                            std::to_string(b.overhead_estimate) + " + safety reserve " +
                            std::to_string(b.safety_reserve) + " exceeds the budget " +
                            std::to_string(b.requested_budget) + " at context " + std::to_string(context_tokens),
                        model_alone ? "Use a device with more memory or split the model across devices."
                                    : "Lower --context or raise the memory budget.");
}

}  // namespace tuckmill
