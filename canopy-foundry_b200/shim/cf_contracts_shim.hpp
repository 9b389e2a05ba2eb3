// Publishes what the dispatch front end of libcanopy_fp8 leaves on the device through the reference's own planner
// contracts, so that its trainer can keep the forward-owned route identity and the schedule identity it expects:
//   RoutePlan / RoutePlanStore                     include/canopy_foundry/moe/route_plan.hpp, src/moe/route_plan.cpp
//   SchedulerKey / SchedulerWorkspace / ...Cache   include/canopy_foundry/moe/scheduler.hpp,  src/moe/scheduler.cpp
// Both contracts speak in opaque 64-bit "tokens" that name backend storage; here a token is the device address of the
// buffer. Nothing in this header touches the device or synchronises with it: the counts stay on the GPU (the grouped
// GEMMs read them there), so the fields that would need them on the host (active_expert_count, actual_rows, active_tiles,
// routing_load_cv) are published as "unavailable" (-1), which the contract allows.
//
// One layer, forward:
//   cf_moe_route_dispatch_lists(...)                          fills counts / offsets / row_indices / route weights
//   plan = cf_shim::publish_dispatch(store, key, generation, buffers)
//   ws   = cf_shim::require_schedule(cache, generation, buffers, N, K, orientation)
//   cf_moe_gather_all_u8 / cf_gemm_fp8_nt_grouped / ...       consume the same buffers
// Backward: store.require_for_backward(key, generation) returns the same plan, hence the same lists (the row order the
// backward must reuse), and cf_shim::buffers_of(plan) gives the device pointers back.
//
// Weights: ExecutionViewCache (include/canopy_foundry/precision/execution_view.hpp, src/precision/execution_view.cpp) keeps
// one packed view per (tensor, role, format, layout) and tensor generation. cf_shim::require_weight_view maps the E4M3
// caches of a cf_fp8_weight onto it: the forward role is the [out, in] cache, the dgrad roles either the transposed
// [in, out] cache (NT dgrad) or the forward cache read MN-major (cf_gemm_fp8_nn: no second cache). The caches are
// re-quantised (cf_refresh_fp8_weight, or nothing when the optimiser pass wrote them itself) at most once per tensor
// generation: the optimiser advances the generation (cache.invalidate), the first consumer of the new generation
// triggers the refresh, later consumers of the same generation reuse it.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>

#include "canopy_foundry/moe/route_plan.hpp"
#include "canopy_foundry/moe/scheduler.hpp"
#include "canopy_foundry/precision/execution_view.hpp"
#include "canopy_fp8.h"

namespace cf_shim {

// Device buffers of one dispatch (the outputs of cf_moe_route_dispatch_lists, or of the four separate calls).
struct DispatchBuffers {
    const int* d_counts = nullptr;         // int[lists]
    const int* d_offsets = nullptr;        // int[lists]
    const int* d_row_indices = nullptr;    // int[lists, rows]: ascending row numbers per list
    const float* d_route_weights = nullptr;   // float[rows, lists]: a row's non-zero columns are its selected lists, the
                                              // values its renormalised top-k probabilities
    int lists = 0;                         // experts, or expert replicas in the expert-parallel layer
    int rows = 0;                          // tokens routed by this call
    int top_k = 0;
};

inline std::uint64_t token_of(const void* p) { return static_cast<std::uint64_t>(reinterpret_cast<std::uintptr_t>(p)); }

// FNV-1a over the buffer identities and the shape: another buffer set, shape or top_k gives another fingerprint.
inline std::uint64_t dispatch_fingerprint(const DispatchBuffers& b) {
    const std::uint64_t words[7] = {token_of(b.d_counts), token_of(b.d_offsets), token_of(b.d_row_indices),
                                    token_of(b.d_route_weights), static_cast<std::uint64_t>(b.lists),
                                    static_cast<std::uint64_t>(b.rows), static_cast<std::uint64_t>(b.top_k)};
    std::uint64_t h = 1469598103934665603ull;
    for (std::uint64_t w : words)
        for (int i = 0; i < 8; ++i) { h ^= (w >> (8 * i)) & 0xffu; h *= 1099511628211ull; }
    return h ? h : 1;
}

inline canopy_foundry::RoutePlan make_route_plan(canopy_foundry::RoutePlanKey key, canopy_foundry::RouteGeneration generation,
                                                 const DispatchBuffers& b) {
    canopy_foundry::RoutePlan p;
    p.key = key;
    p.generation = generation;
    p.counts_token = token_of(b.d_counts);
    p.row_indices_token = token_of(b.d_row_indices);
    p.offsets_token = token_of(b.d_offsets);
    // the sparse route-weight matrix carries both the selection (its non-zero pattern) and the probabilities
    p.selected_experts_token = token_of(b.d_route_weights);
    p.topk_probabilities_token = token_of(b.d_route_weights);
    p.schedule_fingerprint = dispatch_fingerprint(b);
    p.experts = b.lists;
    p.source_rows = b.rows;
    p.routes = b.rows * b.top_k;
    p.top_k = b.top_k;
    p.forward_owned = true;
    return p;               // active_expert_count, actual_rows, active_tiles, routing_load_cv: -1 (not read back)
}

// Throws canopy_foundry::RoutePlanError exactly where the store does (invalid plan, generation not advancing, duplicate key).
inline const canopy_foundry::RoutePlan& publish_dispatch(canopy_foundry::RoutePlanStore& store, canopy_foundry::RoutePlanKey key,
                                                         canopy_foundry::RouteGeneration generation, const DispatchBuffers& b) {
    return store.publish(make_route_plan(key, generation, b));
}

inline DispatchBuffers buffers_of(const canopy_foundry::RoutePlan& p) {
    DispatchBuffers b;
    b.d_counts = reinterpret_cast<const int*>(static_cast<std::uintptr_t>(p.counts_token));
    b.d_offsets = reinterpret_cast<const int*>(static_cast<std::uintptr_t>(p.offsets_token));
    b.d_row_indices = reinterpret_cast<const int*>(static_cast<std::uintptr_t>(p.row_indices_token));
    b.d_route_weights = reinterpret_cast<const float*>(static_cast<std::uintptr_t>(p.topk_probabilities_token));
    b.lists = p.experts;
    b.rows = p.source_rows;
    b.top_k = p.top_k;
    return b;
}

// The grouped GEMM of this library schedules itself on the device from counts / offsets (tile = one list's 256-row block x
// 256 output columns, K in 128-byte chunks), so the "schedule" of a route generation IS those two buffers and its
// workspace needs no allocation. orientation: 0 = NT forward (cf_gemm_fp8_nt_grouped and its fused forms), 1 = NN dgrad
// (cf_gemm_fp8_nn_grouped).
inline canopy_foundry::SchedulerKey schedule_key(canopy_foundry::RouteGeneration generation, const DispatchBuffers& b, int N, int K,
                                                 int orientation) {
    canopy_foundry::SchedulerKey k;
    k.route_generation = generation;
    k.experts = b.lists;
    k.max_rows = b.rows * b.top_k;
    k.n_tiles = (N + 255) / 256;
    k.k_chunks = (K + 127) / 128;
    k.orientation = orientation;
    return k;
}

inline const canopy_foundry::SchedulerWorkspace& require_schedule(canopy_foundry::SchedulerWorkspaceCache& cache,
                                                                  canopy_foundry::RouteGeneration generation,
                                                                  const DispatchBuffers& b, int N, int K, int orientation) {
    const canopy_foundry::SchedulerKey key = schedule_key(generation, b, N, K, orientation);
    return cache.require(key, [&b](const canopy_foundry::SchedulerKey& k) {
        canopy_foundry::SchedulerWorkspace w;
        w.key = k;
        w.schedule_token = token_of(b.d_counts);
        w.workspace_token = token_of(b.d_offsets);
        // upper bound of the tiles a launch can see: every list may end in a partly filled row block
        w.tile_capacity = (static_cast<std::size_t>(k.max_rows + 255) / 256 + static_cast<std::size_t>(k.experts)) *
                          static_cast<std::size_t>(k.n_tiles);
        w.expert_capacity = static_cast<std::size_t>(k.experts);
        w.schedule_valid = true;
        return w;
    });
}

// ---- weights ------------------------------------------------------------------------------------------------------
// Key of the packed view a role consumes. Forward / ExpertForward: fwd8 [out, in], row-major. BackwardDx / ExpertDx:
// bwd8 [in, out] (PackedOrientation::Transposed) when the weight keeps one, else the forward cache consumed MN-major
// (PackedOrientation::ColumnMajor). The GEMM's tile is 256 x 128 bytes in either case.
inline canopy_foundry::ExecutionViewKey weight_view_key(canopy_foundry::TensorId tensor, canopy_foundry::ExecutionRole role,
                                                        const cf_fp8_weight& w) {
    using namespace canopy_foundry;
    ExecutionViewKey k;
    k.tensor = tensor;
    k.role = role;
    k.format = NumericFormat::FP8E4M3;
    const bool dx = role == ExecutionRole::BackwardDx || role == ExecutionRole::ExpertDx;
    k.layout.rows = static_cast<std::uint32_t>(dx && w.bwd8 ? w.in_dim : w.out_dim);
    k.layout.columns = static_cast<std::uint32_t>(dx && w.bwd8 ? w.out_dim : w.in_dim);
    k.layout.tile_rows = 256;
    k.layout.tile_columns = 128;
    k.layout.orientation = !dx ? PackedOrientation::RowMajor : (w.bwd8 ? PackedOrientation::Transposed : PackedOrientation::ColumnMajor);
    return k;
}

// `refresh` brings both caches of the weight up to date with its bf16 master (default: cf_refresh_fp8_weight with the
// amax the optimiser left, recompute_amax = 0, on `stream`); it runs only when the cache holds no view of this generation
// for this key AND no other role of the same tensor has already refreshed this generation (one refresh writes both caches).
// Returns the view; its storage_token is the device address of the E4M3 bytes the role's GEMM reads.
inline const canopy_foundry::PackedExecutionView& require_weight_view(
    canopy_foundry::ExecutionViewCache& cache, canopy_foundry::TensorId tensor, canopy_foundry::TensorGeneration generation,
    canopy_foundry::ExecutionRole role, const cf_fp8_weight& w, void* stream,
    const std::function<int(const cf_fp8_weight&, void*)>& refresh = nullptr) {
    using namespace canopy_foundry;
    const ExecutionViewKey key = weight_view_key(tensor, role, w);
    return cache.require(key, generation, [&](const ExecutionViewKey& k, TensorGeneration g) {
        // another role's view of the same generation means the caches are current already
        bool current = false;
        for (ExecutionRole other : {ExecutionRole::Forward, ExecutionRole::BackwardDx, ExecutionRole::ExpertForward,
                                    ExecutionRole::ExpertDx}) {
            if (other == role) continue;
            if (cache.lookup(weight_view_key(tensor, other, w), g) != nullptr) { current = true; break; }
        }
        if (!current) {
            const int rc = refresh ? refresh(w, stream) : cf_refresh_fp8_weight(&w, 0, stream);
            if (rc != CF_OK) throw ExecutionViewError("FP8 weight refresh failed");
        }
        PackedExecutionView v;
        v.key = k;
        v.source_generation = g;
        const bool dx = role == ExecutionRole::BackwardDx || role == ExecutionRole::ExpertDx;
        v.storage_token = token_of(dx && w.bwd8 ? w.bwd8 : w.fwd8);
        v.payload_bytes = static_cast<std::size_t>(w.in_dim) * static_cast<std::size_t>(w.out_dim);
        v.scale_bytes = sizeof(float);
        v.ready = true;
        return v;
    });
}

}  // namespace cf_shim
