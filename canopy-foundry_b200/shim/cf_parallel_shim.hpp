// Handling for the reference's ParallelMode::ExpertSharded (include/canopy_foundry/parallel/plan.hpp:9-13), which its
// src/parallel/plan.cpp only names: turns a ParallelPlan of that mode plus the expected expert load into the layout the
// expert-parallel entry points of libcanopy_fp8 consume, in the reference's own terms:
//   plan.devices     one rank per listed device (the reference drives several devices from one process, one thread
//                    per training body: include/ida_native/kernels.hpp:599-604)
//   plan.transport   must be TransportKind::CudaP2P: rows are stored straight into the serving rank's buffers, so every
//                    pair of listed devices needs peer access (cudaDeviceEnablePeerAccess) and the receive / return
//                    buffers are plain cudaMalloc (or arena) allocations on their own device, addressed by every rank
//                    through the same pointer value
// Per rank r the trainer then allocates, once, from its arena (capacity = tokens_per_rank * top_k * world rows):
//   recv8  [capacity, H] bytes, recv_dx float[capacity], back [tokens_per_rank * top_k, H] bf16,
// builds the device tables (d_replica_start / d_replica_cum_share / d_range_lo / d_range_hi from this layout, the
// arrays of all ranks' recv8 / recv_dx / back pointers), and runs per layer on its own stream:
//   cf_moe_topk_route_f32 -> cf_moe_expand_route_replicas -> cf_moe_build_expert_row_lists ->
//   cf_moe_expert_offsets_from_counts -> [exchange the counts: every rank copies its int[V] row into every rank's
//   counts_all table with cudaMemcpyPeerAsync, then a cross-device event] -> cf_fp8_quant_act -> cf_moe_ep_plan ->
//   cf_moe_send_row_runs -> [cross-device event: all rows have arrived] -> cf_gemm_fp8_swiglu_quant_act ->
//   cf_gemm_fp8_nt_grouped_return -> [cross-device event: all results are back] -> cf_moe_combine_sorted_bf16.
// The two "[cross-device event]" points are cudaEventRecord on every rank's stream + cudaStreamWaitEvent on every
// other rank's stream (no host synchronisation), which is what the one-float all-reduces of the Python mirror
// (canopy-foundry_b200/parallel.py, EpMoeSwigluFp8Direct) stand for in a one-process-per-GPU job.
#pragma once

#include <stdexcept>
#include <string>
#include <vector>

#include "canopy_foundry/parallel/plan.hpp"
#include "canopy_fp8.h"

namespace cf_shim {

struct ExpertShardedLayout {
    cf_ep_placement placement;          // replicas, shares, per-rank replica ranges
    std::vector<int> devices;           // rank -> CUDA device ordinal (ParallelPlan::devices)
    int world() const { return placement.world; }
    // experts whose weights rank r holds, in the order the stacked local weight tensors must use
    std::vector<int> local_experts(int r) const {
        std::vector<int> out;
        for (int v = placement.rank_lo[r]; v < placement.rank_hi[r]; ++v) out.push_back(placement.replica_expert[v]);
        return out;
    }
};

// expected_load[e]: rows expert e is expected to receive (any positive scale; a trainer takes it from the previous
// steps' routing counts). min_share: overlaps below this fraction of a rank's piece get no weight copy.
// expected_total_rows > 0 (selected rows of all ranks per layer, tokens * top_k) sizes the ranks' pieces for equal tile
// work of the grouped GEMM instead of equal rows (cf_ep_placement_build_balanced); rank_speed, one positive number per
// device, additionally shortens the pieces of slower devices (cf_ep_placement_build_weighted).
inline ExpertShardedLayout expert_sharded_layout(const canopy_foundry::ParallelPlan& plan,
                                                 const std::vector<double>& expected_load, double min_share = 0.02,
                                                 double expected_total_rows = 0.0, const std::vector<double>& rank_speed = {}) {
    using canopy_foundry::ParallelMode;
    using canopy_foundry::TransportKind;
    if (plan.mode != ParallelMode::ExpertSharded)
        throw std::invalid_argument("expert_sharded_layout: plan mode is " + canopy_foundry::parallel_mode_name(plan.mode));
    if (plan.devices.empty()) throw std::invalid_argument("expert_sharded_layout: the plan lists no devices");
    if (plan.devices.size() > 1 && plan.transport != TransportKind::CudaP2P)
        throw std::invalid_argument("expert_sharded_layout: rows are stored into peer buffers, transport must be cuda_p2p, not " +
                                    canopy_foundry::transport_kind_name(plan.transport));
    ExpertShardedLayout out;
    out.devices = plan.devices;
    const int experts = static_cast<int>(expected_load.size()), world = static_cast<int>(plan.devices.size());
    if (!rank_speed.empty() && (rank_speed.size() != plan.devices.size() || expected_total_rows <= 0.0))
        throw std::invalid_argument("expert_sharded_layout: rank_speed needs one entry per device and expected_total_rows");
    const int rc = expected_total_rows > 0.0
                       ? cf_ep_placement_build_weighted(expected_load.data(), experts, world, min_share, expected_total_rows, 256,
                                                        rank_speed.empty() ? nullptr : rank_speed.data(), &out.placement)
                       : cf_ep_placement_build(expected_load.data(), experts, world, min_share, &out.placement);
    if (rc != CF_OK) throw std::runtime_error(std::string("expert_sharded_layout: ") + cf_last_error());
    return out;
}

}  // namespace cf_shim
