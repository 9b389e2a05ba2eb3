// Internal launch interface of the tcgen05 FP8 GEMM (shared by the API and MoE translation units).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

#include "canopy_fp8.h"

namespace cf {

struct GemmParams {
    int groups = 1;                 // experts stacked along the rows of B; 1 = dense
    int M = 0;                      // dense row count (ignored when d_counts is set)
    int N = 0;                      // output columns (per expert)
    int K = 0;
    const int* d_counts = nullptr;  // grouped: rows per expert (device)
    const int* d_offsets = nullptr; // grouped: first compact row per expert (device)
    const int* d_group_weight = nullptr; // grouped: weight-block index per group (device); null = group index
    void* const* d_group_out = nullptr;  // grouped: per-group output base (device array; may point into a peer GPU); null = C
    const long long* d_group_out_row0 = nullptr;  // grouped: first output row of the group inside its base
    const float* d_a_descale = nullptr;
    int a_descale_per_group = 0;
    const float* d_b_descale = nullptr;
    const float* d_a_row_descale = nullptr;
    const float* d_b_col_descale = nullptr;
    void* C = nullptr;
    long long ldc = 0;
    int out_kind = 0;               // 0 bf16 store, 1 f32 store, 2 f32 +=, 3 bf16 +=, 4 SwiGLU -> E4M3 [., N/2] (ldc in bytes),
                                    // 5 SwiGLU -> bf16 [., N/2] (ldc in elements) + per-row amax
    const float* d_quant_scale = nullptr;   // out_kind 4: scale the SwiGLU product is quantised with
    float* d_amax_out = nullptr;            // out_kind 4: amax of the bf16 SwiGLU product (integer atomicMax)
    float* d_row_amax_out = nullptr;        // out_kind 5: per-row amax of the bf16 SwiGLU product, indexed like d_a_row_descale
    const uint16_t* bias = nullptr;
    int bias_mode = 0;
    int c_vec = 0;                  // filled by the launcher
    int tma_store = 0;              // filled by the launcher: bf16 output goes through shared memory + TMA stores
    int tma_reduce = 0;             // filled by the launcher: fp32 beta=1 output goes through TMA reduce-add
    long long c_rows = 0;           // filled by the launcher: row extent of C for the store tensor map
    // Reduce-scatter form (out_kind 2 only): rows [r * rows_per_peer, (r + 1) * rows_per_peer) of the product are added
    // into peer_out_host[r], rank r's fp32 [rows_per_peer, N] slice as mapped in this process (may be a peer GPU's
    // memory). The launcher encodes one tensor map per slice into d_peer_maps (device, peer_count * 128 bytes).
    void* const* peer_out_host = nullptr;
    int peer_count = 0;
    int rows_per_peer = 0;
    void* d_peer_maps = nullptr;
    // Return form (out_kind 0, grouped): the rows of group g are runs d_out_runs[g * runs_per_group + s] (ascending
    // src_row in the compact row space of A); run s goes to rows dst_row.. of destination buffer `dst` (bf16
    // [rows_per_peer, N], pitch ldc), whose tensor maps sit at d_peer_maps and whose base pointers at d_peer_bases.
    const cf_row_run* d_out_runs = nullptr;
    int runs_per_group = 0;
    void* const* d_peer_bases = nullptr;
    int peer_maps_ready = 0;        // the maps at d_peer_maps already describe peer_out_host (cached by the caller)
    int mn_major = 0;               // operands are [K, M] and [K, N] in memory (un-transposed weight-gradient form)
    int b_mn_major = 0;             // only B is [K, N] in memory (weight blocks [weights * K, N] read as they lie): C = A . B
    long long ldb = 0;              // mn_major / b_mn_major: row pitch of B in bytes
    int a_e5m2 = 0;
    int b_e5m2 = 0;
    int* d_status = nullptr;        // context status word (bounded-wait failures)
    int raster_m = 8;               // row blocks per rasterisation band
};

// a_rows / b_rows: row extents of the two byte matrices as the tensor maps should see them.
// tile_upper_bound: number of (128 x 256) tiles at most (sizes the persistent grid).
int launch_gemm_fp8_nt(const void* d_A, long long lda, long long a_rows, const void* d_B, long long b_rows,
                       GemmParams p, int tile_upper_bound, cudaStream_t st);
int launch_wait_selftest(int* d_status, unsigned long long limit_ns, cudaStream_t st);
int gemm_tile_m();
int gemm_tile_n();

struct Ctx;
}  // namespace cf
