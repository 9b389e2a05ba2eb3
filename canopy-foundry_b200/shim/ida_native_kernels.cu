// Drop-in definitions of the reference's operator symbols (namespace ida_native, declared in
// include/ida_native/kernels.hpp) for the FP8 / MoE hot path. Each function forwards to the C ABI of
// libcanopy_fp8.so and converts a non-zero status into the std::runtime_error the reference's callers
// expect (IDA_CUDA_CHECK convention, include/ida_native/cuda_check.hpp:10-18).
//
// Integration: compile this file INSTEAD of the FP8 half of kernels/fp8.cu and the dispatch / grouped part
// of kernels/moe.cu, with the reference's include directories on the path, and link libcanopy_fp8.so.
// Signatures, default arguments and argument meaning are the reference's; nothing in trainer.cu changes
// for these calls.
#include "ida_native/kernels.hpp"
#include "ida_native/pack_trace.hpp"

#include <stdexcept>
#include <string>

#include "canopy_fp8.h"
#include "cf_trainer_shim.hpp"

namespace {
inline void cf_check(int rc, const char* fn) {
    if (rc != CF_OK) throw std::runtime_error(std::string(fn) + ": " + cf_last_error());
}
// Operators whose reference signature has no context parameter but whose tensor-core implementation needs one
// (status word, workspace) use the context the integrator registered for the calling thread with
// cf_shim::set_thread_context (cf_trainer_shim.hpp): created once at set-up next to the trainer's own Fp8Ctx, with its
// workspace reserved there, and destroyed by its owner. Nothing on the call path allocates.
cf_ctx* thread_ctx(const char* fn) {
    cf_ctx* ctx = cf_shim::thread_context();
    if (!ctx)
        throw std::runtime_error(std::string(fn) + ": no cf_ctx registered for this thread (call cf_shim::set_thread_context "
                                                   "at set-up, after cf_ctx_create and cf_ctx_reserve_workspace)");
    return ctx;
}
}  // namespace

namespace ida_native {

// kernels/fp8.cu:250-330, 396-417
void fp8_amax_bf16(const __nv_bfloat16* d_x, std::size_t n, float* d_amax, cudaStream_t s) {
    cf_check(cf_fp8_amax_bf16(d_x, n, d_amax, s), "fp8_amax_bf16");
}
void fp8_scale_from_amax(const float* d_amax, float fp8_max, float* d_scale, float* d_descale, cudaStream_t s) {
    cf_check(cf_fp8_scale_from_amax(d_amax, fp8_max, d_scale, d_descale, s), "fp8_scale_from_amax");
}
void fp8_quantize_e4m3(const __nv_bfloat16* d_x, void* d_out, const float* d_scale, std::size_t n, cudaStream_t s) {
    pack_trace::record(pack_trace::K_FP8_PACK, n, n * sizeof(__nv_bfloat16), n);      // kernels/fp8.cu:264-266
    cf_check(cf_fp8_quantize_e4m3(d_x, d_out, d_scale, n, s), "fp8_quantize_e4m3");
}
void fp8_quantize_e5m2(const __nv_bfloat16* d_x, void* d_out, const float* d_scale, std::size_t n, cudaStream_t s) {
    pack_trace::record(pack_trace::K_FP8_PACK, n, n * sizeof(__nv_bfloat16), n);      // kernels/fp8.cu:274-276
    cf_check(cf_fp8_quantize_e5m2(d_x, d_out, d_scale, n, s), "fp8_quantize_e5m2");
}
void fp8_quantize_transpose_e4m3(const __nv_bfloat16* d_w, void* d_out, const float* d_scale, int K, int N, cudaStream_t s) {
    const std::size_t elements = static_cast<std::size_t>(K) * N;
    pack_trace::record(pack_trace::K_FP8_PACK_TRANSPOSE, elements, elements * sizeof(__nv_bfloat16), elements);   // :285-287
    cf_check(cf_fp8_quantize_transpose_e4m3(d_w, d_out, d_scale, K, N, s), "fp8_quantize_transpose_e4m3");
}
void fp8_quant_and_transpose_e4m3(const __nv_bfloat16* d_in, void* d_act8_out, void* d_snap_out, const float* d_scale,
                                  int K, int N, cudaStream_t s) {
    const std::size_t elements = static_cast<std::size_t>(K) * N;
    pack_trace::record(pack_trace::K_FP8_PACK_FUSED_TRANSPOSE, elements, elements * sizeof(__nv_bfloat16), 2 * elements);   // :297-299
    cf_check(cf_fp8_quant_and_transpose_e4m3(d_in, d_act8_out, d_snap_out, d_scale, K, N, s), "fp8_quant_and_transpose_e4m3");
}
void fp8_quantize_e4m3_record(const __nv_bfloat16* d_x, void* d_out, const float* d_scale, float* d_amax, std::size_t n,
                              cudaStream_t s) {
    pack_trace::record(pack_trace::K_FP8_PACK, n, n * sizeof(__nv_bfloat16), n);      // kernels/fp8.cu:314-316
    cf_check(cf_fp8_quantize_e4m3_record(d_x, d_out, d_scale, d_amax, n, s), "fp8_quantize_e4m3_record");
}
void fp8_quantize_e5m2_record(const __nv_bfloat16* d_x, void* d_out, const float* d_scale, float* d_amax, std::size_t n,
                              cudaStream_t s) {
    pack_trace::record(pack_trace::K_FP8_PACK, n, n * sizeof(__nv_bfloat16), n);      // kernels/fp8.cu:325-327
    cf_check(cf_fp8_quantize_e5m2_record(d_x, d_out, d_scale, d_amax, n, s), "fp8_quantize_e5m2_record");
}
void fp8_clip_probe(const float* d_amax, const float* d_scale, float fp8_max, float* d_stats, cudaStream_t s) {
    cf_check(cf_fp8_clip_probe(d_amax, d_scale, fp8_max, d_stats, s), "fp8_clip_probe");
}
void fp8_elem_clip_count(const __nv_bfloat16* d_x, const float* d_scale, float fp8_max, std::size_t n, float* d_out,
                         cudaStream_t s) {
    cf_check(cf_fp8_elem_clip_count(d_x, d_scale, fp8_max, n, d_out, s), "fp8_elem_clip_count");
}
void fp8_update_delayed_scale(const float* d_amax, float fp8_max, float* d_scale, float* d_descale, float* d_history,
                              int history_len, int* d_history_cursor, int* d_history_count, cudaStream_t s) {
    cf_check(cf_fp8_update_delayed_scale(d_amax, fp8_max, d_scale, d_descale, d_history, history_len, d_history_cursor,
                                         d_history_count, s), "fp8_update_delayed_scale");
}
// kernels/fp8.cu:491-528
void fp8_pack_bf16_e4m3_raw(const __nv_bfloat16* d_x, std::uint8_t* d_out, float* d_amax, float* d_scale, float* d_descale,
                            int* d_bad_count, std::size_t n, cudaStream_t s) {
    pack_trace::record(pack_trace::K_FP8_PACK, n, n * sizeof(__nv_bfloat16), n);      // kernels/fp8.cu:502
    cf_check(cf_fp8_pack_bf16_e4m3_raw(d_x, d_out, d_amax, d_scale, d_descale, d_bad_count, n, s), "fp8_pack_bf16_e4m3_raw");
}
void fp8_pack_bf16_e4m3_raw_and_dequant(const __nv_bfloat16* d_x, std::uint8_t* d_out, __nv_bfloat16* d_dequant,
                                        float* d_amax, float* d_scale, float* d_descale, int* d_bad_count, std::size_t n,
                                        cudaStream_t s) {
    pack_trace::record(pack_trace::K_FP8_PACK_DEQUANT, n, n * sizeof(__nv_bfloat16),
                       n * sizeof(std::uint8_t) + n * sizeof(__nv_bfloat16));          // kernels/fp8.cu:517-520
    cf_check(cf_fp8_pack_bf16_e4m3_raw_and_dequant(d_x, d_out, d_dequant, d_amax, d_scale, d_descale, d_bad_count, n, s),
             "fp8_pack_bf16_e4m3_raw_and_dequant");
}
void fp8_unpack_e4m3_raw_bf16(const std::uint8_t* d_in, const float* d_descale, __nv_bfloat16* d_out, std::size_t n,
                              cudaStream_t s) {
    cf_check(cf_fp8_unpack_e4m3_raw_bf16(d_in, d_descale, d_out, n, s), "fp8_unpack_e4m3_raw_bf16");
}

// kernels/lion.cu:121-144
void lion_step(__nv_bfloat16* d_w, float* d_m, const float* d_grad, std::size_t n, float lr, float beta1, float beta2,
               float wd, cudaStream_t stream, float* d_weight_amax, unsigned sr_seed) {
    cf_check(cf_lion_step_f32_state(d_w, d_m, d_grad, n, lr, beta1, beta2, wd, stream, d_weight_amax, sr_seed), "lion_step");
}
void lion_step(__nv_bfloat16* d_w, __nv_bfloat16* d_m, const float* d_grad, std::size_t n, float lr, float beta1,
               float beta2, float wd, cudaStream_t stream, float* d_weight_amax, unsigned sr_seed) {
    cf_check(cf_lion_step_bf16_state(d_w, d_m, d_grad, n, lr, beta1, beta2, wd, stream, d_weight_amax, sr_seed), "lion_step");
}

// kernels/rmsnorm.cu:101-108 (the forward only: rmsnorm_backward stays in the reference's translation unit)
void rmsnorm_forward(const __nv_bfloat16* d_x, const __nv_bfloat16* d_scale, __nv_bfloat16* d_out, float* d_rms, int rows, int H,
                     float eps, cudaStream_t stream) {
    cf_check(cf_rmsnorm_forward(d_x, d_scale, d_out, d_rms, rows, H, eps, stream), "rmsnorm_forward");
}

// kernels/activations.cu:76-87; kernels/moe.cu:338-345, 519-521
void swiglu_forward(const __nv_bfloat16* d_gate, const __nv_bfloat16* d_up, __nv_bfloat16* d_out, int N, cudaStream_t stream) {
    const int rc = cf_swiglu_forward(d_gate, d_up, d_out, N, stream);
    if (rc == CF_ERR_INVALID_ARG) throw std::invalid_argument(cf_last_error());   // activations.cu:61-72
    cf_check(rc, "swiglu_forward");
}
void gelu_forward(const __nv_bfloat16* d_x, __nv_bfloat16* d_out, std::size_t n, cudaStream_t stream) {
    cf_check(cf_gelu_forward(d_x, d_out, n, stream), "gelu_forward");
}
void bias_add_strided_bf16(__nv_bfloat16* d_inout, const __nv_bfloat16* d_bias, int rows, int cols, int row_stride,
                           int base, cudaStream_t stream) {
    cf_check(cf_bias_add_strided_bf16(d_inout, d_bias, rows, cols, row_stride, base, stream), "bias_add_strided_bf16");
}

// kernels/moe.cu:410-422, 677-738, 859-863, 1062-1127
void moe_topk_route_f32(float* d_scores, int rows, int num_experts, int top_k, cudaStream_t stream, float* d_row_sum_save,
                        float* d_scores_save, bool normalize_topk) {
    cf_check(cf_moe_topk_route_f32(d_scores, rows, num_experts, top_k, stream, d_row_sum_save, d_scores_save,
                                   normalize_topk ? 1 : 0), "moe_topk_route_f32");
}
void moe_scale_accumulate_bf16(__nv_bfloat16* d_mixed, const __nv_bfloat16* d_term, const float* d_route_weights, int rows,
                               int expert_idx, int num_experts, int H, cudaStream_t stream) {
    cf_check(cf_moe_scale_accumulate_bf16(d_mixed, d_term, d_route_weights, rows, expert_idx, num_experts, H, stream),
             "moe_scale_accumulate_bf16");
}
void moe_build_expert_row_lists(const float* d_route_weights, int* d_counts, int* d_row_indices, int rows, int num_experts,
                                cudaStream_t stream) {
    cf_check(cf_moe_build_expert_row_lists(d_route_weights, d_counts, d_row_indices, rows, num_experts, stream),
             "moe_build_expert_row_lists");
}
void moe_gather_rows_bf16(const __nv_bfloat16* d_src, __nv_bfloat16* d_dst, const int* d_row_indices, int n_rows, int width,
                          cudaStream_t stream) {
    cf_check(cf_moe_gather_rows_bf16(d_src, d_dst, d_row_indices, n_rows, width, stream), "moe_gather_rows_bf16");
}
void moe_gather_rows_u8(const std::uint8_t* d_src, std::uint8_t* d_dst, const int* d_row_indices, int n_rows, int width,
                        cudaStream_t stream) {
    cf_check(cf_moe_gather_rows_u8(d_src, d_dst, d_row_indices, n_rows, width, stream), "moe_gather_rows_u8");
}
void moe_scatter_accumulate_rows_bf16(__nv_bfloat16* d_mixed, const __nv_bfloat16* d_compact, const float* d_route_weights,
                                      const int* d_row_indices, int n_rows, int expert_idx, int num_experts, int H,
                                      cudaStream_t stream) {
    cf_check(cf_moe_scatter_accumulate_rows_bf16(d_mixed, d_compact, d_route_weights, d_row_indices, n_rows, expert_idx,
                                                 num_experts, H, stream), "moe_scatter_accumulate_rows_bf16");
}
void moe_expert_offsets_from_counts(const int* d_counts, int* d_offsets, int num_experts, cudaStream_t stream) {
    cf_check(cf_moe_expert_offsets_from_counts(d_counts, d_offsets, num_experts, stream), "moe_expert_offsets_from_counts");
}
void moe_grouped_expert_forward_fp8(const void* d_hidden, const float* d_fcin_descale, int fcin_is_e5m2,
                                    const float* d_route_weights, const int* d_counts, const int* d_offsets,
                                    const int* d_row_indices, const void* d_fc_in_w, const float* d_fc_in_descale,
                                    const void* d_fc_out_w, const float* d_fc_out_descale, __nv_bfloat16* d_mixed, int rows,
                                    int H, int Ie, int num_experts, int total_selected_rows, cudaStream_t stream) {
    // The tensor-core form needs total_selected_rows * (3 H + 4 Ie) + 4 KiB of workspace from the registered context;
    // with less reserved the call fails with CF_ERR_LIMIT (surfaced as std::runtime_error) instead of allocating.
    cf_ctx* ctx = thread_ctx("moe_grouped_expert_forward_fp8");
    cf_check(cf_moe_grouped_expert_forward_fp8(ctx, d_hidden, d_fcin_descale, fcin_is_e5m2, d_route_weights, d_counts,
                                               d_offsets, d_row_indices, d_fc_in_w, d_fc_in_descale, d_fc_out_w,
                                               d_fc_out_descale, d_mixed, rows, H, Ie, num_experts, total_selected_rows,
                                               stream), "moe_grouped_expert_forward_fp8");
}

}  // namespace ida_native
