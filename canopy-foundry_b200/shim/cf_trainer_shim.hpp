// Same-named replacements for the FILE-STATIC FP8 helpers of the reference's src/trainer.cu, so that its
// ~70 call sites compile unchanged once the originals are removed:
//   lt_gemm_fp8_nt            src/trainer.cu:4498-4534   (cublasLtMatmul, bf16 out)
//   lt_gemm_fp8_tn_accum_f32  src/trainer.cu:4596-4625, :4670-4691 (fp32 and bf16 accumulators)
//   fp8_quant_act             src/trainer.cu:4732-4851
//   transpose_u8              src/trainer.cu:1441-1448
// The one structural change on the reference side: Fp8Ctx gains a member `cf_ctx* cf` created next to
// cublasLtCreate in build_fp8_ctx (src/trainer.cu:4205) with cf_ctx_create(&f.cf, act8_bytes), and ActSlot
// gains a `cf_act_slot cfs` whose pointer members alias the slot's existing device scalars (same names).
// Errors surface as std::runtime_error, like CUBLAS_CHECK / IDA_CUDA_CHECK.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <library_types.h>

#include <cstddef>
#include <stdexcept>
#include <string>

#include "canopy_fp8.h"
#include "ida_native/gemm_trace.hpp"

namespace cf_shim {
inline void check(int rc, const char* fn) {
    if (rc != CF_OK) throw std::runtime_error(std::string(fn) + ": " + cf_last_error());
}
// The context the ida_native:: operators without a context parameter (moe_grouped_expert_forward_fp8) use on this
// thread. The trainer owns it: cf_ctx_create + cf_ctx_reserve_workspace in build_fp8_ctx, set_thread_context on every
// training-body thread that shares it (the reference runs one body per thread, include/ida_native/kernels.hpp:599-604),
// set_thread_context(nullptr) and cf_ctx_destroy at teardown. The shim never creates, grows or frees a context.
inline cf_ctx*& thread_context_slot() {
    thread_local cf_ctx* ctx = nullptr;
    return ctx;
}
inline void set_thread_context(cf_ctx* ctx) { thread_context_slot() = ctx; }
inline cf_ctx* thread_context() { return thread_context_slot(); }
}  // namespace cf_shim

template <class Fp8CtxT>
static void lt_gemm_fp8_nt(Fp8CtxT& f, int M, int N, int K, const void* A, int lda, cudaDataType_t a_type,
                           const float* a_descale, const void* B, const float* b_descale, __nv_bfloat16* C, int ldc,
                           cudaStream_t s) {
    ::ida_native::gemm_trace::record_current(static_cast<long long>(M), static_cast<long long>(N), static_cast<long long>(K));   // :4506
    cf_shim::check(cf_gemm_fp8_nt(f.cf, M, N, K, A, lda, a_type == CUDA_R_8F_E5M2 ? 1 : 0, a_descale, B, b_descale, C, ldc,
                                  nullptr, s), "lt_gemm_fp8_nt");
}

template <class Fp8CtxT>
static void lt_gemm_fp8_tn_accum_f32(Fp8CtxT& f, int M, int N, int K, const void* Xt_e4m3, const float* ds_x,
                                     const void* dYt_e5m2, const float* ds_dy, float* dW, int ldc_dw, cudaStream_t s) {
    ::ida_native::gemm_trace::record_current(static_cast<long long>(M), static_cast<long long>(N), static_cast<long long>(K));   // :4606
    cf_shim::check(cf_gemm_fp8_tn_accum_f32(f.cf, M, N, K, Xt_e4m3, ds_x, dYt_e5m2, ds_dy, dW, ldc_dw, s),
                   "lt_gemm_fp8_tn_accum_f32");
}

template <class Fp8CtxT>
static void lt_gemm_fp8_tn_accum_f32(Fp8CtxT& f, int M, int N, int K, const void* Xt_e4m3, const float* ds_x,
                                     const void* dYt_e5m2, const float* ds_dy, __nv_bfloat16* dW, int ldc_dw,
                                     cudaStream_t s) {
    ::ida_native::gemm_trace::record_current(static_cast<long long>(M), static_cast<long long>(N), static_cast<long long>(K));   // :4678
    cf_shim::check(cf_gemm_fp8_tn_accum_bf16(f.cf, M, N, K, Xt_e4m3, ds_x, dYt_e5m2, ds_dy, dW, ldc_dw, s),
                   "lt_gemm_fp8_tn_accum_f32(bf16)");
}

template <class Fp8CtxT, class ActSlotT>
static void fp8_quant_act(Fp8CtxT& f, ActSlotT& slot, const __nv_bfloat16* x, std::size_t n, cudaStream_t s,
                          bool is_recompute = false) {
    // host-side state (fp8_max, init, calibration counters) lives in slot.cfs and is mirrored back
    cf_shim::check(cf_fp8_quant_act(f.cf, &slot.cfs, x, n, f.act8, s, is_recompute ? 1 : 0), "fp8_quant_act");
    slot.fp8_max = slot.cfs.fp8_max;
    slot.init = slot.cfs.init != 0;
    slot.calib_remaining = slot.cfs.calib_remaining;
    slot.calib_commit_pending = slot.cfs.calib_commit_pending != 0;
}

static inline void transpose_u8(const void* in, void* out, int rows, int cols, cudaStream_t s) {
    cf_shim::check(cf_transpose_u8(in, out, rows, cols, s), "transpose_u8");
}
