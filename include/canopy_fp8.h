/*
 * canopy_fp8.h — C ABI of libcanopy_fp8.so, the sm_100a implementation of
 * Canopy-Foundry's FP8 quantize-and-GEMM hot path.
 *
 * Conventions (they follow the reference's operator layer, include/ida_native/kernels.hpp):
 *   - every pointer named d_* is a DEVICE pointer; scalars such as scales, amax and ring
 *     cursors live on the device and are read at kernel time;
 *   - `stream` is a cudaStream_t passed as void*; all work is stream-ordered, no entry
 *     point synchronises the host unless its comment says so;
 *   - operators allocate nothing: buffers come from the caller, workspace from a cf_ctx;
 *   - bf16 tensors are passed as const void* / void* (2-byte elements, __nv_bfloat16 bits),
 *     FP8 tensors as 1-byte codes (E4M3 "fn" or E5M2);
 *   - return value: CF_OK or a CF_ERR_* code; cf_last_error() gives the text for the calling
 *     thread. The reference's functions return void and throw std::runtime_error; the C++
 *     shim (canopy-foundry_b200/shim) converts a non-zero status into that exception.
 *   - the library runs on compute capability 10.x only and has no CPU or library fallback.
 *
 * Each declaration cites the reference interface it replaces (path:line inside the
 * reference project).
 */
#ifndef CANOPY_FP8_H
#define CANOPY_FP8_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    CF_OK = 0,
    CF_ERR_INVALID_ARG = 1,   /* null pointer, negative size, misaligned scale pointer, ... */
    CF_ERR_UNSUPPORTED = 2,   /* shape or device this build cannot serve */
    CF_ERR_CUDA = 3,          /* a CUDA runtime / driver call failed; see cf_last_error() */
    CF_ERR_DEVICE_WAIT = 4,   /* a bounded device-side wait gave up (reported by cf_ctx_poll_status) */
    CF_ERR_LIMIT = 5,         /* size beyond a documented fixed limit */
    CF_ERR_DEVICE_RANGE = 6   /* a device-side plan pointed outside a destination buffer; the store was skipped
                                 (reported by cf_ctx_poll_status) */
};

#define CF_E4M3_MAX 448.0f     /* src/trainer.cu:3179 */
#define CF_E5M2_MAX 57344.0f   /* src/trainer.cu:3212 */

const char* cf_last_error(void);
/* ABI version of this header; bumped when a signature changes. */
int cf_abi_version(void);

/* ------------------------------------------------------------------ quantize / cast */

/* kernels/fp8.cu:250-253, include/ida_native/kernels.hpp:983.
 * *d_amax = max |x[i]| over n bf16 values (NaN ignored, +Inf propagates). Zeroes d_amax itself. */
int cf_fp8_amax_bf16(const void* d_x, size_t n, float* d_amax, void* stream);

/* kernels/fp8.cu:255-259, kernels.hpp:1003-1004.
 * a = max(*d_amax, 1e-12); *d_scale = fp8_max / a; *d_descale = a / fp8_max (IEEE divides). */
int cf_fp8_scale_from_amax(const float* d_amax, float fp8_max, float* d_scale, float* d_descale, void* stream);

/* kernels/fp8.cu:261-279, kernels.hpp:1005-1008.
 * out[i] = fp8(float(x[i]) * *d_scale), round-to-nearest-even, saturate to finite. */
int cf_fp8_quantize_e4m3(const void* d_x, void* d_out, const float* d_scale, size_t n, void* stream);
int cf_fp8_quantize_e5m2(const void* d_x, void* d_out, const float* d_scale, size_t n, void* stream);

/* kernels/fp8.cu:310-330, kernels.hpp:1021-1026.
 * As above and, in the same pass, *d_amax = max(*d_amax, max|x|) of the UNSCALED input
 * (integer atomicMax on the float bits; the caller zeroes d_amax first). */
int cf_fp8_quantize_e4m3_record(const void* d_x, void* d_out, const float* d_scale, float* d_amax, size_t n, void* stream);
int cf_fp8_quantize_e5m2_record(const void* d_x, void* d_out, const float* d_scale, float* d_amax, size_t n, void* stream);

/* kernels/fp8.cu:396-417, kernels.hpp:1042-1052.
 * Ring of the last history_len clamped amaxes; scale = fp8_max / max(ring). history_len <= 0
 * behaves like cf_fp8_scale_from_amax. Cursor outside [0,len) restarts at 0. */
int cf_fp8_update_delayed_scale(const float* d_amax, float fp8_max, float* d_scale, float* d_descale,
                                float* d_history, int history_len, int* d_history_cursor,
                                int* d_history_count, void* stream);

/* kernels/fp8.cu:281-290, kernels.hpp:1010-1011.  w[K,N] bf16 -> out[N,K] E4M3. */
int cf_fp8_quantize_transpose_e4m3(const void* d_w, void* d_out, const float* d_scale, int K, int N, void* stream);

/* kernels/fp8.cu:292-308, kernels.hpp:1016-1018.  in[K,N] bf16 -> act8[K,N] and snap[N,K] E4M3.
 * Either output pointer may be NULL to skip that layout (src/trainer.cu:8225-8228 uses snap only). */
int cf_fp8_quant_and_transpose_e4m3(const void* d_in, void* d_act8_out, void* d_snap_out,
                                    const float* d_scale, int K, int N, void* stream);

/* src/trainer.cu:1441-1448 (file-static transpose_u8).  in[rows,cols] bytes -> out[cols,rows]. */
int cf_transpose_u8(const void* d_in, void* d_out, int rows, int cols, void* stream);

/* kernels/fp8.cu:358-363, kernels.hpp:1029-1032.  stats = [clipped_calls, max_ratio, total_calls]. */
int cf_fp8_clip_probe(const float* d_amax, const float* d_scale, float fp8_max, float* d_stats, void* stream);
/* kernels/fp8.cu:389-394, kernels.hpp:1034-1037.  out[0] += clipped elements, out[1] += n. */
int cf_fp8_elem_clip_count(const void* d_x, const float* d_scale, float fp8_max, size_t n, float* d_out, void* stream);

/* kernels/fp8.cu:491-528, kernels.hpp:988-1002: raw-byte E4M3 storage path. Encoder semantics are those
 * of include/ida_native/fp8_e4m3.hpp (non-finite products become sign|0x7f and are counted in d_bad_count). */
int cf_fp8_pack_bf16_e4m3_raw(const void* d_x, uint8_t* d_out, float* d_amax, float* d_scale, float* d_descale,
                              int* d_bad_count, size_t n, void* stream);
int cf_fp8_pack_bf16_e4m3_raw_and_dequant(const void* d_x, uint8_t* d_out, void* d_dequant, float* d_amax,
                                          float* d_scale, float* d_descale, int* d_bad_count, size_t n, void* stream);
int cf_fp8_unpack_e4m3_raw_bf16(const uint8_t* d_in, const float* d_descale, void* d_out, size_t n, void* stream);

/* src/trainer.cu:3789-3795 (k_calib_minmax_update): running min/max of the clamped amax. */
int cf_fp8_calib_minmax_update(const float* d_amax, float* d_calib_min, float* d_calib_max, void* stream);

/* ------------------------------------------------------------------ context */

/* Replaces the reference's Fp8Ctx (src/trainer.cu:3296-3345) as far as this path needs it: it owns the
 * device status word the tensor-core kernels report bounded-wait failures into, the shared act8 scratch
 * and the scalar pool ActSlots are carved from. Created once per device; creation allocates, calls on
 * the hot path do not. act8_bytes may be 0 when cf_fp8_quant_act is not used. */
typedef struct cf_ctx cf_ctx;
int cf_ctx_create(cf_ctx** out, size_t act8_bytes);
int cf_ctx_destroy(cf_ctx* ctx);
/* Device pointer of the shared quantised-activation scratch (Fp8Ctx::act8, src/trainer.cu:3339-3340). */
void* cf_ctx_act8(cf_ctx* ctx);
/* Synchronises `stream`, then returns CF_OK, CF_ERR_DEVICE_WAIT if any kernel launched through this context since
 * the last poll abandoned a bounded wait, or CF_ERR_DEVICE_RANGE if a planned run of rows was refused because it
 * left its destination buffer (the output is invalid in both cases). Clears the word. */
int cf_ctx_poll_status(cf_ctx* ctx, void* stream);
/* Failure-detection self-test (no counterpart in the reference): launches one small kernel whose only wait is on a
 * barrier nothing ever signals; the wait gives up after limit_ms (1..1000), the kernel records a status code and
 * returns normally, and the next cf_ctx_poll_status reports CF_ERR_DEVICE_WAIT. Nothing faults or hangs; the context
 * stays usable. It checks the path a starved tensor-core pipeline would take. */
int cf_ctx_selftest_bounded_wait(cf_ctx* ctx, int limit_ms, void* stream);
/* Number of kernels this library launched through any entry point since load (process-wide counter). */
uint64_t cf_launch_count(void);

/* ------------------------------------------------------------------ FP8 GEMM */

/* Epilogue description shared by the GEMM entry points. Zero-initialise for the reference behaviour. */
typedef struct cf_gemm_epilogue {
    const void* d_bias;          /* bf16[N] or NULL */
    int bias_mode;               /* 0 none; 1 add in fp32 before the single bf16 rounding (fused);
                                    2 reference order: round to bf16, then bf16(float(c)+float(bias))
                                      as kernels/moe.cu:325-336 does after the GEMM */
    const float* d_a_row_descale; /* NULL, or float[M]: per-row (per-token) scales replace *d_a_descale */
    const float* d_b_col_descale; /* NULL, or float[N]: per-output-channel scales replace *d_b_descale */
    int out_fp32;                /* 0: C is bf16 (the reference's output type); 1: C is float[M, ldc] and no bias is
                                    applied — the partial product of a K-sharded (row-parallel) GEMM, to be summed
                                    across ranks in fp32 */
} cf_gemm_epilogue;

/* src/trainer.cu:4498-4534 (file-static lt_gemm_fp8_nt, the cuBLASLt call).
 * C[M,N] bf16 (row stride ldc) = (*d_a_descale * *d_b_descale) * sum_k A8[m,k] * B8[n,k], fp32 accumulate.
 * A8: row-major [M,K], row stride lda bytes, E4M3 (a_is_e5m2 = 0) or E5M2 (1).
 * B8: row-major [N,K] contiguous, E4M3.   epi may be NULL. */
int cf_gemm_fp8_nt(cf_ctx* ctx, int M, int N, int K, const void* d_A, int lda, int a_is_e5m2,
                   const float* d_a_descale, const void* d_B, const float* d_b_descale, void* d_C, int ldc,
                   const cf_gemm_epilogue* epi, void* stream);

/* No counterpart in the reference (it runs on one GPU). Row-parallel (K-sharded) form of lt_gemm_fp8_nt with the
 * reduce-scatter fused into the epilogue: this rank multiplies its K slice, A8[M, K_local] . B8[N, K_local]^T, and ADDS
 * rows [r * M/num_slices, (r + 1) * M/num_slices) of the scaled fp32 product into slices[r], rank r's fp32
 * [M/num_slices, N] accumulation slice as mapped in this process (symmetric / peer-mapped memory for r != own rank).
 * The tiles leave the SM as bulk reduce-add copies (whole 128-byte lines, one fp32 addition per element at the
 * destination), so the transfer over NVLink overlaps the main loop tile by tile. `slices` is a HOST array of
 * num_slices (1..16) device pointers, 16-byte aligned. The caller zeroes its own slice beforehand and orders the
 * readers behind every rank's launch (a barrier after the call). Needs M/num_slices % 256 == 0, N % 32 == 0,
 * 16-byte aligned operands, K % 16 == 0. Scales: per tensor, or per row of A (float[M]) and / or per output column
 * (float[N], 16-byte aligned) when those pointers are given; ranks that share one set of row / column scales sum
 * products that are already scaled. The context keeps the tensor maps of the last four slice sets on the device; calls
 * that share a context must be on one stream. */
int cf_gemm_fp8_nt_reduce_scatter_f32(cf_ctx* ctx, int M, int N, int K, const void* d_A, int lda, int a_is_e5m2,
                                      const float* d_a_descale, const void* d_B, const float* d_b_descale,
                                      const float* d_a_row_descale_or_null, const float* d_b_col_descale_or_null,
                                      void* const* slices, int num_slices, void* stream);
/* Finishes a reduce-scatter: out[i] = bf16(acc[i]) and acc[i] = 0 (ready for the next accumulation). */
int cf_f32_to_bf16_and_zero(float* d_acc, void* d_out, size_t n, void* stream);

/* src/trainer.cu:4596-4625 and :4670-4691 (lt_gemm_fp8_tn_accum_f32, fp32 and bf16 accumulators).
 * dW[M,N] += (*d_ds_x * *d_ds_dy) * sum_k Xt[m,k] * dYt[n,k]; Xt E4M3 [M,K], dYt E5M2 [N,K], both
 * contiguous with leading dimension K. */
int cf_gemm_fp8_tn_accum_f32(cf_ctx* ctx, int M, int N, int K, const void* d_Xt_e4m3, const float* d_ds_x,
                             const void* d_dYt_e5m2, const float* d_ds_dy, float* d_dW, int ldc, void* stream);
int cf_gemm_fp8_tn_accum_bf16(cf_ctx* ctx, int M, int N, int K, const void* d_Xt_e4m3, const float* d_ds_x,
                              const void* d_dYt_e5m2, const float* d_ds_dy, void* d_dW, int ldc, void* stream);

/* The weight-gradient GEMM of src/trainer.cu:8269-8317 without its two byte transposes: the reference transposes the
 * activation snapshot and the gradient (transpose_u8 / the dual quantise kernel) so that cuBLASLt can run the TN form;
 * here the tensor cores read both operands as they lie in memory,
 *   dW[M,N] += (*d_ds_x * *d_ds_dy) * sum_k X8[k,m] * dY8[k,n],
 * X8 E4M3 [K, M] with row pitch ldx, dY8 E5M2 [K, N] with row pitch ldy (K = tokens), dW fp32 or bf16 with pitch ldc.
 * Needs 16-byte aligned bases and pitches and the CTA-pair form (CF_ERR_UNSUPPORTED otherwise: use the transposes and
 * cf_gemm_fp8_tn_accum_*). No counterpart in the reference. */
int cf_gemm_fp8_dw_accum_f32(cf_ctx* ctx, int M, int N, int K, const void* d_X_e4m3, int ldx, const float* d_ds_x,
                             const void* d_dY_e5m2, int ldy, const float* d_ds_dy, float* d_dW, int ldc, void* stream);
int cf_gemm_fp8_dw_accum_bf16(cf_ctx* ctx, int M, int N, int K, const void* d_X_e4m3, int ldx, const float* d_ds_x,
                              const void* d_dY_e5m2, int ldy, const float* d_ds_dy, void* d_dW, int ldc, void* stream);

/* The data-gradient direction of the FP8 linear, dX[M,N] = dY[M,K] . W[K,N], reading the weight from the FORWARD cache
 * as it lies ([out, in] = [K, N] row-major with pitch ldb): the tensor cores take B as an MN-major operand, so the second,
 * transposed weight cache of src/trainer.cu:3284-3294 (bwd8) and the transposed quantise that fills it (kernels/fp8.cu:
 * 281-290) are not needed for src/trainer.cu:8282-8314. A is E5M2 (a_is_e5m2 = 1, the gradient) or E4M3, [M, K] with row
 * pitch lda; C is bf16 [M, N] with pitch ldc, stored (accumulate = 0) or added to in fp32 with one rounding
 * (accumulate = 1, the beta = 1 calls of the reference). Results equal cf_gemm_fp8_nt on the transposed weight.
 * Needs 16-byte aligned bases and pitches, K % 16 == 0, N % 16 == 0, the CTA-pair form. */
int cf_gemm_fp8_nn(cf_ctx* ctx, int M, int N, int K, const void* d_A, int lda, int a_is_e5m2, const float* d_a_descale,
                   const void* d_B_kn, int ldb, const float* d_b_descale, void* d_C, int ldc, int accumulate, void* stream);
/* The same for ragged expert groups: group g multiplies compact rows [d_offsets[g], +d_counts[g]) of A with block g of
 * the stacked forward cache [num_groups, K, N] (contiguous blocks). This is the dgrad of the MoE expert bank that
 * src/trainer.cu:7829-7856 leaves in bf16 because the reference's transposed cache of a multi-expert block is not
 * per-expert-correct: here no transposed cache exists, every expert's own [K, N] block is read in place. K % 128 == 0. */
int cf_gemm_fp8_nn_grouped(cf_ctx* ctx, int num_groups, int max_total_rows, int N, int K, const int* d_counts,
                           const int* d_offsets, const void* d_A, int lda, int a_is_e5m2, const float* d_a_descale,
                           const void* d_B_stacked_kn, const float* d_b_descale, void* d_C, int ldc, int accumulate,
                           void* stream);

/* The ragged per-expert GEMMs of src/trainer.cu:6893-6927 as ONE launch with a device-side schedule:
 * for every expert e, rows [d_offsets[e], d_offsets[e]+d_counts[e]) of the compact A8 [total_rows,K]
 * are multiplied with B8[e] ([N,K] slice of a [E,N,K] block) into the same rows of compact C [.,ldc].
 * No host synchronisation; max_total_rows bounds sum(counts) (tile budget only). d_a_descale / d_b_descale
 * are one per-tensor scalar each unless per_expert_a_descale != 0, in which case d_a_descale is float[E]. */
int cf_gemm_fp8_nt_grouped(cf_ctx* ctx, int num_experts, int max_total_rows, int N, int K, const int* d_counts,
                           const int* d_offsets, const void* d_A, int lda, int a_is_e5m2, const float* d_a_descale,
                           int per_expert_a_descale, const void* d_B, const float* d_b_descale, void* d_C, int ldc,
                           void* stream);

/* The same launch over arbitrary row segments: segment g multiplies rows [d_offsets[g], +d_counts[g]) with weight block
 * d_segment_weight[g] (0 <= index < num_weights; NULL = g) of the stacked [num_weights, N, K] tensor, optionally with
 * its own activation descale (per_segment_a_descale: d_a_descale is float[num_segments]). Expert parallelism uses it:
 * rows received from different ranks for the same local expert are separate segments with that rank's scale. No
 * counterpart in the reference (it has no expert parallelism, include/ida_native/arena.hpp:24-26). */
int cf_gemm_fp8_nt_segments(cf_ctx* ctx, int num_segments, int num_weights, const int* d_segment_weight,
                            int max_total_rows, int N, int K, const int* d_counts, const int* d_offsets, const void* d_A,
                            int lda, int a_is_e5m2, const float* d_a_descale, int per_segment_a_descale, const void* d_B,
                            const float* d_b_descale, void* d_C, int ldc, void* stream);

/* GEMM fused with the return leg of an expert-parallel exchange: like cf_gemm_fp8_nt_segments, but the rows of segment g
 * are written to d_segment_out[g] (a device array of 16-byte aligned bf16 base pointers, row stride ldc) starting at
 * row d_segment_out_row0[g] of that buffer. The bases may be peer-GPU buffers mapped into this process (NVLink P2P
 * stores from the epilogue), which replaces the all-to-all that would otherwise carry the expert outputs back to the
 * ranks that own the tokens; the caller orders the consumers behind the kernel with its own cross-rank barrier.
 * d_C is unused when d_segment_out is given. No counterpart in the reference. */
int cf_gemm_fp8_nt_segments_scatter(cf_ctx* ctx, int num_segments, int num_weights, const int* d_segment_weight,
                                    int max_total_rows, int N, int K, const int* d_counts, const int* d_offsets,
                                    const void* d_A, int lda, int a_is_e5m2, const float* d_a_descale,
                                    int per_segment_a_descale, const void* d_B, const float* d_b_descale, void* d_C,
                                    void* const* d_segment_out, const long long* d_segment_out_row0, int ldc,
                                    void* stream);

/* ------------------------------------------------------------------ delayed-scaling slot + fused linear */

/* Mirror of ActSlot (src/trainer.cu:3248-3279). All pointer members are device scalars; cf_act_slot_init
 * carves them from the context's scalar pool (16-byte aligned, src/trainer.cu:4239-4242). */
typedef struct cf_act_slot {
    float* amax;
    float* scale;
    float* descale;
    float* history;          /* float[8] (kActHistoryLen, src/trainer.cu:3213) */
    int* history_cursor;
    int* history_count;
    float* scale_snapshot;
    float* descale_snapshot;
    float fp8_max;           /* CF_E4M3_MAX or CF_E5M2_MAX */
    int init;
    int calib_remaining;
    int calib_commit_pending;
    float* calib_min;
    float* calib_max;
    unsigned* ticket;        /* optional pair of zero-initialised device words, 8 bytes (not in the reference's ActSlot):
                                when set, a steady-state cf_fp8_quant_act is ONE launch (snapshot, record-quantise and
                                ring update fused); NULL = the reference's sequence of small launches */
} cf_act_slot;

int cf_act_slot_init(cf_ctx* ctx, cf_act_slot* slot, float fp8_max, int calib_calls, void* stream);

/* src/trainer.cu:4732-4851 (file-static fp8_quant_act): quantise x into d_out8 (the reference always
 * writes Fp8Ctx::act8; pass cf_ctx_act8(ctx) for that) following the slot's state machine — recompute,
 * calibration, first use, steady state (snapshot, record-quantise, ring update). A pending calibration
 * commit synchronises the stream and reads two floats back, exactly like the reference (:4750-4752). */
int cf_fp8_quant_act(cf_ctx* ctx, cf_act_slot* slot, const void* d_x, size_t n, void* d_out8, void* stream,
                     int is_recompute);

/* swiglu_forward (src/trainer.cu:6322) followed by fp8_quant_act on its output (:7138-7140) as one pass over gate and
 * up: the bf16 SwiGLU product is rounded exactly as swiglu_forward would write it, quantised with the slot's
 * delayed scale, its amax recorded and the ring advanced. E4M3 slots without calibration; the first call takes an
 * exact amax first. gate/up are [rows, cols] views with row stride ld_in; d_out8 is [rows, cols] contiguous. */
int cf_fp8_swiglu_quant_act(cf_ctx* ctx, cf_act_slot* slot, const void* d_gate, const void* d_up, int ld_in, int rows,
                            int cols, void* d_out8, void* stream);

/* Gate and up projection, SwiGLU and the re-quantisation that feeds the down projection in ONE GEMM launch: the
 * epilogue turns each (gate, up) accumulator pair into bf16(silu(bf16 gate) * bf16 up), quantises it with the slot's
 * delayed scale and records its amax, so the [rows, 2F] bf16 intermediate of src/trainer.cu:6304-6322 and :7138-7140
 * never exists in HBM. Rounding points are those of the unfused sequence (bit-identical output). The weight is the
 * stacked [num_weights, 2F, K] E4M3 tensor with gate and up rows interleaved in groups of 32 (cf_fp8_interleave_gate_up);
 * d_h8 is E4M3 [rows, F] with row pitch ldh bytes (16-byte aligned). Dense form: d_counts = d_offsets = NULL,
 * num_segments = 1, max_total_rows = M. Segment form: as cf_gemm_fp8_nt_segments. per_segment_a_descale: 0 = one
 * descale, 1 = d_a_descale[segment], 2 = d_a_descale[row] (one float per row of A). The first call on a fresh slot
 * runs the GEMM twice (exact amax first). The reference's row clip of the SwiGLU output (act_row_clip,
 * src/trainer.cu:7138, L2 norm of a whole row against a fixed ceiling, 1000 by default) is NOT applied: a row norm
 * spans every column tile; results equal the reference's whenever no row exceeds that ceiling. */
int cf_gemm_fp8_swiglu_quant_act(cf_ctx* ctx, cf_act_slot* slot, int num_segments, int num_weights,
                                 const int* d_segment_weight, int max_total_rows, int F, int K, const int* d_counts,
                                 const int* d_offsets, const void* d_A, int lda, int a_is_e5m2, const float* d_a_descale,
                                 int per_segment_a_descale, const void* d_W_interleaved, const float* d_w_descale,
                                 void* d_h8, int ldh, void* stream);
/* The per-token form of the same fusion (no counterpart in the reference, which scales per tensor): gate and up
 * projection and SwiGLU in one GEMM launch, output h = bf16(silu(bf16 gate) * bf16 up) as bf16 [M, F] (row pitch ldh
 * elements, ldh % 8 == 0, 16-byte aligned) together with max|h| of every row accumulated into d_row_amax[M] (integer
 * atomicMax on the float bits; the caller zeroes it). cf_fp8_quantize_rowwise_given_amax_e4m3 then quantises h in one
 * read: the [M, 2F] bf16 gate/up intermediate of the unfused sequence never reaches HBM, and the rows, their amax and
 * the codes equal those of cf_gemm_fp8_nt + cf_swiglu_quantize_rowwise_e4m3 bit for bit. When the F dimension is
 * sharded over ranks, max-reduce d_row_amax across them before quantising. Scales: *d_a_descale or one per row
 * (d_a_row_descale, float[M]); *d_w_descale or one per interleaved weight row (float[2F] in the same 32-row
 * interleaved order as the weight, 16-byte aligned). Dense rows only. */
int cf_gemm_fp8_swiglu_bf16_rowamax(cf_ctx* ctx, int M, int F, int K, const void* d_A, int lda, int a_is_e5m2,
                                    const float* d_a_descale, const float* d_a_row_descale_or_null,
                                    const void* d_W_interleaved, const float* d_w_descale,
                                    const float* d_w_col_descale_interleaved_or_null, void* d_h, int ldh, float* d_row_amax,
                                    void* stream);
/* out[e, (f/32)*64 + f%32, :] = gate[e, f, :], out[e, (f/32)*64 + 32 + f%32, :] = up[e, f, :]; F % 32 == 0, K % 16 == 0. */
int cf_fp8_interleave_gate_up(const void* d_gate8, const void* d_up8, void* d_out8, int num_experts, int F, int K, void* stream);

/* One FP8-cached weight (Fp8Slot, src/trainer.cu:3284-3294) and its refresh (:4694-4712): [amax] -> scale ->
 * quantise into the native layout cache -> quantise-transpose into the other one. */
typedef struct cf_fp8_weight {
    const void* w;      /* bf16 master */
    void* fwd8;         /* [out,in] E4M3 */
    void* bwd8;         /* [in,out] E4M3 */
    float* amax;
    float* scale;
    float* descale;
    int in_dim;
    int out_dim;
    int stored_out_major;
} cf_fp8_weight;
int cf_refresh_fp8_weight(const cf_fp8_weight* slot, int recompute_amax, void* stream);

/* The forward FP8 linear of src/trainer.cu:6114-6132 as one call: fp8_quant_act(x) into the context's act8
 * scratch, then lt_gemm_fp8_nt against the cached weight with the slot's snapshot descale, then the bias
 * step. y[M,N] bf16. */
int cf_fp8_linear_forward(cf_ctx* ctx, cf_act_slot* slot, const void* d_x, int M, int K, const void* d_w8,
                          const float* d_w_descale, int N, const void* d_bias, int bias_mode, void* d_y, int ldy,
                          void* stream);

/* No counterpart in the reference. The same computation as the quantise + GEMM + bias part of
 * cf_fp8_linear_forward, for callers that may not allocate device memory and therefore cannot create a
 * cf_ctx: a trainer whose arena already owns the device-memory budget, or a latency-critical thread that
 * cannot afford the device-wide stall of cudaMalloc / cudaFree. The E4M3 copy of the activation is kept in
 * a 4 MiB array that is part of the library image (every GPU that loads the library holds it until exit),
 * so M*K must not exceed 4 MiB (4,194,304 elements); larger calls return CF_ERR_LIMIT. The caller passes
 * the scale pair to quantise with (for delayed scaling: an ActSlot's snapshot pair) and all inputs and
 * outputs; the call itself uses no cudaMalloc, cudaFree or other allocating routine.
 *   y[M,N] bf16 (row stride ldy) = (*d_x_descale * *d_w_descale) * e4m3(x * *d_x_scale) . w8^T  [+ bias]
 * d_status_or_null: optional device int that receives a non-zero code if a bounded device-side wait gave up
 * (d_y is then incomplete). Without it the code goes to a word inside the array that no entry point reads, so
 * such a failure is only observable when the caller passes its own word (and clears it before the call).
 * The first call on each device looks up the array's device address. All calls share the one array and it
 * keeps the previous call's contents (the call clears the word it needs zeroed): two calls that overlap on
 * the GPU, e.g. on different streams, race on it. */
int cf_fp8_linear_static_scratch(const void* d_x, int M, int K, const float* d_x_scale, const float* d_x_descale,
                                 const void* d_w8, const float* d_w_descale, int N, const void* d_bias, int bias_mode,
                                 void* d_y, int ldy, int* d_status_or_null, void* stream);

/* kernels/lion.cu:121-144, include/ida_native/kernels.hpp:1089-1108 (both lion_step overloads): Lion update with the
 * stochastic-rounding bf16 weight write and, when d_weight_amax is non-NULL, max |w_new| of the fp32 value before
 * rounding accumulated into it (integer atomicMax; the caller zeroes it) — the amax cf_refresh_fp8_weight consumes with
 * recompute_amax = 0. Momentum state fp32 or bf16 (bf16 state is itself rounded stochastically). */
int cf_lion_step_f32_state(void* d_w, float* d_m, const float* d_grad, size_t n, float lr, float beta1, float beta2, float wd,
                           void* stream, float* d_weight_amax, unsigned sr_seed);
int cf_lion_step_bf16_state(void* d_w, void* d_m, const float* d_grad, size_t n, float lr, float beta1, float beta2, float wd,
                            void* stream, float* d_weight_amax, unsigned sr_seed);
/* kernels/lion.cu:39-119 and src/trainer.cu:4694-4712 in ONE pass (no counterpart as a single call): the Lion step of a
 * [rows, cols] weight that also writes its E4M3 caches, so the weight refresh needs no pass of its own. Weights,
 * momentum and the amax recorded into d_weight_amax (caller-zeroed) equal cf_lion_step_*_state bit for bit. The
 * stochastically rounded bf16 value just written is quantised with scale = 448 / max(*d_quant_amax, 1e-12) (published to
 * d_scale_out / d_descale_out like cf_refresh_fp8_weight does) into d_w8, the cache in the master's own layout
 * [rows, cols], and, when d_w8_transposed_or_null is given, into the other layout [cols, rows]: the bytes
 * cf_refresh_fp8_weight(recompute_amax = 0) would produce from that amax. *d_quant_amax is the amax an EARLIER step left
 * (delayed by one step: this step's amax is complete only when the pass ends), so it must be a different word from
 * d_weight_amax; a trainer alternates two words per weight. Needs cols % 8 == 0, 16-byte aligned master, gradient and
 * state, an 8-byte aligned d_w8; CF_ERR_UNSUPPORTED otherwise (run
 * the plain step and cf_refresh_fp8_weight then). With cf_gemm_fp8_nn the dgrad GEMMs read the native-layout cache as
 * it lies, so the transposed cache is only needed by callers that keep the reference's NT dgrad. */
int cf_lion_step_f32_state_quantize(void* d_w, float* d_m, const float* d_grad, int rows, int cols, float lr, float beta1,
                                    float beta2, float wd, void* stream, float* d_weight_amax, unsigned sr_seed,
                                    const float* d_quant_amax, float* d_scale_out, float* d_descale_out, void* d_w8,
                                    void* d_w8_transposed_or_null);
int cf_lion_step_bf16_state_quantize(void* d_w, void* d_m, const float* d_grad, int rows, int cols, float lr, float beta1,
                                     float beta2, float wd, void* stream, float* d_weight_amax, unsigned sr_seed,
                                     const float* d_quant_amax, float* d_scale_out, float* d_descale_out, void* d_w8,
                                     void* d_w8_transposed_or_null);

/* ------------------------------------------------------------------ RMSNorm feeding the quantiser */

/* kernels/rmsnorm.cu:13-54,101-108, include/ida_native/kernels.hpp:117-124 (rmsnorm_forward): out = bf16((x / rms) * scale),
 * rms = sqrt(mean(x^2) + eps) per row, rms values kept for the backward pass when d_rms_or_null is given. Same
 * summation order as the reference kernel (bit-identical rows). x, out: bf16 [rows, H] contiguous; d_scale: bf16 [H].
 * H below 512 must be a multiple of 32 (the reference's reduction is undefined otherwise); H <= 16384. */
int cf_rmsnorm_forward(const void* d_x, const void* d_scale, void* d_out, float* d_rms_or_null, int rows, int H, float eps,
                       void* stream);
/* rmsnorm_forward followed by fp8_quantize_e4m3_record on its output (kernels/fp8.cu:67-84) in one pass over x: the
 * normalised row is rounded to bf16 exactly as rmsnorm_forward would store it, then quantised with *d_quant_scale and
 * its amax accumulated into the caller-zeroed *d_amax. d_normed_or_null: also keep the bf16 row (the backward pass of
 * the reference reads it). */
int cf_rmsnorm_quantize_e4m3_record(const void* d_x, const void* d_scale, void* d_normed_or_null, float* d_rms_or_null,
                                    void* d_out8, const float* d_quant_scale, float* d_amax, int rows, int H, float eps,
                                    void* stream);
/* No counterpart in the reference (it scales per tensor): the same pass with one scale per token, as
 * cf_fp8_quantize_rowwise_e4m3 would compute from the normalised row. */
int cf_rmsnorm_quantize_rowwise_e4m3(const void* d_x, const void* d_scale, void* d_normed_or_null, float* d_rms_or_null,
                                     void* d_out8, float* d_row_scale_or_null, float* d_row_descale, int rows, int H,
                                     float eps, void* stream);
/* src/trainer.cu:6097 + :6115 (rmsnorm_forward, then fp8_quant_act on sb.normed) as one call: the slot's delayed-scale
 * state machine around cf_rmsnorm_quantize_e4m3_record. E4M3 slots without calibration; the first call on a fresh slot
 * takes an exact amax first. With slot->ticket set a steady-state call is two launches (snapshot, fused pass). */
int cf_fp8_rmsnorm_quant_act(cf_ctx* ctx, cf_act_slot* slot, const void* d_x, const void* d_norm_scale, void* d_normed_or_null,
                             float* d_rms_or_null, int rows, int H, float eps, void* d_out8, void* stream);
/* The same passes with the row clip the reference runs between the norm and the quantiser (act_row_clip in its default
 * fixed-ceiling mode, src/trainer.cu:3822-3845, 3940-3991: rows of the normalised bf16 tensor whose L2 norm exceeds
 * clip_ceiling are multiplied by clip_ceiling / norm and rounded to bf16 again; the norm uses the reference kernel's
 * summation order). One read of x replaces rmsnorm_forward + the clip's norm pass + its conditional rewrite (+ the
 * quantiser's read). clip_ceiling <= 0: no clip. Needs H % 512 == 0, H <= 8192, 16-byte aligned rows. The statistics
 * counters of the reference's clip (g_rowclip_stats) are not kept. */
int cf_rmsnorm_clip_forward(const void* d_x, const void* d_scale, void* d_out, float* d_rms_or_null, int rows, int H, float eps,
                            float clip_ceiling, void* stream);
int cf_rmsnorm_clip_quantize_e4m3_record(const void* d_x, const void* d_scale, void* d_normed_or_null, float* d_rms_or_null,
                                         void* d_out8, const float* d_quant_scale, float* d_amax, int rows, int H, float eps,
                                         float clip_ceiling, void* stream);
/* cf_fp8_rmsnorm_quant_act with that clip in between: the sequence of src/trainer.cu:6097-6115 as one pass. */
int cf_fp8_rmsnorm_clip_quant_act(cf_ctx* ctx, cf_act_slot* slot, const void* d_x, const void* d_norm_scale,
                                  void* d_normed_or_null, float* d_rms_or_null, int rows, int H, float eps,
                                  float clip_ceiling, void* d_out8, void* stream);

/* ------------------------------------------------------------------ elementwise neighbours of the GEMMs */

/* kernels/moe.cu:338-345, kernels.hpp:243-247. */
int cf_bias_add_strided_bf16(void* d_inout, const void* d_bias, int rows, int cols, int row_stride, int base, void* stream);
/* kernels/activations.cu:76-87, kernels.hpp:159-165.  out = bf16(silu(gate) * up). */
int cf_swiglu_forward(const void* d_gate, const void* d_up, void* d_out, int n, void* stream);
/* kernels/moe.cu:519-521, kernels.hpp:334.  exact-erf GELU. */
int cf_gelu_forward(const void* d_x, void* d_out, size_t n, void* stream);

/* Per-token (row-wise) scaling (the granularity of the per-token / per-channel SwiGLU MLP); the reference scales per tensor only, so
 * these generalise kernels/fp8.cu:34-49 per row: a_r = max(amax_r, 1e-12), scale_r = 448/a_r, descale_r = a_r/448,
 * out[r,c] = e4m3(x[r,c] * scale_r). d_row_scale may be NULL. At most 16384 columns. The GEMM consumes d_row_descale
 * through cf_gemm_epilogue.d_a_row_descale. */
int cf_fp8_quantize_rowwise_e4m3(const void* d_x, int ld_x, void* d_out, int ld_out, float* d_row_scale,
                                 float* d_row_descale, int rows, int cols, void* stream);
/* The same quantiser for rows whose amax is already known (recorded by the kernel that produced them, e.g.
 * cf_gemm_fp8_swiglu_bf16_rowamax, and max-reduced over ranks where the row is split): one read, one write. */
int cf_fp8_quantize_rowwise_given_amax_e4m3(const void* d_x, int ld_x, void* d_out, int ld_out, const float* d_row_amax,
                                            float* d_row_scale, float* d_row_descale, int rows, int cols, void* stream);
/* The same on bf16(silu(gate) * up): swiglu_forward (kernels/activations.cu:28-40) and the re-quantisation before the
 * down projection (src/trainer.cu:7138-7146) in one pass; gate and up are [rows, cols] views with row stride ld_in. */
int cf_swiglu_quantize_rowwise_e4m3(const void* d_gate, const void* d_up, int ld_in, void* d_out, int ld_out,
                                    float* d_row_scale, float* d_row_descale, int rows, int cols, void* stream);
/* Per-tensor delayed-scaling form of the same fusion: swiglu_forward + fp8_quantize_e4m3_record
 * (kernels/fp8.cu:310-319) without the bf16 intermediate in HBM. The caller zeroes d_amax. */
int cf_swiglu_quantize_e4m3_record(const void* d_gate, const void* d_up, int ld_in, void* d_out, int ld_out,
                                   const float* d_scale, float* d_amax, int rows, int cols, void* stream);

/* ------------------------------------------------------------------ MoE routing, permute, combine */

/* kernels/moe.cu:410-422, kernels.hpp:313-317: softmax in place, hard top-k (lowest index wins ties),
 * zero the rest, renormalise kept. Save pointers may be NULL. */
int cf_moe_topk_route_f32(float* d_scores, int rows, int num_experts, int top_k, void* stream,
                          float* d_row_sum_save, float* d_scores_save, int normalize_topk);
/* kernels/moe.cu:702-710, kernels.hpp:361-364. Zeroes d_counts itself (the reference relies on the caller);
 * row order inside one expert is ascending (the reference's is atomic-order dependent). */
int cf_moe_build_expert_row_lists(const float* d_route_weights, int* d_counts, int* d_row_indices, int rows,
                                  int num_experts, void* stream);
/* kernels/moe.cu:859-863, kernels.hpp:396-398. */
int cf_moe_expert_offsets_from_counts(const int* d_counts, int* d_offsets, int num_experts, void* stream);
/* kernels/moe.cu:712-728, kernels.hpp:365-372. */
int cf_moe_gather_rows_u8(const uint8_t* d_src, uint8_t* d_dst, const int* d_row_indices, int n_rows, int width, void* stream);
int cf_moe_gather_rows_bf16(const void* d_src, void* d_dst, const int* d_row_indices, int n_rows, int width, void* stream);
/* kernels/moe.cu:730-738, kernels.hpp:373-377. */
int cf_moe_scatter_accumulate_rows_bf16(void* d_mixed, const void* d_compact, const float* d_route_weights,
                                        const int* d_row_indices, int n_rows, int expert_idx, int num_experts, int H,
                                        void* stream);
/* kernels/moe.cu:677-683, kernels.hpp:341-344. */
int cf_moe_scale_accumulate_bf16(void* d_mixed, const void* d_term, const float* d_route_weights, int rows,
                                 int expert_idx, int num_experts, int H, void* stream);

/* Device-scheduled forms of the two passes above for all experts at once (no host copy of the counts):
 * gather every expert's rows into one compact [sum(counts), width] buffer at d_offsets[e], and combine
 * every expert's compact output back, one expert after the other per row in expert order (same rounding
 * sequence as running cf_moe_scatter_accumulate_rows_bf16 for e = 0..E-1). */
int cf_moe_gather_all_u8(const uint8_t* d_src, uint8_t* d_dst, const int* d_row_indices, const int* d_counts,
                         const int* d_offsets, int rows, int num_experts, int width, void* stream);
int cf_moe_combine_all_bf16(void* d_mixed, const void* d_compact, const float* d_route_weights,
                            const int* d_row_indices, const int* d_counts, const int* d_offsets, int rows,
                            int num_experts, int H, void* stream);
/* The same combine in one pass over the token rows, for dispatch lists in ascending row order (what
 * cf_moe_build_expert_row_lists writes; the reference's own builder orders them arbitrarily, use cf_moe_combine_all_bf16
 * for those): every row of mixed is read (accumulate != 0) or started from zero (accumulate == 0) and written once, the
 * selected experts are added in ascending expert order with one bf16 rounding each, so the result equals zero-fill +
 * cf_moe_combine_all_bf16 bit for bit. */
int cf_moe_combine_sorted_bf16(void* d_mixed, const void* d_compact, const float* d_route_weights, const int* d_row_indices,
                               const int* d_counts, const int* d_offsets, int rows, int num_experts, int H, int accumulate,
                               void* stream);
/* No counterpart in the reference (single GPU). Expert parallelism under a skewed load: a popular expert is held by
 * several ranks, each replica being a "virtual expert". Rewrites sparse route weights [rows, num_experts] as
 * [rows, num_replicas]: expert e owns the replica ids [d_replica_start[e], d_replica_start[e + 1]); every selected
 * (row, e) keeps its weight on exactly one of them, chosen by a hash of (first_row + row, e) against the replicas'
 * cumulative shares d_replica_cum_share (ascending inside each expert, the last one 1). Replica ids ascend with the
 * expert id, so combining over replicas in ascending id order adds the experts in the single-GPU order. */
int cf_moe_expand_route_replicas(const float* d_route_weights, float* d_replica_weights, int rows, int num_experts,
                                 int num_replicas, const int* d_replica_start, const float* d_replica_cum_share,
                                 unsigned first_row, void* stream);
/* Dispatch front end of a routed layer in one call (two launches, no block waits for another): what
 * cf_moe_topk_route_f32 (kernels/moe.cu:374-422), [cf_moe_expand_route_replicas,] cf_moe_build_expert_row_lists
 * (kernels/moe.cu:565-580, 702-710) and cf_moe_expert_offsets_from_counts (kernels/moe.cu:785-795, 859-863) produce one
 * after the other, bit for bit and list entry for list entry: d_scores [rows, num_experts] is overwritten by the sparse
 * route weights; with d_replica_weights_or_null != NULL the replica form [rows, num_replicas] is written too and the lists
 * are built over the replicas, otherwise over the experts (the replica arguments are then ignored). The lists hold the row
 * numbers in ascending order; d_counts, d_offsets: one int per list; d_row_indices: [lists, rows]. It replaces the
 * host-synchronised list building of src/trainer.cu:6876-6880. d_scratch: cf_moe_route_dispatch_scratch_ints(rows, lists)
 * ints owned by the caller, contents irrelevant (CF_ERR_LIMIT if too small); more than 64 lists run the separate
 * kernels. Every 256-row chunk sums the counts of the chunks in front of it, so the second launch reads
 * (rows / 256)^2 / 2 x lists integers in total: negligible up to a few hundred thousand rows per call, which is what a
 * layer routes. */
size_t cf_moe_route_dispatch_scratch_ints(int rows, int num_lists);
int cf_moe_route_dispatch_lists(float* d_scores, int rows, int num_experts, int top_k, int normalize_topk,
                                float* d_row_sum_save_or_null, float* d_scores_save_or_null, float* d_replica_weights_or_null,
                                int num_replicas, const int* d_replica_start, const float* d_replica_cum_share,
                                unsigned first_row, int* d_counts, int* d_offsets, int* d_row_indices, int* d_scratch,
                                size_t scratch_ints, void* stream);

/* ------------------------------------------------------------------ sharding glue (host side, no device work) */

/* Contiguous balanced shard [*lo, *hi) of range(n) for `rank` of `world`; shard sizes are multiples of `multiple`
 * except possibly the last one. Used for column-sharded weights (output columns) and row-parallel GEMMs (K). */
int cf_shard_range(long long n, int world, int rank, int multiple, long long* lo, long long* hi);

/* Expert placement of an expert-parallel MoE layer under a skewed load: the layout behind the reference's
 * ParallelMode::ExpertSharded (include/canopy_foundry/parallel/plan.hpp:9-13, a mode name with no handling in
 * src/parallel/plan.cpp:5-12). The experts are laid end to end on a line, each as long as its expected share of the rows
 * (popularity[e], any positive scale), and the line is cut into `world` equal pieces, one per rank: every
 * (expert, rank) overlap is a replica of that expert on that rank and receives the overlapping fraction of the expert's
 * rows; overlaps below min_share of a piece are merged into the expert's largest replica. Replica ids ascend along the
 * line, so every rank owns a contiguous id range [rank_lo, rank_hi), ids ascend with the expert id, and every rank
 * expects the same number of rows. A uniform load with world | num_experts degenerates to plain expert sharding. The
 * arrays feed cf_moe_expand_route_replicas (replica_start, replica_cum_share) and cf_moe_ep_plan (rank_lo, rank_hi). */
#define CF_EP_MAX_EXPERTS 256
#define CF_EP_MAX_RANKS 64
#define CF_EP_MAX_REPLICAS (CF_EP_MAX_EXPERTS + CF_EP_MAX_RANKS)
typedef struct cf_ep_placement {
    int world;
    int num_experts;
    int num_replicas;
    int replica_expert[CF_EP_MAX_REPLICAS];        /* expert of each replica */
    int replica_rank[CF_EP_MAX_REPLICAS];          /* rank that holds it */
    double replica_share[CF_EP_MAX_REPLICAS];      /* fraction of its expert's rows it takes */
    double replica_cum_share[CF_EP_MAX_REPLICAS];  /* cumulative share inside the expert (last replica of an expert: 1) */
    int replica_start[CF_EP_MAX_EXPERTS + 1];      /* first replica id of each expert */
    int rank_lo[CF_EP_MAX_RANKS];                  /* replica id range served by each rank */
    int rank_hi[CF_EP_MAX_RANKS];
} cf_ep_placement;
int cf_ep_placement_build(const double* popularity, int num_experts, int world, double min_share, cf_ep_placement* out);
/* The same placement with the pieces of the line sized so that the ranks share the TILE WORK rather than the rows: the
 * grouped GEMM processes every replica in tiles of tile_rows rows (256 in the CTA-pair form), so a rank that holds
 * several small replicas pays about tile_rows / 2 padded rows for each of them (at 8 ranks and a Zipf load the rank
 * with four replicas does 9 % more tile work than the rank with one, and every rank waits for it). expected_total_rows:
 * selected rows of all ranks per layer (tokens * top_k). Never worse than the equal-rows placement by its own cost model. */
int cf_ep_placement_build_balanced(const double* popularity, int num_experts, int world, double min_share,
                                   double expected_total_rows, int tile_rows, cf_ep_placement* out);
/* The balanced placement for ranks of unequal speed: rank_speed_or_null[g] > 0 is rank g's measured throughput on this
 * work in any common unit (rows of tile work per millisecond of its GEMM stages, say; NULL = all equal). The GPUs of one box
 * differ by several percent under their power cap, and every rank waits for the slowest at the closing barrier of a layer;
 * the pieces of the line are sized so that tile work / speed is what the ranks have in common. */
int cf_ep_placement_build_weighted(const double* popularity, int num_experts, int world, double min_share,
                                   double expected_total_rows, int tile_rows, const double* rank_speed_or_null,
                                   cf_ep_placement* out);

/* A run of rows on its way to another buffer: `rows` rows starting at src_row (ignored when the call gathers through an
 * index table) go to row dst_row of destination buffer number dst. */
typedef struct cf_row_run {
    long long src_row;
    long long dst_row;
    int rows;
    int dst;
} cf_row_run;

/* No counterpart in the reference (single GPU). Device-side plan of one expert-parallel layer, computed by every rank
 * from the same table d_counts_all[world, num_replicas] (rows each source rank routes to each replica; gathered with
 * one collective, never copied to the host). Replica v is served by the rank whose id range
 * [d_range_lo[g], d_range_hi[g]) holds it; a serving rank receives its replicas one after the other and, inside a
 * replica, the sources in rank order, so every replica is one ragged GEMM group.
 *   d_send_runs[num_replicas]          where this rank's rows for each replica land (dst = serving rank)
 *   d_group_counts/offsets[n_local]    the ragged groups this rank serves (n_local = its range length)
 *   d_return_runs[n_local * world]     where each (replica, source) block of results returns to (dst = source rank,
 *                                      dst_row = that replica's offset in the source's own compact order)
 * recv_capacity_rows (> 0): rows of this rank's receive buffer; a group that would run past it is cut to what fits and a
 * code is left in ctx_or_null's status word (CF_ERR_DEVICE_RANGE at the next poll). 0 = unchecked. */
int cf_moe_ep_plan(const int* d_counts_all, int world, int rank, int num_replicas, const int* d_range_lo, const int* d_range_hi,
                   cf_row_run* d_send_runs, int* d_group_counts, int* d_group_offsets, cf_row_run* d_return_runs,
                   long long recv_capacity_rows, cf_ctx* ctx_or_null, void* stream);
/* Copies the runs of a device plan: whole rows of row_bytes (a multiple of 16) from d_src to
 * d_dst_bases[run.dst] + run.dst_row * row_bytes; the destinations may be peer GPUs' buffers mapped into this process
 * (plain stores over NVLink). With an index table the i-th row of run r is row d_row_indices[r * index_stride + i] of
 * d_src (permute and send in one pass). With a tag, *d_tag_value is also stored at d_tag_bases[run.dst][run.dst_row + i]
 * for every row (the sender's activation descale travelling with its rows). d_dst_bases / d_tag_bases are DEVICE arrays
 * of num_dst base pointers, each buffer dst_rows rows long; max_rows_per_run only sizes the grid. A run with dst outside
 * [0, num_dst) or rows outside [0, dst_rows) is not stored at all (the destinations may be other GPUs' memory) and
 * leaves a code in ctx_or_null's status word: CF_ERR_DEVICE_RANGE at the next cf_ctx_poll_status. */
int cf_moe_send_row_runs(const void* d_src, const int* d_row_indices_or_null, long long index_stride, const cf_row_run* d_runs,
                         int num_runs, int max_rows_per_run, void* const* d_dst_bases, long long row_bytes,
                         const float* d_tag_value_or_null, float* const* d_tag_bases_or_null, int num_dst, long long dst_rows,
                         cf_ctx* ctx_or_null, void* stream);
/* No counterpart in the reference (single GPU). Barrier between the ranks of one box without a collective launch: every
 * rank calls it with the same epoch (a counter that grows by one per barrier; the flag words start at zero). The kernel
 * stores `epoch` into word `rank` of every rank's flag array and waits until all `world` words of its own array have
 * reached it, so the work enqueued behind it on `stream` starts once every rank's earlier work on ITS stream, including
 * its stores into peers' buffers, is complete and visible. d_flag_arrays is a DEVICE array of `world` pointers, entry r =
 * rank r's array of `world` unsigned words as mapped in this process (peer-mapped memory for r != rank). The ranks must
 * run on different GPUs. The wait is bounded: after limit_ms (1..60000) the kernel gives up, the launches behind it still
 * run (on incomplete data) and the next cf_ctx_poll_status returns CF_ERR_DEVICE_WAIT. */
int cf_peer_barrier(cf_ctx* ctx, unsigned* const* d_flag_arrays, int world, int rank, unsigned epoch, int limit_ms,
                    void* stream);

/* A small all-gather done the same way, in the same launch as the barrier: this rank's n words (1..4096) are stored into
 * row `rank` of every rank's [world, n] table (d_tables: DEVICE array of `world` table pointers as mapped here), then the
 * barrier protocol of cf_peer_barrier runs with `epoch`, so the work behind the call sees every rank's row in its own
 * table. The expert-parallel layer exchanges its per-replica row counts with it (a library all-gather of 36 integers
 * costs several times as much). Same bounded wait and status reporting. No counterpart in the reference. */
int cf_peer_share_i32(cf_ctx* ctx, const int* d_src, int n, int* const* d_tables, unsigned* const* d_flag_arrays, int world,
                      int rank, unsigned epoch, int limit_ms, void* stream);

/* The down projection of a device-planned expert-parallel layer with the return leg in its epilogue: a ragged grouped
 * NT GEMM (as cf_gemm_fp8_nt_grouped) whose output rows leave straight for the buffers of the ranks that own the tokens.
 * Inside group g the rows are the runs d_return_runs[g * runs_per_group + s] in ascending src_row (compact rows of A);
 * run s is written to rows dst_row.. of dst_buffers[run.dst], bf16 [dst_rows, N] with pitch ldc (peer-mapped memory
 * for other ranks). 32-row boxes that lie inside one run leave as TMA stores, boxes that straddle two runs row by row.
 * dst_buffers is a HOST array of num_dst (1..16) device pointers; the context caches their tensor maps on the device.
 * Needs N % 64 == 0, ldc % 8 == 0, 16-byte aligned operands, K % 16 == 0. */
int cf_gemm_fp8_nt_grouped_return(cf_ctx* ctx, int num_groups, int max_total_rows, int N, int K, const int* d_counts,
                                  const int* d_offsets, const void* d_A, int lda, int a_is_e5m2, const float* d_a_descale,
                                  const void* d_B, const float* d_b_descale, const cf_row_run* d_return_runs,
                                  int runs_per_group, void* const* dst_buffers, int num_dst, int dst_rows, int ldc,
                                  void* stream);

/* kernels/moe.cu:1062-1127, kernels.hpp:414-423: grouped selected-expert FP8 forward with exact-erf GELU,
 * accumulating rw*y into d_mixed. The tensor-core implementation needs workspace, which the reference
 * signature has no room for, hence the ctx parameter: it uses about
 *   total_selected_rows * (3*H + 4*Ie) + 2 KiB bytes of ctx workspace (cf_ctx_reserve_workspace, done once
 * outside the hot path; the call fails with CF_ERR_LIMIT when too little is reserved). The fc_in output is
 * rounded to bf16 and the GELU output is carried into fc_out as a two-term E4M3 split (hi + lo, ~2^-8
 * relative) where the reference keeps it in fp32: outputs agree within the path's 1e-2 relative-Frobenius
 * tolerance, not bit for bit. */
int cf_ctx_reserve_workspace(cf_ctx* ctx, size_t bytes);
int cf_moe_grouped_expert_forward_fp8(cf_ctx* ctx, const void* d_hidden, const float* d_fcin_descale, int fcin_is_e5m2,
                                      const float* d_route_weights, const int* d_counts, const int* d_offsets,
                                      const int* d_row_indices, const void* d_fc_in_w, const float* d_fc_in_descale,
                                      const void* d_fc_out_w, const float* d_fc_out_descale, void* d_mixed, int rows,
                                      int H, int Ie, int num_experts, int total_selected_rows, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CANOPY_FP8_H */
