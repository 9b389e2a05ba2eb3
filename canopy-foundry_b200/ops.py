"""Operator mirror of the reference's FP8 / MoE interface on torch CUDA tensors.

Function names, argument order and meaning follow include/ida_native/kernels.hpp:983-1052 (FP8),
:313-423 (MoE) and the file-static helpers of src/trainer.cu (lt_gemm_fp8_nt :4498, fp8_quant_act
:4732, refresh_fp8_weights :4694). torch supplies device memory and streams only; every operator
runs in libcanopy_fp8.so on the current torch stream. A failing call raises CanopyError, where the
reference throws std::runtime_error.
"""
import ctypes as C

import torch

from . import _capi
from ._capi import E4M3_MAX, E5M2_MAX, CanopyError, check

__all__ = [
    "E4M3_MAX", "E5M2_MAX", "CanopyError", "Fp8Ctx", "ActSlot", "Fp8Weight",
    "fp8_amax_bf16", "fp8_scale_from_amax", "fp8_quantize_e4m3", "fp8_quantize_e5m2",
    "fp8_quantize_e4m3_record", "fp8_quantize_e5m2_record", "fp8_update_delayed_scale",
    "fp8_quantize_transpose_e4m3", "fp8_quant_and_transpose_e4m3", "transpose_u8", "fp8_clip_probe",
    "fp8_elem_clip_count", "fp8_pack_bf16_e4m3_raw", "fp8_pack_bf16_e4m3_raw_and_dequant",
    "fp8_unpack_e4m3_raw_bf16", "lt_gemm_fp8_nt", "gemm_fp8_nn", "gemm_fp8_nn_grouped", "lt_gemm_fp8_tn_accum_f32", "gemm_fp8_dw_accum", "gemm_fp8_nt_reduce_scatter", "f32_to_bf16_and_zero", "gemm_fp8_nt_grouped", "gemm_fp8_nt_segments", "gemm_fp8_nt_segments_scatter",
    "fp8_quant_act", "fp8_swiglu_quant_act", "gemm_fp8_swiglu_quant_act", "fp8_interleave_gate_up", "refresh_fp8_weight", "fp8_linear_forward", "bias_add_strided_bf16", "swiglu_forward",
    "gelu_forward", "lion_step", "lion_step_quantize", "fp8_quantize_rowwise_e4m3", "fp8_quantize_rowwise_given_amax_e4m3", "gemm_fp8_swiglu_bf16_rowamax", "interleave_gate_up_vector", "swiglu_mlp_fp8_rowwise_fused", "swiglu_quantize_rowwise_e4m3", "swiglu_quantize_e4m3_record",
    "rmsnorm_forward", "rmsnorm_quantize_e4m3_record", "rmsnorm_quantize_rowwise_e4m3", "fp8_rmsnorm_quant_act", "rmsnorm_clip_forward", "rmsnorm_clip_quantize_e4m3_record", "fp8_rmsnorm_clip_quant_act",
    "moe_topk_route_f32", "moe_build_expert_row_lists", "moe_expert_offsets_from_counts",
    "moe_gather_rows_u8", "moe_gather_rows_bf16", "moe_scatter_accumulate_rows_bf16",
    "moe_scale_accumulate_bf16", "moe_gather_all_u8", "moe_combine_all_bf16", "moe_combine_sorted_bf16", "moe_expand_route_replicas", "moe_route_dispatch_lists", "moe_route_dispatch_scratch_ints", "moe_ep_plan", "gemm_fp8_nt_grouped_return", "moe_send_row_runs", "peer_barrier", "peer_share_i32", "ROW_RUN_BYTES",
    "moe_grouped_expert_forward_fp8", "launch_count", "swiglu_mlp_fp8_rowwise", "MoeSwigluFp8", "FfnSwigluFp8",
]


def _s():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    if t is None:
        return None
    assert t.is_cuda, "device tensor expected"
    return C.c_void_p(t.data_ptr())


def _L():
    return _capi.lib()


_rt = None


def _cudart():
    """The CUDA runtime torch already loaded (used only for debug read-backs of slot scalars)."""
    global _rt
    if _rt is None:
        for name in ("libcudart.so.12", "libcudart.so.13", "libcudart.so"):
            try:
                _rt = C.CDLL(name)
                break
            except OSError:
                continue
        if _rt is None:
            raise ImportError("libcudart not found")
        _rt.cudaMemcpy.restype = C.c_int
    return _rt


def launch_count():
    return int(_L().cf_launch_count())


# ---------------------------------------------------------------- quantize / cast
def fp8_amax_bf16(x, amax):
    check(_L().cf_fp8_amax_bf16(_p(x), x.numel(), _p(amax), _s()))


def fp8_scale_from_amax(amax, fp8_max, scale, descale):
    check(_L().cf_fp8_scale_from_amax(_p(amax), fp8_max, _p(scale), _p(descale), _s()))


def fp8_quantize_e4m3(x, out, scale, n=None):
    check(_L().cf_fp8_quantize_e4m3(_p(x), _p(out), _p(scale), x.numel() if n is None else n, _s()))


def fp8_quantize_e5m2(x, out, scale, n=None):
    check(_L().cf_fp8_quantize_e5m2(_p(x), _p(out), _p(scale), x.numel() if n is None else n, _s()))


def fp8_quantize_e4m3_record(x, out, scale, amax, n=None):
    check(_L().cf_fp8_quantize_e4m3_record(_p(x), _p(out), _p(scale), _p(amax), x.numel() if n is None else n, _s()))


def fp8_quantize_e5m2_record(x, out, scale, amax, n=None):
    check(_L().cf_fp8_quantize_e5m2_record(_p(x), _p(out), _p(scale), _p(amax), x.numel() if n is None else n, _s()))


def fp8_update_delayed_scale(amax, fp8_max, scale, descale, history, history_len, cursor, count):
    check(_L().cf_fp8_update_delayed_scale(_p(amax), fp8_max, _p(scale), _p(descale), _p(history), history_len,
                                           _p(cursor), _p(count), _s()))


def fp8_quantize_transpose_e4m3(w, out, scale, K, N):
    check(_L().cf_fp8_quantize_transpose_e4m3(_p(w), _p(out), _p(scale), K, N, _s()))


def fp8_quant_and_transpose_e4m3(x, act8, snap, scale, K, N):
    check(_L().cf_fp8_quant_and_transpose_e4m3(_p(x), _p(act8), _p(snap), _p(scale), K, N, _s()))


def transpose_u8(src, dst, rows, cols):
    check(_L().cf_transpose_u8(_p(src), _p(dst), rows, cols, _s()))


def fp8_clip_probe(amax, scale, fp8_max, stats):
    check(_L().cf_fp8_clip_probe(_p(amax), _p(scale), fp8_max, _p(stats), _s()))


def fp8_elem_clip_count(x, scale, fp8_max, out):
    check(_L().cf_fp8_elem_clip_count(_p(x), _p(scale), fp8_max, x.numel(), _p(out), _s()))


def fp8_pack_bf16_e4m3_raw(x, out, amax, scale, descale, bad_count):
    check(_L().cf_fp8_pack_bf16_e4m3_raw(_p(x), _p(out), _p(amax), _p(scale), _p(descale), _p(bad_count), x.numel(), _s()))


def fp8_pack_bf16_e4m3_raw_and_dequant(x, out, dequant, amax, scale, descale, bad_count):
    check(_L().cf_fp8_pack_bf16_e4m3_raw_and_dequant(_p(x), _p(out), _p(dequant), _p(amax), _p(scale), _p(descale),
                                                     _p(bad_count), x.numel(), _s()))


def fp8_unpack_e4m3_raw_bf16(codes, descale, out):
    check(_L().cf_fp8_unpack_e4m3_raw_bf16(_p(codes), _p(descale), _p(out), codes.numel(), _s()))


# ---------------------------------------------------------------- context, slots
class Fp8Ctx:
    """Counterpart of the reference's Fp8Ctx (src/trainer.cu:3296-3345): owns the shared act8 scratch,
    the scalar pool ActSlots live in and the status word of the tensor-core kernels."""

    def __init__(self, act8_bytes=0):
        h = C.c_void_p()
        check(_L().cf_ctx_create(C.byref(h), act8_bytes))
        self.handle = h
        self.act8_bytes = act8_bytes

    def act8_ptr(self):
        return _L().cf_ctx_act8(self.handle)

    def reserve_workspace(self, nbytes):
        check(_L().cf_ctx_reserve_workspace(self.handle, nbytes))

    def poll_status(self):
        """Synchronises the current stream; raises CanopyError(CF_ERR_DEVICE_WAIT) if a kernel gave up a wait."""
        check(_L().cf_ctx_poll_status(self.handle, _s()))

    def selftest_bounded_wait(self, limit_ms=5):
        """Launches the wait that is designed to run out; the following poll_status() raises CF_ERR_DEVICE_WAIT."""
        check(_L().cf_ctx_selftest_bounded_wait(self.handle, limit_ms, _s()))

    def close(self):
        if self.handle:
            _L().cf_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ActSlot:
    """Delayed-scaling state of one activation/gradient call site (ActSlot, src/trainer.cu:3248-3279)."""

    def __init__(self, ctx, fp8_max=E4M3_MAX, calib_calls=0):
        self.ctx = ctx
        self.c = _capi.ActSlotStruct()
        check(_L().cf_act_slot_init(ctx.handle, C.byref(self.c), fp8_max, calib_calls, _s()))

    def _read(self, ptr, dtype=torch.float32, n=1):
        """Debug read-back of slot scalars (device pointers owned by the context's pool)."""
        torch.cuda.current_stream().synchronize()
        host = torch.empty(n, dtype=dtype)
        rc = _cudart().cudaMemcpy(C.c_void_p(host.data_ptr()), C.c_void_p(ptr), C.c_size_t(n * host.element_size()),
                                  C.c_int(2))
        if rc != 0:
            raise CanopyError(_capi.CF_ERR_CUDA, f"cudaMemcpy device->host failed with {rc}")
        return host

    def scalars(self):
        c = self.c
        return {
            "amax": self._read(c.amax).item(), "scale": self._read(c.scale).item(),
            "descale": self._read(c.descale).item(), "scale_snapshot": self._read(c.scale_snapshot).item(),
            "descale_snapshot": self._read(c.descale_snapshot).item(),
            "history": self._read(c.history, n=8).tolist(),
            "cursor": self._read(c.history_cursor, torch.int32).item(),
            "count": self._read(c.history_count, torch.int32).item(),
            "fp8_max": c.fp8_max, "init": c.init, "calib_remaining": c.calib_remaining,
        }


class Fp8Weight:
    """One FP8-cached weight (Fp8Slot, src/trainer.cu:3284-3294): bf16 master plus both E4M3 layouts."""

    def __init__(self, w, stored_out_major):
        assert w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous()
        self.w = w
        if stored_out_major:
            self.out_dim, self.in_dim = w.shape
        else:
            self.in_dim, self.out_dim = w.shape
        self.fwd8 = torch.empty(self.out_dim, self.in_dim, dtype=torch.uint8, device=w.device)
        self.bwd8 = torch.empty(self.in_dim, self.out_dim, dtype=torch.uint8, device=w.device)
        self.scalars = torch.zeros(12, dtype=torch.float32, device=w.device)   # 16-byte aligned amax/scale/descale
        self.amax, self.scale, self.descale = self.scalars[0:1], self.scalars[4:5], self.scalars[8:9]
        self.c = _capi.Fp8WeightStruct(w.data_ptr(), self.fwd8.data_ptr(), self.bwd8.data_ptr(), self.amax.data_ptr(),
                                       self.scale.data_ptr(), self.descale.data_ptr(), self.in_dim, self.out_dim,
                                       int(stored_out_major))


def refresh_fp8_weight(weight, recompute_amax=True):
    check(_L().cf_refresh_fp8_weight(C.byref(weight.c), int(recompute_amax), _s()))


def fp8_quant_act(ctx, slot, x, out8=None, is_recompute=False, n=None):
    dst = C.c_void_p(ctx.act8_ptr()) if out8 is None else _p(out8)
    check(_L().cf_fp8_quant_act(ctx.handle, C.byref(slot.c), _p(x), x.numel() if n is None else n, dst, _s(),
                                int(is_recompute)))


def fp8_swiglu_quant_act(ctx, slot, gate, up, ld_in, rows, cols, out8):
    check(_L().cf_fp8_swiglu_quant_act(ctx.handle, C.byref(slot.c), _p(gate), _p(up), ld_in, rows, cols, _p(out8), _s()))


def fp8_interleave_gate_up(w_gateup8):
    """[E, 2F, K] with gate rows first -> the 32-row interleaved layout the fused SwiGLU GEMM reads."""
    E, F2, K = w_gateup8.shape
    F = F2 // 2
    out = torch.empty_like(w_gateup8)
    gate = w_gateup8[:, :F].contiguous()
    up = w_gateup8[:, F:].contiguous()
    check(_L().cf_fp8_interleave_gate_up(_p(gate), _p(up), _p(out), E, F, K, _s()))
    return out


def gemm_fp8_swiglu_quant_act(ctx, slot, num_segments, num_weights, segment_weight, max_total_rows, F, K, counts, offsets, A,
                              lda, a_is_e5m2, a_descale, per_segment_a_descale, w_interleaved, w_descale, h8, ldh):
    check(_L().cf_gemm_fp8_swiglu_quant_act(ctx.handle, C.byref(slot.c), num_segments, num_weights, _p(segment_weight),
                                            max_total_rows, F, K, _p(counts), _p(offsets), _p(A), lda, int(a_is_e5m2),
                                            _p(a_descale), int(per_segment_a_descale), _p(w_interleaved), _p(w_descale),
                                            _p(h8), ldh, _s()))


# ---------------------------------------------------------------- GEMMs
def _epi(bias, bias_mode, a_row_descale, b_col_descale, out_fp32=False):
    if bias is None and a_row_descale is None and b_col_descale is None and not out_fp32:
        return None
    return C.byref(_capi.GemmEpilogue(bias.data_ptr() if bias is not None else None, bias_mode,
                                      a_row_descale.data_ptr() if a_row_descale is not None else None,
                                      b_col_descale.data_ptr() if b_col_descale is not None else None, int(out_fp32)))


def lt_gemm_fp8_nt(ctx, M, N, K, A, lda, a_is_e5m2, a_descale, B, b_descale, Cout, ldc, bias=None, bias_mode=0,
                   a_row_descale=None, b_col_descale=None):
    """C[M,N] = (dA*dB) * A8[M,K] . B8[N,K]^T  (src/trainer.cu:4498-4534). C is bf16 like the reference's output;
    a float32 C selects the fp32 partial-product form used by row-parallel (K-sharded) GEMMs."""
    out_fp32 = Cout.dtype == torch.float32
    check(_L().cf_gemm_fp8_nt(ctx.handle, M, N, K, _p(A), lda, int(a_is_e5m2), _p(a_descale), _p(B), _p(b_descale),
                              _p(Cout), ldc, _epi(bias, bias_mode, a_row_descale, b_col_descale, out_fp32), _s()))


def lt_gemm_fp8_tn_accum_f32(ctx, M, N, K, Xt, ds_x, dYt, ds_dy, dW, ldc):
    """dW[M,N] += (dsx*dsdy) * Xt[M,K] . dYt[N,K]^T; dW fp32 or bf16 (src/trainer.cu:4596-4691)."""
    fn = _L().cf_gemm_fp8_tn_accum_f32 if dW.dtype == torch.float32 else _L().cf_gemm_fp8_tn_accum_bf16
    check(fn(ctx.handle, M, N, K, _p(Xt), _p(ds_x), _p(dYt), _p(ds_dy), _p(dW), ldc, _s()))


def gemm_fp8_dw_accum(ctx, M, N, K, X8, ldx, ds_x, dY8, ldy, ds_dy, dW, ldc):
    """dW[M,N] += X8[K,M]^T . dY8[K,N] straight from the un-transposed operands (fp32 or bf16 dW)."""
    fn = _L().cf_gemm_fp8_dw_accum_f32 if dW.dtype == torch.float32 else _L().cf_gemm_fp8_dw_accum_bf16
    check(fn(ctx.handle, M, N, K, _p(X8), ldx, _p(ds_x), _p(dY8), ldy, _p(ds_dy), _p(dW), ldc, _s()))


def gemm_fp8_nt_reduce_scatter(ctx, M, N, K_local, A, lda, a_is_e5m2, a_descale, B, b_descale, slice_ptrs,
                               a_row_descale=None, b_col_descale=None):
    """Row-parallel GEMM whose epilogue adds every row slice of the fp32 product into its owner's accumulation slice
    (slice_ptrs: device addresses, one per rank, as mapped in this process)."""
    arr = (C.c_void_p * len(slice_ptrs))(*[C.c_void_p(int(x)) for x in slice_ptrs])
    check(_L().cf_gemm_fp8_nt_reduce_scatter_f32(ctx.handle, M, N, K_local, _p(A), lda, int(a_is_e5m2), _p(a_descale), _p(B),
                                                 _p(b_descale), _p(a_row_descale), _p(b_col_descale), arr, len(slice_ptrs), _s()))


def f32_to_bf16_and_zero(acc, out):
    check(_L().cf_f32_to_bf16_and_zero(_p(acc), _p(out), acc.numel(), _s()))


def gemm_fp8_nn(ctx, M, N, K, A, lda, a_is_e5m2, a_descale, B_kn, ldb, b_descale, Cout, ldc, accumulate=False):
    """C[M,N] = A[M,K] . B[K,N]: the dgrad direction, reading the forward weight cache ([out,in] = [K,N]) as it lies."""
    check(_L().cf_gemm_fp8_nn(ctx.handle, M, N, K, _p(A), lda, int(a_is_e5m2), _p(a_descale), _p(B_kn), ldb, _p(b_descale),
                              _p(Cout), ldc, int(accumulate), _s()))


def gemm_fp8_nn_grouped(ctx, num_groups, max_total_rows, N, K, counts, offsets, A, lda, a_is_e5m2, a_descale, B_stacked_kn,
                        b_descale, Cout, ldc, accumulate=False):
    """Ragged per-expert dgrad over the stacked forward cache [E, K, N] (no transposed cache)."""
    check(_L().cf_gemm_fp8_nn_grouped(ctx.handle, num_groups, max_total_rows, N, K, _p(counts), _p(offsets), _p(A), lda,
                                      int(a_is_e5m2), _p(a_descale), _p(B_stacked_kn), _p(b_descale), _p(Cout), ldc,
                                      int(accumulate), _s()))


def gemm_fp8_nt_grouped(ctx, num_experts, max_total_rows, N, K, counts, offsets, A, lda, a_is_e5m2, a_descale,
                        per_expert_a_descale, B, b_descale, Cout, ldc):
    check(_L().cf_gemm_fp8_nt_grouped(ctx.handle, num_experts, max_total_rows, N, K, _p(counts), _p(offsets), _p(A),
                                      lda, int(a_is_e5m2), _p(a_descale), int(per_expert_a_descale), _p(B),
                                      _p(b_descale), _p(Cout), ldc, _s()))


def gemm_fp8_nt_segments(ctx, num_segments, num_weights, segment_weight, max_total_rows, N, K, counts, offsets, A, lda,
                         a_is_e5m2, a_descale, per_segment_a_descale, B, b_descale, Cout, ldc):
    check(_L().cf_gemm_fp8_nt_segments(ctx.handle, num_segments, num_weights, _p(segment_weight), max_total_rows, N, K,
                                       _p(counts), _p(offsets), _p(A), lda, int(a_is_e5m2), _p(a_descale),
                                       int(per_segment_a_descale), _p(B), _p(b_descale), _p(Cout), ldc, _s()))


def gemm_fp8_nt_segments_scatter(ctx, num_segments, num_weights, segment_weight, max_total_rows, N, K, counts, offsets, A,
                                 lda, a_is_e5m2, a_descale, per_segment_a_descale, B, b_descale, segment_out,
                                 segment_out_row0, ldc):
    """segment_out: int64 device tensor of output base addresses; segment_out_row0: int64 device tensor of first rows."""
    check(_L().cf_gemm_fp8_nt_segments_scatter(ctx.handle, num_segments, num_weights, _p(segment_weight), max_total_rows, N,
                                               K, _p(counts), _p(offsets), _p(A), lda, int(a_is_e5m2), _p(a_descale),
                                               int(per_segment_a_descale), _p(B), _p(b_descale), None, _p(segment_out),
                                               _p(segment_out_row0), ldc, _s()))


def fp8_linear_forward(ctx, slot, x, w8, w_descale, y, bias=None, bias_mode=2):
    M, K = x.shape
    N = w8.shape[0]
    check(_L().cf_fp8_linear_forward(ctx.handle, C.byref(slot.c), _p(x), M, K, _p(w8), _p(w_descale), N, _p(bias),
                                     bias_mode if bias is not None else 0, _p(y), y.stride(0), _s()))


# ---------------------------------------------------------------- elementwise + MoE
def bias_add_strided_bf16(inout, bias, rows, cols, row_stride, base):
    check(_L().cf_bias_add_strided_bf16(_p(inout), _p(bias), rows, cols, row_stride, base, _s()))


def swiglu_forward(gate, up, out, n=None):
    check(_L().cf_swiglu_forward(_p(gate), _p(up), _p(out), gate.numel() if n is None else n, _s()))


def lion_step(w, m, grad, lr, beta1, beta2, wd, weight_amax=None, sr_seed=0):
    """lion_step (include/ida_native/kernels.hpp:1089-1108); m float32 or bfloat16 selects the overload."""
    fn = _L().cf_lion_step_f32_state if m.dtype == torch.float32 else _L().cf_lion_step_bf16_state
    check(fn(_p(w), _p(m), _p(grad), w.numel(), lr, beta1, beta2, wd, _s(), _p(weight_amax), sr_seed))


def lion_step_quantize(w, m, grad, lr, beta1, beta2, wd, weight_amax, quant_amax, scale_out, descale_out, w8,
                       w8_transposed=None, sr_seed=0):
    """lion_step that also writes the E4M3 cache(s) of the [rows, cols] weight in the same pass (scale from quant_amax,
    the amax an earlier step left; this step's amax goes to weight_amax)."""
    rows, cols = w.shape
    fn = _L().cf_lion_step_f32_state_quantize if m.dtype == torch.float32 else _L().cf_lion_step_bf16_state_quantize
    check(fn(_p(w), _p(m), _p(grad), rows, cols, lr, beta1, beta2, wd, _s(), _p(weight_amax), sr_seed, _p(quant_amax),
             _p(scale_out), _p(descale_out), _p(w8), _p(w8_transposed)))


def gelu_forward(x, out):
    check(_L().cf_gelu_forward(_p(x), _p(out), x.numel(), _s()))


def fp8_quantize_rowwise_e4m3(x, out, row_descale, row_scale=None, rows=None, cols=None, ld_x=None, ld_out=None):
    rows = x.shape[0] if rows is None else rows
    cols = x.shape[1] if cols is None else cols
    check(_L().cf_fp8_quantize_rowwise_e4m3(_p(x), x.stride(0) if ld_x is None else ld_x, _p(out),
                                            out.stride(0) if ld_out is None else ld_out, _p(row_scale), _p(row_descale),
                                            rows, cols, _s()))


def fp8_quantize_rowwise_given_amax_e4m3(x, out, row_amax, row_descale, row_scale=None, rows=None, cols=None):
    rows = x.shape[0] if rows is None else rows
    cols = x.shape[1] if cols is None else cols
    check(_L().cf_fp8_quantize_rowwise_given_amax_e4m3(_p(x), x.stride(0), _p(out), out.stride(0), _p(row_amax),
                                                       _p(row_scale), _p(row_descale), rows, cols, _s()))


def gemm_fp8_swiglu_bf16_rowamax(ctx, M, F, K, A, lda, a_is_e5m2, a_descale, a_row_descale, w_interleaved, w_descale,
                                 w_col_descale_interleaved, h, row_amax):
    """Gate/up GEMM + SwiGLU in one launch: h bf16 [M, F] and max|h| per row (row_amax, zeroed by the caller)."""
    check(_L().cf_gemm_fp8_swiglu_bf16_rowamax(ctx.handle, M, F, K, _p(A), lda, int(a_is_e5m2), _p(a_descale),
                                               _p(a_row_descale), _p(w_interleaved), _p(w_descale),
                                               _p(w_col_descale_interleaved), _p(h), h.stride(0), _p(row_amax), _s()))


def interleave_gate_up_vector(v, F):
    """A per-output-row vector of the [2F, K] gate/up weight (gate rows first) in the 32-row interleaved order of
    fp8_interleave_gate_up: [g0..g31, u0..u31, g32..g63, u32..u63, ...]."""
    g, u = v[:F].reshape(F // 32, 32), v[F:].reshape(F // 32, 32)
    return torch.stack([g, u], dim=1).reshape(2 * F).contiguous()


def swiglu_quantize_rowwise_e4m3(gate, up, out, row_descale, rows, cols, ld_in, ld_out=None, row_scale=None):
    check(_L().cf_swiglu_quantize_rowwise_e4m3(_p(gate), _p(up), ld_in, _p(out), cols if ld_out is None else ld_out,
                                               _p(row_scale), _p(row_descale), rows, cols, _s()))


def rmsnorm_forward(x, scale, out, rms, rows, H, eps=1e-6):
    """out = bf16(x / rms * scale) per row, rms kept for the backward pass (kernels/rmsnorm.cu:101-108)."""
    check(_L().cf_rmsnorm_forward(_p(x), _p(scale), _p(out), _p(rms), rows, H, eps, _s()))


def rmsnorm_quantize_e4m3_record(x, scale, normed, rms, out8, quant_scale, amax, rows, H, eps=1e-6):
    """rmsnorm_forward + fp8_quantize_e4m3_record in one pass; normed / rms may be None."""
    check(_L().cf_rmsnorm_quantize_e4m3_record(_p(x), _p(scale), _p(normed), _p(rms), _p(out8), _p(quant_scale), _p(amax),
                                               rows, H, eps, _s()))


def rmsnorm_quantize_rowwise_e4m3(x, scale, normed, rms, out8, row_descale, rows, H, eps=1e-6, row_scale=None):
    check(_L().cf_rmsnorm_quantize_rowwise_e4m3(_p(x), _p(scale), _p(normed), _p(rms), _p(out8), _p(row_scale),
                                                _p(row_descale), rows, H, eps, _s()))


def fp8_rmsnorm_quant_act(ctx, slot, x, scale, normed, rms, rows, H, out8, eps=1e-6):
    """rmsnorm_forward followed by fp8_quant_act on its output (src/trainer.cu:6097,6115) as one pass."""
    check(_L().cf_fp8_rmsnorm_quant_act(ctx.handle, C.byref(slot.c), _p(x), _p(scale), _p(normed), _p(rms), rows, H, eps,
                                        _p(out8), _s()))


def rmsnorm_clip_forward(x, scale, out, rms, rows, H, clip_ceiling, eps=1e-6):
    """rmsnorm_forward followed by act_row_clip (fixed ceiling) in one pass."""
    check(_L().cf_rmsnorm_clip_forward(_p(x), _p(scale), _p(out), _p(rms), rows, H, eps, clip_ceiling, _s()))


def rmsnorm_clip_quantize_e4m3_record(x, scale, normed, rms, out8, quant_scale, amax, rows, H, clip_ceiling, eps=1e-6):
    check(_L().cf_rmsnorm_clip_quantize_e4m3_record(_p(x), _p(scale), _p(normed), _p(rms), _p(out8), _p(quant_scale),
                                                    _p(amax), rows, H, eps, clip_ceiling, _s()))


def fp8_rmsnorm_clip_quant_act(ctx, slot, x, scale, normed, rms, rows, H, out8, clip_ceiling, eps=1e-6):
    """rmsnorm_forward, act_row_clip and fp8_quant_act (src/trainer.cu:6097-6115) as one pass."""
    check(_L().cf_fp8_rmsnorm_clip_quant_act(ctx.handle, C.byref(slot.c), _p(x), _p(scale), _p(normed), _p(rms), rows, H, eps,
                                             clip_ceiling, _p(out8), _s()))


def swiglu_quantize_e4m3_record(gate, up, out, scale, amax, rows, cols, ld_in, ld_out=None):
    check(_L().cf_swiglu_quantize_e4m3_record(_p(gate), _p(up), ld_in, _p(out), cols if ld_out is None else ld_out,
                                              _p(scale), _p(amax), rows, cols, _s()))


def moe_topk_route_f32(scores, rows, num_experts, top_k, row_sum_save=None, scores_save=None, normalize_topk=True):
    check(_L().cf_moe_topk_route_f32(_p(scores), rows, num_experts, top_k, _s(), _p(row_sum_save), _p(scores_save),
                                     int(normalize_topk)))


def moe_build_expert_row_lists(route_weights, counts, row_indices, rows, num_experts):
    check(_L().cf_moe_build_expert_row_lists(_p(route_weights), _p(counts), _p(row_indices), rows, num_experts, _s()))


def moe_expert_offsets_from_counts(counts, offsets, num_experts):
    check(_L().cf_moe_expert_offsets_from_counts(_p(counts), _p(offsets), num_experts, _s()))


def moe_gather_rows_u8(src, dst, row_indices, n_rows, width):
    check(_L().cf_moe_gather_rows_u8(_p(src), _p(dst), _p(row_indices), n_rows, width, _s()))


def moe_gather_rows_bf16(src, dst, row_indices, n_rows, width):
    check(_L().cf_moe_gather_rows_bf16(_p(src), _p(dst), _p(row_indices), n_rows, width, _s()))


def moe_scatter_accumulate_rows_bf16(mixed, compact, route_weights, row_indices, n_rows, expert_idx, num_experts, H):
    check(_L().cf_moe_scatter_accumulate_rows_bf16(_p(mixed), _p(compact), _p(route_weights), _p(row_indices), n_rows,
                                                   expert_idx, num_experts, H, _s()))


def moe_scale_accumulate_bf16(mixed, term, route_weights, rows, expert_idx, num_experts, H):
    check(_L().cf_moe_scale_accumulate_bf16(_p(mixed), _p(term), _p(route_weights), rows, expert_idx, num_experts, H, _s()))


def moe_gather_all_u8(src, dst, row_indices, counts, offsets, rows, num_experts, width):
    check(_L().cf_moe_gather_all_u8(_p(src), _p(dst), _p(row_indices), _p(counts), _p(offsets), rows, num_experts, width, _s()))


def moe_combine_all_bf16(mixed, compact, route_weights, row_indices, counts, offsets, rows, num_experts, H):
    check(_L().cf_moe_combine_all_bf16(_p(mixed), _p(compact), _p(route_weights), _p(row_indices), _p(counts),
                                       _p(offsets), rows, num_experts, H, _s()))


def moe_combine_sorted_bf16(mixed, compact, route_weights, row_indices, counts, offsets, rows, num_experts, H,
                            accumulate=True):
    """One pass over the token rows (ascending dispatch lists): mixed is read (accumulate) or started from zero, and
    written once; equals zero-fill + moe_combine_all_bf16 bit for bit."""
    check(_L().cf_moe_combine_sorted_bf16(_p(mixed), _p(compact), _p(route_weights), _p(row_indices), _p(counts),
                                          _p(offsets), rows, num_experts, H, int(accumulate), _s()))


def moe_expand_route_replicas(route_weights, replica_weights, rows, num_experts, num_replicas, replica_start,
                              replica_cum_share, first_row=0):
    """[rows, E] sparse route weights -> [rows, V] over expert replicas (one replica per selected expert and row)."""
    check(_L().cf_moe_expand_route_replicas(_p(route_weights), _p(replica_weights), rows, num_experts, num_replicas,
                                            _p(replica_start), _p(replica_cum_share), int(first_row) & 0xffffffff, _s()))


def moe_route_dispatch_scratch_ints(rows, num_lists):
    return int(_L().cf_moe_route_dispatch_scratch_ints(rows, num_lists))


def moe_route_dispatch_lists(scores, rows, num_experts, top_k, counts, offsets, row_indices, scratch, normalize=True,
                             replica_weights=None, num_replicas=0, replica_start=None, replica_cum_share=None, first_row=0,
                             row_sum_save=None, scores_save=None):
    """Route + (replica choice) + ascending dispatch lists + counts + offsets in one call: the outputs of
    moe_topk_route_f32, [moe_expand_route_replicas,] moe_build_expert_row_lists and moe_expert_offsets_from_counts."""
    check(_L().cf_moe_route_dispatch_lists(_p(scores), rows, num_experts, top_k, int(normalize), _p(row_sum_save),
                                           _p(scores_save), _p(replica_weights), num_replicas, _p(replica_start),
                                           _p(replica_cum_share), int(first_row) & 0xffffffff, _p(counts), _p(offsets),
                                           _p(row_indices), _p(scratch), scratch.numel(), _s()))


def peer_barrier(ctx, flag_arrays, world, rank, epoch, limit_ms=2000):
    """Barrier between the ranks of one box done by the GPUs (flag words in peer-mapped memory); flag_arrays: int64
    device tensor of the ranks' flag-array addresses as mapped in this process."""
    check(_L().cf_peer_barrier(ctx.handle, _p(flag_arrays), world, rank, int(epoch) & 0xffffffff, int(limit_ms), _s()))


def peer_share_i32(ctx, src, n, tables, flag_arrays, world, rank, epoch, limit_ms=2000):
    """This rank's n int32 words into row `rank` of every rank's [world, n] table, then the flag-word barrier, in one
    launch (tables / flag_arrays: int64 device tensors of addresses as mapped in this process)."""
    check(_L().cf_peer_share_i32(ctx.handle, _p(src), int(n), _p(tables), _p(flag_arrays), world, rank,
                                 int(epoch) & 0xffffffff, int(limit_ms), _s()))


ROW_RUN_BYTES = 24      # sizeof(cf_row_run): two int64 and two int32


def moe_ep_plan(counts_all, world, rank, num_replicas, range_lo, range_hi, send_runs, group_counts, group_offsets,
                return_runs, recv_capacity_rows=0, ctx=None):
    """Device-side plan of one expert-parallel layer from the gathered count table (no host copy)."""
    check(_L().cf_moe_ep_plan(_p(counts_all), world, rank, num_replicas, _p(range_lo), _p(range_hi), _p(send_runs),
                              _p(group_counts), _p(group_offsets), _p(return_runs), int(recv_capacity_rows),
                              ctx.handle if ctx is not None else None, _s()))


def moe_send_row_runs(src, row_indices, index_stride, runs, num_runs, max_rows_per_run, dst_bases, row_bytes,
                      num_dst, dst_rows, tag_value=None, tag_bases=None, ctx=None):
    """Copies planned runs of rows into (peer) destination buffers; optional gather through an index table and a
    per-row float tag. dst_bases / tag_bases: int64 device tensors of num_dst base addresses of dst_rows rows each; a
    run that leaves its destination is skipped and reported through ctx.poll_status()."""
    check(_L().cf_moe_send_row_runs(_p(src), _p(row_indices), index_stride, _p(runs), num_runs, max_rows_per_run,
                                    _p(dst_bases), row_bytes, _p(tag_value), _p(tag_bases), int(num_dst), int(dst_rows),
                                    ctx.handle if ctx is not None else None, _s()))


def gemm_fp8_nt_grouped_return(ctx, num_groups, max_total_rows, N, K, counts, offsets, A, lda, a_is_e5m2, a_descale, B,
                               b_descale, return_runs, runs_per_group, dst_ptrs, dst_rows, ldc):
    """Ragged grouped GEMM whose epilogue stores every run of rows into its destination buffer (dst_ptrs: device
    addresses as mapped in this process, one per rank)."""
    arr = (C.c_void_p * len(dst_ptrs))(*[C.c_void_p(int(x)) for x in dst_ptrs])
    check(_L().cf_gemm_fp8_nt_grouped_return(ctx.handle, num_groups, max_total_rows, N, K, _p(counts), _p(offsets), _p(A),
                                             lda, int(a_is_e5m2), _p(a_descale), _p(B), _p(b_descale), _p(return_runs),
                                             runs_per_group, arr, len(dst_ptrs), dst_rows, ldc, _s()))


def moe_grouped_expert_forward_fp8(ctx, hidden, fcin_descale, fcin_is_e5m2, route_weights, counts, offsets, row_indices,
                                   fc_in_w, fc_in_descale, fc_out_w, fc_out_descale, mixed, rows, H, Ie, num_experts,
                                   total_selected_rows):
    check(_L().cf_moe_grouped_expert_forward_fp8(ctx.handle, _p(hidden), _p(fcin_descale), int(fcin_is_e5m2),
                                                 _p(route_weights), _p(counts), _p(offsets), _p(row_indices),
                                                 _p(fc_in_w), _p(fc_in_descale), _p(fc_out_w), _p(fc_out_descale),
                                                 _p(mixed), rows, H, Ie, num_experts, total_selected_rows, _s()))


# ---------------------------------------------------------------- composites: SwiGLU MLP (per-token scales) and MoE SwiGLU experts
def swiglu_mlp_fp8_rowwise(ctx, x, w_gateup8, w_gateup_descale, w_down8, w_down_descale, y, work=None):
    """Llama-style SwiGLU MLP in FP8 with per-token activation scales and per-output-channel weight scales
    (the reference has per-tensor scales only, so this follows the documented generalisation
    C[m,n] = dA[m] * dW[n] * acc):
        x8, dx   = rowwise_quant(x)                      [M,H]
        gu       = x8 . w_gateup8^T  (scales dx, dWgu)   [M,2F]  gate = gu[:, :F], up = gu[:, F:]
        h8, dh   = rowwise_quant(bf16(silu(gate) * up))  [M,F]
        y        = h8 . w_down8^T    (scales dh, dWd)    [M,H]
    w_gateup8 is [2F,H] (gate rows first), w_down8 is [H,F]; descales are float[2F] / float[H]."""
    M, H = x.shape
    F2 = w_gateup8.shape[0]
    F = F2 // 2
    dev = x.device
    if work is None:
        work = {}
    x8 = work.setdefault("x8", torch.empty((M, H), dtype=torch.uint8, device=dev))
    dx = work.setdefault("dx", torch.empty(M, dtype=torch.float32, device=dev))
    gu = work.setdefault("gu", torch.empty((M, F2), dtype=torch.bfloat16, device=dev))
    h8 = work.setdefault("h8", torch.empty((M, F), dtype=torch.uint8, device=dev))
    dh = work.setdefault("dh", torch.empty(M, dtype=torch.float32, device=dev))
    one = work.setdefault("one", torch.ones(4, dtype=torch.float32, device=dev))
    fp8_quantize_rowwise_e4m3(x, x8, dx)
    lt_gemm_fp8_nt(ctx, M, F2, H, x8, H, False, one, w_gateup8, one, gu, F2, a_row_descale=dx,
                   b_col_descale=w_gateup_descale)
    swiglu_quantize_rowwise_e4m3(gu, gu.view(-1)[F:], h8, dh, M, F, F2)
    lt_gemm_fp8_nt(ctx, M, y.shape[1], F, h8, F, False, one, w_down8, one, y, y.stride(0), a_row_descale=dh,
                   b_col_descale=w_down_descale)
    return work


def swiglu_mlp_fp8_rowwise_fused(ctx, x, w_gateup8_il, w_gateup_descale_il, w_down8, w_down_descale, y, work=None,
                                 amax_allreduce=None, down=None):
    """The same MLP as swiglu_mlp_fp8_rowwise with the [M, 2F] bf16 gate/up intermediate fused away: the gate/up GEMM's
    epilogue writes h = bf16(silu(gate) * up) as bf16 [M, F] and records max|h| per row, one row-wise pass quantises h
    with that amax, the down GEMM follows. Bit-identical to the unfused composite. w_gateup8_il is the [2F, H] weight in
    the 32-row interleaved layout (fp8_interleave_gate_up) with its per-row descales interleaved the same way
    (interleave_gate_up_vector).
    Sharded use (gate/up split by output features, down by its contraction dimension): F is this rank's share,
    amax_allreduce(row_amax) max-reduces the per-row amax over the ranks before the quantiser, and down(h8, dh) replaces
    the local down GEMM (partial products that the caller sums across ranks)."""
    M, H = x.shape
    F = w_gateup8_il.shape[0] // 2
    dev = x.device
    if work is None:
        work = {}
    x8 = work.setdefault("x8", torch.empty((M, H), dtype=torch.uint8, device=dev))
    dx = work.setdefault("dx", torch.empty(M, dtype=torch.float32, device=dev))
    h = work.setdefault("h", torch.empty((M, F), dtype=torch.bfloat16, device=dev))
    h8 = work.setdefault("h8", torch.empty((M, F), dtype=torch.uint8, device=dev))
    hmax = work.setdefault("hmax", torch.empty(M, dtype=torch.float32, device=dev))
    dh = work.setdefault("dh", torch.empty(M, dtype=torch.float32, device=dev))
    one = work.setdefault("one", torch.ones(4, dtype=torch.float32, device=dev))
    fp8_quantize_rowwise_e4m3(x, x8, dx)
    hmax.zero_()
    gemm_fp8_swiglu_bf16_rowamax(ctx, M, F, H, x8, H, False, None, dx, w_gateup8_il, None, w_gateup_descale_il, h, hmax)
    if amax_allreduce is not None:
        amax_allreduce(hmax)
    fp8_quantize_rowwise_given_amax_e4m3(h, h8, hmax, dh)
    if down is not None:
        down(h8, dh)
    else:
        lt_gemm_fp8_nt(ctx, M, y.shape[1], F, h8, F, False, one, w_down8, one, y, y.stride(0), a_row_descale=dh,
                       b_col_descale=w_down_descale)
    return work


class MoeSwigluFp8:
    """Top-k routed SwiGLU experts in FP8: route -> dispatch lists -> per-tensor delayed-scale
    quantise of x -> permute -> ragged gate/up GEMM -> SwiGLU + delayed-scale re-quantise -> ragged down GEMM ->
    unpermute + weighted combine. Everything is scheduled on the device (no host copy of the counts); the
    rounding points are those of the reference's SwiGLU expert maths (src/trainer.cu:6510-6529) combined with its
    FP8 quantise / GEMM semantics. Weights: w_gateup8 [E,2F,H] and w_down8 [E,H,F] with one per-tensor descale each."""

    def __init__(self, ctx, rows, H, F, E, top_k, device="cuda", fused_swiglu=False):
        """fused_swiglu: gate/up GEMM, SwiGLU and re-quantise run as one launch (cf_gemm_fp8_swiglu_quant_act) and the
        [T, 2F] bf16 intermediate is never materialised; forward() then expects w_gateup8 in the interleaved layout."""
        self.ctx, self.rows, self.H, self.F, self.E, self.k = ctx, rows, H, F, E, top_k
        self.fused_swiglu = fused_swiglu
        T = rows * top_k
        self.T = T
        self.counts = torch.zeros(E, dtype=torch.int32, device=device)
        self.offsets = torch.zeros(E, dtype=torch.int32, device=device)
        self.idx = torch.zeros((E, rows), dtype=torch.int32, device=device)
        self.x8 = torch.empty((rows, H), dtype=torch.uint8, device=device)
        self.xc = torch.empty((T, H), dtype=torch.uint8, device=device)
        self.gu = None if fused_swiglu else torch.empty((T, 2 * F), dtype=torch.bfloat16, device=device)
        self.h8 = torch.empty((T, F), dtype=torch.uint8, device=device)
        self.yc = torch.empty((T, H), dtype=torch.bfloat16, device=device)
        self.slot_x = ActSlot(ctx, E4M3_MAX)
        self.slot_h = ActSlot(ctx, E4M3_MAX)
        self.front_scratch = torch.empty(max(1, moe_route_dispatch_scratch_ints(rows, E)), dtype=torch.int32, device=device)

    def forward(self, x, route_weights, w_gateup8, w_gateup_descale, w_down8, w_down_descale, mixed, accumulate=True):
        """route_weights: float32 [rows,E] router logits, overwritten in place by the sparse route weights.
        accumulate=False: mixed is overwritten (as if it had been zero-filled first) instead of added to."""
        rows, H, F, E, T = self.rows, self.H, self.F, self.E, self.T
        moe_route_dispatch_lists(route_weights, rows, E, self.k, self.counts, self.offsets, self.idx, self.front_scratch)
        fp8_quant_act(self.ctx, self.slot_x, x, self.x8)
        moe_gather_all_u8(self.x8, self.xc, self.idx, self.counts, self.offsets, rows, E, H)
        if self.fused_swiglu:
            gemm_fp8_swiglu_quant_act(self.ctx, self.slot_h, E, E, None, T, F, H, self.counts, self.offsets, self.xc, H, False,
                                      _DevPtr(self.slot_x.c.descale_snapshot), False, w_gateup8, w_gateup_descale, self.h8, F)
        else:
            gemm_fp8_nt_grouped(self.ctx, E, T, 2 * F, H, self.counts, self.offsets, self.xc, H, False,
                                _DevPtr(self.slot_x.c.descale_snapshot), False, w_gateup8, w_gateup_descale, self.gu, 2 * F)
            fp8_swiglu_quant_act(self.ctx, self.slot_h, self.gu, self.gu.view(-1)[F:], 2 * F, T, F, self.h8)
        gemm_fp8_nt_grouped(self.ctx, E, T, H, F, self.counts, self.offsets, self.h8, F, False,
                            _DevPtr(self.slot_h.c.descale_snapshot), False, w_down8, w_down_descale, self.yc, H)
        moe_combine_sorted_bf16(mixed, self.yc, route_weights, self.idx, self.counts, self.offsets, rows, E, H, accumulate)


class _DevPtr:
    """Wraps a raw device address so that it can be passed where a tensor is expected."""

    is_cuda = True

    def __init__(self, addr):
        self._addr = addr

    def data_ptr(self):
        return self._addr


class FfnSwigluFp8:
    """The reference's dense FP8 FFN (src/trainer.cu:6296-6322 and :7138-7146) with per-tensor delayed scaling:
    fp8_quant_act(x) -> gate and up GEMMs -> swiglu_forward -> fp8_quant_act -> down GEMM, here as three launches
    after the activation quantise: the gate/up GEMM carries SwiGLU and the re-quantise in its epilogue
    (cf_gemm_fp8_swiglu_quant_act), so the [M, 2F] bf16 intermediate is never written. `w_gateup8_interleaved` is the
    [2F, H] E4M3 tensor in the 32-row interleaved layout (fp8_interleave_gate_up), w_down8 is [H, F]."""

    def __init__(self, ctx, M, H, F, device="cuda"):
        self.ctx, self.M, self.H, self.F = ctx, M, H, F
        self.x8 = torch.empty((M, H), dtype=torch.uint8, device=device)
        self.h8 = torch.empty((M, F), dtype=torch.uint8, device=device)
        self.slot_x = ActSlot(ctx, E4M3_MAX)
        self.slot_h = ActSlot(ctx, E4M3_MAX)

    def forward(self, x, w_gateup8_interleaved, w_gateup_descale, w_down8, w_down_descale, y, bias=None, bias_mode=2):
        M, H, F = self.M, self.H, self.F
        fp8_quant_act(self.ctx, self.slot_x, x, self.x8)
        gemm_fp8_swiglu_quant_act(self.ctx, self.slot_h, 1, 1, None, M, F, H, None, None, self.x8, H, False,
                                  _DevPtr(self.slot_x.c.descale_snapshot), False, w_gateup8_interleaved, w_gateup_descale,
                                  self.h8, F)
        lt_gemm_fp8_nt(self.ctx, M, y.shape[1], F, self.h8, F, False, _DevPtr(self.slot_h.c.descale_snapshot), w_down8,
                       w_down_descale, y, y.stride(0), bias=bias, bias_mode=bias_mode)
