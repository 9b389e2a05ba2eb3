"""ctypes binding of libcanopy_fp8.so (the C ABI declared in include/canopy_fp8.h).

The library is the product; this module only loads it and declares signatures. There is no
fallback: when the shared object is missing the import fails with a build hint.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libcanopy_fp8.so")

CF_OK, CF_ERR_INVALID_ARG, CF_ERR_UNSUPPORTED, CF_ERR_CUDA, CF_ERR_DEVICE_WAIT, CF_ERR_LIMIT, CF_ERR_DEVICE_RANGE = range(7)
ABI_VERSION = 3        # cf_abi_version() of the library this table was written for
E4M3_MAX = 448.0
E5M2_MAX = 57344.0

vp = C.c_void_p
fp = C.c_void_p      # float* on the device
ip = C.c_void_p      # int* on the device
sz = C.c_size_t
ci = C.c_int
cf = C.c_float


class GemmEpilogue(C.Structure):
    _fields_ = [("d_bias", vp), ("bias_mode", ci), ("d_a_row_descale", fp), ("d_b_col_descale", fp), ("out_fp32", ci)]


class ActSlotStruct(C.Structure):
    _fields_ = [("amax", fp), ("scale", fp), ("descale", fp), ("history", fp), ("history_cursor", ip),
                ("history_count", ip), ("scale_snapshot", fp), ("descale_snapshot", fp), ("fp8_max", cf),
                ("init", ci), ("calib_remaining", ci), ("calib_commit_pending", ci), ("calib_min", fp),
                ("calib_max", fp), ("ticket", vp)]


EP_MAX_EXPERTS, EP_MAX_RANKS = 256, 64
EP_MAX_REPLICAS = EP_MAX_EXPERTS + EP_MAX_RANKS


class EpPlacementStruct(C.Structure):
    _fields_ = [("world", ci), ("num_experts", ci), ("num_replicas", ci), ("replica_expert", ci * EP_MAX_REPLICAS),
                ("replica_rank", ci * EP_MAX_REPLICAS), ("replica_share", C.c_double * EP_MAX_REPLICAS),
                ("replica_cum_share", C.c_double * EP_MAX_REPLICAS), ("replica_start", ci * (EP_MAX_EXPERTS + 1)),
                ("rank_lo", ci * EP_MAX_RANKS), ("rank_hi", ci * EP_MAX_RANKS)]


class Fp8WeightStruct(C.Structure):
    _fields_ = [("w", vp), ("fwd8", vp), ("bwd8", vp), ("amax", fp), ("scale", fp), ("descale", fp),
                ("in_dim", ci), ("out_dim", ci), ("stored_out_major", ci)]


# name -> (restype, argtypes); every symbol include/canopy_fp8.h declares
SIGNATURES = {
    "cf_last_error": (C.c_char_p, []),
    "cf_abi_version": (ci, []),
    "cf_launch_count": (C.c_uint64, []),
    "cf_fp8_amax_bf16": (ci, [vp, sz, fp, vp]),
    "cf_fp8_scale_from_amax": (ci, [fp, cf, fp, fp, vp]),
    "cf_fp8_quantize_e4m3": (ci, [vp, vp, fp, sz, vp]),
    "cf_fp8_quantize_e5m2": (ci, [vp, vp, fp, sz, vp]),
    "cf_fp8_quantize_e4m3_record": (ci, [vp, vp, fp, fp, sz, vp]),
    "cf_fp8_quantize_e5m2_record": (ci, [vp, vp, fp, fp, sz, vp]),
    "cf_fp8_update_delayed_scale": (ci, [fp, cf, fp, fp, fp, ci, ip, ip, vp]),
    "cf_fp8_quantize_transpose_e4m3": (ci, [vp, vp, fp, ci, ci, vp]),
    "cf_fp8_quant_and_transpose_e4m3": (ci, [vp, vp, vp, fp, ci, ci, vp]),
    "cf_transpose_u8": (ci, [vp, vp, ci, ci, vp]),
    "cf_fp8_clip_probe": (ci, [fp, fp, cf, fp, vp]),
    "cf_fp8_elem_clip_count": (ci, [vp, fp, cf, sz, fp, vp]),
    "cf_fp8_pack_bf16_e4m3_raw": (ci, [vp, vp, fp, fp, fp, ip, sz, vp]),
    "cf_fp8_pack_bf16_e4m3_raw_and_dequant": (ci, [vp, vp, vp, fp, fp, fp, ip, sz, vp]),
    "cf_fp8_unpack_e4m3_raw_bf16": (ci, [vp, fp, vp, sz, vp]),
    "cf_fp8_calib_minmax_update": (ci, [fp, fp, fp, vp]),
    "cf_ctx_create": (ci, [C.POINTER(vp), sz]),
    "cf_ctx_destroy": (ci, [vp]),
    "cf_ctx_act8": (vp, [vp]),
    "cf_ctx_poll_status": (ci, [vp, vp]),
    "cf_ctx_reserve_workspace": (ci, [vp, sz]),
    "cf_ctx_selftest_bounded_wait": (ci, [vp, ci, vp]),
    "cf_gemm_fp8_nt": (ci, [vp, ci, ci, ci, vp, ci, ci, fp, vp, fp, vp, ci, C.POINTER(GemmEpilogue), vp]),
    "cf_gemm_fp8_tn_accum_f32": (ci, [vp, ci, ci, ci, vp, fp, vp, fp, vp, ci, vp]),
    "cf_gemm_fp8_tn_accum_bf16": (ci, [vp, ci, ci, ci, vp, fp, vp, fp, vp, ci, vp]),
    "cf_gemm_fp8_dw_accum_f32": (ci, [vp, ci, ci, ci, vp, ci, fp, vp, ci, fp, vp, ci, vp]),
    "cf_gemm_fp8_dw_accum_bf16": (ci, [vp, ci, ci, ci, vp, ci, fp, vp, ci, fp, vp, ci, vp]),
    "cf_gemm_fp8_nt_reduce_scatter_f32": (ci, [vp, ci, ci, ci, vp, ci, ci, fp, vp, fp, fp, fp, C.POINTER(vp), ci, vp]),
    "cf_gemm_fp8_swiglu_bf16_rowamax": (ci, [vp, ci, ci, ci, vp, ci, ci, fp, fp, vp, fp, fp, vp, ci, fp, vp]),
    "cf_fp8_quantize_rowwise_given_amax_e4m3": (ci, [vp, ci, vp, ci, fp, fp, fp, ci, ci, vp]),
    "cf_f32_to_bf16_and_zero": (ci, [fp, vp, sz, vp]),
    "cf_gemm_fp8_nn": (ci, [vp, ci, ci, ci, vp, ci, ci, fp, vp, ci, fp, vp, ci, ci, vp]),
    "cf_gemm_fp8_nn_grouped": (ci, [vp, ci, ci, ci, ci, ip, ip, vp, ci, ci, fp, vp, fp, vp, ci, ci, vp]),
    "cf_gemm_fp8_nt_grouped": (ci, [vp, ci, ci, ci, ci, ip, ip, vp, ci, ci, fp, ci, vp, fp, vp, ci, vp]),
    "cf_gemm_fp8_nt_segments": (ci, [vp, ci, ci, ip, ci, ci, ci, ip, ip, vp, ci, ci, fp, ci, vp, fp, vp, ci, vp]),
    "cf_gemm_fp8_nt_segments_scatter": (ci, [vp, ci, ci, ip, ci, ci, ci, ip, ip, vp, ci, ci, fp, ci, vp, fp, vp, vp, vp, ci, vp]),
    "cf_act_slot_init": (ci, [vp, C.POINTER(ActSlotStruct), cf, ci, vp]),
    "cf_fp8_quant_act": (ci, [vp, C.POINTER(ActSlotStruct), vp, sz, vp, vp, ci]),
    "cf_fp8_swiglu_quant_act": (ci, [vp, C.POINTER(ActSlotStruct), vp, vp, ci, ci, ci, vp, vp]),
    "cf_gemm_fp8_swiglu_quant_act": (ci, [vp, C.POINTER(ActSlotStruct), ci, ci, ip, ci, ci, ci, ip, ip, vp, ci, ci, fp, ci, vp, fp, vp, ci, vp]),
    "cf_fp8_interleave_gate_up": (ci, [vp, vp, vp, ci, ci, ci, vp]),
    "cf_refresh_fp8_weight": (ci, [C.POINTER(Fp8WeightStruct), ci, vp]),
    "cf_fp8_linear_forward": (ci, [vp, C.POINTER(ActSlotStruct), vp, ci, ci, vp, fp, ci, vp, ci, vp, ci, vp]),
    "cf_fp8_linear_static_scratch": (ci, [vp, ci, ci, fp, fp, vp, fp, ci, vp, ci, vp, ci, ip, vp]),
    "cf_lion_step_f32_state": (ci, [vp, fp, fp, sz, cf, cf, cf, cf, vp, fp, C.c_uint]),
    "cf_lion_step_bf16_state": (ci, [vp, vp, fp, sz, cf, cf, cf, cf, vp, fp, C.c_uint]),
    "cf_lion_step_f32_state_quantize": (ci, [vp, fp, fp, ci, ci, cf, cf, cf, cf, vp, fp, C.c_uint, fp, fp, fp, vp, vp]),
    "cf_lion_step_bf16_state_quantize": (ci, [vp, vp, fp, ci, ci, cf, cf, cf, cf, vp, fp, C.c_uint, fp, fp, fp, vp, vp]),
    "cf_rmsnorm_forward": (ci, [vp, vp, vp, fp, ci, ci, cf, vp]),
    "cf_rmsnorm_quantize_e4m3_record": (ci, [vp, vp, vp, fp, vp, fp, fp, ci, ci, cf, vp]),
    "cf_rmsnorm_quantize_rowwise_e4m3": (ci, [vp, vp, vp, fp, vp, fp, fp, ci, ci, cf, vp]),
    "cf_fp8_rmsnorm_quant_act": (ci, [vp, C.POINTER(ActSlotStruct), vp, vp, vp, fp, ci, ci, cf, vp, vp]),
    "cf_rmsnorm_clip_forward": (ci, [vp, vp, vp, fp, ci, ci, cf, cf, vp]),
    "cf_rmsnorm_clip_quantize_e4m3_record": (ci, [vp, vp, vp, fp, vp, fp, fp, ci, ci, cf, cf, vp]),
    "cf_fp8_rmsnorm_clip_quant_act": (ci, [vp, C.POINTER(ActSlotStruct), vp, vp, vp, fp, ci, ci, cf, cf, vp, vp]),
    "cf_bias_add_strided_bf16": (ci, [vp, vp, ci, ci, ci, ci, vp]),
    "cf_swiglu_forward": (ci, [vp, vp, vp, ci, vp]),
    "cf_gelu_forward": (ci, [vp, vp, sz, vp]),
    "cf_fp8_quantize_rowwise_e4m3": (ci, [vp, ci, vp, ci, fp, fp, ci, ci, vp]),
    "cf_swiglu_quantize_rowwise_e4m3": (ci, [vp, vp, ci, vp, ci, fp, fp, ci, ci, vp]),
    "cf_swiglu_quantize_e4m3_record": (ci, [vp, vp, ci, vp, ci, fp, fp, ci, ci, vp]),
    "cf_moe_topk_route_f32": (ci, [fp, ci, ci, ci, vp, fp, fp, ci]),
    "cf_moe_build_expert_row_lists": (ci, [fp, ip, ip, ci, ci, vp]),
    "cf_moe_expert_offsets_from_counts": (ci, [ip, ip, ci, vp]),
    "cf_moe_gather_rows_u8": (ci, [vp, vp, ip, ci, ci, vp]),
    "cf_moe_gather_rows_bf16": (ci, [vp, vp, ip, ci, ci, vp]),
    "cf_moe_scatter_accumulate_rows_bf16": (ci, [vp, vp, fp, ip, ci, ci, ci, ci, vp]),
    "cf_moe_scale_accumulate_bf16": (ci, [vp, vp, fp, ci, ci, ci, ci, vp]),
    "cf_moe_gather_all_u8": (ci, [vp, vp, ip, ip, ip, ci, ci, ci, vp]),
    "cf_moe_combine_all_bf16": (ci, [vp, vp, fp, ip, ip, ip, ci, ci, ci, vp]),
    "cf_moe_combine_sorted_bf16": (ci, [vp, vp, fp, ip, ip, ip, ci, ci, ci, ci, vp]),
    "cf_moe_expand_route_replicas": (ci, [fp, fp, ci, ci, ci, ip, fp, C.c_uint, vp]),
    "cf_moe_route_dispatch_scratch_ints": (C.c_size_t, [ci, ci]),
    "cf_moe_route_dispatch_lists": (ci, [fp, ci, ci, ci, ci, fp, fp, fp, ci, ip, fp, C.c_uint, ip, ip, ip, ip, C.c_size_t, vp]),
    "cf_shard_range": (ci, [C.c_longlong, ci, ci, ci, C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)]),
    "cf_ep_placement_build": (ci, [C.POINTER(C.c_double), ci, ci, C.c_double, C.POINTER(EpPlacementStruct)]),
    "cf_ep_placement_build_balanced": (ci, [C.POINTER(C.c_double), ci, ci, C.c_double, C.c_double, ci, C.POINTER(EpPlacementStruct)]),
    "cf_ep_placement_build_weighted": (ci, [C.POINTER(C.c_double), ci, ci, C.c_double, C.c_double, ci, C.POINTER(C.c_double),
                                            C.POINTER(EpPlacementStruct)]),
    "cf_peer_barrier": (ci, [vp, vp, ci, ci, C.c_uint, ci, vp]),
    "cf_peer_share_i32": (ci, [vp, ip, ci, vp, vp, ci, ci, C.c_uint, ci, vp]),
    "cf_moe_ep_plan": (ci, [ip, ci, ci, ci, ip, ip, vp, ip, ip, vp, C.c_longlong, vp, vp]),
    "cf_moe_send_row_runs": (ci, [vp, ip, C.c_longlong, vp, ci, ci, vp, C.c_longlong, fp, vp, ci, C.c_longlong, vp, vp]),
    "cf_gemm_fp8_nt_grouped_return": (ci, [vp, ci, ci, ci, ci, ip, ip, vp, ci, ci, fp, vp, fp, vp, ci, C.POINTER(vp), ci, ci, ci, vp]),
    "cf_moe_grouped_expert_forward_fp8": (ci, [vp, vp, fp, ci, fp, ip, ip, ip, vp, fp, vp, fp, vp, ci, ci, ci, ci, ci, vp]),
}


class CanopyError(RuntimeError):
    """Raised when a C-ABI call returns a non-zero status (the reference's operators throw
    std::runtime_error in the same situations)."""

    def __init__(self, code, message):
        super().__init__(f"libcanopy_fp8 status {code}: {message}")
        self.code = code


def load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "or `make -C canopy-foundry_b200/csrc`. There is no fallback path.")
    lib = C.CDLL(LIB_PATH)
    lib.cf_abi_version.restype = ci
    if lib.cf_abi_version() != ABI_VERSION:
        raise ImportError(f"{LIB_PATH} has ABI version {lib.cf_abi_version()}, this binding expects {ABI_VERSION}: rebuild it")
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)      # AttributeError here means the header and the library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = load()
    return _lib


def check(code):
    if code != CF_OK:
        raise CanopyError(code, lib().cf_last_error().decode("utf-8", "replace"))
