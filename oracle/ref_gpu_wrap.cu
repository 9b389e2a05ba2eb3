// C-linkage doorway to the REFERENCE's own CUDA operators (namespace
// ida_native, include/ida_native/kernels.hpp), linked from the reference's
// kernels/fp8.cu, kernels/moe.cu, kernels/activations.cu,
// kernels/lion.cu and kernels/cross_entropy.cu compiled where they lie for sm_100a. Output goes to
// oracle/_ref/libref_gpu.so and is used by the GPU parity tests as the
// reference-on-the-same-GPU comparator. Test infrastructure only.
#include "ida_native/kernels.hpp"
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

using namespace ida_native;
#define S(x) static_cast<cudaStream_t>(x)
#define BF(x) static_cast<const __nv_bfloat16*>(x)
#define BFW(x) static_cast<__nv_bfloat16*>(x)

extern "C" {
int ref_fp8_amax_bf16(const void* x, size_t n, float* amax, void* s) { try { fp8_amax_bf16(BF(x), n, amax, S(s)); } catch (...) { return 1; } return 0; }
int ref_fp8_scale_from_amax(const float* amax, float mx, float* sc, float* de, void* s) { try { fp8_scale_from_amax(amax, mx, sc, de, S(s)); } catch (...) { return 1; } return 0; }
int ref_fp8_quantize_e4m3(const void* x, void* o, const float* sc, size_t n, void* s) { try { fp8_quantize_e4m3(BF(x), o, sc, n, S(s)); } catch (...) { return 1; } return 0; }
int ref_fp8_quantize_e5m2(const void* x, void* o, const float* sc, size_t n, void* s) { try { fp8_quantize_e5m2(BF(x), o, sc, n, S(s)); } catch (...) { return 1; } return 0; }
int ref_fp8_quantize_e4m3_record(const void* x, void* o, const float* sc, float* am, size_t n, void* s) { try { fp8_quantize_e4m3_record(BF(x), o, sc, am, n, S(s)); } catch (...) { return 1; } return 0; }
int ref_fp8_quantize_e5m2_record(const void* x, void* o, const float* sc, float* am, size_t n, void* s) { try { fp8_quantize_e5m2_record(BF(x), o, sc, am, n, S(s)); } catch (...) { return 1; } return 0; }
int ref_fp8_quantize_transpose_e4m3(const void* w, void* o, const float* sc, int K, int N, void* s) { try { fp8_quantize_transpose_e4m3(BF(w), o, sc, K, N, S(s)); } catch (...) { return 1; } return 0; }
int ref_fp8_quant_and_transpose_e4m3(const void* in, void* a8, void* sn, const float* sc, int K, int N, void* s) { try { fp8_quant_and_transpose_e4m3(BF(in), a8, sn, sc, K, N, S(s)); } catch (...) { return 1; } return 0; }
int ref_fp8_update_delayed_scale(const float* am, float mx, float* sc, float* de, float* h, int len, int* cur, int* cnt, void* s) { try { fp8_update_delayed_scale(am, mx, sc, de, h, len, cur, cnt, S(s)); } catch (...) { return 1; } return 0; }
int ref_fp8_clip_probe(const float* am, const float* sc, float mx, float* st, void* s) { try { fp8_clip_probe(am, sc, mx, st, S(s)); } catch (...) { return 1; } return 0; }
int ref_fp8_elem_clip_count(const void* x, const float* sc, float mx, size_t n, float* o, void* s) { try { fp8_elem_clip_count(BF(x), sc, mx, n, o, S(s)); } catch (...) { return 1; } return 0; }
int ref_fp8_pack_bf16_e4m3_raw(const void* x, uint8_t* o, float* am, float* sc, float* de, int* bad, size_t n, void* s) { try { fp8_pack_bf16_e4m3_raw(BF(x), o, am, sc, de, bad, n, S(s)); } catch (...) { return 1; } return 0; }
int ref_fp8_pack_bf16_e4m3_raw_and_dequant(const void* x, uint8_t* o, void* dq, float* am, float* sc, float* de, int* bad, size_t n, void* s) { try { fp8_pack_bf16_e4m3_raw_and_dequant(BF(x), o, BFW(dq), am, sc, de, bad, n, S(s)); } catch (...) { return 1; } return 0; }
int ref_fp8_unpack_e4m3_raw_bf16(const uint8_t* in, const float* de, void* o, size_t n, void* s) { try { fp8_unpack_e4m3_raw_bf16(in, de, BFW(o), n, S(s)); } catch (...) { return 1; } return 0; }

int ref_lion_step_f32(void* w, float* m, const float* g, size_t n, float lr, float b1, float b2, float wd, void* s, float* amax, unsigned seed) { try { lion_step(BFW(w), m, g, n, lr, b1, b2, wd, S(s), amax, seed); } catch (...) { return 1; } return 0; }
int ref_lion_step_bf16(void* w, void* m, const float* g, size_t n, float lr, float b1, float b2, float wd, void* s, float* amax, unsigned seed) { try { lion_step(BFW(w), BFW(m), g, n, lr, b1, b2, wd, S(s), amax, seed); } catch (...) { return 1; } return 0; }

int ref_rmsnorm_forward(const void* x, const void* g, void* o, float* rms, int rows, int H, float eps, void* s) { try { rmsnorm_forward(BF(x), BF(g), BFW(o), rms, rows, H, eps, S(s)); } catch (...) { return 1; } return 0; }
int ref_swiglu_forward(const void* g, const void* u, void* o, int n, void* s) { try { swiglu_forward(BF(g), BF(u), BFW(o), n, S(s)); } catch (...) { return 1; } return 0; }
int ref_gelu_forward(const void* x, void* o, size_t n, void* s) { try { gelu_forward(BF(x), BFW(o), n, S(s)); } catch (...) { return 1; } return 0; }
int ref_bias_add_strided_bf16(void* io, const void* b, int rows, int cols, int stride, int base, void* s) { try { bias_add_strided_bf16(BFW(io), BF(b), rows, cols, stride, base, S(s)); } catch (...) { return 1; } return 0; }
int ref_moe_topk_route_f32(float* sc, int rows, int E, int k, void* s) { try { moe_topk_route_f32(sc, rows, E, k, S(s)); } catch (...) { return 1; } return 0; }
int ref_moe_build_expert_row_lists(const float* rw, int* cnt, int* idx, int rows, int E, void* s) { try { moe_build_expert_row_lists(rw, cnt, idx, rows, E, S(s)); } catch (...) { return 1; } return 0; }
int ref_moe_expert_offsets_from_counts(const int* cnt, int* off, int E, void* s) { try { moe_expert_offsets_from_counts(cnt, off, E, S(s)); } catch (...) { return 1; } return 0; }
int ref_moe_gather_rows_u8(const uint8_t* src, uint8_t* dst, const int* idx, int n, int w, void* s) { try { moe_gather_rows_u8(src, dst, idx, n, w, S(s)); } catch (...) { return 1; } return 0; }
int ref_moe_gather_rows_bf16(const void* src, void* dst, const int* idx, int n, int w, void* s) { try { moe_gather_rows_bf16(BF(src), BFW(dst), idx, n, w, S(s)); } catch (...) { return 1; } return 0; }
int ref_moe_scatter_accumulate_rows_bf16(void* mixed, const void* compact, const float* rw, const int* idx, int n, int e, int E, int H, void* s) { try { moe_scatter_accumulate_rows_bf16(BFW(mixed), BF(compact), rw, idx, n, e, E, H, S(s)); } catch (...) { return 1; } return 0; }
int ref_moe_scale_accumulate_bf16(void* mixed, const void* term, const float* rw, int rows, int e, int E, int H, void* s) { try { moe_scale_accumulate_bf16(BFW(mixed), BF(term), rw, rows, e, E, H, S(s)); } catch (...) { return 1; } return 0; }
int ref_moe_grouped_expert_forward_fp8(const void* hid, const float* dx, int e5, const float* rw, const int* cnt, const int* off, const int* idx, const void* win, const float* dwin, const void* wout, const float* dwout, void* mixed, int rows, int H, int Ie, int E, int total, void* s) {
    // The reference kernel covers at most 1024 threads x 8 = 8192 output columns
    // (kernels/moe.cu:1089-1091); wider layers are outside its valid range.
    if (H > 8192 || Ie > 8192) return 2;
    try { moe_grouped_expert_forward_fp8(hid, dx, e5, rw, cnt, off, idx, win, dwin, wout, dwout, BFW(mixed), rows, H, Ie, E, total, S(s)); } catch (...) { return 1; }
    return 0;
}
}
