// Lion optimiser step with stochastic-rounding bf16 weight write and the fused per-tensor weight amax that feeds
// the FP8 weight refresh (kernels/lion.cu:39-144). The amax is taken on the fp32 value BEFORE rounding, as the
// reference does; refresh_fp8_weights(recompute_amax = false) then quantises with it (src/trainer.cu:10795-10855).
//
// Arithmetic is written expression for expression like the reference kernel so that the compiler contracts the same
// multiply-adds; the hash that drives the stochastic rounding is a pure function of (element index, seed).
#include "cf_common.cuh"
#include "cf_lion.cuh"

namespace cf {
namespace {

constexpr int kLT = 256;

// 8 elements per thread and iteration: 16-byte weight access, two 16-byte gradient / fp32-momentum accesses (the
// gradient is read once: streaming loads).
__device__ __forceinline__ float4 ld_stream_f4(const float* p) {
    float4 v;
    asm volatile("ld.global.cs.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

template <bool BF16_STATE>
__global__ void __launch_bounds__(kLT) k_lion(uint16_t* __restrict__ w, void* __restrict__ mstate,
                                              const float* __restrict__ grad, size_t n, float lr, float beta1, float beta2,
                                              float wd, float* __restrict__ amax_out, unsigned sr_seed, int vec) {
    float local = 0.0f;
    const size_t stride = static_cast<size_t>(gridDim.x) * kLT;
    const size_t nvec = vec ? n / 8 : 0;
    for (size_t v = static_cast<size_t>(blockIdx.x) * kLT + threadIdx.x; v < nvec; v += stride) {
        const size_t i0 = v * 8;
        const float4 g0 = ld_stream_f4(grad + i0), g1 = ld_stream_f4(grad + i0 + 4);
        const uint4 w4 = *reinterpret_cast<const uint4*>(w + i0);
        float mp[8];
        if (BF16_STATE) {
            const uint4 m4 = *reinterpret_cast<const uint4*>(static_cast<uint16_t*>(mstate) + i0);
            mp[0] = __uint_as_float(m4.x << 16); mp[1] = __uint_as_float(m4.x & 0xffff0000u);
            mp[2] = __uint_as_float(m4.y << 16); mp[3] = __uint_as_float(m4.y & 0xffff0000u);
            mp[4] = __uint_as_float(m4.z << 16); mp[5] = __uint_as_float(m4.z & 0xffff0000u);
            mp[6] = __uint_as_float(m4.w << 16); mp[7] = __uint_as_float(m4.w & 0xffff0000u);
        } else {
            const float4 m0 = *reinterpret_cast<const float4*>(static_cast<float*>(mstate) + i0);
            const float4 m1 = *reinterpret_cast<const float4*>(static_cast<float*>(mstate) + i0 + 4);
            mp[0] = m0.x; mp[1] = m0.y; mp[2] = m0.z; mp[3] = m0.w; mp[4] = m1.x; mp[5] = m1.y; mp[6] = m1.z; mp[7] = m1.w;
        }
        const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const float wf[8] = {__uint_as_float(w4.x << 16), __uint_as_float(w4.x & 0xffff0000u),
                             __uint_as_float(w4.y << 16), __uint_as_float(w4.y & 0xffff0000u),
                             __uint_as_float(w4.z << 16), __uint_as_float(w4.z & 0xffff0000u),
                             __uint_as_float(w4.w << 16), __uint_as_float(w4.w & 0xffff0000u)};
        uint16_t wn[8], mn16[8];
        float mn[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float w_new;
            lion_elem(g[e], mp[e], wf[e], lr, beta1, beta2, wd, mn[e], w_new);
            const unsigned h = sr_hash(i0 + e, sr_seed);
            if (BF16_STATE) mn16[e] = f32_to_bf16_sr(mn[e], h ^ 0x9e3779b9u);
            wn[e] = f32_to_bf16_sr(w_new, h);
            local = fmaxf(local, fabsf(w_new));
        }
        *reinterpret_cast<uint4*>(w + i0) =
            make_uint4(wn[0] | (static_cast<uint32_t>(wn[1]) << 16), wn[2] | (static_cast<uint32_t>(wn[3]) << 16),
                       wn[4] | (static_cast<uint32_t>(wn[5]) << 16), wn[6] | (static_cast<uint32_t>(wn[7]) << 16));
        if (BF16_STATE) {
            *reinterpret_cast<uint4*>(static_cast<uint16_t*>(mstate) + i0) =
                make_uint4(mn16[0] | (static_cast<uint32_t>(mn16[1]) << 16), mn16[2] | (static_cast<uint32_t>(mn16[3]) << 16),
                           mn16[4] | (static_cast<uint32_t>(mn16[5]) << 16), mn16[6] | (static_cast<uint32_t>(mn16[7]) << 16));
        } else {
            float* md = static_cast<float*>(mstate) + i0;
            *reinterpret_cast<float4*>(md) = make_float4(mn[0], mn[1], mn[2], mn[3]);
            *reinterpret_cast<float4*>(md + 4) = make_float4(mn[4], mn[5], mn[6], mn[7]);
        }
    }
    for (size_t i = nvec * 8 + static_cast<size_t>(blockIdx.x) * kLT + threadIdx.x; i < n; i += stride) {
        const float gg = grad[i];
        const float m_prev = BF16_STATE ? bf16_bits_to_f32(static_cast<uint16_t*>(mstate)[i]) : static_cast<float*>(mstate)[i];
        const float w_f32 = bf16_bits_to_f32(w[i]);
        float m_new, w_new;
        lion_elem(gg, m_prev, w_f32, lr, beta1, beta2, wd, m_new, w_new);
        const unsigned h = sr_hash(i, sr_seed);
        if (BF16_STATE) static_cast<uint16_t*>(mstate)[i] = f32_to_bf16_sr(m_new, h ^ 0x9e3779b9u);
        else static_cast<float*>(mstate)[i] = m_new;
        w[i] = f32_to_bf16_sr(w_new, h);
        local = fmaxf(local, fabsf(w_new));
    }
    if (amax_out) block_amax_commit(local, amax_out);
}

template <bool BF16_STATE>
int launch_lion(void* w, void* m, const float* grad, size_t n, float lr, float b1, float b2, float wd, float* amax,
                unsigned seed, cudaStream_t st) {
    if (n == 0) return CF_OK;
    const int vec = ((reinterpret_cast<uintptr_t>(w) % 16) == 0) && ((reinterpret_cast<uintptr_t>(grad) % 16) == 0) &&
                    ((reinterpret_cast<uintptr_t>(m) % 16) == 0);
    size_t blocks = (n / 8 + kLT - 1) / kLT;
    if (blocks < 1) blocks = 1;
    const size_t cap = static_cast<size_t>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    k_lion<BF16_STATE><<<static_cast<unsigned>(blocks), kLT, 0, st>>>(static_cast<uint16_t*>(w), m, grad, n, lr, b1, b2, wd,
                                                                      amax, seed, vec);
    CF_LAUNCH_CHECK("lion_step");
    return CF_OK;
}

}  // namespace
}  // namespace cf

using namespace cf;

static int lion_quant_entry(void* w, void* m, const float* grad, int rows, int cols, float lr, float b1, float b2, float wd,
                            float* amax, unsigned seed, const float* quant_amax, float* scale_out, float* descale_out, void* w8,
                            void* w8_t, int bf16_state, cudaStream_t st) {
    if (rows == 0 || cols == 0) return CF_OK;
    LionArgs la;
    la.w = static_cast<uint16_t*>(w); la.mstate = m; la.grad = grad;
    la.lr = lr; la.beta1 = b1; la.beta2 = b2; la.wd = wd;
    la.amax_out = amax; la.sr_seed = seed; la.bf16_state = bf16_state;
    ScaleFromAmax sfa;
    sfa.amax = quant_amax; sfa.fp8_max = CF_E4M3_MAX; sfa.scale_out = scale_out; sfa.descale_out = descale_out;
    return lion_quant_tile_launch(la, w8, w8_t, sfa, rows, cols, st);
}

extern "C" {

int cf_lion_step_f32_state(void* d_w, float* d_m, const float* d_grad, size_t n, float lr, float beta1, float beta2, float wd,
                           void* stream, float* d_weight_amax, unsigned sr_seed) {
    CF_REQUIRE(n == 0 || (d_w && d_m && d_grad), "cf_lion_step_f32_state: null pointer");
    return launch_lion<false>(d_w, d_m, d_grad, n, lr, beta1, beta2, wd, d_weight_amax, sr_seed, as_stream(stream));
}

int cf_lion_step_bf16_state(void* d_w, void* d_m, const float* d_grad, size_t n, float lr, float beta1, float beta2, float wd,
                            void* stream, float* d_weight_amax, unsigned sr_seed) {
    CF_REQUIRE(n == 0 || (d_w && d_m && d_grad), "cf_lion_step_bf16_state: null pointer");
    return launch_lion<true>(d_w, d_m, d_grad, n, lr, beta1, beta2, wd, d_weight_amax, sr_seed, as_stream(stream));
}

int cf_lion_step_f32_state_quantize(void* d_w, float* d_m, const float* d_grad, int rows, int cols, float lr, float beta1,
                                    float beta2, float wd, void* stream, float* d_weight_amax, unsigned sr_seed,
                                    const float* d_quant_amax, float* d_scale_out, float* d_descale_out, void* d_w8,
                                    void* d_w8_transposed_or_null) {
    CF_REQUIRE(rows >= 0 && cols >= 0, "cf_lion_step_f32_state_quantize: negative shape");
    CF_REQUIRE((rows == 0 || cols == 0) || (d_w && d_m && d_grad && d_quant_amax && d_scale_out && d_descale_out && d_w8),
               "cf_lion_step_f32_state_quantize: null pointer");
    CF_REQUIRE(d_weight_amax != d_quant_amax, "cf_lion_step_f32_state_quantize: the amax to quantise with and the amax being recorded must be different words");
    return lion_quant_entry(d_w, d_m, d_grad, rows, cols, lr, beta1, beta2, wd, d_weight_amax, sr_seed, d_quant_amax, d_scale_out,
                            d_descale_out, d_w8, d_w8_transposed_or_null, 0, as_stream(stream));
}

int cf_lion_step_bf16_state_quantize(void* d_w, void* d_m, const float* d_grad, int rows, int cols, float lr, float beta1,
                                     float beta2, float wd, void* stream, float* d_weight_amax, unsigned sr_seed,
                                     const float* d_quant_amax, float* d_scale_out, float* d_descale_out, void* d_w8,
                                     void* d_w8_transposed_or_null) {
    CF_REQUIRE(rows >= 0 && cols >= 0, "cf_lion_step_bf16_state_quantize: negative shape");
    CF_REQUIRE((rows == 0 || cols == 0) || (d_w && d_m && d_grad && d_quant_amax && d_scale_out && d_descale_out && d_w8),
               "cf_lion_step_bf16_state_quantize: null pointer");
    CF_REQUIRE(d_weight_amax != d_quant_amax, "cf_lion_step_bf16_state_quantize: the amax to quantise with and the amax being recorded must be different words");
    return lion_quant_entry(d_w, d_m, d_grad, rows, cols, lr, beta1, beta2, wd, d_weight_amax, sr_seed, d_quant_amax, d_scale_out,
                            d_descale_out, d_w8, d_w8_transposed_or_null, 1, as_stream(stream));
}

}  // extern "C"
