// Lion optimiser step with stochastic-rounding bf16 weight write and the fused per-tensor weight amax that feeds
// the FP8 weight refresh (kernels/lion.cu:39-144). The amax is taken on the fp32 value BEFORE rounding, as the
// reference does; refresh_fp8_weights(recompute_amax = false) then quantises with it (src/trainer.cu:10795-10855).
//
// Arithmetic is written expression for expression like the reference kernel so that the compiler contracts the same
// multiply-adds; the hash that drives the stochastic rounding is a pure function of (element index, seed).
#include "cf_common.cuh"

namespace cf {
namespace {

constexpr int kLT = 256;

// kernels/lion.cu:17-25
__device__ __forceinline__ uint16_t f32_to_bf16_sr(float x, unsigned rnd) {
    unsigned bits = __float_as_uint(x);
    if ((bits & 0x7f800000u) == 0x7f800000u) return __bfloat16_as_ushort(__float2bfloat16(x));
    bits += (rnd & 0xffffu);
    return static_cast<uint16_t>(bits >> 16);
}

__device__ __forceinline__ unsigned sr_hash(size_t i, unsigned seed) {   // kernels/lion.cu:67-68
    unsigned h = static_cast<unsigned>(i) * 2654435761u ^ seed;
    h ^= h >> 16; h *= 0x85ebca6bu; h ^= h >> 13; h *= 0xc2b2ae35u; h ^= h >> 16;
    return h;
}

// One element, written expression for expression like kernels/lion.cu:57-66 / :95-108 so that the compiler makes
// the same multiply-add contraction choices on both the vector and the scalar path.
__device__ __forceinline__ void lion_elem(float g, float m_prev, float w_f32, float lr, float beta1, float beta2, float wd,
                                          float& m_new, float& w_new) {
    const float blend = beta1 * m_prev + (1.0f - beta1) * g;
    const float update = (blend > 0.0f) - (blend < 0.0f);
    m_new = beta2 * m_prev + (1.0f - beta2) * g;
    w_new = w_f32 - lr * (update + wd * w_f32);
}

// 4 elements per thread: 8-byte weight access, 16-byte gradient / fp32-momentum access.
template <bool BF16_STATE>
__global__ void __launch_bounds__(kLT) k_lion(uint16_t* __restrict__ w, void* __restrict__ mstate,
                                              const float* __restrict__ grad, size_t n, float lr, float beta1, float beta2,
                                              float wd, float* __restrict__ amax_out, unsigned sr_seed, int vec) {
    float local = 0.0f;
    const size_t stride = static_cast<size_t>(gridDim.x) * kLT;
    const size_t nvec = vec ? n / 4 : 0;
    for (size_t v = static_cast<size_t>(blockIdx.x) * kLT + threadIdx.x; v < nvec; v += stride) {
        const size_t i0 = v * 4;
        const float4 g4 = *reinterpret_cast<const float4*>(grad + i0);
        const uint2 w2 = *reinterpret_cast<const uint2*>(w + i0);
        float mp[4];
        if (BF16_STATE) {
            const uint2 m2 = *reinterpret_cast<const uint2*>(static_cast<uint16_t*>(mstate) + i0);
            mp[0] = __uint_as_float(m2.x << 16); mp[1] = __uint_as_float(m2.x & 0xffff0000u);
            mp[2] = __uint_as_float(m2.y << 16); mp[3] = __uint_as_float(m2.y & 0xffff0000u);
        } else {
            const float4 m4 = *reinterpret_cast<const float4*>(static_cast<float*>(mstate) + i0);
            mp[0] = m4.x; mp[1] = m4.y; mp[2] = m4.z; mp[3] = m4.w;
        }
        const float g[4] = {g4.x, g4.y, g4.z, g4.w};
        const float wf[4] = {__uint_as_float(w2.x << 16), __uint_as_float(w2.x & 0xffff0000u),
                             __uint_as_float(w2.y << 16), __uint_as_float(w2.y & 0xffff0000u)};
        uint16_t wn[4], mn16[4];
        float mn[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float w_new;
            lion_elem(g[e], mp[e], wf[e], lr, beta1, beta2, wd, mn[e], w_new);
            const unsigned h = sr_hash(i0 + e, sr_seed);
            if (BF16_STATE) mn16[e] = f32_to_bf16_sr(mn[e], h ^ 0x9e3779b9u);
            wn[e] = f32_to_bf16_sr(w_new, h);
            local = fmaxf(local, fabsf(w_new));
        }
        *reinterpret_cast<uint2*>(w + i0) = make_uint2(wn[0] | (static_cast<uint32_t>(wn[1]) << 16),
                                                       wn[2] | (static_cast<uint32_t>(wn[3]) << 16));
        if (BF16_STATE)
            *reinterpret_cast<uint2*>(static_cast<uint16_t*>(mstate) + i0) =
                make_uint2(mn16[0] | (static_cast<uint32_t>(mn16[1]) << 16), mn16[2] | (static_cast<uint32_t>(mn16[3]) << 16));
        else
            *reinterpret_cast<float4*>(static_cast<float*>(mstate) + i0) = make_float4(mn[0], mn[1], mn[2], mn[3]);
    }
    for (size_t i = nvec * 4 + static_cast<size_t>(blockIdx.x) * kLT + threadIdx.x; i < n; i += stride) {
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
    const int vec = ((reinterpret_cast<uintptr_t>(w) % 8) == 0) && ((reinterpret_cast<uintptr_t>(grad) % 16) == 0) &&
                    ((reinterpret_cast<uintptr_t>(m) % (BF16_STATE ? 8 : 16)) == 0);
    size_t blocks = (n / 4 + kLT - 1) / kLT;
    if (blocks < 1) blocks = 1;
    const size_t cap = static_cast<size_t>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    k_lion<BF16_STATE><<<static_cast<unsigned>(blocks), kLT, 0, st>>>(static_cast<uint16_t*>(w), m, grad, n, lr, b1, b2, wd,
                                                                      amax, seed, vec);
    CF_LAUNCH_CHECK("lion_step");
    return CF_OK;
}

// Lion step that also emits the weight's FP8 caches: the pass that reads the gradient and the momentum and writes the
// bf16 master quantises what it just wrote (the stochastically rounded bf16 value times the scale, exactly what the
// refresh pass would read back) into the native-layout E4M3 cache and, when asked, the transposed one, so the weight
// refresh of src/trainer.cu:4694-4712 needs no pass of its own. The scale comes from *quant_amax, the amax an earlier
// step left (delayed by one step: this step's amax is only complete when the pass ends; it goes to amax_out, a
// different word). 64 x 64 element tiles: 16 threads x 4 columns across, 16 rows per pass, four passes; the codes of
// the tile stay in shared memory for the transposed write (16 contiguous rows per thread, one 16-byte store).
constexpr int kTile = 64, kTilePitch = kTile + 4;

template <bool BF16_STATE>
__global__ void __launch_bounds__(kLT) k_lion_quant_tile(uint16_t* __restrict__ w, void* __restrict__ mstate,
                                                         const float* __restrict__ grad, int rows, int cols, float lr,
                                                         float beta1, float beta2, float wd, float* __restrict__ amax_out,
                                                         unsigned sr_seed, const float* __restrict__ quant_amax,
                                                         float* __restrict__ scale_out, float* __restrict__ descale_out,
                                                         uint8_t* __restrict__ out8, uint8_t* __restrict__ out8_t, int t_vec) {
    __shared__ __align__(16) uint8_t tile[kTile * kTilePitch];
    const float a = fmaxf(*quant_amax, 1e-12f);
    const float scale = __fdiv_rn(448.0f, a);                 // kernels/fp8.cu:34-40
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        *scale_out = scale;
        *descale_out = __fdiv_rn(a, 448.0f);
    }
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int tiles_x = (cols + kTile - 1) / kTile, tiles_y = (rows + kTile - 1) / kTile;
    float local = 0.0f;
    for (long long t = blockIdx.x; t < static_cast<long long>(tiles_x) * tiles_y; t += gridDim.x) {
        const int r0 = static_cast<int>(t / tiles_x) * kTile, c0 = static_cast<int>(t % tiles_x) * kTile;
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
            const int rl = ty + 16 * pass;
            const int r = r0 + rl, c = c0 + 4 * tx;
            uint32_t q = 0u;
            if (r < rows && c < cols) {                           // cols % 4 == 0: the four columns are all inside
                const size_t i0 = static_cast<size_t>(r) * cols + c;
                const float4 g4 = *reinterpret_cast<const float4*>(grad + i0);
                const uint2 w2 = *reinterpret_cast<const uint2*>(w + i0);
                float mp[4];
                if (BF16_STATE) {
                    const uint2 m2 = *reinterpret_cast<const uint2*>(static_cast<uint16_t*>(mstate) + i0);
                    mp[0] = __uint_as_float(m2.x << 16); mp[1] = __uint_as_float(m2.x & 0xffff0000u);
                    mp[2] = __uint_as_float(m2.y << 16); mp[3] = __uint_as_float(m2.y & 0xffff0000u);
                } else {
                    const float4 m4 = *reinterpret_cast<const float4*>(static_cast<float*>(mstate) + i0);
                    mp[0] = m4.x; mp[1] = m4.y; mp[2] = m4.z; mp[3] = m4.w;
                }
                const float g[4] = {g4.x, g4.y, g4.z, g4.w};
                const float wf[4] = {__uint_as_float(w2.x << 16), __uint_as_float(w2.x & 0xffff0000u),
                                     __uint_as_float(w2.y << 16), __uint_as_float(w2.y & 0xffff0000u)};
                uint16_t wn[4], mn16[4];
                float mn[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float w_new;
                    lion_elem(g[e], mp[e], wf[e], lr, beta1, beta2, wd, mn[e], w_new);
                    const unsigned h = sr_hash(i0 + e, sr_seed);
                    if (BF16_STATE) mn16[e] = f32_to_bf16_sr(mn[e], h ^ 0x9e3779b9u);
                    wn[e] = f32_to_bf16_sr(w_new, h);
                    local = fmaxf(local, fabsf(w_new));
                }
                *reinterpret_cast<uint2*>(w + i0) = make_uint2(wn[0] | (static_cast<uint32_t>(wn[1]) << 16),
                                                               wn[2] | (static_cast<uint32_t>(wn[3]) << 16));
                if (BF16_STATE)
                    *reinterpret_cast<uint2*>(static_cast<uint16_t*>(mstate) + i0) =
                        make_uint2(mn16[0] | (static_cast<uint32_t>(mn16[1]) << 16), mn16[2] | (static_cast<uint32_t>(mn16[3]) << 16));
                else
                    *reinterpret_cast<float4*>(static_cast<float*>(mstate) + i0) = make_float4(mn[0], mn[1], mn[2], mn[3]);
                q = cvt_fp8x4<false>(bf16_bits_to_f32(wn[0]) * scale, bf16_bits_to_f32(wn[1]) * scale,
                                     bf16_bits_to_f32(wn[2]) * scale, bf16_bits_to_f32(wn[3]) * scale);
                *reinterpret_cast<uint32_t*>(out8 + i0) = q;
            }
            *reinterpret_cast<uint32_t*>(tile + rl * kTilePitch + 4 * tx) = q;
        }
        if (out8_t != nullptr) {
            __syncthreads();
            const int col = threadIdx.x >> 2, chunk = threadIdx.x & 3;       // 64 columns x 4 chunks of 16 rows
            const int c = c0 + col, rr = r0 + 16 * chunk;
            if (c < cols && rr < rows) {
                uint32_t v[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    v[j >> 2] |= static_cast<uint32_t>(tile[(16 * chunk + j) * kTilePitch + col]) << (8 * (j & 3));
                uint8_t* dst = out8_t + static_cast<size_t>(c) * rows + rr;
                if (t_vec && rr + 16 <= rows) {
                    *reinterpret_cast<uint4*>(dst) = make_uint4(v[0], v[1], v[2], v[3]);
                } else {
                    for (int j = 0; j < 16 && rr + j < rows; ++j) dst[j] = static_cast<uint8_t>(v[j >> 2] >> (8 * (j & 3)));
                }
            }
            __syncthreads();
        }
    }
    if (amax_out) block_amax_commit(local, amax_out);
}

template <bool BF16_STATE>
int launch_lion_quant(void* w, void* m, const float* grad, int rows, int cols, float lr, float b1, float b2, float wd,
                      float* amax, unsigned seed, const float* quant_amax, float* scale_out, float* descale_out, void* out8,
                      void* out8_t, cudaStream_t st) {
    if (rows == 0 || cols == 0) return CF_OK;
    const bool ok = (cols % 4 == 0) && ((reinterpret_cast<uintptr_t>(w) % 8) == 0) && ((reinterpret_cast<uintptr_t>(grad) % 16) == 0) &&
                    ((reinterpret_cast<uintptr_t>(m) % (BF16_STATE ? 8 : 16)) == 0) && ((reinterpret_cast<uintptr_t>(out8) % 4) == 0);
    if (!ok) {
        set_error("lion step with fused quantise: needs cols %% 4 == 0, 8-byte aligned weights, 16-byte aligned gradients and state, a 4-byte aligned E4M3 output; run the plain step and cf_refresh_fp8_weight instead");
        return CF_ERR_UNSUPPORTED;
    }
    const long long tiles = static_cast<long long>((rows + kTile - 1) / kTile) * ((cols + kTile - 1) / kTile);
    long long blocks = tiles;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    const int t_vec = out8_t && (reinterpret_cast<uintptr_t>(out8_t) % 16 == 0) && (rows % 16 == 0);
    k_lion_quant_tile<BF16_STATE><<<static_cast<unsigned>(blocks), kLT, 0, st>>>(
        static_cast<uint16_t*>(w), m, grad, rows, cols, lr, b1, b2, wd, amax, seed, quant_amax, scale_out, descale_out,
        static_cast<uint8_t*>(out8), static_cast<uint8_t*>(out8_t), t_vec);
    CF_LAUNCH_CHECK("lion_step_quantize");
    return CF_OK;
}

}  // namespace
}  // namespace cf

using namespace cf;

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
    return launch_lion_quant<false>(d_w, d_m, d_grad, rows, cols, lr, beta1, beta2, wd, d_weight_amax, sr_seed, d_quant_amax,
                                    d_scale_out, d_descale_out, d_w8, d_w8_transposed_or_null, as_stream(stream));
}

int cf_lion_step_bf16_state_quantize(void* d_w, void* d_m, const float* d_grad, int rows, int cols, float lr, float beta1,
                                     float beta2, float wd, void* stream, float* d_weight_amax, unsigned sr_seed,
                                     const float* d_quant_amax, float* d_scale_out, float* d_descale_out, void* d_w8,
                                     void* d_w8_transposed_or_null) {
    CF_REQUIRE(rows >= 0 && cols >= 0, "cf_lion_step_bf16_state_quantize: negative shape");
    CF_REQUIRE((rows == 0 || cols == 0) || (d_w && d_m && d_grad && d_quant_amax && d_scale_out && d_descale_out && d_w8),
               "cf_lion_step_bf16_state_quantize: null pointer");
    CF_REQUIRE(d_weight_amax != d_quant_amax, "cf_lion_step_bf16_state_quantize: the amax to quantise with and the amax being recorded must be different words");
    return launch_lion_quant<true>(d_w, d_m, d_grad, rows, cols, lr, beta1, beta2, wd, d_weight_amax, sr_seed, d_quant_amax,
                                   d_scale_out, d_descale_out, d_w8, d_w8_transposed_or_null, as_stream(stream));
}

}  // extern "C"
