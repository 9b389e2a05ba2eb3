// Device helpers of the Lion step shared by the plain kernel (cf_lion.cu) and the tile kernel that also writes the
// weight's E4M3 caches (cf_quant.cu), plus the argument block of the latter.
#pragma once
#include "cf_common.cuh"
#include "cf_internal.cuh"

namespace cf {

struct LionArgs {
    uint16_t* w = nullptr;          // bf16 master [rows, cols]
    void* mstate = nullptr;         // fp32 or bf16 momentum
    const float* grad = nullptr;
    float lr = 0.0f, beta1 = 0.0f, beta2 = 0.0f, wd = 0.0f;
    float* amax_out = nullptr;      // this step's amax (may be null)
    unsigned sr_seed = 0;
    int bf16_state = 0;
};

int lion_quant_tile_launch(const LionArgs& la, void* d_direct, void* d_transposed_or_null, const ScaleFromAmax& sfa, int rows,
                           int cols, cudaStream_t st);

#ifdef __CUDACC__
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
#endif

}  // namespace cf
