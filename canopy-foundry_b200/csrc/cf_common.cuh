// Shared host/device helpers for libcanopy_fp8 (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "canopy_fp8.h"

namespace cf {

// ---- error plumbing -----------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
extern std::atomic<uint64_t> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }
// Number of SMs of the current device (cached per device index).
int sm_count();
// CF_OK when the current device is compute capability 10.x, else CF_ERR_UNSUPPORTED.
int require_sm100();

#define CF_REQUIRE(cond, ...)                      \
    do {                                           \
        if (!(cond)) {                             \
            ::cf::set_error(__VA_ARGS__);          \
            return CF_ERR_INVALID_ARG;             \
        }                                          \
    } while (0)

#define CF_CUDA(call)                                              \
    do {                                                           \
        cudaError_t e__ = (call);                                  \
        if (e__ != cudaSuccess) return ::cf::cuda_fail(e__, #call); \
    } while (0)

#define CF_LAUNCH_CHECK(name)                                          \
    do {                                                               \
        cudaError_t e__ = cudaPeekAtLastError();                       \
        if (e__ != cudaSuccess) return ::cf::cuda_fail(e__, name);     \
        ::cf::count_launch();                                          \
    } while (0)

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

// Launch with programmatic dependent launch: the grid may be scheduled while its predecessor in the stream is
// still draining; the kernel itself orders its memory accesses with pdl_wait() (griddepcontrol.wait), so only
// launch latency and the kernel's prologue overlap with the predecessor's tail.
template <class... KArgs, class... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- device helpers -----------------------------------------------------------------
#ifdef __CUDACC__

// Waits until the grids this one depends on have completed and their writes are visible, then lets the next
// grid of the stream be scheduled behind this one. No-ops for launches without the attribute.
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// Two floats -> two FP8 codes (lo = a, hi = b); cvt.rn.satfinite is the instruction
// __nv_fp8_e4m3(float) / __nv_fp8_e5m2(float) execute on sm_89+.
template <bool E5M2>
__device__ __forceinline__ uint32_t cvt_fp8x2(float a, float b) {
    uint16_t r;
    if constexpr (E5M2) {
        asm("cvt.rn.satfinite.e5m2x2.f32 %0, %2, %1;" : "=h"(r) : "f"(a), "f"(b));
    } else {
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(a), "f"(b));
    }
    return r;
}

template <bool E5M2>
__device__ __forceinline__ uint8_t cvt_fp8(float a) { return static_cast<uint8_t>(cvt_fp8x2<E5M2>(a, 0.0f) & 0xffu); }

// Four floats -> four packed FP8 codes (byte i = value i).
template <bool E5M2>
__device__ __forceinline__ uint32_t cvt_fp8x4(float a, float b, float c, float d) {
    return cvt_fp8x2<E5M2>(a, b) | (cvt_fp8x2<E5M2>(c, d) << 16);
}

// Exact decode of an FP8 code through the half-precision converter.
template <bool E5M2>
__device__ __forceinline__ float fp8_to_f32(uint8_t code) {
    if constexpr (E5M2) {
        return __half2float(__ushort_as_half(static_cast<unsigned short>(code) << 8));
    } else {
        uint32_t h2;
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(code)));
        return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xffffu)));
    }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

// Block-wide max of non-negative floats followed by one integer atomicMax on the float bits
// (valid because non-negative IEEE floats order like their bit patterns).
__device__ __forceinline__ void block_amax_commit(float local, float* amax_out) {
    __shared__ float s_part[32];
    local = warp_max(local);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) s_part[warp] = local;
    __syncthreads();
    if (warp == 0) {
        const int nwarps = (blockDim.x + 31) >> 5;
        float v = lane < nwarps ? s_part[lane] : 0.0f;
        v = warp_max(v);
        if (lane == 0) atomicMax(reinterpret_cast<int*>(amax_out), __float_as_int(v));
    }
}

#endif  // __CUDACC__

}  // namespace cf
