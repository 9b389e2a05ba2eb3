// Internal (non-ABI) entry points shared between translation units of libcanopy_fp8.
#pragma once
#include <cuda_runtime.h>
#include <cstddef>

namespace cf {

// Delayed-scale ring update fused into the tail of a record-quantise launch (ticket != nullptr enables it).
struct RingTail {
    float fp8_max = 0.0f;
    float* scale = nullptr;
    float* descale = nullptr;
    float* history = nullptr;
    int history_len = 0;
    int* history_cursor = nullptr;
    int* history_count = nullptr;
    unsigned* ticket = nullptr;      // zero-initialised device word owned by the slot
    // single-launch form (all three set): amax accumulates in *work_amax (zero between calls), the kernel
    // snapshots the pair it quantises with, and the tail publishes the amax
    float* work_amax = nullptr;
    float* snap_scale = nullptr;
    float* snap_descale = nullptr;
};

// Scale derived inside the quantise kernel from a device amax (amax != nullptr enables it).
struct ScaleFromAmax {
    const float* amax = nullptr;
    float fp8_max = 0.0f;
    float* scale_out = nullptr;
    float* descale_out = nullptr;
};

int slot_begin(const float* scale, const float* descale, float* snap_scale, float* snap_descale, float* amax,
               cudaStream_t st);
int quantize_record_fused(const void* d_x, void* d_out, const float* d_scale, float* d_amax, size_t n, bool e5m2,
                          const RingTail& tail, cudaStream_t st);
int quant_dual_from_amax(const void* d_in, void* d_direct, void* d_transposed, const ScaleFromAmax& sfa, int R, int Ccols,
                         cudaStream_t st);

int swiglu_record_launch(const void* d_gate, const void* d_up, int ld_in, void* d_out, int ld_out, const float* d_scale,
                         float* d_amax, int rows, int cols, const RingTail& tail, cudaStream_t st);

}  // namespace cf
