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

// mode 0: normalise only; 1: + per-tensor E4M3 codes with *d_scale, amax of the normalised bf16 row recorded;
// 2: + per-row scale derived from the row's own amax (row_scale / row_descale written).
// clip_ceiling > 0: rows of the normalised bf16 tensor whose L2 norm exceeds it are rescaled first (act_row_clip).
int rmsnorm_launch(int mode, const void* d_x, const void* d_gamma, void* d_normed_or_null, float* d_rms_or_null, void* d_out8,
                   const float* d_scale, float* d_amax, float* d_row_scale, float* d_row_descale, int rows, int H, float eps,
                   const RingTail& tail, cudaStream_t st, float clip_ceiling = 0.0f);

int swiglu_record_launch(const void* d_gate, const void* d_up, int ld_in, void* d_out, int ld_out, const float* d_scale,
                         float* d_amax, int rows, int cols, const RingTail& tail, cudaStream_t st);

#ifdef __CUDACC__
// Called by one thread of every block after the block's amax has been committed: the last block to arrive runs the
// delayed-scale ring update of kernels/fp8.cu:105-142 on the finished amax and re-arms the ticket.
__device__ __forceinline__ void ring_tail_last_block(const RingTail& tail, float* amax) {
    __threadfence();
    if (atomicAdd(tail.ticket, 1u) != gridDim.x - 1) return;
    __threadfence();
    const float a = fmaxf(__int_as_float(atomicMax(reinterpret_cast<int*>(amax), 0)), 1e-12f);
    int cursor = *tail.history_cursor, count = *tail.history_count;
    if (cursor < 0 || cursor >= tail.history_len) cursor = 0;
    tail.history[cursor] = a;
    cursor = (cursor + 1) % tail.history_len;
    if (count < tail.history_len) ++count;
    float m = tail.history[0];
    for (int i = 1; i < count; ++i) m = fmaxf(m, tail.history[i]);
    m = fmaxf(m, 1e-12f);
    *tail.history_cursor = cursor;
    *tail.history_count = count;
    *tail.scale = __fdiv_rn(tail.fp8_max, m);
    *tail.descale = __fdiv_rn(m, tail.fp8_max);
    *tail.ticket = 0;
}
#endif

}  // namespace cf
