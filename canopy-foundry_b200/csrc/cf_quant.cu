// FP8 quantize / cast / amax / transpose kernels: HBM-streaming, 16-byte vectorised.
//
// Arithmetic contract (bit-exact with the reference's kernels/fp8.cu):
//   code = cvt.rn.satfinite.{e4m3,e5m2}(float(x) * scale)      (fp8.cu:49,59,78,97)
//   amax = integer atomicMax over fmaxf(|x|) partials           (fp8.cu:27-31)
// max() is order-free, so wider threads/vectors change no bit of the result.
#include "cf_common.cuh"
#include "cf_internal.cuh"
#include "cf_lion.cuh"

namespace cf {
namespace {

constexpr int kThreads = 256;

// Delayed-scale ring update (kernels/fp8.cu:105-142), shared by the stand-alone kernel and the fused tail.
__device__ __forceinline__ void ring_update(float amax, float fp8_max, float* scale, float* descale, float* history,
                                            int history_len, int* history_cursor, int* history_count) {
    const float a = fmaxf(amax, 1e-12f);
    if (history_len <= 0) {
        *scale = __fdiv_rn(fp8_max, a);
        *descale = __fdiv_rn(a, fp8_max);
        return;
    }
    int cursor = *history_cursor;
    int count = *history_count;
    if (cursor < 0 || cursor >= history_len) cursor = 0;
    history[cursor] = a;
    cursor = (cursor + 1) % history_len;
    if (count < history_len) ++count;
    float m = history[0];
    for (int i = 1; i < count; ++i) m = fmaxf(m, history[i]);
    m = fmaxf(m, 1e-12f);
    *history_cursor = cursor;
    *history_count = count;
    *scale = __fdiv_rn(fp8_max, m);
    *descale = __fdiv_rn(m, fp8_max);
}

// After the block's amax has been committed: the last block of the grid to get here runs the ring update,
// so the record pass and the scale update are one launch.
__device__ __forceinline__ void fused_tail(const RingTail& t, float* amax) {
    if (t.ticket == nullptr) return;
    if (threadIdx.x == 0) {
        __threadfence();                                    // this block's atomicMax is visible before its ticket
        const unsigned prev = atomicAdd(t.ticket, 1u);
        if (prev == gridDim.x - 1) {
            __threadfence();
            float a;
            if (t.work_amax) {
                // single-launch form: the blocks accumulated into the slot's work word; publish it as the call's
                // amax and leave the work word zero for the next call
                a = __int_as_float(atomicExch(reinterpret_cast<int*>(t.work_amax), 0));
                *amax = a;
            } else {
                a = __int_as_float(atomicMax(reinterpret_cast<int*>(amax), 0));   // coherent read
            }
            ring_update(a, t.fp8_max, t.scale, t.descale, t.history, t.history_len, t.history_cursor, t.history_count);
            *t.ticket = 0;                                  // ready for the next call
        }
    }
}

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ float4 ldg_stream_f4(const float* p) {
    float4 v;
    asm volatile("ld.global.cs.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

// 8 bf16 (one uint4) -> 8 floats
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}

template <bool E5M2>
__device__ __forceinline__ uint2 quant8(const float (&f)[8], float s) {
    uint2 r;
    r.x = cvt_fp8x4<E5M2>(f[0] * s, f[1] * s, f[2] * s, f[3] * s);
    r.y = cvt_fp8x4<E5M2>(f[4] * s, f[5] * s, f[6] * s, f[7] * s);
    return r;
}

__device__ __forceinline__ float amax8(float local, const float (&f)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) local = fmaxf(local, fabsf(f[i]));
    return local;
}

// Streaming kernel over [head | nvec vectors of 16 elements | tail]; head/tail (< 16 elements
// each) are handled by block 0 with scalar accesses. QUANT=false is the amax-only pass.
template <bool E5M2, bool QUANT, bool RECORD>
__global__ void __launch_bounds__(kThreads) k_stream(const uint16_t* __restrict__ x, uint8_t* __restrict__ out,
                                                     const float* __restrict__ scale, float* __restrict__ amax,
                                                     size_t n, size_t head, size_t nvec, const RingTail tail) {
    pdl_wait();
    const float s = QUANT ? *scale : 0.0f;
    if (RECORD && tail.snap_scale && blockIdx.x == 0 && threadIdx.x == 0) {
        // single-launch form: the pair this call quantises with is snapshotted here (nobody reads the snapshot
        // words during this kernel; the live pair is rewritten only by the last block's tail)
        *tail.snap_scale = s;
        *tail.snap_descale = *tail.descale;
    }
    float local = 0.0f;
    const uint16_t* xv = x + head;
    uint8_t* ov = out + head;
    const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
    size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x;
    // two vectors (32 elements, four 16-byte loads) in flight per thread
    for (; i + stride < nvec; i += 2 * stride) {
        const uint4 a0 = ldg_stream16(xv + i * 16), a1 = ldg_stream16(xv + i * 16 + 8);
        const uint4 b0 = ldg_stream16(xv + (i + stride) * 16), b1 = ldg_stream16(xv + (i + stride) * 16 + 8);
        float f[8], g[8];
        unpack8(a0, f); unpack8(a1, g);
        if (RECORD) { local = amax8(local, f); local = amax8(local, g); }
        if (QUANT) {
            const uint2 q0 = quant8<E5M2>(f, s), q1 = quant8<E5M2>(g, s);
            *reinterpret_cast<uint4*>(ov + i * 16) = make_uint4(q0.x, q0.y, q1.x, q1.y);
        }
        unpack8(b0, f); unpack8(b1, g);
        if (RECORD) { local = amax8(local, f); local = amax8(local, g); }
        if (QUANT) {
            const uint2 q0 = quant8<E5M2>(f, s), q1 = quant8<E5M2>(g, s);
            *reinterpret_cast<uint4*>(ov + (i + stride) * 16) = make_uint4(q0.x, q0.y, q1.x, q1.y);
        }
    }
    for (; i < nvec; i += stride) {
        const uint4 a0 = ldg_stream16(xv + i * 16), a1 = ldg_stream16(xv + i * 16 + 8);
        float f[8], g[8];
        unpack8(a0, f); unpack8(a1, g);
        if (RECORD) { local = amax8(local, f); local = amax8(local, g); }
        if (QUANT) {
            const uint2 q0 = quant8<E5M2>(f, s), q1 = quant8<E5M2>(g, s);
            *reinterpret_cast<uint4*>(ov + i * 16) = make_uint4(q0.x, q0.y, q1.x, q1.y);
        }
    }
    if (blockIdx.x == 0) {
        const size_t tail0 = head + nvec * 16;
        const size_t edge = head + (n - tail0);   // scalar elements in total (< 32)
        for (size_t e = threadIdx.x; e < edge; e += kThreads) {
            const size_t idx = e < head ? e : tail0 + (e - head);
            const float v = bf16_bits_to_f32(x[idx]);
            if (RECORD) local = fmaxf(local, fabsf(v));
            if (QUANT) out[idx] = cvt_fp8<E5M2>(v * s);
        }
    }
    if (RECORD) {
        block_amax_commit(local, tail.work_amax ? tail.work_amax : amax);
        fused_tail(tail, amax);
    }
}

// Fully scalar form for pointers whose relative alignment rules out 16-byte accesses.
template <bool E5M2, bool QUANT, bool RECORD>
__global__ void __launch_bounds__(kThreads) k_stream_scalar(const uint16_t* __restrict__ x, uint8_t* __restrict__ out,
                                                            const float* __restrict__ scale,
                                                            float* __restrict__ amax, size_t n, const RingTail tail) {
    pdl_wait();
    const float s = QUANT ? *scale : 0.0f;
    if (RECORD && tail.snap_scale && blockIdx.x == 0 && threadIdx.x == 0) {
        *tail.snap_scale = s;
        *tail.snap_descale = *tail.descale;
    }
    float local = 0.0f;
    for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * kThreads) {
        const float v = bf16_bits_to_f32(x[i]);
        if (RECORD) local = fmaxf(local, fabsf(v));
        if (QUANT) out[i] = cvt_fp8<E5M2>(v * s);
    }
    if (RECORD) {
        block_amax_commit(local, tail.work_amax ? tail.work_amax : amax);
        fused_tail(tail, amax);
    }
}

__global__ void k_ring_update_only(float* amax, const RingTail t) {
    if (t.snap_scale) {                 // empty tensor in the single-launch form: snapshot, amax = 0, ring update
        *t.snap_scale = *t.scale;
        *t.snap_descale = *t.descale;
        *amax = 0.0f;
    }
    ring_update(*amax, t.fp8_max, t.scale, t.descale, t.history, t.history_len, t.history_cursor, t.history_count);
}

template <bool E5M2, bool QUANT, bool RECORD>
int launch_stream(const void* d_x, void* d_out, const float* d_scale, float* d_amax, size_t n, cudaStream_t st,
                  const char* name, const RingTail tail = RingTail()) {
    if (n == 0) {
        if (tail.ticket) {     // nothing to scan: the ring still advances with the caller-zeroed amax
            k_ring_update_only<<<1, 1, 0, st>>>(d_amax, tail);
            CF_LAUNCH_CHECK(name);
        }
        return CF_OK;
    }
    const uintptr_t xa = reinterpret_cast<uintptr_t>(d_x);
    const uintptr_t oa = reinterpret_cast<uintptr_t>(d_out);
    // Peel `head` elements so that the input is 16-byte aligned; the vector path also needs the
    // output (1 byte per element) 16-byte aligned at the same element.
    size_t head = ((16 - (xa & 15)) & 15) / 2;
    bool vec_ok = (xa & 1) == 0;
    if (QUANT && ((oa + head) & 15) != 0) {
        // try the other input phase: adding 8 elements keeps x aligned and moves out by 8 bytes
        if (((oa + head + 8) & 15) == 0) head += 8; else vec_ok = false;
    }
    if (head > n) head = n;
    const int sms = sm_count();
    if (!vec_ok) {
        const size_t blocks = (n + kThreads - 1) / kThreads;
        const unsigned grid = static_cast<unsigned>(blocks < static_cast<size_t>(sms) * 16 ? blocks : static_cast<size_t>(sms) * 16);
        CF_CUDA(launch_pdl(k_stream_scalar<E5M2, QUANT, RECORD>, dim3(grid), dim3(kThreads), 0, st,
                           static_cast<const uint16_t*>(d_x), static_cast<uint8_t*>(d_out), d_scale, d_amax, n, tail));
    } else {
        const size_t nvec = (n - head) / 16;
        size_t blocks = (nvec + 2 * kThreads - 1) / (2 * kThreads);
        if (blocks < 1) blocks = 1;
        const size_t cap = static_cast<size_t>(sms) * 8;
        const unsigned grid = static_cast<unsigned>(blocks < cap ? blocks : cap);
        CF_CUDA(launch_pdl(k_stream<E5M2, QUANT, RECORD>, dim3(grid), dim3(kThreads), 0, st,
                           static_cast<const uint16_t*>(d_x), static_cast<uint8_t*>(d_out), d_scale, d_amax, n, head, nvec, tail));
    }
    CF_LAUNCH_CHECK(name);
    return CF_OK;
}

// ---- scalar bookkeeping kernels (one thread; latency only) ---------------------------------
__global__ void k_scale_from_amax(const float* amax, float fp8_max, float* scale, float* descale) {
    const float a = fmaxf(*amax, 1e-12f);
    *scale = __fdiv_rn(fp8_max, a);
    *descale = __fdiv_rn(a, fp8_max);
}

__global__ void k_update_delayed_scale(const float* amax, float fp8_max, float* scale, float* descale, float* history,
                                       int history_len, int* history_cursor, int* history_count) {
    ring_update(*amax, fp8_max, scale, descale, history, history_len, history_cursor, history_count);
}

// Start of a steady-state fp8_quant_act call: snapshot the pair the forward pass is about to use and zero the
// amax slot (src/trainer.cu:4823-4827 does this with two scalar copies and a memset).
__global__ void k_slot_begin(const float* scale, const float* descale, float* snap_scale, float* snap_descale, float* amax) {
    pdl_wait();
    *snap_scale = *scale;
    *snap_descale = *descale;
    *amax = 0.0f;
}

__global__ void k_calib_minmax(const float* amax, float* cmin, float* cmax) {
    const float a = fmaxf(*amax, 1e-12f);
    *cmin = fminf(*cmin, a);
    *cmax = fmaxf(*cmax, a);
}

__global__ void k_clip_probe(const float* amax, const float* scale, float fp8_max, float* stats) {
    const float a = *amax, s = *scale;
    stats[2] += 1.0f;
    if (fp8_max > 0.0f && s > 0.0f) {
        const float ratio = __fdiv_rn(__fmul_rn(a, s), fp8_max);
        if (ratio > 1.0f) {
            stats[0] += 1.0f;
            if (ratio > stats[1]) stats[1] = ratio;
        }
    }
}

__global__ void __launch_bounds__(kThreads) k_elem_clip_count(const uint16_t* __restrict__ x, const float* scale,
                                                              float fp8_max, size_t n, float* out, int vec) {
    const float s = *scale;
    unsigned long long clipped = 0;
    const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
    const size_t nvec = vec ? n / 8 : 0;                          // 16-byte loads when the base is aligned
    for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < nvec; i += stride) {
        const uint4 v = __ldcs(reinterpret_cast<const uint4*>(x) + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (fabsf(__uint_as_float(w[j] << 16)) * s > fp8_max) ++clipped;
            if (fabsf(__uint_as_float(w[j] & 0xffff0000u)) * s > fp8_max) ++clipped;
        }
    }
    for (size_t i = nvec * 8 + static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride)
        if (fabsf(bf16_bits_to_f32(x[i])) * s > fp8_max) ++clipped;
    // one float atomic per warp instead of per thread: integer partial sums stay exact below 2^24
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) clipped += __shfl_xor_sync(0xffffffffu, clipped, off);
    if ((threadIdx.x & 31) == 0 && clipped) atomicAdd(&out[0], static_cast<float>(clipped));
    if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&out[1], static_cast<float>(n));
}

// ---- raw-byte E4M3 storage path (include/ida_native/fp8_e4m3.hpp semantics) -----------------
__global__ void __launch_bounds__(kThreads) k_pack_raw_stats(const uint16_t* __restrict__ x, size_t n, float* amax, int* bad,
                                                             int vec) {
    float local = 0.0f;
    int local_bad = 0;
    const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
    const size_t nvec = vec ? n / 8 : 0;
    for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < nvec; i += stride) {
        const uint4 v = __ldcs(reinterpret_cast<const uint4*>(x) + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t b = h ? (w[j] >> 16) : (w[j] & 0xffffu);
                if ((b & 0x7f80u) == 0x7f80u) local_bad = 1;        // Inf or NaN
                else local = fmaxf(local, bf16_bits_to_f32(b & 0x7fffu));
            }
        }
    }
    for (size_t i = nvec * 8 + static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
        const uint32_t b = x[i];
        if ((b & 0x7f80u) == 0x7f80u) local_bad = 1;            // Inf or NaN
        else local = fmaxf(local, bf16_bits_to_f32(b & 0x7fffu));
    }
    local_bad = __any_sync(0xffffffffu, local_bad);
    if ((threadIdx.x & 31) == 0 && local_bad) atomicAdd(bad, 1);
    block_amax_commit(local, amax);
}

// pack(): finite products use the hardware converter (same codes for every finite input);
// non-finite products become sign|0x7f and are counted.
__device__ __forceinline__ uint8_t pack_e4m3(float v, int& nonfinite) {
    const uint32_t u = __float_as_uint(v);
    if ((u & 0x7f800000u) == 0x7f800000u) {
        nonfinite = 1;
        return static_cast<uint8_t>(((u >> 24) & 0x80u) | 0x7fu);
    }
    return cvt_fp8<false>(v);
}

// unpack(): exact decode; 0x7f / 0xff are NaN.
__device__ __forceinline__ float unpack_e4m3(uint8_t c) { return fp8_to_f32<false>(c); }

template <bool DEQUANT>
__global__ void __launch_bounds__(kThreads) k_pack_raw(const uint16_t* __restrict__ x, uint8_t* __restrict__ out,
                                                       uint16_t* __restrict__ dequant, const float* scale,
                                                       const float* descale, int* bad, size_t n, int vec) {
    const float s = *scale;
    const float d = DEQUANT ? *descale : 0.0f;
    int nbad = 0;
    const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
    const size_t nvec = vec ? n / 8 : 0;          // 8 elements per thread: 16 bytes in, 8 bytes (+16 bytes) out
    for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < nvec; i += stride) {
        const uint4 v = __ldcs(reinterpret_cast<const uint4*>(x) + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t codes[2] = {0u, 0u}, dq[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int nf0 = 0, nf1 = 0;
            const uint32_t c0 = pack_e4m3(__uint_as_float(w[j] << 16) * s, nf0);
            const uint32_t c1 = pack_e4m3(__uint_as_float(w[j] & 0xffff0000u) * s, nf1);
            nbad += nf0 + nf1;
            codes[j >> 1] |= (c0 | (c1 << 8)) << (16 * (j & 1));
            if (DEQUANT)
                dq[j] = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16(unpack_e4m3(static_cast<uint8_t>(c0)) * d))) |
                        (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16(unpack_e4m3(static_cast<uint8_t>(c1)) * d))) << 16);
        }
        reinterpret_cast<uint2*>(out)[i] = make_uint2(codes[0], codes[1]);
        if (DEQUANT) reinterpret_cast<uint4*>(dequant)[i] = make_uint4(dq[0], dq[1], dq[2], dq[3]);
    }
    for (size_t i = nvec * 8 + static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
        int nf = 0;
        const uint8_t c = pack_e4m3(bf16_bits_to_f32(x[i]) * s, nf);
        nbad += nf;
        out[i] = c;
        if (DEQUANT) dequant[i] = __bfloat16_as_ushort(__float2bfloat16(unpack_e4m3(c) * d));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) nbad += __shfl_xor_sync(0xffffffffu, nbad, off);
    if ((threadIdx.x & 31) == 0 && nbad) atomicAdd(bad, nbad);
}

__global__ void __launch_bounds__(kThreads) k_unpack_raw(const uint8_t* __restrict__ in, const float* descale,
                                                         uint16_t* __restrict__ out, size_t n, int vec) {
    const float d = *descale;
    const size_t stride = static_cast<size_t>(gridDim.x) * kThreads;
    const size_t nvec = vec ? n / 8 : 0;          // 8 codes in, 16 bytes of bf16 out
    for (size_t i = static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < nvec; i += stride) {
        const uint2 c = __ldcs(reinterpret_cast<const uint2*>(in) + i);
        const uint32_t w[2] = {c.x, c.y};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t pair = (w[j >> 1] >> (16 * (j & 1))) & 0xffffu;
            o[j] = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16(unpack_e4m3(static_cast<uint8_t>(pair & 0xffu)) * d))) |
                   (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16(unpack_e4m3(static_cast<uint8_t>(pair >> 8)) * d))) << 16);
        }
        reinterpret_cast<uint4*>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    for (size_t i = nvec * 8 + static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride)
        out[i] = __bfloat16_as_ushort(__float2bfloat16(unpack_e4m3(in[i]) * d));
}

unsigned flat_grid(size_t n, int per_block) {
    const size_t blocks = (n + per_block - 1) / per_block;
    const size_t cap = static_cast<size_t>(sm_count()) * 16;
    return static_cast<unsigned>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

// ---- tiled transpose family ----------------------------------------------------------------
// One block moves a tile of 256 source rows x 64 source columns through shared memory and writes it
// transposed: 64 output rows x 256 contiguous bytes, each output row written by one warp-wide store
// instruction (32 lanes x 8 bytes). Source is bf16 (quantised on the way in, optionally also written
// un-transposed) or bytes (plain transpose).
constexpr int kTR = 256;          // source rows per tile  -> 256 contiguous output bytes per row
constexpr int kTC = 64;           // source columns per tile (16 words of quantised bytes per source row)

// Shared-memory word index of (source row k, word column wc). Rows are 16 words with no padding; the word
// column is XOR-swizzled by the 8-row group and the two halves of the tile are offset by one row, which makes
// the column-wise reads of the write-out phase hit 32 different banks.
__device__ __forceinline__ int tile_word(int k, int wc) {
    return ((k ^ ((k >> 7) & 1)) << 4) + (wc ^ ((k >> 3) & 15));
}

// SRC: 0 = byte source (plain transpose), 1 = bf16 source (quantised on the way in), 2 = the Lion step: the tile's
// weights are updated in place (gradient, momentum and master read and written as kernels/lion.cu does) and the value
// just stored is what gets quantised, so the optimiser pass leaves both E4M3 caches behind.
template <int SRC>
__global__ void __launch_bounds__(kThreads) k_tile_transpose(const void* __restrict__ src, uint8_t* __restrict__ direct,
                                                             uint8_t* __restrict__ transposed,
                                                             const float* __restrict__ scale, int R, int Ccols,
                                                             int src_vec, int direct_vec, int trans_vec,
                                                             const ScaleFromAmax sfa, const LionArgs la) {
    constexpr bool SRC_BF16 = SRC != 0;
    __shared__ uint32_t tile[kTR * 16];
    const int r0 = blockIdx.y * kTR, c0 = blockIdx.x * kTC;
    const int tid = threadIdx.x;
    pdl_wait();
    float s = 0.0f;
    if (SRC_BF16) {
        if (sfa.amax) {
            // every block derives the same scale from the amax (kernels/fp8.cu:34-40); one thread publishes it
            const float a = fmaxf(*sfa.amax, 1e-12f);
            s = __fdiv_rn(sfa.fp8_max, a);
            if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 0) {
                *sfa.scale_out = s;
                *sfa.descale_out = __fdiv_rn(a, sfa.fp8_max);
            }
        } else {
            s = *scale;
        }
    }

    if (SRC == 2) {
        // 8 threads x 8 columns per row, 32 rows per pass, 8 passes (vector accesses: the launcher requires
        // cols % 8 == 0 and aligned bases); rows and columns outside the tensor leave zeros in the tile
        const int cg = (tid & 7) * 8, rl = tid >> 3;
        float local = 0.0f;
#pragma unroll 2
        for (int p = 0; p < kTR / 32; ++p) {
            const int k = p * 32 + rl;
            const int r = r0 + k, c = c0 + cg;
            uint2 q = make_uint2(0u, 0u);
            if (r < R && c < Ccols) {
                const size_t off = static_cast<size_t>(r) * Ccols + c;
                const uint4 wv = *reinterpret_cast<const uint4*>(la.w + off);
                const float4 g0 = ldg_stream_f4(la.grad + off), g1 = ldg_stream_f4(la.grad + off + 4);
                float wf[8], mp[8];
                unpack8(wv, wf);
                if (la.bf16_state) {
                    unpack8(*reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(la.mstate) + off), mp);
                } else {
                    const float4 m0 = *reinterpret_cast<const float4*>(static_cast<const float*>(la.mstate) + off);
                    const float4 m1 = *reinterpret_cast<const float4*>(static_cast<const float*>(la.mstate) + off + 4);
                    mp[0] = m0.x; mp[1] = m0.y; mp[2] = m0.z; mp[3] = m0.w; mp[4] = m1.x; mp[5] = m1.y; mp[6] = m1.z; mp[7] = m1.w;
                }
                const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                uint16_t wn[8], mn16[8];
                float mn[8], f[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float w_new;
                    lion_elem(g[e], mp[e], wf[e], la.lr, la.beta1, la.beta2, la.wd, mn[e], w_new);
                    const unsigned h = sr_hash(off + e, la.sr_seed);
                    if (la.bf16_state) mn16[e] = f32_to_bf16_sr(mn[e], h ^ 0x9e3779b9u);
                    wn[e] = f32_to_bf16_sr(w_new, h);
                    local = fmaxf(local, fabsf(w_new));
                    f[e] = bf16_bits_to_f32(wn[e]);
                }
                *reinterpret_cast<uint4*>(la.w + off) =
                    make_uint4(wn[0] | (static_cast<uint32_t>(wn[1]) << 16), wn[2] | (static_cast<uint32_t>(wn[3]) << 16),
                               wn[4] | (static_cast<uint32_t>(wn[5]) << 16), wn[6] | (static_cast<uint32_t>(wn[7]) << 16));
                if (la.bf16_state) {
                    *reinterpret_cast<uint4*>(static_cast<uint16_t*>(la.mstate) + off) =
                        make_uint4(mn16[0] | (static_cast<uint32_t>(mn16[1]) << 16), mn16[2] | (static_cast<uint32_t>(mn16[3]) << 16),
                                   mn16[4] | (static_cast<uint32_t>(mn16[5]) << 16), mn16[6] | (static_cast<uint32_t>(mn16[7]) << 16));
                } else {
                    float* md = static_cast<float*>(la.mstate) + off;
                    *reinterpret_cast<float4*>(md) = make_float4(mn[0], mn[1], mn[2], mn[3]);
                    *reinterpret_cast<float4*>(md + 4) = make_float4(mn[4], mn[5], mn[6], mn[7]);
                }
                q = quant8<false>(f, s);
                if (direct) *reinterpret_cast<uint2*>(direct + off) = q;
            }
            tile[tile_word(k, cg >> 2)] = q.x;
            tile[tile_word(k, (cg >> 2) + 1)] = q.y;
        }
        if (la.amax_out) block_amax_commit(local, la.amax_out);      // a block barrier: every thread gets here
    } else if (SRC_BF16) {
        // 8 threads x 8 columns per source row, 32 rows per pass, 8 passes; all loads of a thread issued first
        const uint16_t* in = static_cast<const uint16_t*>(src);
        const int cg = (tid & 7) * 8, rl = tid >> 3;
        uint4 raw[kTR / 32];
#pragma unroll
        for (int p = 0; p < kTR / 32; ++p) {
            const int r = r0 + p * 32 + rl, c = c0 + cg;
            raw[p] = make_uint4(0u, 0u, 0u, 0u);
            if (r < R && c < Ccols) {
                const size_t off = static_cast<size_t>(r) * Ccols + c;
                if (src_vec && c + 8 <= Ccols) {
                    raw[p] = ldg_stream16(in + off);
                } else {
                    uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                    for (int b = 0; b < 8; ++b)
                        if (c + b < Ccols) w[b >> 1] |= static_cast<uint32_t>(in[off + b]) << (16 * (b & 1));
                    raw[p] = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
#pragma unroll
        for (int p = 0; p < kTR / 32; ++p) {
            const int k = p * 32 + rl;
            const int r = r0 + k, c = c0 + cg;
            float f[8];
            unpack8(raw[p], f);
            const uint2 q = quant8<false>(f, s);
            if (direct && r < R && c < Ccols) {
                const size_t off = static_cast<size_t>(r) * Ccols + c;
                if (direct_vec && c + 8 <= Ccols) {
                    *reinterpret_cast<uint2*>(direct + off) = q;
                } else {
                    const uint64_t qq = (static_cast<uint64_t>(q.y) << 32) | q.x;
#pragma unroll
                    for (int b = 0; b < 8; ++b)
                        if (c + b < Ccols) direct[off + b] = static_cast<uint8_t>(qq >> (8 * b));
                }
            }
            tile[tile_word(k, cg >> 2)] = q.x;
            tile[tile_word(k, (cg >> 2) + 1)] = q.y;
        }
    } else {
        // 4 threads x 16 bytes per source row, 64 rows per pass, 4 passes
        const uint8_t* in = static_cast<const uint8_t*>(src);
        const int cg = (tid & 3) * 16, rl = tid >> 2;
#pragma unroll
        for (int p = 0; p < kTR / 64; ++p) {
            const int k = p * 64 + rl;
            const int r = r0 + k, c = c0 + cg;
            uint4 q = make_uint4(0u, 0u, 0u, 0u);
            if (r < R && c < Ccols) {
                const size_t off = static_cast<size_t>(r) * Ccols + c;
                if (src_vec && c + 16 <= Ccols) {
                    q = ldg_stream16(in + off);
                } else {
                    uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                    for (int b = 0; b < 16; ++b)
                        if (c + b < Ccols) w[b >> 2] |= static_cast<uint32_t>(in[off + b]) << (8 * (b & 3));
                    q = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            const int wc = cg >> 2;
            tile[tile_word(k, wc)] = q.x;
            tile[tile_word(k, wc + 1)] = q.y;
            tile[tile_word(k, wc + 2)] = q.z;
            tile[tile_word(k, wc + 3)] = q.w;
        }
    }
    __syncthreads();
    if (!transposed) return;

    // Lane = 8 consecutive source rows (kc8), warp = two word columns (ng): 8 word reads, two 4x4 byte
    // transposes, four 8-byte stores; the 32 lanes of one store cover one whole 256-byte output row.
    const int kc8 = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int ng = warp * 2 + half;
        uint32_t w[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) w[r] = tile[tile_word(kc8 * 8 + r, ng)];
        uint32_t o[4][2];
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            const uint32_t w0 = w[blk * 4], w1 = w[blk * 4 + 1], w2 = w[blk * 4 + 2], w3 = w[blk * 4 + 3];
            const uint32_t a = __byte_perm(w0, w1, 0x5140), b = __byte_perm(w2, w3, 0x5140);
            const uint32_t c = __byte_perm(w0, w1, 0x7362), d = __byte_perm(w2, w3, 0x7362);
            o[0][blk] = __byte_perm(a, b, 0x5410);
            o[1][blk] = __byte_perm(a, b, 0x7632);
            o[2][blk] = __byte_perm(c, d, 0x5410);
            o[3][blk] = __byte_perm(c, d, 0x7632);
        }
        const int ocol = r0 + kc8 * 8;           // output column = source row
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int orow = c0 + ng * 4 + j;    // output row = source column
            if (orow >= Ccols || ocol >= R) continue;
            uint8_t* dst = transposed + static_cast<size_t>(orow) * R + ocol;
            if (trans_vec && ocol + 8 <= R) {
                *reinterpret_cast<uint2*>(dst) = make_uint2(o[j][0], o[j][1]);
            } else {
#pragma unroll
                for (int b = 0; b < 8; ++b)
                    if (ocol + b < R) dst[b] = static_cast<uint8_t>(o[j][b >> 2] >> (8 * (b & 3)));
            }
        }
    }
}

template <int SRC>
int launch_tile_transpose(const void* src, void* direct, void* transposed, const float* scale, int R, int Ccols,
                          cudaStream_t st, const char* name, const ScaleFromAmax sfa = ScaleFromAmax(),
                          const LionArgs la = LionArgs()) {
    constexpr bool SRC_BF16 = SRC != 0;
    if (R == 0 || Ccols == 0) return CF_OK;
    const uintptr_t sa = reinterpret_cast<uintptr_t>(src), da = reinterpret_cast<uintptr_t>(direct),
                    ta = reinterpret_cast<uintptr_t>(transposed);
    const int esz = SRC_BF16 ? 2 : 1;
    const int src_vec = (sa % 16 == 0) && ((static_cast<size_t>(Ccols) * esz) % 16 == 0);
    const int direct_vec = direct && (da % 8 == 0) && (Ccols % 8 == 0);
    const int trans_vec = transposed && (ta % 8 == 0) && (R % 8 == 0);
    dim3 grid((Ccols + kTC - 1) / kTC, (R + kTR - 1) / kTR);
    CF_CUDA(launch_pdl(k_tile_transpose<SRC>, grid, dim3(kThreads), 0, st, src, static_cast<uint8_t*>(direct),
                       static_cast<uint8_t*>(transposed), scale, R, Ccols, src_vec, direct_vec, trans_vec, sfa, la));
    CF_LAUNCH_CHECK(name);
    return CF_OK;
}

}  // namespace

int slot_begin(const float* scale, const float* descale, float* snap_scale, float* snap_descale, float* amax,
               cudaStream_t st) {
    CF_CUDA(launch_pdl(k_slot_begin, dim3(1), dim3(1), 0, st, scale, descale, snap_scale, snap_descale, amax));
    CF_LAUNCH_CHECK("slot_begin");
    return CF_OK;
}

int quantize_record_fused(const void* d_x, void* d_out, const float* d_scale, float* d_amax, size_t n, bool e5m2,
                          const RingTail& tail, cudaStream_t st) {
    return e5m2 ? launch_stream<true, true, true>(d_x, d_out, d_scale, d_amax, n, st, "quantize_e5m2_record_fused", tail)
                : launch_stream<false, true, true>(d_x, d_out, d_scale, d_amax, n, st, "quantize_e4m3_record_fused", tail);
}

int lion_quant_tile_launch(const LionArgs& la, void* d_direct, void* d_transposed_or_null, const ScaleFromAmax& sfa, int rows,
                           int cols, cudaStream_t st) {
    const bool ok = (cols % 8 == 0) && (reinterpret_cast<uintptr_t>(la.w) % 16 == 0) &&
                    (reinterpret_cast<uintptr_t>(la.grad) % 16 == 0) && (reinterpret_cast<uintptr_t>(la.mstate) % 16 == 0) &&
                    (reinterpret_cast<uintptr_t>(d_direct) % 8 == 0);
    if (!ok) {
        set_error("lion step with fused quantise: needs cols %% 8 == 0, 16-byte aligned weights, gradients and state, an 8-byte aligned E4M3 output; run the plain step and cf_refresh_fp8_weight instead");
        return CF_ERR_UNSUPPORTED;
    }
    return launch_tile_transpose<2>(la.w, d_direct, d_transposed_or_null, nullptr, rows, cols, st, "lion_step_quantize", sfa, la);
}

int quant_dual_from_amax(const void* d_in, void* d_direct, void* d_transposed, const ScaleFromAmax& sfa, int R, int Ccols,
                         cudaStream_t st) {
    return launch_tile_transpose<1>(d_in, d_direct, d_transposed, nullptr, R, Ccols, st, "quant_dual_from_amax", sfa);
}

}  // namespace cf

using namespace cf;

extern "C" {

int cf_fp8_amax_bf16(const void* d_x, size_t n, float* d_amax, void* stream) {
    CF_REQUIRE(d_amax != nullptr && (d_x != nullptr || n == 0), "cf_fp8_amax_bf16: null pointer");
    cudaStream_t st = as_stream(stream);
    CF_CUDA(cudaMemsetAsync(d_amax, 0, sizeof(float), st));
    return launch_stream<false, false, true>(d_x, nullptr, nullptr, d_amax, n, st, "amax_bf16");
}

int cf_fp8_scale_from_amax(const float* d_amax, float fp8_max, float* d_scale, float* d_descale, void* stream) {
    CF_REQUIRE(d_amax && d_scale && d_descale, "cf_fp8_scale_from_amax: null pointer");
    k_scale_from_amax<<<1, 1, 0, as_stream(stream)>>>(d_amax, fp8_max, d_scale, d_descale);
    CF_LAUNCH_CHECK("scale_from_amax");
    return CF_OK;
}

int cf_fp8_quantize_e4m3(const void* d_x, void* d_out, const float* d_scale, size_t n, void* stream) {
    CF_REQUIRE(d_scale && (n == 0 || (d_x && d_out)), "cf_fp8_quantize_e4m3: null pointer");
    return launch_stream<false, true, false>(d_x, d_out, d_scale, nullptr, n, as_stream(stream), "quantize_e4m3");
}
int cf_fp8_quantize_e5m2(const void* d_x, void* d_out, const float* d_scale, size_t n, void* stream) {
    CF_REQUIRE(d_scale && (n == 0 || (d_x && d_out)), "cf_fp8_quantize_e5m2: null pointer");
    return launch_stream<true, true, false>(d_x, d_out, d_scale, nullptr, n, as_stream(stream), "quantize_e5m2");
}
int cf_fp8_quantize_e4m3_record(const void* d_x, void* d_out, const float* d_scale, float* d_amax, size_t n, void* stream) {
    CF_REQUIRE(d_scale && d_amax && (n == 0 || (d_x && d_out)), "cf_fp8_quantize_e4m3_record: null pointer");
    return launch_stream<false, true, true>(d_x, d_out, d_scale, d_amax, n, as_stream(stream), "quantize_e4m3_record");
}
int cf_fp8_quantize_e5m2_record(const void* d_x, void* d_out, const float* d_scale, float* d_amax, size_t n, void* stream) {
    CF_REQUIRE(d_scale && d_amax && (n == 0 || (d_x && d_out)), "cf_fp8_quantize_e5m2_record: null pointer");
    return launch_stream<true, true, true>(d_x, d_out, d_scale, d_amax, n, as_stream(stream), "quantize_e5m2_record");
}

int cf_fp8_update_delayed_scale(const float* d_amax, float fp8_max, float* d_scale, float* d_descale, float* d_history,
                                int history_len, int* d_history_cursor, int* d_history_count, void* stream) {
    CF_REQUIRE(d_amax && d_scale && d_descale, "cf_fp8_update_delayed_scale: null pointer");
    CF_REQUIRE(history_len <= 0 || (d_history && d_history_cursor && d_history_count),
               "cf_fp8_update_delayed_scale: history pointers required when history_len > 0");
    k_update_delayed_scale<<<1, 1, 0, as_stream(stream)>>>(d_amax, fp8_max, d_scale, d_descale, d_history, history_len,
                                                          d_history_cursor, d_history_count);
    CF_LAUNCH_CHECK("update_delayed_scale");
    return CF_OK;
}

int cf_fp8_calib_minmax_update(const float* d_amax, float* d_calib_min, float* d_calib_max, void* stream) {
    CF_REQUIRE(d_amax && d_calib_min && d_calib_max, "cf_fp8_calib_minmax_update: null pointer");
    k_calib_minmax<<<1, 1, 0, as_stream(stream)>>>(d_amax, d_calib_min, d_calib_max);
    CF_LAUNCH_CHECK("calib_minmax_update");
    return CF_OK;
}

int cf_fp8_quantize_transpose_e4m3(const void* d_w, void* d_out, const float* d_scale, int K, int N, void* stream) {
    CF_REQUIRE(K >= 0 && N >= 0, "cf_fp8_quantize_transpose_e4m3: negative shape");
    CF_REQUIRE(d_scale && (K == 0 || N == 0 || (d_w && d_out)), "cf_fp8_quantize_transpose_e4m3: null pointer");
    return launch_tile_transpose<1>(d_w, nullptr, d_out, d_scale, K, N, as_stream(stream), "quantize_transpose_e4m3");
}

int cf_fp8_quant_and_transpose_e4m3(const void* d_in, void* d_act8_out, void* d_snap_out, const float* d_scale, int K,
                                    int N, void* stream) {
    CF_REQUIRE(K >= 0 && N >= 0, "cf_fp8_quant_and_transpose_e4m3: negative shape");
    CF_REQUIRE(d_scale && (K == 0 || N == 0 || d_in), "cf_fp8_quant_and_transpose_e4m3: null pointer");
    CF_REQUIRE(d_act8_out || d_snap_out, "cf_fp8_quant_and_transpose_e4m3: both outputs null");
    return launch_tile_transpose<1>(d_in, d_act8_out, d_snap_out, d_scale, K, N, as_stream(stream),
                                       "quant_and_transpose_e4m3");
}

int cf_transpose_u8(const void* d_in, void* d_out, int rows, int cols, void* stream) {
    CF_REQUIRE(rows >= 0 && cols >= 0, "cf_transpose_u8: negative shape");
    CF_REQUIRE(rows == 0 || cols == 0 || (d_in && d_out), "cf_transpose_u8: null pointer");
    return launch_tile_transpose<0>(d_in, nullptr, d_out, nullptr, rows, cols, as_stream(stream), "transpose_u8");
}

int cf_fp8_clip_probe(const float* d_amax, const float* d_scale, float fp8_max, float* d_stats, void* stream) {
    CF_REQUIRE(d_amax && d_scale && d_stats, "cf_fp8_clip_probe: null pointer");
    k_clip_probe<<<1, 1, 0, as_stream(stream)>>>(d_amax, d_scale, fp8_max, d_stats);
    CF_LAUNCH_CHECK("clip_probe");
    return CF_OK;
}

int cf_fp8_elem_clip_count(const void* d_x, const float* d_scale, float fp8_max, size_t n, float* d_out, void* stream) {
    CF_REQUIRE(d_scale && d_out && (n == 0 || d_x), "cf_fp8_elem_clip_count: null pointer");
    k_elem_clip_count<<<flat_grid(n, kThreads * 16), kThreads, 0, as_stream(stream)>>>(
        static_cast<const uint16_t*>(d_x), d_scale, fp8_max, n, d_out, reinterpret_cast<uintptr_t>(d_x) % 16 == 0);
    CF_LAUNCH_CHECK("elem_clip_count");
    return CF_OK;
}

static int pack_raw_common(const void* d_x, uint8_t* d_out, void* d_dequant, float* d_amax, float* d_scale,
                           float* d_descale, int* d_bad, size_t n, cudaStream_t st) {
    CF_REQUIRE(d_amax && d_scale && d_descale && d_bad && (n == 0 || (d_x && d_out)), "cf_fp8_pack_bf16_e4m3_raw: null pointer");
    CF_CUDA(cudaMemsetAsync(d_amax, 0, sizeof(float), st));
    CF_CUDA(cudaMemsetAsync(d_bad, 0, sizeof(int), st));
    const unsigned grid = flat_grid(n, kThreads * 16);
    const int vec_in = reinterpret_cast<uintptr_t>(d_x) % 16 == 0;
    const int vec = vec_in && reinterpret_cast<uintptr_t>(d_out) % 8 == 0 && reinterpret_cast<uintptr_t>(d_dequant) % 16 == 0;
    k_pack_raw_stats<<<grid, kThreads, 0, st>>>(static_cast<const uint16_t*>(d_x), n, d_amax, d_bad, vec_in);
    CF_LAUNCH_CHECK("pack_raw_stats");
    k_scale_from_amax<<<1, 1, 0, st>>>(d_amax, 448.0f, d_scale, d_descale);
    CF_LAUNCH_CHECK("scale_from_amax");
    if (d_dequant)
        k_pack_raw<true><<<grid, kThreads, 0, st>>>(static_cast<const uint16_t*>(d_x), d_out,
                                                    static_cast<uint16_t*>(d_dequant), d_scale, d_descale, d_bad, n, vec);
    else
        k_pack_raw<false><<<grid, kThreads, 0, st>>>(static_cast<const uint16_t*>(d_x), d_out, nullptr, d_scale,
                                                     d_descale, d_bad, n, vec);
    CF_LAUNCH_CHECK("pack_raw");
    return CF_OK;
}

int cf_fp8_pack_bf16_e4m3_raw(const void* d_x, uint8_t* d_out, float* d_amax, float* d_scale, float* d_descale,
                              int* d_bad_count, size_t n, void* stream) {
    return pack_raw_common(d_x, d_out, nullptr, d_amax, d_scale, d_descale, d_bad_count, n, as_stream(stream));
}
int cf_fp8_pack_bf16_e4m3_raw_and_dequant(const void* d_x, uint8_t* d_out, void* d_dequant, float* d_amax,
                                          float* d_scale, float* d_descale, int* d_bad_count, size_t n, void* stream) {
    CF_REQUIRE(d_dequant || n == 0, "cf_fp8_pack_bf16_e4m3_raw_and_dequant: null dequant pointer");
    return pack_raw_common(d_x, d_out, d_dequant, d_amax, d_scale, d_descale, d_bad_count, n, as_stream(stream));
}
int cf_fp8_unpack_e4m3_raw_bf16(const uint8_t* d_in, const float* d_descale, void* d_out, size_t n, void* stream) {
    CF_REQUIRE(d_descale && (n == 0 || (d_in && d_out)), "cf_fp8_unpack_e4m3_raw_bf16: null pointer");
    const int vec = reinterpret_cast<uintptr_t>(d_in) % 8 == 0 && reinterpret_cast<uintptr_t>(d_out) % 16 == 0;
    k_unpack_raw<<<flat_grid(n, kThreads * 16), kThreads, 0, as_stream(stream)>>>(d_in, d_descale,
                                                                                 static_cast<uint16_t*>(d_out), n, vec);
    CF_LAUNCH_CHECK("unpack_raw");
    return CF_OK;
}

}  // extern "C"
