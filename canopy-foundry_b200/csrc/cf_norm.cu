// RMSNorm that emits the FP8 operand of the following GEMM in the same pass.
//
// The reference normalises (kernels/rmsnorm.cu:13-54), writes the bf16 row, and a second kernel reads it back to
// quantise it (src/trainer.cu:6097 then :6115, fp8_quant_act): 7 bytes of HBM traffic per element. Here the row is
// read once, normalised in shared memory, and leaves as bf16 (optional) and E4M3 together: 5 bytes per element,
// 3 without the bf16 copy.
//
// The arithmetic and the order of every fp32 operation are the reference kernel's, so the bf16 row, the rms value
// and the E4M3 bytes are bit-identical to the two-kernel sequence: one block of T = min(H, 512) threads per row,
// thread t accumulates x[h]^2 for h = t, t+T, ... in that order, xor-butterfly inside the warp, warp leaders through
// shared memory, a second butterfly over the warp count; rms = sqrtf(sum / H + eps);
// out = bf16((x * (1 / rms)) * scale[h]). What differs is the data movement: 16-byte loads fill a shared-memory copy
// of the row, each thread picks its strided elements from there, and results return to HBM as 16-byte stores.
#include "cf_common.cuh"

#include "cf_internal.cuh"

namespace cf {
namespace {

constexpr int kNormThreads = 512;
constexpr int kNormMaxH = 16384;            // shared memory: 2 bytes (bf16 row) + 1 byte (codes) per column

template <int MODE>
__global__ void __launch_bounds__(kNormThreads) k_rmsnorm(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gamma,
                                                          uint16_t* __restrict__ out, float* __restrict__ rms_out,
                                                          uint8_t* __restrict__ out8, const float* __restrict__ scale,
                                                          float* __restrict__ amax, float* __restrict__ row_scale,
                                                          float* __restrict__ row_descale, int H, float eps, int vec,
                                                          const RingTail tail) {
    extern __shared__ __align__(16) uint8_t s_raw[];
    uint16_t* s_x = reinterpret_cast<uint16_t*>(s_raw);
    uint8_t* s_q = s_raw + static_cast<size_t>((H + 7) & ~7) * 2;
    __shared__ float s_red[32];
    const long long row = blockIdx.x;
    const int t = threadIdx.x, T = blockDim.x;
    const uint16_t* xr = x + row * H;

    if (vec & 1) {
        const uint4* src = reinterpret_cast<const uint4*>(xr);
        uint4* dst = reinterpret_cast<uint4*>(s_x);
        for (int v = t; v < H / 8; v += T) dst[v] = __ldcs(src + v);
    } else {
        for (int h = t; h < H; h += T) s_x[h] = xr[h];
    }
    __syncthreads();

    float ms = 0.0f;
    for (int h = t; h < H; h += T) {
        const float v = bf16_bits_to_f32(s_x[h]);
        ms = fmaf(v, v, ms);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ms += __shfl_xor_sync(0xffffffffu, ms, off);
    if ((t & 31) == 0) s_red[t >> 5] = ms;
    __syncthreads();
    if (t < 32) {
        ms = (t < (T + 31) / 32) ? s_red[t] : 0.0f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ms += __shfl_xor_sync(0xffffffffu, ms, off);
    }
    if (t == 0) s_red[0] = ms;
    __syncthreads();
    const float rms_val = sqrtf(__fadd_rn(__fdiv_rn(s_red[0], static_cast<float>(H)), eps));
    if (t == 0 && rms_out) rms_out[row] = rms_val;
    const float inv_rms = __fdiv_rn(1.0f, rms_val);
    __syncthreads();                       // s_red is reused by the row maximum below

    const float s1 = MODE == 1 ? *scale : 0.0f;
    float local = 0.0f;
    for (int h = t; h < H; h += T) {
        const float v = __fmul_rn(__fmul_rn(bf16_bits_to_f32(s_x[h]), inv_rms), bf16_bits_to_f32(gamma[h]));
        const uint16_t b = __bfloat16_as_ushort(__float2bfloat16_rn(v));
        s_x[h] = b;                        // only this thread ever reads element h
        const float n = bf16_bits_to_f32(b);
        local = fmaxf(local, fabsf(n));
        if (MODE == 1) s_q[h] = cvt_fp8<false>(n * s1);
    }
    if (MODE == 2) {
        // per-token scale from the row's own amax (kernels/fp8.cu:34-40 applied per row)
        float m = warp_max(local);
        if ((t & 31) == 0) s_red[t >> 5] = m;
        __syncthreads();
        if (t < 32) {
            m = (t < (T + 31) / 32) ? s_red[t] : 0.0f;
            m = warp_max(m);
            if (t == 0) s_red[0] = m;
        }
        __syncthreads();
        const float a = fmaxf(s_red[0], 1e-12f);
        const float s2 = __fdiv_rn(448.0f, a);
        if (t == 0) {
            if (row_scale) row_scale[row] = s2;
            row_descale[row] = __fdiv_rn(a, 448.0f);
        }
        for (int h = t; h < H; h += T) s_q[h] = cvt_fp8<false>(bf16_bits_to_f32(s_x[h]) * s2);
    }
    __syncthreads();

    if (out) {
        uint16_t* orow = out + row * H;
        if (vec & 1) {
            const uint4* src = reinterpret_cast<const uint4*>(s_x);
            uint4* dst = reinterpret_cast<uint4*>(orow);
            for (int v = t; v < H / 8; v += T) dst[v] = src[v];
        } else {
            for (int h = t; h < H; h += T) orow[h] = s_x[h];
        }
    }
    if (MODE != 0) {
        uint8_t* qrow = out8 + row * H;
        if (vec & 2) {
            const uint4* src = reinterpret_cast<const uint4*>(s_q);
            uint4* dst = reinterpret_cast<uint4*>(qrow);
            for (int v = t; v < H / 16; v += T) dst[v] = src[v];
        } else {
            for (int h = t; h < H; h += T) qrow[h] = s_q[h];
        }
    }
    if (MODE == 1) {
        block_amax_commit(local, amax);
        if (tail.ticket != nullptr && t == 0) ring_tail_last_block(tail, amax);
    }
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(lo))) |
           (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(hi))) << 16);
}

// Fast form for H % 512 == 0 (the reference then runs 512 threads, each owning H/512 elements): 64 threads per row,
// thread j loads the 16-byte vectors j, j+64, j+128, ... and so holds, in registers and in the reference's order,
// every element of the reference's threads 8j .. 8j+7. Their eight partial sums are kept apart; the reference's
// xor-butterfly over a warp (offsets 16, 8, 4, 2, 1) becomes two shuffles between neighbouring lanes (offsets 16 and
// 8 map to lanes j^2 and j^1) and three in-register steps, since every lane of a butterfly ends with the same bits.
// The sixteen warp sums meet in shared memory and are combined in the order of the reference's second butterfly.
// Blocks stride over rows, so the amax and ticket atomics are per block, not per row.
constexpr int kFastThreads = 64;

template <int MODE, int NV>
__global__ void __launch_bounds__(kFastThreads) k_rmsnorm_fast(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gamma,
                                                               uint16_t* __restrict__ out, float* __restrict__ rms_out,
                                                               uint8_t* __restrict__ out8, const float* __restrict__ scale,
                                                               float* __restrict__ amax, float* __restrict__ row_scale,
                                                               float* __restrict__ row_descale, int rows, int H, float eps,
                                                               const RingTail tail) {
    __shared__ float s_w[2][16];
    __shared__ float s_m[2][2];
    const int j = threadIdx.x;
    const int nv = H / 512;
    const float s1 = MODE == 1 ? *scale : 0.0f;
    const uint4* g4 = reinterpret_cast<const uint4*>(gamma);
    float local = 0.0f;
    int par = 0;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x, par ^= 1) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
        uint4 v[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (i < nv) v[i] = __ldcs(xr + j + kFastThreads * i);
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (i < nv) {
                float f[8];
                unpack8(v[i], f);
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] = fmaf(f[e], f[e], acc[e]);
            }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = __fadd_rn(acc[e], __shfl_xor_sync(0xffffffffu, acc[e], 2));
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = __fadd_rn(acc[e], __shfl_xor_sync(0xffffffffu, acc[e], 1));
        const float a0 = __fadd_rn(acc[0], acc[4]), a1 = __fadd_rn(acc[1], acc[5]);
        const float a2 = __fadd_rn(acc[2], acc[6]), a3 = __fadd_rn(acc[3], acc[7]);
        const float wsum = __fadd_rn(__fadd_rn(a0, a2), __fadd_rn(a1, a3));
        if ((j & 3) == 0) s_w[par][j >> 2] = wsum;
        __syncthreads();
        float b[16];
#pragma unroll
        for (int w = 0; w < 16; ++w) b[w] = __fadd_rn(s_w[par][w], 0.0f);
#pragma unroll
        for (int w = 0; w < 8; ++w) b[w] = __fadd_rn(b[w], b[w + 8]);
#pragma unroll
        for (int w = 0; w < 4; ++w) b[w] = __fadd_rn(b[w], b[w + 4]);
        const float total = __fadd_rn(__fadd_rn(b[0], b[2]), __fadd_rn(b[1], b[3]));
        const float rms_val = sqrtf(__fadd_rn(__fdiv_rn(total, static_cast<float>(H)), eps));
        if (j == 0 && rms_out) rms_out[row] = rms_val;
        const float inv_rms = __fdiv_rn(1.0f, rms_val);

        float rmax = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (i < nv) {
                const int vi = j + kFastThreads * i;
                float f[8], gg[8];
                unpack8(v[i], f);
                unpack8(__ldg(g4 + vi), gg);
                uint4 o;
                o.x = pack2(__fmul_rn(__fmul_rn(f[0], inv_rms), gg[0]), __fmul_rn(__fmul_rn(f[1], inv_rms), gg[1]));
                o.y = pack2(__fmul_rn(__fmul_rn(f[2], inv_rms), gg[2]), __fmul_rn(__fmul_rn(f[3], inv_rms), gg[3]));
                o.z = pack2(__fmul_rn(__fmul_rn(f[4], inv_rms), gg[4]), __fmul_rn(__fmul_rn(f[5], inv_rms), gg[5]));
                o.w = pack2(__fmul_rn(__fmul_rn(f[6], inv_rms), gg[6]), __fmul_rn(__fmul_rn(f[7], inv_rms), gg[7]));
                if (out) reinterpret_cast<uint4*>(out + row * H)[vi] = o;
                if (MODE != 0) {
                    unpack8(o, f);
#pragma unroll
                    for (int e = 0; e < 8; ++e) rmax = fmaxf(rmax, fabsf(f[e]));
                    if (MODE == 1) {
                        uint2 q;
                        q.x = cvt_fp8x4<false>(f[0] * s1, f[1] * s1, f[2] * s1, f[3] * s1);
                        q.y = cvt_fp8x4<false>(f[4] * s1, f[5] * s1, f[6] * s1, f[7] * s1);
                        reinterpret_cast<uint2*>(out8 + row * H)[vi] = q;
                    } else {
                        v[i] = o;
                    }
                }
            }
        }
        if (MODE == 1) local = fmaxf(local, rmax);
        if (MODE == 2) {
            rmax = warp_max(rmax);
            if ((j & 31) == 0) s_m[par][j >> 5] = rmax;
            __syncthreads();
            const float a = fmaxf(fmaxf(s_m[par][0], s_m[par][1]), 1e-12f);
            const float s2 = __fdiv_rn(448.0f, a);
            if (j == 0) {
                if (row_scale) row_scale[row] = s2;
                row_descale[row] = __fdiv_rn(a, 448.0f);
            }
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                if (i < nv) {
                    float f[8];
                    unpack8(v[i], f);
                    uint2 q;
                    q.x = cvt_fp8x4<false>(f[0] * s2, f[1] * s2, f[2] * s2, f[3] * s2);
                    q.y = cvt_fp8x4<false>(f[4] * s2, f[5] * s2, f[6] * s2, f[7] * s2);
                    reinterpret_cast<uint2*>(out8 + row * H)[j + kFastThreads * i] = q;
                }
            }
        }
        // s_w / s_m alternate between two copies: a thread can be at most one row ahead of the slowest one
        // (the barrier above), so the copy it writes next is no longer being read
    }
    if (MODE == 1) {
        block_amax_commit(local, amax);
        if (tail.ticket != nullptr && j == 0) ring_tail_last_block(tail, amax);
    }
}

template <int MODE, int NV>
int launch_fast(const uint16_t* x, const uint16_t* g, uint16_t* o, float* rms, uint8_t* q, const float* scale, float* amax,
                float* row_scale, float* row_descale, int rows, int H, float eps, const RingTail& tail, cudaStream_t st) {
    int per_sm = 0;
    CF_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_rmsnorm_fast<MODE, NV>, kFastThreads, 0));
    if (per_sm < 1) per_sm = 1;
    long long grid = static_cast<long long>(sm_count()) * per_sm;
    if (grid > rows) grid = rows;
    k_rmsnorm_fast<MODE, NV><<<static_cast<unsigned>(grid), kFastThreads, 0, st>>>(x, g, o, rms, q, scale, amax, row_scale,
                                                                                  row_descale, rows, H, eps, tail);
    CF_LAUNCH_CHECK("rmsnorm");
    return CF_OK;
}

template <int MODE>
int launch_fast_nv(int nv, const uint16_t* x, const uint16_t* g, uint16_t* o, float* rms, uint8_t* q, const float* scale,
                   float* amax, float* row_scale, float* row_descale, int rows, int H, float eps, const RingTail& tail,
                   cudaStream_t st) {
    if (nv <= 4) return launch_fast<MODE, 4>(x, g, o, rms, q, scale, amax, row_scale, row_descale, rows, H, eps, tail, st);
    if (nv <= 8) return launch_fast<MODE, 8>(x, g, o, rms, q, scale, amax, row_scale, row_descale, rows, H, eps, tail, st);
    if (nv <= 16) return launch_fast<MODE, 16>(x, g, o, rms, q, scale, amax, row_scale, row_descale, rows, H, eps, tail, st);
    return launch_fast<MODE, 32>(x, g, o, rms, q, scale, amax, row_scale, row_descale, rows, H, eps, tail, st);
}

// Warp-per-row form (H % 512 == 0, H <= 8192), optionally with the row clip the reference runs between the norm and
// the quantiser (act_row_clip, src/trainer.cu:3822-3845 and 3940-3991: squared row norm of the normalised bf16 row by
// a 256-thread block, rows whose norm exceeds an absolute ceiling are rescaled and rounded to bf16 again). Lane j holds
// the vectors j, j+32, j+64, ...: element h = 8(j + 32 i) + e. That one lane owns, complete and in order, both
//   * the reference norm kernel's threads t = 8j + e + 256 (i & 1)   (512 threads, elements t, t+512, ...), and
//   * the clip kernel's threads          t' = 8j + e                 (256 threads, elements t', t'+256, ...),
// so every fused-multiply-add chain of the two reference reductions runs inside one lane, the xor-butterflies of both
// (offsets 16, 8 between lanes j^2, j^1; 4, 2, 1 inside the lane) stay inside the warp, and no block barrier is needed.
constexpr int kWarpRowThreads = 128;

template <int MODE, int NV, bool CLIP>
__global__ void __launch_bounds__(kWarpRowThreads) k_rmsnorm_warp(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gamma,
                                                                  uint16_t* __restrict__ out, float* __restrict__ rms_out,
                                                                  uint8_t* __restrict__ out8, const float* __restrict__ scale,
                                                                  float* __restrict__ amax, float* __restrict__ row_scale,
                                                                  float* __restrict__ row_descale, int rows, int H, float eps,
                                                                  float clip_ceiling, const RingTail tail) {
    const int j = threadIdx.x & 31;
    const int nv = H / 256;                               // vectors per lane
    const float s1 = MODE == 1 ? *scale : 0.0f;
    const uint4* g4 = reinterpret_cast<const uint4*>(gamma);
    const long long warps = (static_cast<long long>(gridDim.x) * kWarpRowThreads) >> 5;
    float local = 0.0f;
    for (long long row = (static_cast<long long>(blockIdx.x) * kWarpRowThreads + threadIdx.x) >> 5; row < rows; row += warps) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
        uint4 v[NV];
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (i < nv) v[i] = __ldcs(xr + j + 32 * i);
        // mean square in the norm kernel's order: acc[p][e] is its thread 8j + e + 256p
        float acc[2][8];
#pragma unroll
        for (int e = 0; e < 8; ++e) { acc[0][e] = 0.0f; acc[1][e] = 0.0f; }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (i < nv) {
                float f[8];
                unpack8(v[i], f);
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[i & 1][e] = fmaf(f[e], f[e], acc[i & 1][e]);
            }
        }
        float wsum[2];
#pragma unroll
        for (int p = 0; p < 2; ++p) {
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[p][e] = __fadd_rn(acc[p][e], __shfl_xor_sync(0xffffffffu, acc[p][e], 2));
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[p][e] = __fadd_rn(acc[p][e], __shfl_xor_sync(0xffffffffu, acc[p][e], 1));
            const float a0 = __fadd_rn(acc[p][0], acc[p][4]), a1 = __fadd_rn(acc[p][1], acc[p][5]);
            const float a2 = __fadd_rn(acc[p][2], acc[p][6]), a3 = __fadd_rn(acc[p][3], acc[p][7]);
            wsum[p] = __fadd_rn(__fadd_rn(a0, a2), __fadd_rn(a1, a3));      // the norm kernel's warp j/4 + 8p
        }
        float b[16];
#pragma unroll
        for (int w = 0; w < 16; ++w) b[w] = __fadd_rn(__shfl_sync(0xffffffffu, wsum[w >> 3], 4 * (w & 7)), 0.0f);
#pragma unroll
        for (int w = 0; w < 8; ++w) b[w] = __fadd_rn(b[w], b[w + 8]);
#pragma unroll
        for (int w = 0; w < 4; ++w) b[w] = __fadd_rn(b[w], b[w + 4]);
        const float total = __fadd_rn(__fadd_rn(b[0], b[2]), __fadd_rn(b[1], b[3]));
        const float rms_val = sqrtf(__fadd_rn(__fdiv_rn(total, static_cast<float>(H)), eps));
        if (j == 0 && rms_out) rms_out[row] = rms_val;
        const float inv_rms = __fdiv_rn(1.0f, rms_val);

        // normalise, round to bf16 (kept packed in v[])
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (i < nv) {
                float f[8], gg[8];
                unpack8(v[i], f);
                unpack8(__ldg(g4 + j + 32 * i), gg);
                v[i].x = pack2(__fmul_rn(__fmul_rn(f[0], inv_rms), gg[0]), __fmul_rn(__fmul_rn(f[1], inv_rms), gg[1]));
                v[i].y = pack2(__fmul_rn(__fmul_rn(f[2], inv_rms), gg[2]), __fmul_rn(__fmul_rn(f[3], inv_rms), gg[3]));
                v[i].z = pack2(__fmul_rn(__fmul_rn(f[4], inv_rms), gg[4]), __fmul_rn(__fmul_rn(f[5], inv_rms), gg[5]));
                v[i].w = pack2(__fmul_rn(__fmul_rn(f[6], inv_rms), gg[6]), __fmul_rn(__fmul_rn(f[7], inv_rms), gg[7]));
            }
        }
        // Largest magnitude of the bf16 row from the packed words (two elements per instruction; a NaN anywhere makes
        // the lane's value NaN). It decides whether the clip's norm has to be computed at all: the row norm cannot
        // exceed sqrt(H) * amax, and the fp32 sum the reference forms exceeds the exact one by far less than the 1 %
        // margin below, so a row that passes the test is left alone by the reference too. Rows with a NaN or an
        // infinity fail the test and take the exact path. With the ceiling the reference uses by default (1000 on
        // normalised rows) every ordinary row passes, and the second reduction over the row is skipped.
        bool need_clip = CLIP;
        float lane_amax = 0.0f;
        if (CLIP || MODE != 0) {
            __nv_bfloat162 pm = __floats2bfloat162_rn(0.0f, 0.0f);
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                if (i < nv) {
                    const uint32_t w4[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) pm = __hmax2_nan(pm, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w4[q])));
                }
            }
            const float lo = __low2float(pm), hi = __high2float(pm);
            lane_amax = (lo != lo || hi != hi) ? __int_as_float(0x7fc00000) : fmaxf(lo, hi);
            if (CLIP) need_clip = __any_sync(0xffffffffu, !(lane_amax * (sqrtf(static_cast<float>(H)) * 1.01f) < clip_ceiling));
        }
        if (CLIP && need_clip) {
            // squared norm of the bf16 row in the clip kernel's order: c[e] is its thread 8j + e
            float c[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) c[e] = 0.0f;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                if (i < nv) {
                    float f[8];
                    unpack8(v[i], f);
#pragma unroll
                    for (int e = 0; e < 8; ++e) c[e] = fmaf(f[e], f[e], c[e]);
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) c[e] = __fadd_rn(c[e], __shfl_xor_sync(0xffffffffu, c[e], 2));
#pragma unroll
            for (int e = 0; e < 8; ++e) c[e] = __fadd_rn(c[e], __shfl_xor_sync(0xffffffffu, c[e], 1));
            const float c0 = __fadd_rn(c[0], c[4]), c1 = __fadd_rn(c[1], c[5]), c2 = __fadd_rn(c[2], c[6]), c3 = __fadd_rn(c[3], c[7]);
            const float cw = __fadd_rn(__fadd_rn(c0, c2), __fadd_rn(c1, c3));            // the clip kernel's warp j/4
            float t = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) t = __fadd_rn(t, __shfl_sync(0xffffffffu, cw, 4 * w));   // thread 0 adds the warps in order
            const float norm = sqrtf(t);
            // the reference's test is `if (norm <= ceiling) return;` (src/trainer.cu:3952): a NaN norm falls through
            // to the rescale and turns the whole row into NaN
            if (!(norm <= clip_ceiling)) {                 // warp-uniform
                const float scalef = __fdiv_rn(clip_ceiling, norm);
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    if (i < nv) {
                        float f[8];
                        unpack8(v[i], f);
                        v[i].x = pack2(__fmul_rn(f[0], scalef), __fmul_rn(f[1], scalef));
                        v[i].y = pack2(__fmul_rn(f[2], scalef), __fmul_rn(f[3], scalef));
                        v[i].z = pack2(__fmul_rn(f[4], scalef), __fmul_rn(f[5], scalef));
                        v[i].w = pack2(__fmul_rn(f[6], scalef), __fmul_rn(f[7], scalef));
                    }
                }
            }
        }
        // amax of the row this lane holds: already known unless the row went through the clip path (rescaled, or holding
        // a NaN, which the recorded amax ignores like fmaxf does): those rows are scanned again below
        const bool rescan = CLIP && need_clip;
        float rmax = rescan ? 0.0f : lane_amax;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (i < nv) {
                const int vi = j + 32 * i;
                if (out) reinterpret_cast<uint4*>(out + row * H)[vi] = v[i];
                if (MODE != 0) {
                    float f[8];
                    unpack8(v[i], f);
                    if (rescan) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) rmax = fmaxf(rmax, fabsf(f[e]));
                    }
                    if (MODE == 1) {
                        uint2 q;
                        q.x = cvt_fp8x4<false>(f[0] * s1, f[1] * s1, f[2] * s1, f[3] * s1);
                        q.y = cvt_fp8x4<false>(f[4] * s1, f[5] * s1, f[6] * s1, f[7] * s1);
                        reinterpret_cast<uint2*>(out8 + row * H)[vi] = q;
                    }
                }
            }
        }
        if (MODE == 1) local = fmaxf(local, rmax);
        if (MODE == 2) {
            const float a = fmaxf(warp_max(rmax), 1e-12f);
            const float s2 = __fdiv_rn(448.0f, a);
            if (j == 0) {
                if (row_scale) row_scale[row] = s2;
                row_descale[row] = __fdiv_rn(a, 448.0f);
            }
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                if (i < nv) {
                    float f[8];
                    unpack8(v[i], f);
                    uint2 q;
                    q.x = cvt_fp8x4<false>(f[0] * s2, f[1] * s2, f[2] * s2, f[3] * s2);
                    q.y = cvt_fp8x4<false>(f[4] * s2, f[5] * s2, f[6] * s2, f[7] * s2);
                    reinterpret_cast<uint2*>(out8 + row * H)[j + 32 * i] = q;
                }
            }
        }
    }
    if (MODE == 1) {
        block_amax_commit(local, amax);
        if (tail.ticket != nullptr && threadIdx.x == 0) ring_tail_last_block(tail, amax);
    }
}

template <int MODE, int NV, bool CLIP>
int launch_warp(const uint16_t* x, const uint16_t* g, uint16_t* o, float* rms, uint8_t* q, const float* scale, float* amax,
                float* row_scale, float* row_descale, int rows, int H, float eps, float ceiling, const RingTail& tail,
                cudaStream_t st) {
    int per_sm = 0;
    CF_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_rmsnorm_warp<MODE, NV, CLIP>, kWarpRowThreads, 0));
    if (per_sm < 1) per_sm = 1;
    long long grid = static_cast<long long>(sm_count()) * per_sm;
    const long long want = (static_cast<long long>(rows) + kWarpRowThreads / 32 - 1) / (kWarpRowThreads / 32);
    if (grid > want) grid = want;
    k_rmsnorm_warp<MODE, NV, CLIP><<<static_cast<unsigned>(grid), kWarpRowThreads, 0, st>>>(
        x, g, o, rms, q, scale, amax, row_scale, row_descale, rows, H, eps, ceiling, tail);
    CF_LAUNCH_CHECK("rmsnorm");
    return CF_OK;
}

template <int MODE, bool CLIP>
int launch_warp_nv(int nv, const uint16_t* x, const uint16_t* g, uint16_t* o, float* rms, uint8_t* q, const float* scale,
                   float* amax, float* row_scale, float* row_descale, int rows, int H, float eps, float ceiling,
                   const RingTail& tail, cudaStream_t st) {
    if (nv <= 4) return launch_warp<MODE, 4, CLIP>(x, g, o, rms, q, scale, amax, row_scale, row_descale, rows, H, eps, ceiling, tail, st);
    if (nv <= 8) return launch_warp<MODE, 8, CLIP>(x, g, o, rms, q, scale, amax, row_scale, row_descale, rows, H, eps, ceiling, tail, st);
    if (nv <= 16) return launch_warp<MODE, 16, CLIP>(x, g, o, rms, q, scale, amax, row_scale, row_descale, rows, H, eps, ceiling, tail, st);
    return launch_warp<MODE, 32, CLIP>(x, g, o, rms, q, scale, amax, row_scale, row_descale, rows, H, eps, ceiling, tail, st);
}

// act_row_clip for the shapes the warp kernel above does not take (src/trainer.cu:3940-3991, fixed-ceiling mode): one
// block of 256 threads per row of the normalised bf16 tensor, thread t adds x[c]^2 for c = t, t+256, ... with fused
// multiply-adds, xor butterfly inside each warp, thread 0 adds the eight warp sums in order, then the conditional
// rescale. The reference splits this over two kernels with the squared norm in a scratch array; here the row norm
// stays in shared memory.
__global__ void __launch_bounds__(256) k_row_clip(uint16_t* __restrict__ x, int cols, float ceiling) {
    __shared__ float s_w[8];
    __shared__ float s_norm;
    uint16_t* xr = x + static_cast<long long>(blockIdx.x) * cols;
    float s = 0.0f;
    for (int c = threadIdx.x; c < cols; c += 256) {
        const float v = bf16_bits_to_f32(xr[c]);
        s = fmaf(v, v, s);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, off));
    if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < 8; ++w) t = __fadd_rn(t, s_w[w]);
        s_norm = sqrtf(t);
    }
    __syncthreads();
    const float norm = s_norm;
    if (norm <= ceiling) return;
    const float scalef = __fdiv_rn(ceiling, norm);
    for (int c = threadIdx.x; c < cols; c += 256)
        xr[c] = __bfloat16_as_ushort(__float2bfloat16_rn(__fmul_rn(bf16_bits_to_f32(xr[c]), scalef)));
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

int rmsnorm_launch(int mode, const void* d_x, const void* d_gamma, void* d_normed_or_null, float* d_rms_or_null, void* d_out8,
                   const float* d_scale, float* d_amax, float* d_row_scale, float* d_row_descale, int rows, int H, float eps,
                   const RingTail& tail, cudaStream_t st, float clip_ceiling) {
    CF_REQUIRE(rows >= 0 && H > 0, "rmsnorm: bad shape");
    if (rows == 0) return CF_OK;
    CF_REQUIRE(d_x && d_gamma, "rmsnorm: null input pointer");
    CF_REQUIRE(mode != 0 || d_normed_or_null, "rmsnorm: no output requested");
    CF_REQUIRE(mode == 0 || d_out8, "rmsnorm: null E4M3 output pointer");
    CF_REQUIRE(mode != 1 || (d_scale && d_amax), "rmsnorm: null scale or amax pointer");
    CF_REQUIRE(mode != 2 || d_row_descale, "rmsnorm: null row descale pointer");
    if (H < 512 && H % 32 != 0) {
        // the reference launches min(H, 512) threads and reduces with full-mask shuffles: undefined for a partial warp
        set_error("rmsnorm: H below 512 must be a multiple of 32 (got %d)", H);
        return CF_ERR_UNSUPPORTED;
    }
    if (H > kNormMaxH) { set_error("rmsnorm: at most %d columns (got %d)", kNormMaxH, H); return CF_ERR_LIMIT; }
    const int rc = require_sm100();
    if (rc != CF_OK) return rc;
    int vec = (H % 8 == 0 && aligned16(d_x) && (d_normed_or_null == nullptr || aligned16(d_normed_or_null))) ? 1 : 0;
    if (mode != 0 && H % 16 == 0 && aligned16(d_out8)) vec |= 2;
    const int T = H < kNormThreads ? H : kNormThreads;
    const size_t smem = static_cast<size_t>((H + 7) & ~7) * 2 + (mode != 0 ? static_cast<size_t>((H + 15) & ~15) : 0);
    const uint16_t* x = static_cast<const uint16_t*>(d_x);
    const uint16_t* g = static_cast<const uint16_t*>(d_gamma);
    uint16_t* o = static_cast<uint16_t*>(d_normed_or_null);
    uint8_t* q = static_cast<uint8_t*>(d_out8);
    const bool fast = H % 512 == 0 && aligned16(d_x) && aligned16(d_gamma) &&
                      (d_normed_or_null == nullptr || aligned16(d_normed_or_null)) &&
                      (mode == 0 || (reinterpret_cast<uintptr_t>(d_out8) & 7) == 0);
    if (clip_ceiling > 0.0f && !(fast && H <= 8192)) {
        // Shapes the one-pass warp kernel does not take run the reference's own sequence: norm into the bf16 row buffer,
        // the row clip in place, then the quantiser over the clipped rows.
        if (d_normed_or_null == nullptr) {
            set_error("rmsnorm with row clip: for H = %d (not a multiple of 512, above 8192, or unaligned rows) the bf16 row buffer is needed", H);
            return CF_ERR_UNSUPPORTED;
        }
        int r = rmsnorm_launch(0, d_x, d_gamma, d_normed_or_null, d_rms_or_null, nullptr, nullptr, nullptr, nullptr, nullptr,
                               rows, H, eps, RingTail(), st, 0.0f);
        if (r != CF_OK) return r;
        k_row_clip<<<rows, 256, 0, st>>>(o, H, clip_ceiling);
        CF_LAUNCH_CHECK("row_clip");
        if (mode == 1) {
            r = cf_fp8_quantize_e4m3_record(d_normed_or_null, d_out8, d_scale, d_amax, static_cast<size_t>(rows) * H, st);
            if (r != CF_OK) return r;
            if (tail.ticket != nullptr)
                r = cf_fp8_update_delayed_scale(d_amax, tail.fp8_max, tail.scale, tail.descale, tail.history, tail.history_len,
                                                tail.history_cursor, tail.history_count, st);
            return r;
        }
        if (mode == 2)
            return cf_fp8_quantize_rowwise_e4m3(d_normed_or_null, H, d_out8, H, d_row_scale, d_row_descale, rows, H, st);
        return CF_OK;
    }
    if (fast && H <= 8192 && clip_ceiling > 0.0f) {
        const int nv = H / 256;
        if (clip_ceiling > 0.0f) {
            if (mode == 0) return launch_warp_nv<0, true>(nv, x, g, o, d_rms_or_null, q, d_scale, d_amax, d_row_scale, d_row_descale, rows, H, eps, clip_ceiling, tail, st);
            if (mode == 1) return launch_warp_nv<1, true>(nv, x, g, o, d_rms_or_null, q, d_scale, d_amax, d_row_scale, d_row_descale, rows, H, eps, clip_ceiling, tail, st);
            return launch_warp_nv<2, true>(nv, x, g, o, d_rms_or_null, q, d_scale, d_amax, d_row_scale, d_row_descale, rows, H, eps, clip_ceiling, tail, st);
        }
    }
    if (fast) {
        const int nv = H / 512;
        if (mode == 0) return launch_fast_nv<0>(nv, x, g, o, d_rms_or_null, q, d_scale, d_amax, d_row_scale, d_row_descale, rows, H, eps, tail, st);
        if (mode == 1) return launch_fast_nv<1>(nv, x, g, o, d_rms_or_null, q, d_scale, d_amax, d_row_scale, d_row_descale, rows, H, eps, tail, st);
        return launch_fast_nv<2>(nv, x, g, o, d_rms_or_null, q, d_scale, d_amax, d_row_scale, d_row_descale, rows, H, eps, tail, st);
    }
    if (smem > 40 * 1024) {
        // the largest rows need more than the default dynamic shared-memory window
        const void* fn = mode == 0 ? reinterpret_cast<const void*>(&k_rmsnorm<0>)
                       : mode == 1 ? reinterpret_cast<const void*>(&k_rmsnorm<1>) : reinterpret_cast<const void*>(&k_rmsnorm<2>);
        CF_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
    }
    if (mode == 0)
        k_rmsnorm<0><<<rows, T, smem, st>>>(x, g, o, d_rms_or_null, q, d_scale, d_amax, d_row_scale, d_row_descale, H, eps, vec, tail);
    else if (mode == 1)
        k_rmsnorm<1><<<rows, T, smem, st>>>(x, g, o, d_rms_or_null, q, d_scale, d_amax, d_row_scale, d_row_descale, H, eps, vec, tail);
    else
        k_rmsnorm<2><<<rows, T, smem, st>>>(x, g, o, d_rms_or_null, q, d_scale, d_amax, d_row_scale, d_row_descale, H, eps, vec, tail);
    CF_LAUNCH_CHECK("rmsnorm");
    return CF_OK;
}

}  // namespace cf

using namespace cf;

extern "C" {

int cf_rmsnorm_forward(const void* d_x, const void* d_scale, void* d_out, float* d_rms_or_null, int rows, int H, float eps,
                       void* stream) {
    return rmsnorm_launch(0, d_x, d_scale, d_out, d_rms_or_null, nullptr, nullptr, nullptr, nullptr, nullptr, rows, H, eps,
                          RingTail(), as_stream(stream));
}

int cf_rmsnorm_quantize_e4m3_record(const void* d_x, const void* d_scale, void* d_normed_or_null, float* d_rms_or_null,
                                    void* d_out8, const float* d_quant_scale, float* d_amax, int rows, int H, float eps,
                                    void* stream) {
    return rmsnorm_launch(1, d_x, d_scale, d_normed_or_null, d_rms_or_null, d_out8, d_quant_scale, d_amax, nullptr, nullptr,
                          rows, H, eps, RingTail(), as_stream(stream));
}

int cf_rmsnorm_quantize_rowwise_e4m3(const void* d_x, const void* d_scale, void* d_normed_or_null, float* d_rms_or_null,
                                     void* d_out8, float* d_row_scale_or_null, float* d_row_descale, int rows, int H,
                                     float eps, void* stream) {
    return rmsnorm_launch(2, d_x, d_scale, d_normed_or_null, d_rms_or_null, d_out8, nullptr, nullptr, d_row_scale_or_null,
                          d_row_descale, rows, H, eps, RingTail(), as_stream(stream));
}

int cf_rmsnorm_clip_quantize_e4m3_record(const void* d_x, const void* d_scale, void* d_normed_or_null, float* d_rms_or_null,
                                         void* d_out8, const float* d_quant_scale, float* d_amax, int rows, int H, float eps,
                                         float clip_ceiling, void* stream) {
    return rmsnorm_launch(1, d_x, d_scale, d_normed_or_null, d_rms_or_null, d_out8, d_quant_scale, d_amax, nullptr, nullptr,
                          rows, H, eps, RingTail(), as_stream(stream), clip_ceiling);
}

int cf_rmsnorm_clip_forward(const void* d_x, const void* d_scale, void* d_out, float* d_rms_or_null, int rows, int H, float eps,
                            float clip_ceiling, void* stream) {
    return rmsnorm_launch(0, d_x, d_scale, d_out, d_rms_or_null, nullptr, nullptr, nullptr, nullptr, nullptr, rows, H, eps,
                          RingTail(), as_stream(stream), clip_ceiling);
}

}  // extern "C"
