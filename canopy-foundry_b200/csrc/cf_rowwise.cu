// Per-token (row-wise) E4M3 quantisation and the SwiGLU -> re-quantise fusions that feed the down projection.
//
// Row-wise scaling has no counterpart in the reference (it scales per tensor); it generalises
// kernels/fp8.cu:34-49 per row:  a_r = max(amax_r, 1e-12), scale_r = 448 / a_r, descale_r = a_r / 448,
// code = e4m3(x * scale_r). The SwiGLU arithmetic and its bf16 rounding point are those of
// kernels/activations.cu:11-40 (the product is rounded to bf16 before it is quantised, exactly as if
// swiglu_forward had written it to memory first).
#include "cf_common.cuh"
#include "cf_internal.cuh"

#define CF_TRY_RET(expr) do { const int rc__ = (expr); if (rc__ != CF_OK) return rc__; } while (0)

namespace cf {
namespace {

constexpr int kRT = 256;          // threads per row
constexpr int kMaxVec = 8;        // 16-byte vectors (8 elements each) a thread keeps in registers: K <= 16384

__device__ __forceinline__ float stable_sigmoid(float x) {
    // Both branches of the reference (1/(1+exp(-x)) for x >= 0, exp(x)/(1+exp(x)) otherwise) share e = exp(-|x|);
    // one IEEE division with the matching numerator gives the same bits without a divergent branch.
    const float e = expf(-fabsf(x));
    return __fdiv_rn(x >= 0.0f ? 1.0f : e, 1.0f + e);
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}

__device__ __forceinline__ float block_max_bcast(float v) {
    __shared__ float s_part[kRT / 32];
    __shared__ float s_res;
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < kRT / 32 ? s_part[threadIdx.x] : 0.0f;
        t = warp_max(t);
        if (threadIdx.x == 0) s_res = t;
    }
    __syncthreads();
    return s_res;
}

// One block per row. SWIGLU: the row is silu(gate)*up rounded to bf16; otherwise the bf16 input itself.
// The row lives in registers between the amax pass and the quantise pass (one read of HBM).
template <bool SWIGLU>
__global__ void __launch_bounds__(kRT) k_rowwise(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b, long long ld_in,
                                                 uint8_t* __restrict__ out, long long ld_out, float* __restrict__ row_scale,
                                                 float* __restrict__ row_descale, int cols, int vec) {
    const long long row = blockIdx.x;
    const uint16_t* ar = a + row * ld_in;
    const uint16_t* br = SWIGLU ? b + row * ld_in : nullptr;
    uint8_t* orow = out + row * ld_out;
    float vals[kMaxVec][8];
    float local = 0.0f;
    const int nvec = vec ? cols / 8 : 0;
#pragma unroll
    for (int j = 0; j < kMaxVec; ++j) {
        const int v = threadIdx.x + j * kRT;
        if (v < nvec) {
            unpack8(*reinterpret_cast<const uint4*>(ar + v * 8), vals[j]);
            if (SWIGLU) {
                float u[8];
                unpack8(*reinterpret_cast<const uint4*>(br + v * 8), u);
#pragma unroll
                for (int e = 0; e < 8; ++e) vals[j][e] = bf16_round(vals[j][e] * stable_sigmoid(vals[j][e]) * u[e]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) local = fmaxf(local, fabsf(vals[j][e]));
        }
    }
    // columns the vector path does not cover (cols % 8, or everything when unaligned): recomputed in pass 2
    for (int c = nvec * 8 + threadIdx.x; c < cols; c += kRT) {
        float x = bf16_bits_to_f32(ar[c]);
        if (SWIGLU) x = bf16_round(x * stable_sigmoid(x) * bf16_bits_to_f32(br[c]));
        local = fmaxf(local, fabsf(x));
    }
    const float amax = fmaxf(block_max_bcast(local), 1e-12f);
    const float s = __fdiv_rn(448.0f, amax);
    if (threadIdx.x == 0) {
        if (row_scale) row_scale[row] = s;
        row_descale[row] = __fdiv_rn(amax, 448.0f);
    }
#pragma unroll
    for (int j = 0; j < kMaxVec; ++j) {
        const int v = threadIdx.x + j * kRT;
        if (v < nvec) {
            uint2 q;
            q.x = cvt_fp8x4<false>(vals[j][0] * s, vals[j][1] * s, vals[j][2] * s, vals[j][3] * s);
            q.y = cvt_fp8x4<false>(vals[j][4] * s, vals[j][5] * s, vals[j][6] * s, vals[j][7] * s);
            *reinterpret_cast<uint2*>(orow + v * 8) = q;
        }
    }
    for (int c = nvec * 8 + threadIdx.x; c < cols; c += kRT) {
        float x = bf16_bits_to_f32(ar[c]);
        if (SWIGLU) x = bf16_round(x * stable_sigmoid(x) * bf16_bits_to_f32(br[c]));
        orow[c] = cvt_fp8<false>(x * s);
    }
}

// Fast form for 16-byte aligned rows with cols % 8 == 0: 64 threads per row, thread j keeps the vectors j, j+64, ...
// of the row in registers (packed bf16) between the amax and the quantise pass, blocks stride over rows. Small blocks
// keep many rows in flight per SM, which is what a one-row-at-a-time kernel needs to reach HBM bandwidth.
constexpr int kFastT = 64;

__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
    return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(lo))) |
           (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(hi))) << 16);
}

template <bool SWIGLU, int NV>
__global__ void __launch_bounds__(kFastT) k_rowwise_fast(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b,
                                                         long long ld_in, uint8_t* __restrict__ out, long long ld_out,
                                                         float* __restrict__ row_scale, float* __restrict__ row_descale,
                                                         int rows, int cols) {
    __shared__ float s_m[2][2];
    const int j = threadIdx.x;
    const int nvec = cols / 8;
    int par = 0;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x, par ^= 1) {
        const uint4* ar = reinterpret_cast<const uint4*>(a + row * ld_in);
        const uint4* br = SWIGLU ? reinterpret_cast<const uint4*>(b + row * ld_in) : nullptr;
        uint4 v[NV];
        float local = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (j + kFastT * i < nvec) v[i] = __ldcs(ar + j + kFastT * i);
        if (SWIGLU) {
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                if (j + kFastT * i < nvec) {
                    float g[8], u[8];
                    unpack8(v[i], g);
                    unpack8(__ldcs(br + j + kFastT * i), u);
                    // the product is rounded to bf16 as swiglu_forward would store it
                    v[i].x = pack2_bf16(g[0] * stable_sigmoid(g[0]) * u[0], g[1] * stable_sigmoid(g[1]) * u[1]);
                    v[i].y = pack2_bf16(g[2] * stable_sigmoid(g[2]) * u[2], g[3] * stable_sigmoid(g[3]) * u[3]);
                    v[i].z = pack2_bf16(g[4] * stable_sigmoid(g[4]) * u[4], g[5] * stable_sigmoid(g[5]) * u[5]);
                    v[i].w = pack2_bf16(g[6] * stable_sigmoid(g[6]) * u[6], g[7] * stable_sigmoid(g[7]) * u[7]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (j + kFastT * i < nvec) {
                float f[8];
                unpack8(v[i], f);
#pragma unroll
                for (int e = 0; e < 8; ++e) local = fmaxf(local, fabsf(f[e]));
            }
        }
        local = warp_max(local);
        if ((j & 31) == 0) s_m[par][j >> 5] = local;
        __syncthreads();
        const float amax = fmaxf(fmaxf(s_m[par][0], s_m[par][1]), 1e-12f);
        const float s = __fdiv_rn(448.0f, amax);
        if (j == 0) {
            if (row_scale) row_scale[row] = s;
            row_descale[row] = __fdiv_rn(amax, 448.0f);
        }
        uint2* orow = reinterpret_cast<uint2*>(out + row * ld_out);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (j + kFastT * i < nvec) {
                float f[8];
                unpack8(v[i], f);
                uint2 q;
                q.x = cvt_fp8x4<false>(f[0] * s, f[1] * s, f[2] * s, f[3] * s);
                q.y = cvt_fp8x4<false>(f[4] * s, f[5] * s, f[6] * s, f[7] * s);
                orow[j + kFastT * i] = q;
            }
        }
        // s_m alternates between two copies: the one written next is read by no thread that is still in this row
    }
}

template <bool SWIGLU, int NV>
int launch_rowwise_fast(const uint16_t* a, const uint16_t* b, long long ld_in, uint8_t* out, long long ld_out, float* row_scale,
                        float* row_descale, int rows, int cols, cudaStream_t st) {
    int per_sm = 0;
    CF_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_rowwise_fast<SWIGLU, NV>, kFastT, 0));
    if (per_sm < 1) per_sm = 1;
    long long grid = static_cast<long long>(sm_count()) * per_sm;
    if (grid > rows) grid = rows;
    k_rowwise_fast<SWIGLU, NV><<<static_cast<unsigned>(grid), kFastT, 0, st>>>(a, b, ld_in, out, ld_out, row_scale, row_descale,
                                                                              rows, cols);
    return CF_OK;
}

// The same scheme for rows that are not 16-byte aligned or whose length is not a multiple of 8: each row is cut into a
// head of up to 7 elements (up to the first 16-byte boundary of the input), whole 16-byte vectors, and a tail of up to 7
// elements. Head and tail live in one register each of the threads 0..6; the vectors are stored as 8-byte words when the
// output address allows it and byte by byte otherwise. SWIGLU: gate and up must share their alignment (checked by the
// launcher).
template <bool SWIGLU, int NV>
__global__ void __launch_bounds__(kFastT) k_rowwise_ragged(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b,
                                                           long long ld_in, uint8_t* __restrict__ out, long long ld_out,
                                                           float* __restrict__ row_scale, float* __restrict__ row_descale,
                                                           int rows, int cols) {
    __shared__ float s_m[2][2];
    const int j = threadIdx.x;
    int par = 0;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x, par ^= 1) {
        const uint16_t* arow = a + row * ld_in;
        const uint16_t* brow = SWIGLU ? b + row * ld_in : nullptr;
        const int head = min(cols, static_cast<int>((8u - static_cast<unsigned>((reinterpret_cast<uintptr_t>(arow) >> 1) & 7u)) & 7u));
        const int nvec = (cols - head) >> 3;
        const int tail0 = head + (nvec << 3), tail = cols - tail0;
        const uint4* ar = reinterpret_cast<const uint4*>(arow + head);
        const uint4* br = SWIGLU ? reinterpret_cast<const uint4*>(brow + head) : nullptr;
        uint4 v[NV];
        float hx = 0.0f, tx = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (j + kFastT * i < nvec) v[i] = __ldcs(ar + j + kFastT * i);
        if (j < head) {
            hx = bf16_bits_to_f32(arow[j]);
            if (SWIGLU) hx = bf16_round(hx * stable_sigmoid(hx) * bf16_bits_to_f32(brow[j]));
        }
        if (j < tail) {
            tx = bf16_bits_to_f32(arow[tail0 + j]);
            if (SWIGLU) tx = bf16_round(tx * stable_sigmoid(tx) * bf16_bits_to_f32(brow[tail0 + j]));
        }
        float local = fmaxf(fabsf(hx), fabsf(tx));
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (j + kFastT * i < nvec) {
                float f[8];
                unpack8(v[i], f);
                if (SWIGLU) {
                    float u[8];
                    unpack8(__ldcs(br + j + kFastT * i), u);
                    v[i].x = pack2_bf16(f[0] * stable_sigmoid(f[0]) * u[0], f[1] * stable_sigmoid(f[1]) * u[1]);
                    v[i].y = pack2_bf16(f[2] * stable_sigmoid(f[2]) * u[2], f[3] * stable_sigmoid(f[3]) * u[3]);
                    v[i].z = pack2_bf16(f[4] * stable_sigmoid(f[4]) * u[4], f[5] * stable_sigmoid(f[5]) * u[5]);
                    v[i].w = pack2_bf16(f[6] * stable_sigmoid(f[6]) * u[6], f[7] * stable_sigmoid(f[7]) * u[7]);
                    unpack8(v[i], f);
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) local = fmaxf(local, fabsf(f[e]));
            }
        }
        local = warp_max(local);
        if ((j & 31) == 0) s_m[par][j >> 5] = local;
        __syncthreads();
        const float amax = fmaxf(fmaxf(s_m[par][0], s_m[par][1]), 1e-12f);
        const float s = __fdiv_rn(448.0f, amax);
        if (j == 0) {
            if (row_scale) row_scale[row] = s;
            row_descale[row] = __fdiv_rn(amax, 448.0f);
        }
        uint8_t* orow = out + row * ld_out;
        if (j < head) orow[j] = cvt_fp8<false>(hx * s);
        if (j < tail) orow[tail0 + j] = cvt_fp8<false>(tx * s);
        uint8_t* ob = orow + head;
        const bool word = (reinterpret_cast<uintptr_t>(ob) & 7u) == 0;      // the same for every vector of the row
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (j + kFastT * i < nvec) {
                float f[8];
                unpack8(v[i], f);
                uint2 q;
                q.x = cvt_fp8x4<false>(f[0] * s, f[1] * s, f[2] * s, f[3] * s);
                q.y = cvt_fp8x4<false>(f[4] * s, f[5] * s, f[6] * s, f[7] * s);
                uint8_t* o = ob + (static_cast<size_t>(j + kFastT * i) << 3);
                if (word) {
                    *reinterpret_cast<uint2*>(o) = q;
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        o[e] = static_cast<uint8_t>(q.x >> (8 * e));
                        o[4 + e] = static_cast<uint8_t>(q.y >> (8 * e));
                    }
                }
            }
        }
    }
}

template <bool SWIGLU, int NV>
int launch_rowwise_ragged(const uint16_t* a, const uint16_t* b, long long ld_in, uint8_t* out, long long ld_out, float* row_scale,
                          float* row_descale, int rows, int cols, cudaStream_t st) {
    int per_sm = 0;
    CF_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_rowwise_ragged<SWIGLU, NV>, kFastT, 0));
    if (per_sm < 1) per_sm = 1;
    long long grid = static_cast<long long>(sm_count()) * per_sm;
    if (grid > rows) grid = rows;
    k_rowwise_ragged<SWIGLU, NV><<<static_cast<unsigned>(grid), kFastT, 0, st>>>(a, b, ld_in, out, ld_out, row_scale, row_descale,
                                                                                rows, cols);
    return CF_OK;
}

static_assert(kFastT * 32 * 8 >= kRT * kMaxVec * 8, "the ragged form covers every row length the entry points accept");

template <bool SWIGLU>
int launch_rowwise_ragged_nv(const uint16_t* a, const uint16_t* b, long long ld_in, uint8_t* out, long long ld_out,
                             float* row_scale, float* row_descale, int rows, int cols, cudaStream_t st) {
    const int nv = (cols / 8 + kFastT - 1) / kFastT;
    if (nv <= 2) return launch_rowwise_ragged<SWIGLU, 2>(a, b, ld_in, out, ld_out, row_scale, row_descale, rows, cols, st);
    if (nv <= 4) return launch_rowwise_ragged<SWIGLU, 4>(a, b, ld_in, out, ld_out, row_scale, row_descale, rows, cols, st);
    if (nv <= 8) return launch_rowwise_ragged<SWIGLU, 8>(a, b, ld_in, out, ld_out, row_scale, row_descale, rows, cols, st);
    if (nv <= 16) return launch_rowwise_ragged<SWIGLU, 16>(a, b, ld_in, out, ld_out, row_scale, row_descale, rows, cols, st);
    return launch_rowwise_ragged<SWIGLU, 32>(a, b, ld_in, out, ld_out, row_scale, row_descale, rows, cols, st);
}

template <bool SWIGLU>
int launch_rowwise_fast_nv(const uint16_t* a, const uint16_t* b, long long ld_in, uint8_t* out, long long ld_out,
                           float* row_scale, float* row_descale, int rows, int cols, cudaStream_t st) {
    const int nv = (cols / 8 + kFastT - 1) / kFastT;
    if (nv <= 2) return launch_rowwise_fast<SWIGLU, 2>(a, b, ld_in, out, ld_out, row_scale, row_descale, rows, cols, st);
    if (nv <= 4) return launch_rowwise_fast<SWIGLU, 4>(a, b, ld_in, out, ld_out, row_scale, row_descale, rows, cols, st);
    if (nv <= 8) return launch_rowwise_fast<SWIGLU, 8>(a, b, ld_in, out, ld_out, row_scale, row_descale, rows, cols, st);
    if (nv <= 16) return launch_rowwise_fast<SWIGLU, 16>(a, b, ld_in, out, ld_out, row_scale, row_descale, rows, cols, st);
    return launch_rowwise_fast<SWIGLU, 32>(a, b, ld_in, out, ld_out, row_scale, row_descale, rows, cols, st);
}

// Per-tensor delayed-scaling form: out = e4m3(bf16(silu(g)*u) * *scale), amax of the bf16 product recorded.
// Fuses swiglu_forward (kernels/activations.cu) with fp8_quantize_e4m3_record (kernels/fp8.cu:67-84):
// the 2-byte intermediate never goes to HBM.
__global__ void __launch_bounds__(kRT) k_swiglu_record(const uint16_t* __restrict__ g, const uint16_t* __restrict__ u,
                                                       long long ld_in, uint8_t* __restrict__ out, long long ld_out,
                                                       const float* __restrict__ scale, float* __restrict__ amax,
                                                       long long rows, int cols, int vec, const RingTail tail) {
    const float s = *scale;
    float local = 0.0f;
    const int vpr = vec ? cols / 8 : 0;                       // vectors per row
    const long long total = rows * vpr;
    for (long long i = static_cast<long long>(blockIdx.x) * kRT + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * kRT) {
        const long long r = i / vpr;
        const int v = static_cast<int>(i - r * vpr);
        float a[8], b[8];
        unpack8(*reinterpret_cast<const uint4*>(g + r * ld_in + v * 8), a);
        unpack8(*reinterpret_cast<const uint4*>(u + r * ld_in + v * 8), b);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            a[e] = bf16_round(a[e] * stable_sigmoid(a[e]) * b[e]);
            local = fmaxf(local, fabsf(a[e]));
        }
        uint2 q;
        q.x = cvt_fp8x4<false>(a[0] * s, a[1] * s, a[2] * s, a[3] * s);
        q.y = cvt_fp8x4<false>(a[4] * s, a[5] * s, a[6] * s, a[7] * s);
        *reinterpret_cast<uint2*>(out + r * ld_out + v * 8) = q;
    }
    const int tail0 = vpr * 8, tailn = cols - tail0;
    const long long ttotal = rows * tailn;
    for (long long i = static_cast<long long>(blockIdx.x) * kRT + threadIdx.x; i < ttotal;
         i += static_cast<long long>(gridDim.x) * kRT) {
        const long long r = i / tailn;
        const int c = tail0 + static_cast<int>(i - r * tailn);
        float x = bf16_bits_to_f32(g[r * ld_in + c]);
        x = bf16_round(x * stable_sigmoid(x) * bf16_bits_to_f32(u[r * ld_in + c]));
        local = fmaxf(local, fabsf(x));
        out[r * ld_out + c] = cvt_fp8<false>(x * s);
    }
    block_amax_commit(local, amax);
    if (tail.ticket != nullptr && threadIdx.x == 0) ring_tail_last_block(tail, amax);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// out = bf16(acc), acc = 0: the reader side of a reduce-scatter into an fp32 accumulation slice.
__global__ void __launch_bounds__(kRT) k_finish_f32(float* __restrict__ acc, uint16_t* __restrict__ out, size_t n, int vec) {
    const size_t stride = static_cast<size_t>(gridDim.x) * kRT;
    const size_t nv = vec ? n / 8 : 0;
    for (size_t i = static_cast<size_t>(blockIdx.x) * kRT + threadIdx.x; i < nv; i += stride) {
        float4* a = reinterpret_cast<float4*>(acc) + 2 * i;
        const float4 lo = a[0], hi = a[1];
        uint4 o;
        o.x = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(lo.x))) | (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(lo.y))) << 16);
        o.y = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(lo.z))) | (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(lo.w))) << 16);
        o.z = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(hi.x))) | (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(hi.y))) << 16);
        o.w = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(hi.z))) | (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(hi.w))) << 16);
        reinterpret_cast<uint4*>(out)[i] = o;
        a[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        a[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (size_t i = nv * 8 + static_cast<size_t>(blockIdx.x) * kRT + threadIdx.x; i < n; i += stride) {
        out[i] = __bfloat16_as_ushort(__float2bfloat16_rn(acc[i]));
        acc[i] = 0.0f;
    }
}

// Row-wise quantiser for rows whose amax is already known (the GEMM that produced them recorded it, possibly reduced
// over the ranks that hold other column slices of the same rows): a pure stream, 16 elements per thread per step (two
// 16-byte loads, one 16-byte store), scale_r = 448 / max(amax_r, 1e-12) derived per row on the fly.
__global__ void __launch_bounds__(kRT) k_rowwise_given_amax(const uint16_t* __restrict__ x, long long ld_x, uint8_t* __restrict__ out,
                                                            long long ld_out, const float* __restrict__ row_amax,
                                                            float* __restrict__ row_scale, float* __restrict__ row_descale,
                                                            long long rows, int cols, int vec) {
    const long long stride = static_cast<long long>(gridDim.x) * kRT;
    if (vec) {
        const int vpr = cols / 16;
        const long long total = rows * vpr;
        for (long long i = static_cast<long long>(blockIdx.x) * kRT + threadIdx.x; i < total; i += stride) {
            const long long r = i / vpr;
            const int c = static_cast<int>(i - r * vpr);
            const uint4* src = reinterpret_cast<const uint4*>(x + r * ld_x) + 2 * c;
            const uint4 v0 = __ldcs(src), v1 = __ldcs(src + 1);
            const float a = fmaxf(row_amax[r], 1e-12f);
            const float sc = __fdiv_rn(448.0f, a);
            if (c == 0) {
                if (row_scale) row_scale[r] = sc;
                row_descale[r] = __fdiv_rn(a, 448.0f);
            }
            float f[8], g[8];
            unpack8(v0, f);
            unpack8(v1, g);
            uint4 q;
            q.x = cvt_fp8x4<false>(f[0] * sc, f[1] * sc, f[2] * sc, f[3] * sc);
            q.y = cvt_fp8x4<false>(f[4] * sc, f[5] * sc, f[6] * sc, f[7] * sc);
            q.z = cvt_fp8x4<false>(g[0] * sc, g[1] * sc, g[2] * sc, g[3] * sc);
            q.w = cvt_fp8x4<false>(g[4] * sc, g[5] * sc, g[6] * sc, g[7] * sc);
            __stcs(reinterpret_cast<uint4*>(out + r * ld_out) + c, q);
        }
        return;
    }
    const long long total = rows * cols;
    for (long long i = static_cast<long long>(blockIdx.x) * kRT + threadIdx.x; i < total; i += stride) {
        const long long r = i / cols;
        const int c = static_cast<int>(i - r * cols);
        const float a = fmaxf(row_amax[r], 1e-12f);
        const float sc = __fdiv_rn(448.0f, a);
        if (c == 0) {
            if (row_scale) row_scale[r] = sc;
            row_descale[r] = __fdiv_rn(a, 448.0f);
        }
        out[r * ld_out + c] = cvt_fp8<false>(bf16_bits_to_f32(x[r * ld_x + c]) * sc);
    }
}

}  // namespace

int swiglu_record_launch(const void* d_gate, const void* d_up, int ld_in, void* d_out, int ld_out, const float* d_scale,
                         float* d_amax, int rows, int cols, const RingTail& tail, cudaStream_t st) {
    const int vec = aligned16(d_gate) && aligned16(d_up) && (ld_in % 8 == 0) &&
                    ((reinterpret_cast<uintptr_t>(d_out) & 7) == 0) && (ld_out % 8 == 0);
    const size_t items = static_cast<size_t>(rows) * (vec ? cols / 8 : cols);
    size_t blocks = (items + kRT * 2 - 1) / (kRT * 2);
    const size_t cap = static_cast<size_t>(sm_count()) * 8;
    if (blocks < 1) blocks = 1;
    if (blocks > cap) blocks = cap;
    k_swiglu_record<<<static_cast<unsigned>(blocks), kRT, 0, st>>>(
        static_cast<const uint16_t*>(d_gate), static_cast<const uint16_t*>(d_up), ld_in, static_cast<uint8_t*>(d_out), ld_out,
        d_scale, d_amax, rows, cols, vec, tail);
    CF_LAUNCH_CHECK("swiglu_quantize_e4m3_record");
    return CF_OK;
}

}  // namespace cf

using namespace cf;

extern "C" {

int cf_fp8_quantize_rowwise_e4m3(const void* d_x, int ld_x, void* d_out, int ld_out, float* d_row_scale,
                                 float* d_row_descale, int rows, int cols, void* stream) {
    CF_REQUIRE(rows >= 0 && cols >= 0 && ld_x >= cols && ld_out >= cols, "cf_fp8_quantize_rowwise_e4m3: bad shape");
    if (rows == 0 || cols == 0) return CF_OK;
    CF_REQUIRE(d_x && d_out && d_row_descale, "cf_fp8_quantize_rowwise_e4m3: null pointer");
    if (cols > kRT * kMaxVec * 8) { set_error("cf_fp8_quantize_rowwise_e4m3: at most %d columns", kRT * kMaxVec * 8); return CF_ERR_LIMIT; }
    const int vec = aligned16(d_x) && (ld_x % 8 == 0) && ((reinterpret_cast<uintptr_t>(d_out) & 7) == 0) && (ld_out % 8 == 0);
    if (vec && cols % 8 == 0) {
        CF_TRY_RET(launch_rowwise_fast_nv<false>(static_cast<const uint16_t*>(d_x), nullptr, ld_x, static_cast<uint8_t*>(d_out), ld_out,
                                                 d_row_scale, d_row_descale, rows, cols, as_stream(stream)));
        CF_LAUNCH_CHECK("quantize_rowwise_e4m3");
        return CF_OK;
    }
    // any other alignment or length (cols <= 16384 was checked above): head / vectors / tail per row
    CF_TRY_RET(launch_rowwise_ragged_nv<false>(static_cast<const uint16_t*>(d_x), nullptr, ld_x, static_cast<uint8_t*>(d_out), ld_out,
                                               d_row_scale, d_row_descale, rows, cols, as_stream(stream)));
    CF_LAUNCH_CHECK("quantize_rowwise_e4m3");
    return CF_OK;
}

int cf_swiglu_quantize_rowwise_e4m3(const void* d_gate, const void* d_up, int ld_in, void* d_out, int ld_out,
                                    float* d_row_scale, float* d_row_descale, int rows, int cols, void* stream) {
    CF_REQUIRE(rows >= 0 && cols >= 0 && ld_in >= cols && ld_out >= cols, "cf_swiglu_quantize_rowwise_e4m3: bad shape");
    if (rows == 0 || cols == 0) return CF_OK;
    CF_REQUIRE(d_gate && d_up && d_out && d_row_descale, "cf_swiglu_quantize_rowwise_e4m3: null pointer");
    if (cols > kRT * kMaxVec * 8) { set_error("cf_swiglu_quantize_rowwise_e4m3: at most %d columns", kRT * kMaxVec * 8); return CF_ERR_LIMIT; }
    const int vec = aligned16(d_gate) && aligned16(d_up) && (ld_in % 8 == 0) &&
                    ((reinterpret_cast<uintptr_t>(d_out) & 7) == 0) && (ld_out % 8 == 0);
    if (vec && cols % 8 == 0) {
        CF_TRY_RET(launch_rowwise_fast_nv<true>(static_cast<const uint16_t*>(d_gate), static_cast<const uint16_t*>(d_up), ld_in,
                                                static_cast<uint8_t*>(d_out), ld_out, d_row_scale, d_row_descale, rows, cols,
                                                as_stream(stream)));
        CF_LAUNCH_CHECK("swiglu_quantize_rowwise_e4m3");
        return CF_OK;
    }
    if (((reinterpret_cast<uintptr_t>(d_gate) ^ reinterpret_cast<uintptr_t>(d_up)) & 15) == 0) {
        // gate and up rows share their alignment: head / vectors / tail per row
        CF_TRY_RET(launch_rowwise_ragged_nv<true>(static_cast<const uint16_t*>(d_gate), static_cast<const uint16_t*>(d_up), ld_in,
                                                  static_cast<uint8_t*>(d_out), ld_out, d_row_scale, d_row_descale, rows, cols,
                                                  as_stream(stream)));
        CF_LAUNCH_CHECK("swiglu_quantize_rowwise_e4m3");
        return CF_OK;
    }
    k_rowwise<true><<<rows, kRT, 0, as_stream(stream)>>>(static_cast<const uint16_t*>(d_gate), static_cast<const uint16_t*>(d_up),
                                                         ld_in, static_cast<uint8_t*>(d_out), ld_out, d_row_scale,
                                                         d_row_descale, cols, vec);
    CF_LAUNCH_CHECK("swiglu_quantize_rowwise_e4m3");
    return CF_OK;
}

int cf_fp8_quantize_rowwise_given_amax_e4m3(const void* d_x, int ld_x, void* d_out, int ld_out, const float* d_row_amax,
                                            float* d_row_scale, float* d_row_descale, int rows, int cols, void* stream) {
    CF_REQUIRE(rows >= 0 && cols >= 0 && ld_x >= cols && ld_out >= cols, "cf_fp8_quantize_rowwise_given_amax_e4m3: bad shape");
    if (rows == 0 || cols == 0) return CF_OK;
    CF_REQUIRE(d_x && d_out && d_row_amax && d_row_descale, "cf_fp8_quantize_rowwise_given_amax_e4m3: null pointer");
    const int vec = aligned16(d_x) && aligned16(d_out) && (ld_x % 8 == 0) && (ld_out % 16 == 0) && (cols % 16 == 0);
    const size_t items = static_cast<size_t>(rows) * (vec ? cols / 16 : cols);
    size_t blocks = (items + kRT - 1) / kRT;
    const size_t cap = static_cast<size_t>(sm_count()) * 8;
    if (blocks < 1) blocks = 1;
    if (blocks > cap) blocks = cap;
    k_rowwise_given_amax<<<static_cast<unsigned>(blocks), kRT, 0, as_stream(stream)>>>(
        static_cast<const uint16_t*>(d_x), ld_x, static_cast<uint8_t*>(d_out), ld_out, d_row_amax, d_row_scale, d_row_descale,
        rows, cols, vec);
    CF_LAUNCH_CHECK("quantize_rowwise_given_amax_e4m3");
    return CF_OK;
}

int cf_f32_to_bf16_and_zero(float* d_acc, void* d_out, size_t n, void* stream) {
    if (n == 0) return CF_OK;
    CF_REQUIRE(d_acc && d_out, "cf_f32_to_bf16_and_zero: null pointer");
    const int vec = aligned16(d_acc) && aligned16(d_out);
    size_t blocks = (n / 8 + kRT * 2 - 1) / (kRT * 2);
    const size_t cap = static_cast<size_t>(sm_count()) * 8;
    if (blocks < 1) blocks = 1;
    if (blocks > cap) blocks = cap;
    k_finish_f32<<<static_cast<unsigned>(blocks), kRT, 0, as_stream(stream)>>>(d_acc, static_cast<uint16_t*>(d_out), n, vec);
    CF_LAUNCH_CHECK("f32_to_bf16_and_zero");
    return CF_OK;
}

int cf_swiglu_quantize_e4m3_record(const void* d_gate, const void* d_up, int ld_in, void* d_out, int ld_out,
                                   const float* d_scale, float* d_amax, int rows, int cols, void* stream) {
    CF_REQUIRE(rows >= 0 && cols >= 0 && ld_in >= cols && ld_out >= cols, "cf_swiglu_quantize_e4m3_record: bad shape");
    CF_REQUIRE(d_scale && d_amax, "cf_swiglu_quantize_e4m3_record: null scalar pointer");
    if (rows == 0 || cols == 0) return CF_OK;
    CF_REQUIRE(d_gate && d_up && d_out, "cf_swiglu_quantize_e4m3_record: null pointer");
    return swiglu_record_launch(d_gate, d_up, ld_in, d_out, ld_out, d_scale, d_amax, rows, cols, RingTail(), as_stream(stream));
}

}  // extern "C"
