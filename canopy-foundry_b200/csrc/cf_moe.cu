// Elementwise neighbours of the FP8 GEMMs and the MoE routing / permute / combine kernels,
// plus the tensor-core grouped expert forward that strings them together.
#include "cf_common.cuh"
#include "cf_gemm.cuh"

namespace cf {

struct Ctx;
// accessors implemented in cf_api.cu
int* ctx_status(cf_ctx* c);
void* ctx_workspace(cf_ctx* c, size_t* bytes);

namespace {

constexpr int kT = 256;

__device__ __forceinline__ uint16_t f2bf(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }

// kernels/activations.cu:11-21
__device__ __forceinline__ float stable_sigmoid(float x) {
    // Both branches of the reference (1/(1+exp(-x)) for x >= 0, exp(x)/(1+exp(x)) otherwise) share e = exp(-|x|);
    // one IEEE division with the matching numerator gives the same bits without a divergent branch.
    const float e = expf(-fabsf(x));
    return __fdiv_rn(x >= 0.0f ? 1.0f : e, 1.0f + e);
}
// kernels/moe.cu:513-514
__device__ __forceinline__ float gelu_erf(float v) { return 0.5f * v * (1.0f + erff(v * 0.7071067811865476f)); }

unsigned grid_for(size_t work_items, int per_block) {
    const size_t b = (work_items + per_block - 1) / per_block;
    const size_t cap = static_cast<size_t>(sm_count()) * 16;
    return static_cast<unsigned>(b < 1 ? 1 : (b < cap ? b : cap));
}

// ---- bias ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kT) k_bias_add(uint16_t* __restrict__ io, const uint16_t* __restrict__ bias, int rows,
                                                 int cols, long long stride, int base, int vec) {
    if (vec) {          // 8 columns (16 bytes) per thread: rows, the slice base and the bias are 16-byte aligned
        const int cpr = cols / 8;
        const long long total = static_cast<long long>(rows) * cpr;
        for (long long i = static_cast<long long>(blockIdx.x) * kT + threadIdx.x; i < total;
             i += static_cast<long long>(gridDim.x) * kT) {
            const long long r = i / cpr;
            const int c = static_cast<int>(i - r * cpr);
            uint4* p = reinterpret_cast<uint4*>(io + r * stride + base) + c;
            const uint4 v = *p, b = __ldg(reinterpret_cast<const uint4*>(bias) + c);
            const uint32_t vw[4] = {v.x, v.y, v.z, v.w}, bw[4] = {b.x, b.y, b.z, b.w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                o[j] = static_cast<uint32_t>(f2bf(__uint_as_float(vw[j] << 16) + __uint_as_float(bw[j] << 16))) |
                       (static_cast<uint32_t>(f2bf(__uint_as_float(vw[j] & 0xffff0000u) + __uint_as_float(bw[j] & 0xffff0000u))) << 16);
            *p = make_uint4(o[0], o[1], o[2], o[3]);
        }
        return;
    }
    const long long total = static_cast<long long>(rows) * cols;
    for (long long i = static_cast<long long>(blockIdx.x) * kT + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * kT) {
        const long long r = i / cols;
        const int c = static_cast<int>(i - r * cols);
        uint16_t* p = io + r * stride + base + c;
        *p = f2bf(bf16_bits_to_f32(*p) + bf16_bits_to_f32(bias[c]));
    }
}

// ---- SwiGLU / GELU: 8 elements (16 bytes) per thread where alignment allows ---------------------
template <int OP>   // 0 = swiglu(gate, up), 1 = gelu(x)
__global__ void __launch_bounds__(kT) k_act(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b,
                                            uint16_t* __restrict__ out, size_t n, int vec) {
    const size_t stride = static_cast<size_t>(gridDim.x) * kT;
    size_t i = static_cast<size_t>(blockIdx.x) * kT + threadIdx.x;
    const size_t nvec = vec ? n / 8 : 0;
    for (; i < nvec; i += stride) {
        const uint4 va = *reinterpret_cast<const uint4*>(a + i * 8);
        uint4 vb = make_uint4(0, 0, 0, 0);
        if (OP == 0) vb = *reinterpret_cast<const uint4*>(b + i * 8);
        const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
        uint32_t wo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a0 = __uint_as_float(wa[j] << 16), a1 = __uint_as_float(wa[j] & 0xffff0000u);
            float r0, r1;
            if (OP == 0) {
                const float b0 = __uint_as_float(wb[j] << 16), b1 = __uint_as_float(wb[j] & 0xffff0000u);
                r0 = a0 * stable_sigmoid(a0) * b0;
                r1 = a1 * stable_sigmoid(a1) * b1;
            } else {
                r0 = gelu_erf(a0);
                r1 = gelu_erf(a1);
            }
            wo[j] = static_cast<uint32_t>(f2bf(r0)) | (static_cast<uint32_t>(f2bf(r1)) << 16);
        }
        *reinterpret_cast<uint4*>(out + i * 8) = make_uint4(wo[0], wo[1], wo[2], wo[3]);
    }
    for (size_t e = nvec * 8 + static_cast<size_t>(blockIdx.x) * kT + threadIdx.x; e < n; e += stride) {
        const float x = bf16_bits_to_f32(a[e]);
        out[e] = f2bf(OP == 0 ? x * stable_sigmoid(x) * bf16_bits_to_f32(b[e]) : gelu_erf(x));
    }
}

// ---- routing: softmax -> hard top-k -> renormalise; one thread per row ---------------------------
// kernels/cross_entropy.cu:167-191 (max-subtract, expf, * 1/sum) then kernels/moe.cu:374-407.
// Returns the set of experts the row keeps (bit e = expert e; E <= 64). The row is worked on in a thread-private
// copy (one read and one write of global memory per element); the arithmetic and its order are those of the reference.
__device__ __forceinline__ unsigned long long route_one_row(float* __restrict__ s, float* __restrict__ row_sum_save,
                                                            float* __restrict__ scores_save, int row, int E, int top_k,
                                                            int normalize) {
    float p[64];
    float mx = -3.402823466e+38f;
    for (int e = 0; e < E; ++e) { p[e] = s[e]; mx = fmaxf(mx, p[e]); }
    float sum = 0.0f;
    for (int e = 0; e < E; ++e) sum += expf(p[e] - mx);
    const float inv = __fdiv_rn(1.0f, sum);
    for (int e = 0; e < E; ++e) {
        p[e] = expf(p[e] - mx) * inv;
        if (scores_save) scores_save[static_cast<size_t>(row) * E + e] = p[e];
    }
    unsigned long long kept = 0;       // E <= 64
    const int k = top_k < E ? top_k : E;
    for (int pick = 0; pick < k; ++pick) {
        int best = -1;
        float best_v = -1.0f;
        for (int e = 0; e < E; ++e)
            if (!((kept >> e) & 1ull) && p[e] > best_v) { best_v = p[e]; best = e; }
        if (best < 0) break;
        kept |= 1ull << best;
    }
    float ks = 0.0f;
    for (int e = 0; e < E; ++e) if ((kept >> e) & 1ull) ks += p[e];
    if (row_sum_save) row_sum_save[row] = ks;
    const float invk = (normalize && ks > 0.0f) ? __fdiv_rn(1.0f, ks) : 1.0f;
    for (int e = 0; e < E; ++e) s[e] = ((kept >> e) & 1ull) ? p[e] * invk : 0.0f;
    return kept;
}

__global__ void __launch_bounds__(128) k_topk_route(float* __restrict__ scores, float* __restrict__ row_sum_save,
                                                    float* __restrict__ scores_save, int rows, int E, int top_k,
                                                    int normalize) {
    const int row = blockIdx.x * 128 + threadIdx.x;
    if (row >= rows) return;
    route_one_row(scores + static_cast<size_t>(row) * E, row_sum_save, scores_save, row, E, top_k, normalize);
}

// ---- dispatch lists: one block per expert, ordered compaction (ascending rows) -------------------
__global__ void __launch_bounds__(1024) k_build_row_lists(const float* __restrict__ rw, int* __restrict__ counts,
                                                          int* __restrict__ row_indices, int rows, int E) {
    __shared__ int s_warp[32];
    __shared__ int s_base;
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) s_base = 0;
    __syncthreads();
    for (int r0 = 0; r0 < rows; r0 += 1024) {
        const int r = r0 + threadIdx.x;
        const bool sel = r < rows && rw[static_cast<size_t>(r) * E + e] > 0.0f;
        const unsigned m = __ballot_sync(0xffffffffu, sel);
        const int before = __popc(m & ((1u << lane) - 1u));
        if (lane == 0) s_warp[warp] = __popc(m);
        __syncthreads();
        int wbase = 0;
        for (int w = 0; w < warp; ++w) wbase += s_warp[w];
        const int base = s_base;
        if (sel) row_indices[static_cast<size_t>(e) * rows + base + wbase + before] = r;
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = 0;
            for (int w = 0; w < 32; ++w) t += s_warp[w];
            s_base = base + t;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[e] = s_base;
}

// Interleaves gate and up weight rows in groups of 32: output row (f/32)*64 + f%32 is gate row f, +32 is up row f.
__global__ void __launch_bounds__(kT) k_interleave_gate_up(const uint8_t* __restrict__ gate, const uint8_t* __restrict__ up,
                                                           uint8_t* __restrict__ out, long long experts, int F, int K) {
    const long long chunks_per_row = K / 16;
    const long long total = experts * 2 * F * chunks_per_row;
    for (long long i = static_cast<long long>(blockIdx.x) * kT + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * kT) {
        const long long row = i / chunks_per_row, c = i - row * chunks_per_row;
        const long long e = row / (2 * F);
        const int r = static_cast<int>(row - e * 2 * F);
        const int f = (r >> 6) * 32 + (r & 31);
        const uint8_t* src = ((r & 32) ? up : gate) + (e * F + f) * static_cast<long long>(K);
        *reinterpret_cast<uint4*>(out + row * K + c * 16) = *reinterpret_cast<const uint4*>(src + c * 16);
    }
}

__global__ void k_offsets(const int* counts, int* offsets, int E) {
    int acc = 0;
    for (int e = 0; e < E; ++e) { offsets[e] = acc; acc += counts[e]; }
}

// ---- row gather (permute). blockIdx.y = expert for the all-experts form --------------------------
// Copies rows of `width_bytes`; 16-byte chunks when vec, bytes otherwise.
__global__ void __launch_bounds__(kT) k_gather_rows(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                    const int* __restrict__ row_indices, const int* __restrict__ counts,
                                                    const int* __restrict__ offsets, int n_rows_host, int rows_stride,
                                                    long long width_bytes, int vec) {
    const int e = blockIdx.y;
    const int n_rows = counts ? counts[e] : n_rows_host;
    const long long dst_row0 = offsets ? offsets[e] : 0;
    const int* idx = row_indices + static_cast<size_t>(e) * rows_stride;
    if (vec) {
        const long long cpr = width_bytes / 16;
        const long long total = static_cast<long long>(n_rows) * cpr;
        for (long long i = static_cast<long long>(blockIdx.x) * kT + threadIdx.x; i < total;
             i += static_cast<long long>(gridDim.x) * kT) {
            const long long r = i / cpr, c = i - r * cpr;
            const uint4 v = *reinterpret_cast<const uint4*>(src + static_cast<long long>(idx[r]) * width_bytes + c * 16);
            *reinterpret_cast<uint4*>(dst + (dst_row0 + r) * width_bytes + c * 16) = v;
        }
    } else {
        const long long total = static_cast<long long>(n_rows) * width_bytes;
        for (long long i = static_cast<long long>(blockIdx.x) * kT + threadIdx.x; i < total;
             i += static_cast<long long>(gridDim.x) * kT) {
            const long long r = i / width_bytes, c = i - r * width_bytes;
            dst[(dst_row0 + r) * width_bytes + c] = src[static_cast<long long>(idx[r]) * width_bytes + c];
        }
    }
}

// ---- unpermute + weighted combine for one expert: mixed[row] = bf16(mixed[row] + w * compact[i]) ----
__global__ void __launch_bounds__(kT) k_scatter_acc(uint16_t* __restrict__ mixed, const uint16_t* __restrict__ compact,
                                                    const float* __restrict__ rw, const int* __restrict__ row_indices,
                                                    const int* __restrict__ counts, const int* __restrict__ offsets,
                                                    int n_rows_host, int expert, int E, int H, int vec) {
    const int n_rows = counts ? counts[expert] : n_rows_host;
    const long long c_row0 = offsets ? offsets[expert] : 0;
    if (vec) {
        const int cpr = H / 8;
        const long long total = static_cast<long long>(n_rows) * cpr;
        for (long long i = static_cast<long long>(blockIdx.x) * kT + threadIdx.x; i < total;
             i += static_cast<long long>(gridDim.x) * kT) {
            const long long r = i / cpr;
            const int c = static_cast<int>(i - r * cpr);
            const long long row = row_indices[r];
            const float w = rw[row * E + expert];
            const uint4 t = *reinterpret_cast<const uint4*>(compact + (c_row0 + r) * H + c * 8);
            uint4* mp = reinterpret_cast<uint4*>(mixed + row * H + c * 8);
            const uint4 m = *mp;
            const uint32_t tw[4] = {t.x, t.y, t.z, t.w}, mw[4] = {m.x, m.y, m.z, m.w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float r0 = __uint_as_float(mw[j] << 16) + w * __uint_as_float(tw[j] << 16);
                const float r1 = __uint_as_float(mw[j] & 0xffff0000u) + w * __uint_as_float(tw[j] & 0xffff0000u);
                o[j] = static_cast<uint32_t>(f2bf(r0)) | (static_cast<uint32_t>(f2bf(r1)) << 16);
            }
            *mp = make_uint4(o[0], o[1], o[2], o[3]);
        }
    } else {
        const long long total = static_cast<long long>(n_rows) * H;
        for (long long i = static_cast<long long>(blockIdx.x) * kT + threadIdx.x; i < total;
             i += static_cast<long long>(gridDim.x) * kT) {
            const long long r = i / H;
            const int h = static_cast<int>(i - r * H);
            const long long row = row_indices[r];
            const float w = rw[row * E + expert];
            uint16_t* d = mixed + row * H + h;
            *d = f2bf(bf16_bits_to_f32(*d) + w * bf16_bits_to_f32(compact[(c_row0 + r) * H + h]));
        }
    }
}

// ---- single-pass combine over ascending dispatch lists ----------------------------------------------
// One warp per token row, no block-wide barrier: lane e finds the row's position in expert e's list by binary search
// (the lists of k_build_row_lists are ascending), a ballot compacts the selected experts into lanes 0..n-1 in
// ascending expert order, then the 32 lanes stream the row, adding the selected experts' rows with the rounding
// points of k_scatter_acc (one bf16 rounding per expert added). mixed is read (accumulate != 0) and written once
// instead of once per expert. Many rows are in flight per SM, which hides the latency of the searches.
constexpr int kCombineMaxE = 64;
constexpr int kCombineThreads = 64;        // small blocks: many rows in flight per SM hide the latency of the searches

__device__ __forceinline__ uint4 combine_add(uint4 m, uint4 t, float w) {
    const uint32_t tw[4] = {t.x, t.y, t.z, t.w}, mw[4] = {m.x, m.y, m.z, m.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float r0 = __uint_as_float(mw[q] << 16) + w * __uint_as_float(tw[q] << 16);
        const float r1 = __uint_as_float(mw[q] & 0xffff0000u) + w * __uint_as_float(tw[q] & 0xffff0000u);
        o[q] = static_cast<uint32_t>(f2bf(r0)) | (static_cast<uint32_t>(f2bf(r1)) << 16);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// One 64-thread block per token row at a time: thread e finds the row's position in expert e's list by binary search
// (the lists of k_build_row_lists are ascending), the first warp compacts the selected experts in ascending order, then
// the block streams the row, adding the selected experts' rows with the rounding points of k_scatter_acc (one bf16
// rounding per expert added). mixed is read (accumulate != 0) and written once instead of once per expert.
__global__ void __launch_bounds__(kCombineThreads) k_combine_rows(uint16_t* __restrict__ mixed, const uint16_t* __restrict__ compact,
                                                                  const float* __restrict__ rw, const int* __restrict__ row_indices,
                                                                  const int* __restrict__ counts, const int* __restrict__ offsets,
                                                                  int rows, int E, int H, int accumulate) {
    __shared__ long long s_pos[2][kCombineMaxE];   // selected experts only, ascending; two copies alternate between rows
    __shared__ float s_w[2][kCombineMaxE];
    __shared__ int s_n[2];
    const int cpr = H / 8;
    const int t = threadIdx.x, lane = t & 31;
    int par = 0;
    for (int row = blockIdx.x; row < rows; row += gridDim.x, par ^= 1) {
        // E <= 64: thread e searches expert e; the two warps compact their halves, the second one after the first
        const float w = t < E ? rw[static_cast<size_t>(row) * E + t] : 0.0f;
        long long pos = -1;
        if (w > 0.0f) {
            const int* list = row_indices + static_cast<size_t>(t) * rows;
            const int n = counts[t];
            int lo = 0, hi = n;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (list[mid] < row) lo = mid + 1; else hi = mid;
            }
            if (lo < n && list[lo] == row) pos = static_cast<long long>(offsets[t]) + lo;
        }
        const unsigned sel = __ballot_sync(0xffffffffu, pos >= 0);
        const int before = __popc(sel & ((1u << lane) - 1u));
        if (t < 32) {
            if (pos >= 0) { s_pos[par][before] = pos; s_w[par][before] = w; }
            if (lane == 0) s_n[par] = __popc(sel);
        }
        __syncthreads();
        if (t >= 32) {
            const int base = s_n[par];
            if (pos >= 0) { s_pos[par][base + before] = pos; s_w[par][base + before] = w; }
        }
        __syncthreads();
        if (t == 32) s_n[par] += __popc(sel);
        __syncthreads();
        const int n = s_n[par];
        uint16_t* mrow = mixed + static_cast<size_t>(row) * H;
        for (int c0 = 0; c0 < cpr; c0 += 2 * kCombineThreads) {
            // two 16-byte columns per thread and pass; the loads of up to four experts are issued before the arithmetic
            const int ca = c0 + t, cb = c0 + kCombineThreads + t;
            const bool ona = ca < cpr, onb = cb < cpr;
            uint4 ma = make_uint4(0u, 0u, 0u, 0u), mb = ma;
            if (accumulate) {
                if (ona) ma = *reinterpret_cast<const uint4*>(mrow + ca * 8);
                if (onb) mb = *reinterpret_cast<const uint4*>(mrow + cb * 8);
            }
            for (int i0 = 0; i0 < n; i0 += 4) {
                uint4 ta[4], tb[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (i0 + j < n) {
                        const uint16_t* src = compact + s_pos[par][i0 + j] * H;
                        if (ona) ta[j] = __ldcs(reinterpret_cast<const uint4*>(src + ca * 8));
                        if (onb) tb[j] = __ldcs(reinterpret_cast<const uint4*>(src + cb * 8));
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (i0 + j < n) {
                        const float wj = s_w[par][i0 + j];
                        ma = combine_add(ma, ta[j], wj);
                        mb = combine_add(mb, tb[j], wj);
                    }
                }
            }
            if (ona) *reinterpret_cast<uint4*>(mrow + ca * 8) = ma;
            if (onb) *reinterpret_cast<uint4*>(mrow + cb * 8) = mb;
        }
        // the next row writes the other copy of s_pos / s_w / s_n; the copy after that is written only behind this
        // row's barriers of the next iteration, which every thread passes after it has left the loop above
    }
}

// ---- expert replicas: spread every expert's tokens over its replicas ------------------------------
// route weights [rows, E] -> [rows, V] over "virtual experts" (expert e owns the virtual ids [vstart[e], vstart[e+1]),
// each one a replica of e's weights on some rank). A selected (row, e) goes to exactly one replica, picked by a hash of
// the global row index against the replicas' cumulative shares, so every replica receives its share of the expert's rows.
__device__ __forceinline__ float replica_u01(unsigned row, unsigned e) {
    unsigned h = (row * 0x9E3779B1u) ^ ((e + 1u) * 0x85EBCA77u);
    h ^= h >> 15; h *= 0x2C1B3C6Du; h ^= h >> 12; h *= 0x297A2D39u; h ^= h >> 15;
    return static_cast<float>(h >> 8) * (1.0f / 16777216.0f);
}
__global__ void __launch_bounds__(kT) k_expand_route(const float* __restrict__ rw, float* __restrict__ rwv, int rows, int E, int V,
                                                     const int* __restrict__ vstart, const float* __restrict__ vcum,
                                                     unsigned row0) {
    const int row = blockIdx.x * kT + threadIdx.x;
    if (row >= rows) return;
    float* out = rwv + static_cast<size_t>(row) * V;
    for (int v = 0; v < V; ++v) out[v] = 0.0f;
    for (int e = 0; e < E; ++e) {
        const float w = rw[static_cast<size_t>(row) * E + e];
        if (!(w > 0.0f)) continue;
        const float u = replica_u01(row0 + static_cast<unsigned>(row), static_cast<unsigned>(e));
        int v = vstart[e];
        const int last = vstart[e + 1] - 1;
        while (v < last && u >= vcum[v]) ++v;
        out[v] = w;
    }
}

// ---- dispatch front end in two launches -----------------------------------------------------------
// Route (kernels/moe.cu:374-407), replica choice, dispatch lists in ascending row order (the order the compaction
// kernel above gives), counts and offsets (kernels/moe.cu:565-580, 702-710, 785-795) for every row in parallel:
// launch 1 routes one row per thread and leaves how many rows of its 256-row chunk go to every list in
// chunk_counts[chunk][list]; launch 2 sums the chunks in front of its own, ranks its rows inside the chunk with warp
// ballots and writes the lists; the block of the last chunk also writes counts and offsets. No block waits for another.
constexpr int kFrontT = 256;

template <bool REPLICAS>
__global__ void __launch_bounds__(kFrontT) k_front_route(float* __restrict__ scores, float* __restrict__ rwv,
                                                         float* __restrict__ row_sum_save, float* __restrict__ scores_save,
                                                         int rows, int E, int V, int top_k, int normalize,
                                                         const int* __restrict__ vstart, const float* __restrict__ vcum,
                                                         unsigned row0, int* __restrict__ chunk_counts) {
    __shared__ int s_cnt[kFrontT / 32][64];
    const int row = blockIdx.x * kFrontT + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int L = REPLICAS ? V : E;
    unsigned long long sel = 0;            // lists this row is on
    if (row < rows) {
        float* sr = scores + static_cast<size_t>(row) * E;
        route_one_row(sr, row_sum_save, scores_save, row, E, top_k, normalize);
        if (REPLICAS) {
            float* out = rwv + static_cast<size_t>(row) * V;
            for (int v = 0; v < V; ++v) out[v] = 0.0f;
            for (int e = 0; e < E; ++e) {
                const float w = sr[e];
                if (!(w > 0.0f)) continue;
                const float u = replica_u01(row0 + static_cast<unsigned>(row), static_cast<unsigned>(e));
                int v = vstart[e];
                const int last = vstart[e + 1] - 1;
                while (v < last && u >= vcum[v]) ++v;
                out[v] = w;
                sel |= 1ull << v;
            }
        } else {
            for (int e = 0; e < E; ++e)
                if (sr[e] > 0.0f) sel |= 1ull << e;
        }
    }
    for (int v = 0; v < L; ++v) {
        const unsigned m = __ballot_sync(0xffffffffu, (sel >> v) & 1ull);
        if (lane == 0) s_cnt[warp][v] = __popc(m);
    }
    __syncthreads();
    if (threadIdx.x < L) {
        int t = 0;
#pragma unroll
        for (int w = 0; w < kFrontT / 32; ++w) t += s_cnt[w][threadIdx.x];
        chunk_counts[static_cast<size_t>(blockIdx.x) * L + threadIdx.x] = t;
    }
}

__global__ void __launch_bounds__(kFrontT) k_front_lists(const float* __restrict__ w, int rows, int L,
                                                         const int* __restrict__ chunk_counts, int* __restrict__ counts,
                                                         int* __restrict__ offsets, int* __restrict__ row_indices) {
    __shared__ int s_base[64];
    __shared__ int s_cnt[kFrontT / 32][64];
    const int row = blockIdx.x * kFrontT + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x < 64) s_base[threadIdx.x] = 0;
    __syncthreads();
    pdl_wait();
    // rows in front of this chunk, per list
    const int before_items = blockIdx.x * L;
    for (int i = threadIdx.x; i < before_items; i += kFrontT) {
        const int c = chunk_counts[i];
        if (c) atomicAdd(&s_base[i % L], c);
    }
    unsigned long long sel = 0;
    if (row < rows) {
        const float* wr = w + static_cast<size_t>(row) * L;
        for (int v = 0; v < L; ++v)
            if (wr[v] > 0.0f) sel |= 1ull << v;
    }
    for (int v = 0; v < L; ++v) {
        const unsigned m = __ballot_sync(0xffffffffu, (sel >> v) & 1ull);
        if (lane == 0) s_cnt[warp][v] = __popc(m);
    }
    __syncthreads();
    for (int v = 0; v < L; ++v) {
        const unsigned m = __ballot_sync(0xffffffffu, (sel >> v) & 1ull);
        if ((sel >> v) & 1ull) {
            int pos = s_base[v] + __popc(m & ((1u << lane) - 1u));
            for (int ww = 0; ww < warp; ++ww) pos += s_cnt[ww][v];
            row_indices[static_cast<size_t>(v) * rows + pos] = row;
        }
    }
    if (blockIdx.x == gridDim.x - 1) {
        __syncthreads();
        if (threadIdx.x < L) {
            int t = s_base[threadIdx.x];
#pragma unroll
            for (int ww = 0; ww < kFrontT / 32; ++ww) t += s_cnt[ww][threadIdx.x];
            counts[threadIdx.x] = t;
            s_base[threadIdx.x] = t;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int acc = 0;
            for (int v = 0; v < L; ++v) { offsets[v] = acc; acc += s_base[v]; }
        }
    }
}

// ---- expert parallelism without a host round trip ---------------------------------------------------
// All ranks hold the same table counts_all[world, V] (rows every source routes to every replica). Replica v lives on the
// rank whose range [lo, hi) contains it; in that rank's receive buffer the replicas follow each other in id order and,
// inside a replica, the sources in rank order ("expert-major"), so each replica is ONE ragged GEMM group whatever the
// number of sources. One thread per replica derives where this rank's rows go, what this rank serves, and where the
// results return to (the source's compact order: replica after replica).
__global__ void k_ep_plan(const int* __restrict__ counts_all, int world, int me, int V, const int* __restrict__ lo,
                          const int* __restrict__ hi, cf_row_run* __restrict__ send_runs, int* __restrict__ grp_counts,
                          int* __restrict__ grp_offsets, cf_row_run* __restrict__ ret_runs, long long capacity,
                          int* __restrict__ status) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= V) return;
    int owner = 0;
    for (int g = 0; g < world; ++g) if (lo[g] <= v && v < hi[g]) owner = g;
    long long base = 0;
    for (int u = lo[owner]; u < v; ++u)
        for (int s = 0; s < world; ++s) base += max(counts_all[s * V + u], 0);
    long long pre_me = 0;
    for (int s = 0; s < me; ++s) pre_me += max(counts_all[s * V + v], 0);
    cf_row_run r;
    r.src_row = 0; r.dst_row = base + pre_me; r.rows = max(counts_all[me * V + v], 0); r.dst = owner;
    send_runs[v] = r;
    if (owner != me) return;
    const int vl = v - lo[me];
    long long pre = 0;
    for (int s = 0; s < world; ++s) {
        const int c = max(counts_all[s * V + v], 0);
        long long off_s = 0;
        for (int u = 0; u < v; ++u) off_s += max(counts_all[s * V + u], 0);
        cf_row_run q;
        q.src_row = base + pre; q.dst_row = off_s; q.rows = c; q.dst = s;
        ret_runs[vl * world + s] = q;
        pre += c;
    }
    // A group that would run past the receive buffer (a count table no sender could have produced honestly) is cut
    // to what fits and reported; the senders skip the same rows (k_send_rows checks every run against the capacity).
    if (capacity > 0 && base + pre > capacity) {
        pre = base < capacity ? capacity - base : 0;
        if (status) atomicExch(status, 0x500 | 2);
    }
    grp_counts[vl] = static_cast<int>(pre);
    grp_offsets[vl] = static_cast<int>(base < capacity || capacity <= 0 ? base : 0);
}

// Copies runs of rows to per-run destinations that may live on peer GPUs (plain 16-byte stores, whole rows contiguous).
// blockIdx.y = run. Source rows: row_indices[run * idx_stride + i] when an index table is given, else src_row + i.
// With a tag, the first thread of every row also stores *tag_value at tag_bases[dst][dst_row + i] (the row's descale).
__global__ void __launch_bounds__(kT) k_send_rows(const uint8_t* __restrict__ src, const int* __restrict__ row_indices,
                                                  long long idx_stride, const cf_row_run* __restrict__ runs,
                                                  void* const* __restrict__ dst_bases, long long width_bytes,
                                                  const float* __restrict__ tag_value, float* const* __restrict__ tag_bases,
                                                  int num_dst, long long dst_rows, int* __restrict__ status) {
    const cf_row_run run = runs[blockIdx.y];
    if (run.rows <= 0) return;
    // The destinations may be other GPUs' memory: a run that names no destination or leaves the destination's rows is
    // not stored at all (nothing faults) and leaves a code in the status word.
    if (run.dst < 0 || run.dst >= num_dst || run.dst_row < 0 || run.dst_row + run.rows > dst_rows) {
        if (status && blockIdx.x == 0 && threadIdx.x == 0) atomicExch(status, 0x500 | 1);
        return;
    }
    uint8_t* dst = static_cast<uint8_t*>(dst_bases[run.dst]) + run.dst_row * width_bytes;
    const int* idx = row_indices ? row_indices + blockIdx.y * idx_stride : nullptr;
    const long long cpr = width_bytes / 16;
    const long long total = static_cast<long long>(run.rows) * cpr;
    const float tag = tag_value ? *tag_value : 0.0f;
    float* tdst = tag_value ? tag_bases[run.dst] + run.dst_row : nullptr;
    for (long long i = static_cast<long long>(blockIdx.x) * kT + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * kT) {
        const long long r = i / cpr, c = i - r * cpr;
        const long long srow = idx ? idx[r] : run.src_row + r;
        *reinterpret_cast<uint4*>(dst + r * width_bytes + c * 16) = *reinterpret_cast<const uint4*>(src + srow * width_bytes + c * 16);
        if (tdst && c == 0) tdst[r] = tag;
    }
}

// ---- dense combine: mixed[row,:] += rw[row,e] * term[row,:] -----------------------------------------
__global__ void __launch_bounds__(kT) k_scale_acc(uint16_t* __restrict__ mixed, const uint16_t* __restrict__ term,
                                                  const float* __restrict__ rw, long long rows, int expert, int E, int H) {
    const long long total = rows * H;
    for (long long i = static_cast<long long>(blockIdx.x) * kT + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * kT) {
        const long long r = i / H;
        const float w = rw[r * E + expert];
        mixed[i] = f2bf(bf16_bits_to_f32(mixed[i]) + w * bf16_bits_to_f32(term[i]));
    }
}

// ---- GELU of the fc_in output over the valid compact rows: amax pass and two-term E4M3 split --------
// g = gelu(h) is represented as hi + lo with hi = e4m3(g*s), lo = e4m3((g*s - dec(hi))): both terms use
// the same scale, so one accumulating GEMM over [hi | lo] reproduces g to ~2^-8 relative.
__device__ __forceinline__ long long valid_elems(const int* counts, int E, int width) {
    long long t = 0;
    for (int e = 0; e < E; ++e) t += max(counts[e], 0);
    return t * width;
}
__global__ void __launch_bounds__(kT) k_gelu_amax(const uint16_t* __restrict__ h, const int* __restrict__ counts, int E,
                                                  int width, float* __restrict__ amax) {
    const long long n = valid_elems(counts, E, width);
    float local = 0.0f;
    for (long long i = static_cast<long long>(blockIdx.x) * kT + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * kT)
        local = fmaxf(local, fabsf(gelu_erf(bf16_bits_to_f32(h[i]))));
    block_amax_commit(local, amax);
}
__global__ void __launch_bounds__(kT) k_gelu_split(const uint16_t* __restrict__ h, const int* __restrict__ counts, int E,
                                                   int width, const float* __restrict__ scale, uint8_t* __restrict__ hi,
                                                   uint8_t* __restrict__ lo) {
    const long long n = valid_elems(counts, E, width);
    const float s = *scale;
    for (long long i = static_cast<long long>(blockIdx.x) * kT + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * kT) {
        const float g = gelu_erf(bf16_bits_to_f32(h[i])) * s;
        const uint8_t c = cvt_fp8<false>(g);
        hi[i] = c;
        lo[i] = cvt_fp8<false>(g - fp8_to_f32<false>(c));
    }
}

}  // namespace
}  // namespace cf

using namespace cf;

#define CF_TRY(call)                    \
    do {                                \
        const int rc__ = (call);        \
        if (rc__ != CF_OK) return rc__; \
    } while (0)

extern "C" {

int cf_bias_add_strided_bf16(void* d_inout, const void* d_bias, int rows, int cols, int row_stride, int base, void* stream) {
    CF_REQUIRE(rows >= 0 && cols >= 0 && base >= 0 && row_stride >= 0, "cf_bias_add_strided_bf16: negative argument");
    if (rows == 0 || cols == 0) return CF_OK;
    CF_REQUIRE(d_inout && d_bias, "cf_bias_add_strided_bf16: null pointer");
    const int vec = cols % 8 == 0 && row_stride % 8 == 0 && base % 8 == 0 &&
                    ((reinterpret_cast<uintptr_t>(d_inout) | reinterpret_cast<uintptr_t>(d_bias)) % 16) == 0;
    k_bias_add<<<grid_for(static_cast<size_t>(rows) * cols, kT * 16), kT, 0, as_stream(stream)>>>(
        static_cast<uint16_t*>(d_inout), static_cast<const uint16_t*>(d_bias), rows, cols, row_stride, base, vec);
    CF_LAUNCH_CHECK("bias_add_strided_bf16");
    return CF_OK;
}

int cf_swiglu_forward(const void* d_gate, const void* d_up, void* d_out, int n, void* stream) {
    // kernels/activations.cu:61-72: negative count and null tensors are argument errors
    CF_REQUIRE(n >= 0, "swiglu element count must be non-negative");
    if (n == 0) return CF_OK;
    CF_REQUIRE(d_gate && d_up && d_out, "swiglu received a null tensor pointer");
    const int vec = ((reinterpret_cast<uintptr_t>(d_gate) | reinterpret_cast<uintptr_t>(d_up) |
                      reinterpret_cast<uintptr_t>(d_out)) % 16) == 0;
    k_act<0><<<grid_for(static_cast<size_t>(n), kT * 16), kT, 0, as_stream(stream)>>>(
        static_cast<const uint16_t*>(d_gate), static_cast<const uint16_t*>(d_up), static_cast<uint16_t*>(d_out),
        static_cast<size_t>(n), vec);
    CF_LAUNCH_CHECK("swiglu_forward");
    return CF_OK;
}

int cf_gelu_forward(const void* d_x, void* d_out, size_t n, void* stream) {
    if (n == 0) return CF_OK;
    CF_REQUIRE(d_x && d_out, "cf_gelu_forward: null pointer");
    const int vec = ((reinterpret_cast<uintptr_t>(d_x) | reinterpret_cast<uintptr_t>(d_out)) % 16) == 0;
    k_act<1><<<grid_for(n, kT * 16), kT, 0, as_stream(stream)>>>(static_cast<const uint16_t*>(d_x), nullptr,
                                                                 static_cast<uint16_t*>(d_out), n, vec);
    CF_LAUNCH_CHECK("gelu_forward");
    return CF_OK;
}

int cf_fp8_interleave_gate_up(const void* d_gate8, const void* d_up8, void* d_out8, int num_experts, int F, int K, void* stream) {
    CF_REQUIRE(num_experts >= 1 && F > 0 && K > 0, "cf_fp8_interleave_gate_up: bad shape");
    CF_REQUIRE(F % 32 == 0 && K % 16 == 0, "cf_fp8_interleave_gate_up: F must be a multiple of 32 and K of 16");
    CF_REQUIRE(d_gate8 && d_up8 && d_out8, "cf_fp8_interleave_gate_up: null pointer");
    CF_REQUIRE(((reinterpret_cast<uintptr_t>(d_gate8) | reinterpret_cast<uintptr_t>(d_up8) | reinterpret_cast<uintptr_t>(d_out8)) % 16) == 0,
               "cf_fp8_interleave_gate_up: pointers must be 16-byte aligned");
    const size_t items = static_cast<size_t>(num_experts) * 2 * F * (K / 16);
    k_interleave_gate_up<<<grid_for(items, kT * 4), kT, 0, as_stream(stream)>>>(
        static_cast<const uint8_t*>(d_gate8), static_cast<const uint8_t*>(d_up8), static_cast<uint8_t*>(d_out8), num_experts, F, K);
    CF_LAUNCH_CHECK("interleave_gate_up");
    return CF_OK;
}

int cf_moe_topk_route_f32(float* d_scores, int rows, int num_experts, int top_k, void* stream, float* d_row_sum_save,
                          float* d_scores_save, int normalize_topk) {
    CF_REQUIRE(rows >= 0 && num_experts >= 1 && num_experts <= 64 && top_k >= 0, "cf_moe_topk_route_f32: bad shape (1 <= experts <= 64)");
    if (rows == 0) return CF_OK;
    CF_REQUIRE(d_scores, "cf_moe_topk_route_f32: null pointer");
    k_topk_route<<<(rows + 127) / 128, 128, 0, as_stream(stream)>>>(d_scores, d_row_sum_save, d_scores_save, rows,
                                                                   num_experts, top_k, normalize_topk);
    CF_LAUNCH_CHECK("moe_topk_route_f32");
    return CF_OK;
}

int cf_moe_build_expert_row_lists(const float* d_route_weights, int* d_counts, int* d_row_indices, int rows,
                                  int num_experts, void* stream) {
    CF_REQUIRE(rows >= 0 && num_experts >= 1, "cf_moe_build_expert_row_lists: bad shape");
    CF_REQUIRE(d_counts && (rows == 0 || (d_route_weights && d_row_indices)), "cf_moe_build_expert_row_lists: null pointer");
    k_build_row_lists<<<num_experts, 1024, 0, as_stream(stream)>>>(d_route_weights, d_counts, d_row_indices, rows, num_experts);
    CF_LAUNCH_CHECK("moe_build_expert_row_lists");
    return CF_OK;
}

int cf_moe_expert_offsets_from_counts(const int* d_counts, int* d_offsets, int num_experts, void* stream) {
    CF_REQUIRE(d_counts && d_offsets && num_experts >= 1, "cf_moe_expert_offsets_from_counts: bad argument");
    k_offsets<<<1, 1, 0, as_stream(stream)>>>(d_counts, d_offsets, num_experts);
    CF_LAUNCH_CHECK("moe_expert_offsets_from_counts");
    return CF_OK;
}

static int gather_rows(const void* src, void* dst, const int* idx, const int* counts, const int* offsets, int n_rows,
                       int rows_stride, int experts, long long width_bytes, cudaStream_t st) {
    if (n_rows == 0 || width_bytes == 0) return CF_OK;
    const int vec = (width_bytes % 16 == 0) && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) % 16 == 0);
    const size_t items = static_cast<size_t>(n_rows) * (vec ? width_bytes / 16 : width_bytes);
    dim3 grid(grid_for(items, kT * 4), experts);
    k_gather_rows<<<grid, kT, 0, st>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), idx, counts, offsets,
                                      n_rows, rows_stride, width_bytes, vec);
    CF_LAUNCH_CHECK("moe_gather_rows");
    return CF_OK;
}

int cf_moe_gather_rows_u8(const uint8_t* d_src, uint8_t* d_dst, const int* d_row_indices, int n_rows, int width, void* stream) {
    CF_REQUIRE(n_rows >= 0 && width >= 0, "cf_moe_gather_rows_u8: negative shape");
    CF_REQUIRE(n_rows == 0 || width == 0 || (d_src && d_dst && d_row_indices), "cf_moe_gather_rows_u8: null pointer");
    return gather_rows(d_src, d_dst, d_row_indices, nullptr, nullptr, n_rows, 0, 1, width, as_stream(stream));
}
int cf_moe_gather_rows_bf16(const void* d_src, void* d_dst, const int* d_row_indices, int n_rows, int width, void* stream) {
    CF_REQUIRE(n_rows >= 0 && width >= 0, "cf_moe_gather_rows_bf16: negative shape");
    CF_REQUIRE(n_rows == 0 || width == 0 || (d_src && d_dst && d_row_indices), "cf_moe_gather_rows_bf16: null pointer");
    return gather_rows(d_src, d_dst, d_row_indices, nullptr, nullptr, n_rows, 0, 1, 2ll * width, as_stream(stream));
}
int cf_moe_gather_all_u8(const uint8_t* d_src, uint8_t* d_dst, const int* d_row_indices, const int* d_counts,
                         const int* d_offsets, int rows, int num_experts, int width, void* stream) {
    CF_REQUIRE(rows >= 0 && width >= 0 && num_experts >= 1, "cf_moe_gather_all_u8: bad shape");
    if (rows == 0 || width == 0) return CF_OK;
    CF_REQUIRE(d_src && d_dst && d_row_indices && d_counts && d_offsets, "cf_moe_gather_all_u8: null pointer");
    return gather_rows(d_src, d_dst, d_row_indices, d_counts, d_offsets, rows, rows, num_experts, width, as_stream(stream));
}

static int scatter_acc(void* mixed, const void* compact, const float* rw, const int* idx, const int* counts,
                       const int* offsets, int n_rows, int expert, int E, int H, cudaStream_t st) {
    if (n_rows == 0 || H == 0) return CF_OK;
    const int vec = (H % 8 == 0) && ((reinterpret_cast<uintptr_t>(mixed) | reinterpret_cast<uintptr_t>(compact)) % 16 == 0);
    const size_t items = static_cast<size_t>(n_rows) * (vec ? H / 8 : H);
    k_scatter_acc<<<grid_for(items, kT * 2), kT, 0, st>>>(static_cast<uint16_t*>(mixed), static_cast<const uint16_t*>(compact),
                                                         rw, idx, counts, offsets, n_rows, expert, E, H, vec);
    CF_LAUNCH_CHECK("moe_scatter_accumulate_rows_bf16");
    return CF_OK;
}

int cf_moe_scatter_accumulate_rows_bf16(void* d_mixed, const void* d_compact, const float* d_route_weights,
                                        const int* d_row_indices, int n_rows, int expert_idx, int num_experts, int H,
                                        void* stream) {
    CF_REQUIRE(n_rows >= 0 && H >= 0 && expert_idx >= 0 && expert_idx < num_experts, "cf_moe_scatter_accumulate_rows_bf16: bad argument");
    CF_REQUIRE(n_rows == 0 || H == 0 || (d_mixed && d_compact && d_route_weights && d_row_indices), "cf_moe_scatter_accumulate_rows_bf16: null pointer");
    return scatter_acc(d_mixed, d_compact, d_route_weights, d_row_indices, nullptr, nullptr, n_rows, expert_idx, num_experts, H, as_stream(stream));
}

int cf_moe_combine_all_bf16(void* d_mixed, const void* d_compact, const float* d_route_weights, const int* d_row_indices,
                            const int* d_counts, const int* d_offsets, int rows, int num_experts, int H, void* stream) {
    CF_REQUIRE(rows >= 0 && H >= 0 && num_experts >= 1, "cf_moe_combine_all_bf16: bad shape");
    if (rows == 0 || H == 0) return CF_OK;
    CF_REQUIRE(d_mixed && d_compact && d_route_weights && d_row_indices && d_counts && d_offsets, "cf_moe_combine_all_bf16: null pointer");
    for (int e = 0; e < num_experts; ++e)
        CF_TRY(scatter_acc(d_mixed, d_compact, d_route_weights, d_row_indices + static_cast<size_t>(e) * rows, d_counts,
                           d_offsets, rows, e, num_experts, H, as_stream(stream)));
    return CF_OK;
}

int cf_moe_combine_sorted_bf16(void* d_mixed, const void* d_compact, const float* d_route_weights, const int* d_row_indices,
                               const int* d_counts, const int* d_offsets, int rows, int num_experts, int H, int accumulate,
                               void* stream) {
    CF_REQUIRE(rows >= 0 && H >= 0 && num_experts >= 1, "cf_moe_combine_sorted_bf16: bad shape");
    if (rows == 0 || H == 0) return CF_OK;
    CF_REQUIRE(d_mixed && d_compact && d_route_weights && d_row_indices && d_counts && d_offsets, "cf_moe_combine_sorted_bf16: null pointer");
    const bool vec = (H % 8 == 0) && ((reinterpret_cast<uintptr_t>(d_mixed) | reinterpret_cast<uintptr_t>(d_compact)) % 16 == 0);
    if (!vec || num_experts > kCombineMaxE) {
        // odd widths: zero fill (when not accumulating) and the per-expert passes
        if (!accumulate) CF_CUDA(cudaMemsetAsync(d_mixed, 0, static_cast<size_t>(rows) * H * 2, as_stream(stream)));
        return cf_moe_combine_all_bf16(d_mixed, d_compact, d_route_weights, d_row_indices, d_counts, d_offsets, rows,
                                       num_experts, H, stream);
    }
    int per_sm = 0;
    CF_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_combine_rows, kCombineThreads, 0));
    if (per_sm < 1) per_sm = 1;
    const long long cap = static_cast<long long>(sm_count()) * per_sm;
    k_combine_rows<<<static_cast<unsigned>(rows < cap ? rows : cap), kCombineThreads, 0, as_stream(stream)>>>(
        static_cast<uint16_t*>(d_mixed), static_cast<const uint16_t*>(d_compact), d_route_weights, d_row_indices, d_counts,
        d_offsets, rows, num_experts, H, accumulate);
    CF_LAUNCH_CHECK("moe_combine_sorted_bf16");
    return CF_OK;
}

int cf_moe_expand_route_replicas(const float* d_route_weights, float* d_replica_weights, int rows, int num_experts,
                                 int num_replicas, const int* d_replica_start, const float* d_replica_cum_share,
                                 unsigned first_row, void* stream) {
    CF_REQUIRE(rows >= 0 && num_experts >= 1 && num_replicas >= num_experts, "cf_moe_expand_route_replicas: bad shape");
    if (rows == 0) return CF_OK;
    CF_REQUIRE(d_route_weights && d_replica_weights && d_replica_start && d_replica_cum_share, "cf_moe_expand_route_replicas: null pointer");
    k_expand_route<<<(rows + kT - 1) / kT, kT, 0, as_stream(stream)>>>(d_route_weights, d_replica_weights, rows, num_experts,
                                                                       num_replicas, d_replica_start, d_replica_cum_share, first_row);
    CF_LAUNCH_CHECK("moe_expand_route_replicas");
    return CF_OK;
}

size_t cf_moe_route_dispatch_scratch_ints(int rows, int num_lists) {
    if (rows <= 0 || num_lists <= 0) return 0;
    return static_cast<size_t>((rows + kFrontT - 1) / kFrontT) * static_cast<size_t>(num_lists);
}

int cf_moe_route_dispatch_lists(float* d_scores, int rows, int num_experts, int top_k, int normalize_topk,
                                float* d_row_sum_save_or_null, float* d_scores_save_or_null, float* d_replica_weights_or_null,
                                int num_replicas, const int* d_replica_start, const float* d_replica_cum_share,
                                unsigned first_row, int* d_counts, int* d_offsets, int* d_row_indices, int* d_scratch,
                                size_t scratch_ints, void* stream) {
    const bool rep = d_replica_weights_or_null != nullptr;
    CF_REQUIRE(rows >= 0 && num_experts >= 1 && num_experts <= 64 && top_k >= 0,
               "cf_moe_route_dispatch_lists: bad shape (1 <= experts <= 64)");
    CF_REQUIRE(!rep || (num_replicas >= num_experts && d_replica_start && d_replica_cum_share),
               "cf_moe_route_dispatch_lists: replica tables missing");
    const int L = rep ? num_replicas : num_experts;
    CF_REQUIRE(d_counts && d_offsets, "cf_moe_route_dispatch_lists: null pointer");
    cudaStream_t st = as_stream(stream);
    if (rows == 0) {
        CF_CUDA(cudaMemsetAsync(d_counts, 0, sizeof(int) * L, st));
        CF_CUDA(cudaMemsetAsync(d_offsets, 0, sizeof(int) * L, st));
        return CF_OK;
    }
    CF_REQUIRE(d_scores && d_row_indices, "cf_moe_route_dispatch_lists: null pointer");
    if (L > 64) {
        // more lists than one 64-bit set per row holds: the same result from the separate kernels
        int rc = cf_moe_topk_route_f32(d_scores, rows, num_experts, top_k, stream, d_row_sum_save_or_null, d_scores_save_or_null,
                                       normalize_topk);
        if (rc != CF_OK) return rc;
        rc = cf_moe_expand_route_replicas(d_scores, d_replica_weights_or_null, rows, num_experts, num_replicas, d_replica_start,
                                          d_replica_cum_share, first_row, stream);
        if (rc != CF_OK) return rc;
        rc = cf_moe_build_expert_row_lists(d_replica_weights_or_null, d_counts, d_row_indices, rows, num_replicas, stream);
        if (rc != CF_OK) return rc;
        return cf_moe_expert_offsets_from_counts(d_counts, d_offsets, num_replicas, stream);
    }
    const size_t need = cf_moe_route_dispatch_scratch_ints(rows, L);
    if (d_scratch == nullptr || scratch_ints < need) {
        set_error("cf_moe_route_dispatch_lists: scratch of %zu ints needed (cf_moe_route_dispatch_scratch_ints)", need);
        return CF_ERR_LIMIT;
    }
    const int chunks = (rows + kFrontT - 1) / kFrontT;
    if (rep)
        k_front_route<true><<<chunks, kFrontT, 0, st>>>(d_scores, d_replica_weights_or_null, d_row_sum_save_or_null,
                                                        d_scores_save_or_null, rows, num_experts, num_replicas, top_k,
                                                        normalize_topk, d_replica_start, d_replica_cum_share, first_row, d_scratch);
    else
        k_front_route<false><<<chunks, kFrontT, 0, st>>>(d_scores, nullptr, d_row_sum_save_or_null, d_scores_save_or_null, rows,
                                                         num_experts, num_experts, top_k, normalize_topk, nullptr, nullptr, first_row,
                                                         d_scratch);
    CF_LAUNCH_CHECK("moe_route_dispatch_lists(route)");
    CF_CUDA(launch_pdl(k_front_lists, dim3(chunks), dim3(kFrontT), 0, st,
                       static_cast<const float*>(rep ? d_replica_weights_or_null : d_scores), rows, L,
                       static_cast<const int*>(d_scratch), d_counts, d_offsets, d_row_indices));
    CF_LAUNCH_CHECK("moe_route_dispatch_lists(lists)");
    return CF_OK;
}

int cf_moe_ep_plan(const int* d_counts_all, int world, int rank, int num_replicas, const int* d_range_lo, const int* d_range_hi,
                   cf_row_run* d_send_runs, int* d_group_counts, int* d_group_offsets, cf_row_run* d_return_runs,
                   long long recv_capacity_rows, cf_ctx* ctx_or_null, void* stream) {
    CF_REQUIRE(recv_capacity_rows >= 0, "cf_moe_ep_plan: negative capacity");
    CF_REQUIRE(world >= 1 && rank >= 0 && rank < world && num_replicas >= 1, "cf_moe_ep_plan: bad shape");
    CF_REQUIRE(d_counts_all && d_range_lo && d_range_hi && d_send_runs && d_group_counts && d_group_offsets && d_return_runs,
               "cf_moe_ep_plan: null pointer");
    k_ep_plan<<<(num_replicas + 63) / 64, 64, 0, as_stream(stream)>>>(d_counts_all, world, rank, num_replicas, d_range_lo,
                                                                      d_range_hi, d_send_runs, d_group_counts, d_group_offsets,
                                                                      d_return_runs, recv_capacity_rows,
                                                                      ctx_or_null ? ctx_status(ctx_or_null) : nullptr);
    CF_LAUNCH_CHECK("moe_ep_plan");
    return CF_OK;
}

int cf_moe_send_row_runs(const void* d_src, const int* d_row_indices_or_null, long long index_stride, const cf_row_run* d_runs,
                         int num_runs, int max_rows_per_run, void* const* d_dst_bases, long long row_bytes,
                         const float* d_tag_value_or_null, float* const* d_tag_bases_or_null, int num_dst, long long dst_rows,
                         cf_ctx* ctx_or_null, void* stream) {
    CF_REQUIRE(num_dst >= 1 && dst_rows >= 0, "cf_moe_send_row_runs: needs the number of destination buffers and their row capacity");
    CF_REQUIRE(num_runs >= 0 && max_rows_per_run >= 0 && row_bytes > 0 && row_bytes % 16 == 0,
               "cf_moe_send_row_runs: rows must be whole 16-byte units");
    if (num_runs == 0 || max_rows_per_run == 0) return CF_OK;
    CF_REQUIRE(d_src && d_runs && d_dst_bases, "cf_moe_send_row_runs: null pointer");
    CF_REQUIRE((d_tag_value_or_null == nullptr) == (d_tag_bases_or_null == nullptr), "cf_moe_send_row_runs: tag value and tag bases go together");
    CF_REQUIRE(reinterpret_cast<uintptr_t>(d_src) % 16 == 0, "cf_moe_send_row_runs: source not 16-byte aligned");
    const size_t items = static_cast<size_t>(max_rows_per_run) * static_cast<size_t>(row_bytes / 16);
    unsigned gx = grid_for(items, kT * 4);
    const unsigned cap = static_cast<unsigned>(sm_count()) * 8u / static_cast<unsigned>(num_runs) + 1u;
    if (gx > cap) gx = cap;
    dim3 grid(gx, num_runs);
    k_send_rows<<<grid, kT, 0, as_stream(stream)>>>(static_cast<const uint8_t*>(d_src), d_row_indices_or_null, index_stride, d_runs,
                                                    d_dst_bases, row_bytes, d_tag_value_or_null, d_tag_bases_or_null, num_dst,
                                                    dst_rows, ctx_or_null ? ctx_status(ctx_or_null) : nullptr);
    CF_LAUNCH_CHECK("moe_send_row_runs");
    return CF_OK;
}

int cf_moe_scale_accumulate_bf16(void* d_mixed, const void* d_term, const float* d_route_weights, int rows, int expert_idx,
                                 int num_experts, int H, void* stream) {
    CF_REQUIRE(rows >= 0 && H >= 0 && expert_idx >= 0 && expert_idx < num_experts, "cf_moe_scale_accumulate_bf16: bad argument");
    if (rows == 0 || H == 0) return CF_OK;
    CF_REQUIRE(d_mixed && d_term && d_route_weights, "cf_moe_scale_accumulate_bf16: null pointer");
    k_scale_acc<<<grid_for(static_cast<size_t>(rows) * H, kT * 4), kT, 0, as_stream(stream)>>>(
        static_cast<uint16_t*>(d_mixed), static_cast<const uint16_t*>(d_term), d_route_weights, rows, expert_idx, num_experts, H);
    CF_LAUNCH_CHECK("moe_scale_accumulate_bf16");
    return CF_OK;
}

int cf_moe_grouped_expert_forward_fp8(cf_ctx* ctx, const void* d_hidden, const float* d_fcin_descale, int fcin_is_e5m2,
                                      const float* d_route_weights, const int* d_counts, const int* d_offsets,
                                      const int* d_row_indices, const void* d_fc_in_w, const float* d_fc_in_descale,
                                      const void* d_fc_out_w, const float* d_fc_out_descale, void* d_mixed, int rows,
                                      int H, int Ie, int num_experts, int total_selected_rows, void* stream) {
    CF_REQUIRE(ctx != nullptr, "cf_moe_grouped_expert_forward_fp8: null context");
    CF_REQUIRE(rows >= 0 && H > 0 && Ie > 0 && num_experts >= 1 && total_selected_rows >= 0, "cf_moe_grouped_expert_forward_fp8: bad shape");
    if (rows == 0 || total_selected_rows == 0) return CF_OK;
    CF_REQUIRE(d_hidden && d_fcin_descale && d_route_weights && d_counts && d_offsets && d_row_indices && d_fc_in_w &&
               d_fc_in_descale && d_fc_out_w && d_fc_out_descale && d_mixed, "cf_moe_grouped_expert_forward_fp8: null pointer");
    CF_REQUIRE(H % 16 == 0 && Ie % 16 == 0, "cf_moe_grouped_expert_forward_fp8: H and Ie must be multiples of 16");
    const size_t T = static_cast<size_t>(total_selected_rows);
    // workspace carve-up (256-byte aligned pieces)
    auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
    const size_t b_xc = up(T * H), b_hc = up(T * Ie * 2), b_g = up(T * Ie * 2), b_yc = up(T * H * 2), b_sc = 256;
    size_t have = 0;
    uint8_t* ws = static_cast<uint8_t*>(ctx_workspace(ctx, &have));
    if (have < b_xc + b_hc + b_g + b_yc + b_sc) {
        set_error("cf_moe_grouped_expert_forward_fp8: needs %zu bytes of context workspace, %zu reserved",
                  b_xc + b_hc + b_g + b_yc + b_sc, have);
        return CF_ERR_LIMIT;
    }
    uint8_t* xc = ws;
    uint16_t* hc = reinterpret_cast<uint16_t*>(ws + b_xc);
    uint8_t* g8 = ws + b_xc + b_hc;                 // [T, 2*Ie]: rows of hi | lo halves are stored as two planes
    uint16_t* yc = reinterpret_cast<uint16_t*>(ws + b_xc + b_hc + b_g);
    float* sc = reinterpret_cast<float*>(ws + b_xc + b_hc + b_g + b_yc);   // [0] amax [4] scale [8] descale [12] descale*wout
    cudaStream_t st = as_stream(stream);

    CF_TRY(cf_moe_gather_all_u8(static_cast<const uint8_t*>(d_hidden), xc, d_row_indices, d_counts, d_offsets, rows,
                                num_experts, H, stream));
    CF_TRY(cf_gemm_fp8_nt_grouped(ctx, num_experts, total_selected_rows, Ie, H, d_counts, d_offsets, xc, H, fcin_is_e5m2,
                                  d_fcin_descale, 0, d_fc_in_w, d_fc_in_descale, hc, Ie, stream));
    CF_CUDA(cudaMemsetAsync(sc, 0, sizeof(float), st));
    const unsigned eg = grid_for(T * Ie, kT * 8);
    k_gelu_amax<<<eg, kT, 0, st>>>(hc, d_counts, num_experts, Ie, sc);
    CF_LAUNCH_CHECK("moe_gelu_amax");
    CF_TRY(cf_fp8_scale_from_amax(sc, CF_E4M3_MAX, sc + 4, sc + 8, stream));
    uint8_t* g_hi = g8;
    uint8_t* g_lo = g8 + T * Ie;
    k_gelu_split<<<eg, kT, 0, st>>>(hc, d_counts, num_experts, Ie, sc + 4, g_hi, g_lo);
    CF_LAUNCH_CHECK("moe_gelu_split");
    // y = dG*dWout * (hi . W^T + lo . W^T): the second launch accumulates into the first one's bf16 result
    CF_TRY(cf_gemm_fp8_nt_grouped(ctx, num_experts, total_selected_rows, H, Ie, d_counts, d_offsets, g_hi, Ie, 0, sc + 8, 0,
                                  d_fc_out_w, d_fc_out_descale, yc, H, stream));
    {
        GemmParams p;
        p.groups = num_experts; p.N = H; p.K = Ie;
        p.d_counts = d_counts; p.d_offsets = d_offsets;
        p.d_a_descale = sc + 8; p.d_b_descale = d_fc_out_descale;
        p.C = yc; p.ldc = H; p.out_kind = 3;
        p.d_status = ctx_status(ctx);
        const int m_blocks = (total_selected_rows + gemm_tile_m() - 1) / gemm_tile_m() + num_experts;
        CF_TRY(launch_gemm_fp8_nt(g_lo, Ie, total_selected_rows, d_fc_out_w, static_cast<long long>(num_experts) * H, p,
                                  m_blocks * ((H + gemm_tile_n() - 1) / gemm_tile_n()), st));
    }
    return cf_moe_combine_all_bf16(d_mixed, yc, d_route_weights, d_row_indices, d_counts, d_offsets, rows, num_experts, H, stream);
}

}  // extern "C"
