// CPU oracle for the FP8 quantize-and-GEMM path. TEST INFRASTRUCTURE ONLY.
//
// This file restates, on the host, the arithmetic of the reference's FP8
// path so that the CUDA kernels of this library can be checked against it.
// It is never linked into the shipped library and no product code path may
// call it: only the test-suite, the smoke check and the benchmark's
// `cpu_baseline` / `--impl reference` legs load it.
//
// Every function cites the reference file:line whose arithmetic it follows.
// Parity pinning: the E4M3 encoder is checked against the reference's own
// header (include/ida_native/fp8_e4m3.hpp, compiled into oracle/_ref) on all
// 65,536 bf16 inputs and on the known-answer codes of tests/fp8_e4m3_probe.cu;
// routing and expert-bank mixing are checked against the golden vectors of
// tests/fixtures/moe_router_parity. The FP8 GEMM itself runs inside cuBLASLt
// in the reference (src/trainer.cu:4516-4533) and the reference holds no
// test vector for it: GEMM parity is "unpinned" and rests on this fp32
// restatement plus a cross-check against cuBLASLt on the GPU box.
//
// Build: make -C oracle   (g++ -O3 -march=native -shared -fPIC)

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

inline float bits_to_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }
inline uint32_t f32_to_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }

// bf16 <-> fp32, matching __bfloat162float / __float2bfloat16 (RN-even,
// NaN -> canonical 0x7fff).
inline float bf16_to_f32(uint16_t h) { return bits_to_f32(static_cast<uint32_t>(h) << 16); }
inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f32_to_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fffu;
    const uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return static_cast<uint16_t>(u >> 16);
}

// Generic "float -> small float" encoder, RN-even, saturate-to-finite.
// EXP_BITS/MAN_BITS/BIAS describe the target; max_code is the largest finite
// code (sign stripped). This follows the documented behaviour of
// cvt.rn.satfinite.{e4m3x2,e5m2x2}.f32, which is what __nv_fp8_e4m3(float) /
// __nv_fp8_e5m2(float) execute in kernels/fp8.cu:49,59,78,97: overflow and
// +-Inf clamp to +-max, any NaN becomes 0x7f.
template <int MAN_BITS, int BIAS, uint8_t MAX_CODE>
inline uint8_t encode_small(float x) {
    const uint32_t u = f32_to_bits(x);
    const uint8_t sign = static_cast<uint8_t>((u >> 24) & 0x80u);
    const uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return 0x7fu;                 // NaN (sign dropped)
    if (a == 0x7f800000u) return sign | MAX_CODE;      // Inf saturates
    if (a == 0) return sign;
    const int e = static_cast<int>(a >> 23) - 127;     // unbiased (denormal floats: -127)
    const int min_normal_e = 1 - BIAS;
    if (e < min_normal_e) {
        // subnormal target: units of 2^(min_normal_e - MAN_BITS)
        const float scaled = std::ldexp(bits_to_f32(a), -(min_normal_e - MAN_BITS));
        const int m = static_cast<int>(std::nearbyintf(scaled));   // RN-even (default mode)
        return sign | static_cast<uint8_t>(m);         // m == 2^MAN_BITS is the smallest normal
    }
    uint32_t man = a & 0x7fffffu;
    const int shift = 23 - MAN_BITS;
    uint32_t m = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    int ee = e;
    if (rem > half || (rem == half && (m & 1u))) {
        ++m;
        if (m == (1u << MAN_BITS)) { m = 0; ++ee; }
    }
    const int code = ((ee + BIAS) << MAN_BITS) | static_cast<int>(m);
    if (code > MAX_CODE) return sign | MAX_CODE;
    return sign | static_cast<uint8_t>(code);
}

inline uint8_t e4m3_sat(float x) { return encode_small<3, 7, 0x7e>(x); }
inline uint8_t e5m2_sat(float x) { return encode_small<2, 15, 0x7b>(x); }

// include/ida_native/fp8_e4m3.hpp:31-67 semantics ("pack"): identical codes
// for finite inputs; non-finite inputs become sign|0x7f with finite=false.
inline uint8_t e4m3_pack(float x, int* finite) {
    const uint32_t u = f32_to_bits(x);
    if ((u & 0x7f800000u) == 0x7f800000u) {
        *finite = 0;
        return static_cast<uint8_t>(((u >> 24) & 0x80u) | 0x7fu);
    }
    *finite = 1;
    return e4m3_sat(x);
}

// include/ida_native/fp8_e4m3.hpp:69-78.
inline float e4m3_decode(uint8_t b) {
    const float sign = (b & 0x80u) ? -1.0f : 1.0f;
    const int e = (b >> 3) & 0xf;
    const int m = b & 7;
    if (e == 0) return sign * std::ldexp(static_cast<float>(m), -9);
    if (e == 15 && m == 7) return std::nanf("");
    return sign * std::ldexp(1.0f + static_cast<float>(m) / 8.0f, e - 7);
}

// E5M2 is the top byte of an IEEE half: Inf = 0x7c, NaN = 0x7d..0x7f.
inline float e5m2_decode(uint8_t b) {
    const float sign = (b & 0x80u) ? -1.0f : 1.0f;
    const int e = (b >> 2) & 0x1f;
    const int m = b & 3;
    if (e == 0) return sign * std::ldexp(static_cast<float>(m), -16);
    if (e == 31) return m == 0 ? sign * INFINITY : std::nanf("");
    return sign * std::ldexp(1.0f + static_cast<float>(m) / 4.0f, e - 15);
}

struct DecodeTables {
    float e4m3[256];
    float e5m2[256];
    DecodeTables() {
        for (int i = 0; i < 256; ++i) {
            e4m3[i] = e4m3_decode(static_cast<uint8_t>(i));
            e5m2[i] = e5m2_decode(static_cast<uint8_t>(i));
        }
    }
};
const DecodeTables& tables() { static DecodeTables t; return t; }

// src/cpu_trainer.cpp:84-108: contiguous row ranges over hardware threads.
template <class F>
void parallel_rows(int64_t rows, int threads, F&& fn) {
    if (threads <= 0) threads = static_cast<int>(std::thread::hardware_concurrency());
    if (threads < 1) threads = 1;
    if (threads > rows) threads = static_cast<int>(rows > 0 ? rows : 1);
    if (threads == 1) { fn(static_cast<int64_t>(0), rows); return; }
    std::vector<std::thread> pool;
    const int64_t chunk = (rows + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        const int64_t lo = t * chunk, hi = std::min<int64_t>(rows, lo + chunk);
        if (lo >= hi) break;
        pool.emplace_back([=, &fn] { fn(lo, hi); });
    }
    for (auto& th : pool) th.join();
}

// kernels/fp8.cu:27 and :29 use fmaxf: a NaN operand is dropped, +Inf wins.
inline float amax_step(float local, float v) { return std::fmax(local, std::fabs(v)); }

inline float dotf(const float* a, const float* b, int64_t k) {
    // fp32 accumulate; 16 independent lanes (any summation order is within
    // the 1e-2 relative-Frobenius GEMM tolerance).
    float acc[16] = {0};
    int64_t i = 0;
    for (; i + 16 <= k; i += 16)
        for (int j = 0; j < 16; ++j) acc[j] += a[i + j] * b[i + j];
    float s = 0.f;
    for (int j = 0; j < 16; ++j) s += acc[j];
    for (; i < k; ++i) s += a[i] * b[i];
    return s;
}

inline float stable_sigmoid(float x) {   // kernels/activations.cu:11-17
    if (x >= 0.0f) return 1.0f / (1.0f + std::exp(-x));
    const float e = std::exp(x);
    return e / (1.0f + e);
}

inline float gelu_erf(float v) {         // kernels/moe.cu:513-514, :1023
    return 0.5f * v * (1.0f + std::erf(v * 0.7071067811865476f));
}

}  // namespace

extern "C" {

int orc_hw_threads() { return static_cast<int>(std::thread::hardware_concurrency()); }

// ---- scalar codecs ---------------------------------------------------------
uint8_t orc_e4m3_encode(float x) { return e4m3_sat(x); }
uint8_t orc_e5m2_encode(float x) { return e5m2_sat(x); }
uint8_t orc_e4m3_pack(float x, int* finite) { return e4m3_pack(x, finite); }
float orc_e4m3_decode(uint8_t b) { return e4m3_decode(b); }
float orc_e5m2_decode(uint8_t b) { return e5m2_decode(b); }
uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
float orc_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }

void orc_f32_to_bf16_array(const float* x, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16(x[i]);
}

// ---- kernels/fp8.cu:22-32,250-253  fp8_amax_bf16 ----------------------------
float orc_amax_bf16(const uint16_t* x, int64_t n) {
    float a = 0.0f;
    for (int64_t i = 0; i < n; ++i) a = amax_step(a, bf16_to_f32(x[i]));
    return a;
}
float orc_amax_f32(const float* x, int64_t n) {
    float a = 0.0f;
    for (int64_t i = 0; i < n; ++i) a = amax_step(a, x[i]);
    return a;
}

// ---- kernels/fp8.cu:34-40  k_scale_from_amax --------------------------------
void orc_scale_from_amax(float amax, float fp8_max, float* scale, float* descale) {
    const float a = std::fmax(amax, 1e-12f);
    *scale = fp8_max / a;
    *descale = a / fp8_max;
}

// ---- kernels/fp8.cu:42-60  k_quant_e4m3 / k_quant_e5m2 ----------------------
void orc_quantize_bf16(const uint16_t* x, uint8_t* out, float scale, int64_t n, int is_e5m2) {
    for (int64_t i = 0; i < n; ++i) {
        const float v = bf16_to_f32(x[i]) * scale;
        out[i] = is_e5m2 ? e5m2_sat(v) : e4m3_sat(v);
    }
}
// fp32-input variant used only by the 256x512x512 CPU configuration.
void orc_quantize_f32(const float* x, uint8_t* out, float scale, int64_t n, int is_e5m2) {
    for (int64_t i = 0; i < n; ++i) {
        const float v = x[i] * scale;
        out[i] = is_e5m2 ? e5m2_sat(v) : e4m3_sat(v);
    }
}

// ---- kernels/fp8.cu:67-103  k_quant_*_record --------------------------------
// amax_inout follows atomicMax on the int bits of a caller-initialised slot.
void orc_quantize_record_bf16(const uint16_t* x, uint8_t* out, float scale, float* amax_inout,
                              int64_t n, int is_e5m2) {
    float local = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        const float v = bf16_to_f32(x[i]);
        local = amax_step(local, v);
        out[i] = is_e5m2 ? e5m2_sat(v * scale) : e4m3_sat(v * scale);
    }
    int32_t cur, loc;
    std::memcpy(&cur, amax_inout, 4);
    std::memcpy(&loc, &local, 4);
    if (loc > cur) std::memcpy(amax_inout, &loc, 4);
}

// ---- kernels/fp8.cu:105-142  k_update_delayed_scale -------------------------
void orc_update_delayed_scale(float amax, float fp8_max, float* scale, float* descale,
                              float* history, int history_len, int* cursor_io, int* count_io) {
    const float a = std::fmax(amax, 1e-12f);
    int cursor = *cursor_io, count = *count_io;
    if (history_len <= 0) {
        *scale = fp8_max / a;
        *descale = a / fp8_max;
        return;
    }
    if (cursor < 0 || cursor >= history_len) cursor = 0;
    history[cursor] = a;
    cursor = (cursor + 1) % history_len;
    if (count < history_len) ++count;
    float hist_max = history[0];
    for (int i = 1; i < count; ++i) hist_max = std::fmax(hist_max, history[i]);
    hist_max = std::fmax(hist_max, 1e-12f);
    *cursor_io = cursor;
    *count_io = count;
    *scale = fp8_max / hist_max;
    *descale = hist_max / fp8_max;
}

// ---- src/trainer.cu:3789-3795  k_calib_minmax_update ------------------------
void orc_calib_minmax_update(float amax, float* cmin, float* cmax) {
    const float a = std::fmax(amax, 1e-12f);
    *cmin = std::fmin(*cmin, a);
    *cmax = std::fmax(*cmax, a);
}

// ---- kernels/fp8.cu:230-243  k_quant_transpose_e4m3: w[K,N] -> out[N,K] -----
void orc_quantize_transpose_e4m3(const uint16_t* w, uint8_t* out, float scale, int K, int N) {
    for (int64_t k = 0; k < K; ++k)
        for (int64_t c = 0; c < N; ++c)
            out[c * K + k] = e4m3_sat(bf16_to_f32(w[k * N + c]) * scale);
}

// ---- kernels/fp8.cu:151-227  k_quant_bf16_e4m3_dual -------------------------
void orc_quant_and_transpose_e4m3(const uint16_t* in, uint8_t* act8, uint8_t* snap, float scale,
                                  int K, int N) {
    for (int64_t k = 0; k < K; ++k)
        for (int64_t c = 0; c < N; ++c) {
            const uint8_t q = e4m3_sat(bf16_to_f32(in[k * N + c]) * scale);
            if (act8) act8[k * N + c] = q;
            if (snap) snap[c * K + k] = q;
        }
}

// ---- src/trainer.cu:1392-1448  transpose_u8 ---------------------------------
void orc_transpose_u8(const uint8_t* in, uint8_t* out, int rows, int cols) {
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) out[c * rows + r] = in[r * cols + c];
}

// ---- kernels/fp8.cu:342-356  k_fp8_clip_probe -------------------------------
void orc_clip_probe(float amax, float scale, float fp8_max, float* stats) {
    stats[2] += 1.0f;
    if (fp8_max > 0.0f && scale > 0.0f) {
        const float ratio = amax * scale / fp8_max;
        if (ratio > 1.0f) {
            stats[0] += 1.0f;
            if (ratio > stats[1]) stats[1] = ratio;
        }
    }
}

// ---- kernels/fp8.cu:373-387  k_fp8_elem_clip_count --------------------------
// The reference adds per-thread counts with float atomics; counts below 2^24
// are exact in any order, which is the range the tests use.
void orc_elem_clip_count(const uint16_t* x, float scale, float fp8_max, int64_t n, float* out) {
    int64_t clipped = 0;
    for (int64_t i = 0; i < n; ++i)
        if (std::fabs(bf16_to_f32(x[i])) * scale > fp8_max) ++clipped;
    out[0] += static_cast<float>(clipped);
    out[1] += static_cast<float>(n);
}

// ---- kernels/fp8.cu:422-521  raw-byte E4M3 storage path ---------------------
// Returns amax over finite inputs; *bad counts what the reference's atomics
// would leave: one per warp holding a non-finite input in the stats pass is
// launch-geometry dependent, so only (bad > 0) is comparable; the pack pass
// adds exactly one per non-finite scaled product (fp8.cu:455).
void orc_pack_raw_e4m3(const uint16_t* x, uint8_t* out, uint16_t* dequant_or_null, float* amax_out,
                       float* scale_out, float* descale_out, int* nonfinite_inputs,
                       int* nonfinite_products, int64_t n) {
    float amax = 0.0f;
    int bad_in = 0;
    for (int64_t i = 0; i < n; ++i) {
        const float v = bf16_to_f32(x[i]);
        if (!std::isfinite(v)) ++bad_in; else amax = std::fmax(amax, std::fabs(v));
    }
    float s, d;
    orc_scale_from_amax(amax, 448.0f, &s, &d);
    int bad_prod = 0;
    for (int64_t i = 0; i < n; ++i) {
        int fin;
        const uint8_t code = e4m3_pack(bf16_to_f32(x[i]) * s, &fin);
        out[i] = code;
        if (!fin) ++bad_prod;
        if (dequant_or_null) dequant_or_null[i] = f32_to_bf16(e4m3_decode(code) * d);
    }
    *amax_out = amax; *scale_out = s; *descale_out = d;
    *nonfinite_inputs = bad_in; *nonfinite_products = bad_prod;
}
void orc_unpack_raw_e4m3_bf16(const uint8_t* in, float descale, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16(e4m3_decode(in[i]) * descale);
}

void orc_decode_fp8(const uint8_t* in, float* out, int64_t n, int is_e5m2) {
    const float* t = is_e5m2 ? tables().e5m2 : tables().e4m3;
    for (int64_t i = 0; i < n; ++i) out[i] = t[in[i]];
}

// ---- src/trainer.cu:4498-4534  lt_gemm_fp8_nt -------------------------------
// C[M,N] (bf16, row stride ldc) = (a_descale*b_descale) * sum_k A8[m,k]*B8[n,k]
// A8 row-major [M,K] stride lda, E4M3 or E5M2; B8 row-major [N,K] contiguous E4M3
// (or E5M2 when b_is_e5m2, used by the TN weight-gradient form). fp32 accumulate.
// Output modes: out_kind 0 = bf16 overwrite, 1 = fp32 overwrite,
//               2 = fp32 accumulate (beta=1), 3 = bf16 accumulate (beta=1).
// Optional bias (bf16[N]): bias_mode 0 none; 1 = added in fp32 before the single
// bf16 rounding (fused epilogue); 2 = the reference order, round to bf16 then
// bf16(float(c)+float(bias)) (kernels/moe.cu:325-336 run after the GEMM).
// Optional per-row a_row_descale[M] / per-column b_col_descale[N] replace the
// per-tensor scalars (documented generalisation; no reference code).
void orc_gemm_fp8_nt(int M, int N, int K, const uint8_t* A, int64_t lda, int a_is_e5m2,
                     const float* a_descale, int a_per_row, const uint8_t* B, int b_is_e5m2,
                     const float* b_descale, int b_per_col, void* C, int64_t ldc, int out_kind,
                     const uint16_t* bias, int bias_mode, int threads) {
    const float* ta = a_is_e5m2 ? tables().e5m2 : tables().e4m3;
    const float* tb = b_is_e5m2 ? tables().e5m2 : tables().e4m3;
    std::vector<float> Bf(static_cast<size_t>(N) * K);
    for (int64_t i = 0; i < static_cast<int64_t>(N) * K; ++i) Bf[i] = tb[B[i]];
    parallel_rows(M, threads, [&](int64_t lo, int64_t hi) {
        std::vector<float> arow(K);
        for (int64_t m = lo; m < hi; ++m) {
            for (int64_t k = 0; k < K; ++k) arow[k] = ta[A[m * lda + k]];
            const float da = a_per_row ? a_descale[m] : a_descale[0];
            for (int64_t n = 0; n < N; ++n) {
                const float db = b_per_col ? b_descale[n] : b_descale[0];
                const float acc = dotf(arow.data(), Bf.data() + n * K, K);
                float v = acc * (da * db);
                if (out_kind == 0) {
                    uint16_t* c = static_cast<uint16_t*>(C) + m * ldc + n;
                    if (bias && bias_mode == 1) v += bf16_to_f32(bias[n]);
                    uint16_t r = f32_to_bf16(v);
                    if (bias && bias_mode == 2) r = f32_to_bf16(bf16_to_f32(r) + bf16_to_f32(bias[n]));
                    *c = r;
                } else if (out_kind == 1) {
                    static_cast<float*>(C)[m * ldc + n] = v;
                } else if (out_kind == 2) {
                    static_cast<float*>(C)[m * ldc + n] += v;
                } else {
                    uint16_t* c = static_cast<uint16_t*>(C) + m * ldc + n;
                    *c = f32_to_bf16(bf16_to_f32(*c) + v);
                }
            }
        }
    });
}

// ---- kernels/moe.cu:325-336  k_bias_add_strided_bf16 ------------------------
void orc_bias_add_strided_bf16(uint16_t* inout, const uint16_t* bias, int rows, int cols,
                               int row_stride, int base) {
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) {
            uint16_t* p = inout + r * row_stride + base + c;
            *p = f32_to_bf16(bf16_to_f32(*p) + bf16_to_f32(bias[c]));
        }
}

// ---- kernels/activations.cu:28-40  k_swiglu_forward -------------------------
// kernels/rmsnorm.cu:13-54,101-108 (k_rmsnorm_fwd, rmsnorm_forward): one block of T = min(H, 512) threads per row.
// Thread t sums x[h]^2 for h = t, t+T, ... in that order (the compiler contracts `ms += v * v` into a fused
// multiply-add), lanes combine with an xor-butterfly (all lanes hold the same value after each step because fp32
// addition commutes), warp leaders' sums go through shared memory and a second butterfly over the warp count with
// zeros in the unused lanes. rms = sqrtf(sum / H + eps); out = bf16((x * (1/rms)) * scale). H must fill whole warps
// (H >= 512 or H % 32 == 0): the reference's full-mask shuffles are undefined otherwise.
void orc_rmsnorm_forward(const uint16_t* x, const uint16_t* scale, uint16_t* out, float* rms_or_null, int64_t rows, int H,
                         float eps) {
    const int T = H < 512 ? H : 512;
    const int warps = (T + 31) / 32;
    std::vector<float> part(static_cast<size_t>(warps) * 32);
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t* xr = x + r * H;
        std::fill(part.begin(), part.end(), 0.0f);
        for (int t = 0; t < T; ++t) {
            float ms = 0.0f;
            for (int h = t; h < H; h += T) { const float v = bf16_to_f32(xr[h]); ms = std::fmaf(v, v, ms); }
            part[t] = ms;
        }
        float wsum[32];
        for (int i = 0; i < 32; ++i) wsum[i] = 0.0f;
        for (int w = 0; w < warps; ++w) {
            float l[32];
            for (int i = 0; i < 32; ++i) l[i] = part[w * 32 + i];
            for (int off = 16; off > 0; off >>= 1) {
                float n[32];
                for (int i = 0; i < 32; ++i) n[i] = l[i] + l[i ^ off];
                std::memcpy(l, n, sizeof(l));
            }
            wsum[w] = l[0];
        }
        for (int off = 16; off > 0; off >>= 1) {
            float n[32];
            for (int i = 0; i < 32; ++i) n[i] = wsum[i] + wsum[i ^ off];
            std::memcpy(wsum, n, sizeof(wsum));
        }
        const float rms = std::sqrt(wsum[0] / static_cast<float>(H) + eps);
        if (rms_or_null) rms_or_null[r] = rms;
        const float inv = 1.0f / rms;
        for (int h = 0; h < H; ++h) out[r * H + h] = f32_to_bf16(bf16_to_f32(xr[h]) * inv * bf16_to_f32(scale[h]));
    }
}

// src/trainer.cu:3822-3845 (k_act_row_normsq), :3940-3962 (k_act_row_clip_apply_abs), :3968-3991 (act_row_clip in its
// default fixed-ceiling mode): a 256-thread block per row sums v*v for c = t, t+256, ... (fused multiply-add chain),
// xor-butterfly inside each warp, thread 0 adds the eight warp sums in order; rows whose norm sqrtf(sum) exceeds the
// ceiling are multiplied by ceiling / norm and rounded to bf16 again. ceiling <= 0 leaves the tensor alone.
void orc_act_row_clip(uint16_t* x, int64_t rows, int cols, float ceiling, float* normsq_or_null) {
    if (!(ceiling > 0.0f)) return;
    for (int64_t r = 0; r < rows; ++r) {
        uint16_t* xr = x + r * cols;
        float part[256];
        for (int t = 0; t < 256; ++t) {
            float s = 0.0f;
            for (int c = t; c < cols; c += 256) { const float v = bf16_to_f32(xr[c]); s = std::fmaf(v, v, s); }
            part[t] = s;
        }
        float total = 0.0f;
        for (int w = 0; w < 8; ++w) {
            float l[32];
            for (int i = 0; i < 32; ++i) l[i] = part[w * 32 + i];
            for (int off = 16; off > 0; off >>= 1) {
                float n[32];
                for (int i = 0; i < 32; ++i) n[i] = l[i] + l[i ^ off];
                std::memcpy(l, n, sizeof(l));
            }
            total += l[0];
        }
        if (normsq_or_null) normsq_or_null[r] = total;
        const float norm = std::sqrt(total);
        if (norm <= ceiling) continue;
        const float scalef = ceiling / norm;
        for (int c = 0; c < cols; ++c) xr[c] = f32_to_bf16(bf16_to_f32(xr[c]) * scalef);
    }
}

void orc_swiglu_forward(const uint16_t* gate, const uint16_t* up, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        const float g = bf16_to_f32(gate[i]);
        out[i] = f32_to_bf16(g * stable_sigmoid(g) * bf16_to_f32(up[i]));
    }
}

// ---- kernels/lion.cu:39-76 (fp32 state) and :78-119 (bf16 state) ------------------------------------------
// The GPU compiler may contract a*b+c into one fused multiply-add; this host restatement keeps the products and
// sums separate (volatile temporaries), so comparisons with the GPU allow the last-bit difference that makes.
static inline uint16_t lion_sr(float x, unsigned rnd) {
    uint32_t bits = f32_to_bits(x);
    if ((bits & 0x7f800000u) == 0x7f800000u) return f32_to_bf16(x);
    bits += (rnd & 0xffffu);
    return static_cast<uint16_t>(bits >> 16);
}
void orc_lion_step(uint16_t* w, void* m, int m_is_bf16, const float* grad, int64_t n, float lr, float beta1, float beta2,
                   float wd, float* amax_io, unsigned seed) {
    float amax = 0.0f;
    for (int64_t i = 0; i < n; ++i) {
        const float g = grad[i];
        const float m_prev = m_is_bf16 ? bf16_to_f32(static_cast<uint16_t*>(m)[i]) : static_cast<float*>(m)[i];
        volatile float t1 = beta1 * m_prev, t2 = (1.0f - beta1) * g;
        const float blend = t1 + t2;
        const float update = static_cast<float>((blend > 0.0f) - (blend < 0.0f));
        volatile float t3 = beta2 * m_prev, t4 = (1.0f - beta2) * g;
        const float m_new = t3 + t4;
        unsigned h = static_cast<unsigned>(i) * 2654435761u ^ seed;
        h ^= h >> 16; h *= 0x85ebca6bu; h ^= h >> 13; h *= 0xc2b2ae35u; h ^= h >> 16;
        if (m_is_bf16) static_cast<uint16_t*>(m)[i] = lion_sr(m_new, h ^ 0x9e3779b9u);
        else static_cast<float*>(m)[i] = m_new;
        const float w_f32 = bf16_to_f32(w[i]);
        volatile float t5 = wd * w_f32;
        volatile float t6 = lr * (update + t5);
        const float w_new = w_f32 - t6;
        w[i] = lion_sr(w_new, h);
        amax = std::fmax(amax, std::fabs(w_new));
    }
    if (amax_io) {
        int32_t cur, loc;
        std::memcpy(&cur, amax_io, 4);
        std::memcpy(&loc, &amax, 4);
        if (loc > cur) std::memcpy(amax_io, &loc, 4);
    }
}

// ---- row-wise (per-token) scaling: kernels/fp8.cu:34-49 applied per row (no reference code; documented
// generalisation for per-token scales). swiglu != 0 quantises bf16(silu(gate)*up) (kernels/activations.cu:28-40).
void orc_quantize_rowwise_e4m3(const uint16_t* a, const uint16_t* b_or_null, int64_t ld_in, uint8_t* out, int64_t ld_out,
                               float* row_scale, float* row_descale, int rows, int cols) {
    std::vector<float> v(cols);
    for (int64_t r = 0; r < rows; ++r) {
        float amax = 0.0f;
        for (int c = 0; c < cols; ++c) {
            float x = bf16_to_f32(a[r * ld_in + c]);
            if (b_or_null) x = bf16_to_f32(f32_to_bf16(x * stable_sigmoid(x) * bf16_to_f32(b_or_null[r * ld_in + c])));
            v[c] = x;
            amax = amax_step(amax, x);
        }
        const float am = std::fmax(amax, 1e-12f);
        const float s = 448.0f / am;
        if (row_scale) row_scale[r] = s;
        row_descale[r] = am / 448.0f;
        for (int c = 0; c < cols; ++c) out[r * ld_out + c] = e4m3_sat(v[c] * s);
    }
}

// ---- kernels/moe.cu:510-516  k_gelu_fwd -------------------------------------
void orc_gelu_forward(const uint16_t* x, uint16_t* out, int64_t n) {
    for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16(gelu_erf(bf16_to_f32(x[i])));
}

// ---- kernels/cross_entropy.cu:167-191 + kernels/moe.cu:374-422 --------------
// softmax (max-subtract, expf, multiply by 1/sum) then hard top-k by strict
// '>' scan (lowest index wins ties), zero the rest, renormalise kept to sum 1.
void orc_moe_topk_route_f32(float* scores, int rows, int E, int top_k, float* row_sum_save,
                            float* scores_save, int normalize_topk) {
    for (int64_t r = 0; r < rows; ++r) {
        float* s = scores + r * E;
        float mx = -3.402823466e+38f;
        for (int e = 0; e < E; ++e) mx = std::fmax(mx, s[e]);
        float sum = 0.0f;
        for (int e = 0; e < E; ++e) sum += std::exp(s[e] - mx);
        const float inv = 1.0f / sum;
        for (int e = 0; e < E; ++e) s[e] = std::exp(s[e] - mx) * inv;
        if (scores_save) std::memcpy(scores_save + r * E, s, sizeof(float) * E);
        bool kept[64] = {false};
        const int k = top_k < E ? top_k : E;
        for (int pick = 0; pick < k; ++pick) {
            int best = -1; float best_v = -1.0f;
            for (int e = 0; e < E; ++e)
                if (!kept[e] && s[e] > best_v) { best_v = s[e]; best = e; }
            if (best < 0) break;
            kept[best] = true;
        }
        float ks = 0.0f;
        for (int e = 0; e < E; ++e) if (kept[e]) ks += s[e];
        if (row_sum_save) row_sum_save[r] = ks;
        const float inv_k = (normalize_topk && ks > 0.0f) ? 1.0f / ks : 1.0f;
        for (int e = 0; e < E; ++e) s[e] = kept[e] ? s[e] * inv_k : 0.0f;
    }
}

// ---- kernels/moe.cu:565-580  k_moe_build_expert_row_lists -------------------
// The reference's slot order inside one expert depends on atomic timing; the
// oracle emits ascending rows, and comparisons sort each expert's list.
void orc_moe_build_expert_row_lists(const float* rw, int* counts, int* row_indices, int rows, int E) {
    for (int e = 0; e < E; ++e) counts[e] = 0;
    for (int r = 0; r < rows; ++r)
        for (int e = 0; e < E; ++e)
            if (rw[static_cast<int64_t>(r) * E + e] > 0.0f)
                row_indices[static_cast<int64_t>(e) * rows + counts[e]++] = r;
}

// ---- kernels/moe.cu:785-795  exclusive prefix sum of counts -----------------
void orc_moe_expert_offsets_from_counts(const int* counts, int* offsets, int E) {
    int acc = 0;
    for (int e = 0; e < E; ++e) { offsets[e] = acc; acc += counts[e]; }
}

// ---- kernels/moe.cu:581-606  row gather -------------------------------------
void orc_moe_gather_rows(const uint8_t* src, uint8_t* dst, const int* row_indices, int n_rows,
                         int width_bytes) {
    for (int64_t i = 0; i < n_rows; ++i)
        std::memcpy(dst + i * width_bytes, src + static_cast<int64_t>(row_indices[i]) * width_bytes,
                    width_bytes);
}

// ---- kernels/moe.cu:607-622  k_moe_scatter_accumulate_rows_bf16 -------------
void orc_moe_scatter_accumulate_rows_bf16(uint16_t* mixed, const uint16_t* compact, const float* rw,
                                          const int* row_indices, int n_rows, int expert, int E, int H) {
    for (int64_t i = 0; i < n_rows; ++i) {
        const int64_t row = row_indices[i];
        const float w = rw[row * E + expert];
        for (int h = 0; h < H; ++h) {
            uint16_t* d = mixed + row * H + h;
            *d = f32_to_bf16(bf16_to_f32(*d) + w * bf16_to_f32(compact[i * H + h]));
        }
    }
}

// ---- kernels/moe.cu:529-542  k_moe_scale_accumulate -------------------------
void orc_moe_scale_accumulate_bf16(uint16_t* mixed, const uint16_t* term, const float* rw, int rows,
                                   int expert, int E, int H) {
    for (int64_t r = 0; r < rows; ++r) {
        const float w = rw[r * E + expert];
        for (int h = 0; h < H; ++h) {
            uint16_t* d = mixed + r * H + h;
            *d = f32_to_bf16(bf16_to_f32(*d) + w * bf16_to_f32(term[r * H + h]));
        }
    }
}

// ---- bf16 NT GEMM used by the expert-bank golden vector ---------------------
// tests/moe_router_parity_check.cu:47-55: C[M,N] bf16 = A[M,K] . B[N,K]^T, fp32 accumulate.
void orc_gemm_bf16_nt(int M, int N, int K, const uint16_t* A, const uint16_t* B, uint16_t* C) {
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            float acc = 0.0f;
            for (int64_t k = 0; k < K; ++k) acc += bf16_to_f32(A[m * K + k]) * bf16_to_f32(B[n * K + k]);
            C[m * N + n] = f32_to_bf16(acc);
        }
}

// ---- kernels/moe.cu:946-1060  k_moe_grouped_expert_forward_fp8_tiled --------
// For each expert e and each of its selected rows: dequantised row (code*dx)
// -> fc_in with dequantised weights (code*dwin), fp32 -> exact-erf GELU kept
// in fp32 (no re-quantisation) -> fc_out (code*dwout), fp32 -> mixed[row] +=
// rw*y through a bf16 read-modify-write (one rounding per expert added).
void orc_moe_grouped_expert_forward_fp8(const uint8_t* hidden, float dx, int x_is_e5m2, const float* rw,
                                        const int* counts, const int* row_indices, const uint8_t* w_in,
                                        float dwin, const uint8_t* w_out, float dwout, uint16_t* mixed,
                                        int rows, int H, int Ie, int E, int threads) {
    const float* tx = x_is_e5m2 ? tables().e5m2 : tables().e4m3;
    const float* tw = tables().e4m3;
    for (int e = 0; e < E; ++e) {
        const int n_active = counts[e];
        if (n_active <= 0) continue;
        std::vector<float> Win(static_cast<size_t>(Ie) * H), Wout(static_cast<size_t>(H) * Ie);
        for (int64_t i = 0; i < static_cast<int64_t>(Ie) * H; ++i) {
            Win[i] = tw[w_in[static_cast<int64_t>(e) * Ie * H + i]] * dwin;
            Wout[i] = tw[w_out[static_cast<int64_t>(e) * H * Ie + i]] * dwout;
        }
        const int* idx = row_indices + static_cast<int64_t>(e) * rows;
        // rows of one expert are distinct, so threads never share a mixed row.
        parallel_rows(n_active, threads, [&](int64_t lo, int64_t hi) {
            std::vector<float> x(H), g(Ie);
            for (int64_t i = lo; i < hi; ++i) {
                const int64_t row = idx[i];
                for (int k = 0; k < H; ++k) x[k] = tx[hidden[row * H + k]] * dx;
                for (int j = 0; j < Ie; ++j) g[j] = gelu_erf(dotf(x.data(), Win.data() + static_cast<int64_t>(j) * H, H));
                const float w = rw[row * E + e];
                for (int h = 0; h < H; ++h) {
                    const float y = dotf(g.data(), Wout.data() + static_cast<int64_t>(h) * Ie, Ie);
                    uint16_t* d = mixed + row * H + h;
                    *d = f32_to_bf16(bf16_to_f32(*d) + w * y);
                }
            }
        });
    }
}

// ---- the CPU reference case (256x512 . 512x512, per-tensor scales), end to end on the host -----------------------
// fp32 A[M,K], W[N,K], bias[N] -> per-tensor amax-scaled E4M3 quantise of both
// (scale = 448/amax), fp32-accumulate GEMM, dequant by dA*dW, + fp32 bias, fp32
// out. Returns nothing; used as correctness case and as a timed CPU sample.
void orc_linear_f32_e4m3(const float* A, const float* W, const float* bias, float* out, int M, int N,
                         int K, int threads) {
    float sa, da, sw, dw;
    orc_scale_from_amax(orc_amax_f32(A, static_cast<int64_t>(M) * K), 448.0f, &sa, &da);
    orc_scale_from_amax(orc_amax_f32(W, static_cast<int64_t>(N) * K), 448.0f, &sw, &dw);
    std::vector<uint8_t> A8(static_cast<size_t>(M) * K), W8(static_cast<size_t>(N) * K);
    orc_quantize_f32(A, A8.data(), sa, static_cast<int64_t>(M) * K, 0);
    orc_quantize_f32(W, W8.data(), sw, static_cast<int64_t>(N) * K, 0);
    orc_gemm_fp8_nt(M, N, K, A8.data(), K, 0, &da, 0, W8.data(), 0, &dw, 0, out, N, 1, nullptr, 0, threads);
    if (bias)
        for (int64_t m = 0; m < M; ++m)
            for (int n = 0; n < N; ++n) out[m * N + n] += bias[n];
}

// ---- timed CPU sample of the bf16 FP8 linear (benchmark leg) ----------------
// One pass over `m_rows` rows of X[.,K] against W[N,K]: record-quantise the
// rows with `x_scale`, GEMM against pre-quantised W8, dequant, + bf16 bias in
// the reference order, bf16 out. Threaded over rows like src/cpu_trainer.cpp.
void orc_linear_bf16_sample(const uint16_t* X, const uint8_t* W8, const uint16_t* bias, uint16_t* out,
                            int m_rows, int N, int K, float x_scale, float x_descale, float w_descale,
                            int threads) {
    std::vector<uint8_t> X8(static_cast<size_t>(m_rows) * K);
    float amax = 0.0f;
    orc_quantize_record_bf16(X, X8.data(), x_scale, &amax, static_cast<int64_t>(m_rows) * K, 0);
    orc_gemm_fp8_nt(m_rows, N, K, X8.data(), K, 0, &x_descale, 0, W8, 0, &w_descale, 0, out, N, 0, bias,
                    bias ? 2 : 0, threads);
}

}  // extern "C"
