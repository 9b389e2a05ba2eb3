// Test infrastructure, not part of the product: a small C++ caller that uses the drop-in the way the reference's trainer
// would. It includes the reference's own declarations (include/ida_native/kernels.hpp, fp8_e4m3.hpp) where they lie, calls
// the ida_native:: operators (defined by canopy-foundry_b200/shim/ida_native_kernels.cu over libcanopy_fp8.so) and the
// same-named trainer helpers of shim/cf_trainer_shim.hpp, and checks the results against plain host arithmetic and the
// reference header's encoder. Built by oracle/Makefile into oracle/_ref/shim_check where the reference tree is present;
// tests/test_gpu_gemm.py runs the binary on the GPU when it exists. Exit code 0 and "shim_check: PASS" on success.
#include "ida_native/fp8_e4m3.hpp"
#include "ida_native/kernels.hpp"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

#include "canopy_fp8.h"
#include "cf_trainer_shim.hpp"

namespace {

struct Fp8CtxLike {          // the two members the trainer helpers use of the reference's Fp8Ctx
    cf_ctx* cf = nullptr;
    void* act8 = nullptr;
};

int g_fail = 0;
void expect(bool ok, const char* what) {
    if (!ok) { std::fprintf(stderr, "shim_check: FAILED: %s\n", what); ++g_fail; }
}
void cu(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
template <class T>
T* dev_alloc(size_t n) {
    T* p = nullptr;
    cu(cudaMalloc(&p, n * sizeof(T) + 16), "cudaMalloc");
    return p;
}
template <class T>
void to_dev(T* d, const std::vector<T>& h) { cu(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice), "H2D"); }
template <class T>
std::vector<T> to_host(const T* d, size_t n) {
    std::vector<T> h(n);
    cu(cudaMemcpy(h.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost), "D2H");
    return h;
}
float bf(const __nv_bfloat16& v) { return __bfloat162float(v); }

void check_quantise(cudaStream_t s) {
    const size_t n = 100003;                       // odd length: vector body and scalar tail
    std::mt19937_64 rng(1);
    std::normal_distribution<float> nd(0.0f, 1.0f);
    std::vector<__nv_bfloat16> x(n);
    float amax_h = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float v = nd(rng) * (i % 997 == 0 ? 20.0f : 1.0f);
        x[i] = __float2bfloat16(v);
        amax_h = std::fmax(amax_h, std::fabs(bf(x[i])));
    }
    auto* d_x = dev_alloc<__nv_bfloat16>(n);
    auto* d_q = dev_alloc<std::uint8_t>(n);
    auto* d_sc = dev_alloc<float>(12);             // amax, scale, descale on 16-byte boundaries
    to_dev(d_x, x);
    ida_native::fp8_amax_bf16(d_x, n, d_sc, s);
    ida_native::fp8_scale_from_amax(d_sc, 448.0f, d_sc + 4, d_sc + 8, s);
    ida_native::fp8_quantize_e4m3(d_x, d_q, d_sc + 4, n, s);
    cu(cudaStreamSynchronize(s), "sync");
    const auto sc = to_host(d_sc, 12);
    const auto q = to_host(d_q, n);
    expect(sc[0] == amax_h, "fp8_amax_bf16 equals the host maximum");
    const float a = std::fmax(amax_h, 1e-12f);
    expect(sc[4] == 448.0f / a && sc[8] == a / 448.0f, "fp8_scale_from_amax: the two IEEE divisions of kernels/fp8.cu:34-40");
    size_t bad = 0;
    for (size_t i = 0; i < n; ++i)
        if (q[i] != ida_native::fp8_e4m3::pack(bf(x[i]) * sc[4]).bits) ++bad;
    expect(bad == 0, "fp8_quantize_e4m3 bytes equal the reference header's pack() on every element");
    cudaFree(d_x); cudaFree(d_q); cudaFree(d_sc);
}

void check_swiglu(cudaStream_t s) {
    const int n = 4099;
    std::mt19937_64 rng(2);
    std::normal_distribution<float> nd(0.0f, 2.0f);
    std::vector<__nv_bfloat16> g(n), u(n);
    for (int i = 0; i < n; ++i) { g[i] = __float2bfloat16(nd(rng)); u[i] = __float2bfloat16(nd(rng)); }
    auto* d_g = dev_alloc<__nv_bfloat16>(n);
    auto* d_u = dev_alloc<__nv_bfloat16>(n);
    auto* d_o = dev_alloc<__nv_bfloat16>(n);
    to_dev(d_g, g); to_dev(d_u, u);
    ida_native::swiglu_forward(d_g, d_u, d_o, n, s);
    cu(cudaStreamSynchronize(s), "sync");
    const auto o = to_host(d_o, n);
    int bad = 0;
    for (int i = 0; i < n; ++i) {
        const float xg = bf(g[i]);
        const float sig = xg >= 0.0f ? 1.0f / (1.0f + std::exp(-xg)) : std::exp(xg) / (1.0f + std::exp(xg));
        const float want = bf(__float2bfloat16(xg * sig * bf(u[i])));
        if (std::fabs(bf(o[i]) - want) > std::fabs(want) * 0.0079f + 1e-6f) ++bad;      // one bf16 step: libm vs device expf
    }
    expect(bad == 0, "swiglu_forward within one bf16 step of the host formula (kernels/activations.cu:11-40)");
    cudaFree(d_g); cudaFree(d_u); cudaFree(d_o);
}

void check_routing(cudaStream_t s) {
    const int rows = 777, E = 8, k = 2;
    std::mt19937_64 rng(3);
    std::normal_distribution<float> nd(0.0f, 1.0f);
    std::vector<float> logits(static_cast<size_t>(rows) * E);
    for (auto& v : logits) v = nd(rng);
    auto* d_s = dev_alloc<float>(logits.size());
    auto* d_counts = dev_alloc<int>(E);
    auto* d_offsets = dev_alloc<int>(E);
    auto* d_idx = dev_alloc<int>(static_cast<size_t>(E) * rows);
    to_dev(d_s, logits);
    ida_native::moe_topk_route_f32(d_s, rows, E, k, s);
    ida_native::moe_build_expert_row_lists(d_s, d_counts, d_idx, rows, E, s);
    ida_native::moe_expert_offsets_from_counts(d_counts, d_offsets, E, s);
    cu(cudaStreamSynchronize(s), "sync");
    const auto rw = to_host(d_s, logits.size());
    const auto counts = to_host(d_counts, E);
    const auto offsets = to_host(d_offsets, E);
    const auto idx = to_host(d_idx, static_cast<size_t>(E) * rows);
    int bad_rows = 0, total = 0;
    std::vector<int> want_counts(E, 0);
    for (int r = 0; r < rows; ++r) {
        int kept = 0;
        float sum = 0.0f;
        for (int e = 0; e < E; ++e) {
            const float w = rw[static_cast<size_t>(r) * E + e];
            if (w > 0.0f) { ++kept; sum += w; ++want_counts[e]; }
        }
        if (kept != k || std::fabs(sum - 1.0f) > 1e-5f) ++bad_rows;
    }
    expect(bad_rows == 0, "moe_topk_route_f32 keeps top_k experts per row with weights that sum to one");
    bool lists_ok = true;
    for (int e = 0; e < E; ++e) {
        lists_ok = lists_ok && counts[e] == want_counts[e] && offsets[e] == total;
        total += counts[e];
        for (int i = 0; i < counts[e] && lists_ok; ++i) {
            const int r = idx[static_cast<size_t>(e) * rows + i];
            lists_ok = r >= 0 && r < rows && rw[static_cast<size_t>(r) * E + e] > 0.0f &&
                       (i == 0 || idx[static_cast<size_t>(e) * rows + i - 1] < r);
        }
    }
    expect(lists_ok && total == rows * k, "dispatch lists: every selected row once, counts and offsets consistent");
    cudaFree(d_s); cudaFree(d_counts); cudaFree(d_offsets); cudaFree(d_idx);
}

void check_gemm(Fp8CtxLike& f, cudaStream_t s) {
    const int M = 384, N = 256, K = 512;
    std::mt19937_64 rng(4);
    std::vector<std::uint8_t> a(static_cast<size_t>(M) * K), b(static_cast<size_t>(N) * K);
    for (auto& v : a) v = static_cast<std::uint8_t>((rng() % 0x60) | ((rng() & 1) << 7));      // finite E4M3 codes of both signs
    for (auto& v : b) v = static_cast<std::uint8_t>((rng() % 0x60) | ((rng() & 1) << 7));
    auto* d_a = dev_alloc<std::uint8_t>(a.size());
    auto* d_b = dev_alloc<std::uint8_t>(b.size());
    auto* d_c = dev_alloc<__nv_bfloat16>(static_cast<size_t>(M) * N);
    auto* d_sc = dev_alloc<float>(8);
    to_dev(d_a, a); to_dev(d_b, b);
    to_dev(d_sc, std::vector<float>{0.5f, 0, 0, 0, 0.25f, 0, 0, 0});
    lt_gemm_fp8_nt(f, M, N, K, d_a, K, CUDA_R_8F_E4M3, d_sc, d_b, d_sc + 4, d_c, N, s);
    cu(cudaStreamSynchronize(s), "sync");
    const auto c = to_host(d_c, static_cast<size_t>(M) * N);
    double num = 0.0, den = 0.0;
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            double acc = 0.0;
            for (int kk = 0; kk < K; ++kk)
                acc += static_cast<double>(ida_native::fp8_e4m3::unpack(a[static_cast<size_t>(m) * K + kk])) *
                       static_cast<double>(ida_native::fp8_e4m3::unpack(b[static_cast<size_t>(n) * K + kk]));
            const double want = acc * 0.125;
            const double got = bf(c[static_cast<size_t>(m) * N + n]);
            num += (got - want) * (got - want);
            den += want * want;
        }
    expect(std::sqrt(num / den) < 5e-3, "lt_gemm_fp8_nt within 5e-3 (relative Frobenius) of the float64 product of the decoded codes");
    cudaFree(d_a); cudaFree(d_b); cudaFree(d_c); cudaFree(d_sc);
}

void check_errors(cudaStream_t s) {
    bool threw = false;
    try { ida_native::fp8_quantize_e4m3(nullptr, nullptr, nullptr, 16, s); } catch (const std::runtime_error&) { threw = true; }
    expect(threw, "a null operand surfaces as std::runtime_error, like IDA_CUDA_CHECK");
    threw = false;
    cf_shim::set_thread_context(nullptr);
    try {
        ida_native::moe_grouped_expert_forward_fp8(nullptr, nullptr, 0, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                                                   nullptr, nullptr, 4, 64, 64, 2, 8, s);
    } catch (const std::runtime_error&) { threw = true; }
    expect(threw, "the grouped forward refuses to run without a registered context (it never creates one)");
    expect(cudaGetLastError() == cudaSuccess, "no CUDA error is left behind by the refused calls");
}

}  // namespace

int main() {
    try {
        cudaStream_t s;
        cu(cudaStreamCreate(&s), "cudaStreamCreate");
        Fp8CtxLike f;
        cf_shim::check(cf_ctx_create(&f.cf, 0), "cf_ctx_create");
        check_quantise(s);
        check_swiglu(s);
        check_routing(s);
        check_gemm(f, s);
        check_errors(s);
        cf_shim::check(cf_ctx_poll_status(f.cf, s), "cf_ctx_poll_status");
        cf_ctx_destroy(f.cf);
        cudaStreamDestroy(s);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "shim_check: exception: %s\n", e.what());
        return 2;
    }
    if (g_fail) return 1;
    std::puts("shim_check: PASS");
    return 0;
}
