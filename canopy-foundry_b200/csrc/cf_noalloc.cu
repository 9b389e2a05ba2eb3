// FP8 linear (quantise -> GEMM -> bias) whose only scratch is a fixed array that is part of the library
// image, for callers that must not allocate device memory.
//
// Who needs this: code that runs after the host application has handed the whole device-memory budget to its
// own arena (the reference's trainer does: every buffer comes from one cudaMemPool and its operators "allocate
// nothing"), and code on latency-critical threads where cudaMalloc / cudaFree would stall the device for every
// other stream. Such callers cannot create a cf_ctx (cf_ctx_create calls cudaMalloc), so the quantised copy of
// the activation, which cf_fp8_linear_forward keeps in the context's act8 buffer, lives here in a file-scope
// __device__ array instead. The cost is that every GPU that loads the library carries these 4 MiB until the
// process exits, and that the activation is limited to that size.
#include <mutex>

#include "cf_common.cuh"
#include "cf_gemm.cuh"

namespace {

constexpr size_t kHeaderBytes = 256;                       // internal status word lives here
constexpr size_t kMaxActBytes = 4u << 20;                  // M*K <= 4 MiB (e.g. 1024 x 4096)
static __device__ __align__(256) unsigned char g_static_scratch[kHeaderBytes + kMaxActBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address: the address has
// to be asked for, once per device, with that device current.
int scratch_address(unsigned char** out) {
    static unsigned char* ptr[64];
    static std::once_flag once[64];
    static cudaError_t err[64];
    int dev = 0;
    CF_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) { cf::set_error("cf_fp8_linear_static_scratch: device index %d out of range", dev); return CF_ERR_LIMIT; }
    std::call_once(once[dev], [dev] {
        void* p = nullptr;
        err[dev] = cudaGetSymbolAddress(&p, g_static_scratch);
        ptr[dev] = static_cast<unsigned char*>(p);
    });
    if (err[dev] != cudaSuccess) return cf::cuda_fail(err[dev], "cudaGetSymbolAddress(g_static_scratch)");
    *out = ptr[dev];
    return CF_OK;
}

}  // namespace

extern "C" int cf_fp8_linear_static_scratch(const void* d_x, int M, int K, const float* d_x_scale,
                                             const float* d_x_descale, const void* d_w8, const float* d_w_descale,
                                             int N, const void* d_bias, int bias_mode, void* d_y, int ldy,
                                             int* d_status_or_null, void* stream) {
    CF_REQUIRE(M >= 0 && N >= 0 && K > 0, "cf_fp8_linear_static_scratch: bad shape");
    if (M == 0 || N == 0) return CF_OK;
    CF_REQUIRE(d_x && d_x_scale && d_x_descale && d_w8 && d_w_descale && d_y, "cf_fp8_linear_static_scratch: null pointer");
    CF_REQUIRE(ldy >= N, "cf_fp8_linear_static_scratch: ldy < N");
    CF_REQUIRE(bias_mode >= 0 && bias_mode <= 2, "cf_fp8_linear_static_scratch: bias_mode out of range");
    const size_t n = static_cast<size_t>(M) * static_cast<size_t>(K);
    if (n > kMaxActBytes) {
        cf::set_error("cf_fp8_linear_static_scratch: M*K = %zu exceeds the built-in scratch of %zu bytes; use "
                      "cf_fp8_linear_forward with a context for larger activations", n, kMaxActBytes);
        return CF_ERR_LIMIT;
    }
    const int rc0 = cf::require_sm100();
    if (rc0 != CF_OK) return rc0;
    unsigned char* base = nullptr;
    const int rc1 = scratch_address(&base);
    if (rc1 != CF_OK) return rc1;
    cudaStream_t st = cf::as_stream(stream);
    int* status = d_status_or_null;
    if (!status) {
        // the array keeps whatever the previous call left: the status word must start at zero
        status = reinterpret_cast<int*>(base);
        CF_CUDA(cudaMemsetAsync(status, 0, sizeof(int), st));
    }
    unsigned char* act8 = base + kHeaderBytes;
    const int rc2 = cf_fp8_quantize_e4m3(d_x, act8, d_x_scale, n, stream);
    if (rc2 != CF_OK) return rc2;
    cf::GemmParams p;
    p.M = M; p.N = N; p.K = K;
    p.d_a_descale = d_x_descale; p.d_b_descale = d_w_descale;
    p.C = d_y; p.ldc = ldy; p.out_kind = 0;
    p.bias = static_cast<const uint16_t*>(d_bias);
    p.bias_mode = d_bias ? bias_mode : 0;
    p.d_status = status;
    const int tiles = ((M + cf::gemm_tile_m() - 1) / cf::gemm_tile_m()) * ((N + cf::gemm_tile_n() - 1) / cf::gemm_tile_n());
    return cf::launch_gemm_fp8_nt(act8, K, M, d_w8, N, p, tiles, st);
}
