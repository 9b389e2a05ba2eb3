// Context, error plumbing, GEMM entry points, delayed-scaling slot state machine, fused linear.
#include <cstring>
#include <mutex>
#include <new>

#include "cf_common.cuh"
#include "cf_gemm.cuh"
#include "cf_internal.cuh"

namespace cf {

std::atomic<uint64_t> g_launches{0};

namespace {
thread_local char t_error[512] = "";
}

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
    return CF_ERR_CUDA;
}

// Per-device caches below are written from any thread: relaxed atomics (every writer stores the same value).
int sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    std::atomic<int>& c = cached[dev & 63];
    int v = c.load(std::memory_order_relaxed);
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        c.store(v, std::memory_order_relaxed);
    }
    return v;
}

int require_sm100() {
    static std::atomic<int> cached[64];   // 0 unknown, 1 ok, 2 unsupported
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { set_error("no CUDA device"); return CF_ERR_CUDA; }
    std::atomic<int>& c = cached[dev & 63];
    int v = c.load(std::memory_order_relaxed);
    if (v == 0) {
        int major = 0;
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        v = (major == 10) ? 1 : 2;
        c.store(v, std::memory_order_relaxed);
    }
    if (v != 1) { set_error("this library runs on compute capability 10.x (sm_100a) only"); return CF_ERR_UNSUPPORTED; }
    return CF_OK;
}

// Context: status word, act8 scratch, scalar pool for ActSlots, optional workspace.
struct Ctx {
    int device = 0;
    int* d_status = nullptr;
    void* act8 = nullptr;
    size_t act8_bytes = 0;
    float* scalar_pool = nullptr;     // blocks of 24 floats per slot
    int scalar_blocks = 0;
    int scalar_used = 0;
    void* workspace = nullptr;
    size_t workspace_bytes = 0;
    // reduce-scatter GEMM: kPeerMapSets sets of 16 tensor maps on the device, each remembered with the slices it
    // describes, so that repeated calls on the same slices re-encode and copy nothing
    void* d_peer_maps = nullptr;
    struct PeerMapKey { int kind = 0, count = 0, rows = 0, n = 0; long long ld = 0; void* ptr[16] = {}; } peer_key[4];
    int peer_next = 0;
    std::mutex mu;
};

constexpr int kPeerSetBytes = 16 * 128 + 16 * 8;   // 16 tensor maps followed by 16 base pointers
constexpr int kSlotFloats = 24;        // 8 scalars padded to 4 floats each is overkill; layout below
constexpr int kMaxSlots = 4096;
constexpr int kHistoryLen = 8;         // kActHistoryLen, src/trainer.cu:3213

int* ctx_status(cf_ctx* c) { return reinterpret_cast<Ctx*>(c)->d_status; }
void* ctx_workspace(cf_ctx* c, size_t* bytes) {
    Ctx* x = reinterpret_cast<Ctx*>(c);
    *bytes = x->workspace_bytes;
    return x->workspace;
}

// Slot of the context's device-side tensor-map sets that describes these buffers, and whether its contents are current.
int peer_set_lookup(Ctx* c, int kind, void* const* ptrs, int count, int rows, int n, long long ld, int* ready) {
    std::lock_guard<std::mutex> lk(c->mu);
    for (int i = 0; i < 4; ++i) {
        const Ctx::PeerMapKey& k = c->peer_key[i];
        if (k.count == count && k.kind == kind && k.rows == rows && k.n == n && k.ld == ld &&
            std::memcmp(k.ptr, ptrs, sizeof(void*) * count) == 0) {
            *ready = 1;
            return i;
        }
    }
    const int set = c->peer_next;
    c->peer_next = (c->peer_next + 1) % 4;
    c->peer_key[set].count = 0;            // invalid until the launch that fills it has been issued
    *ready = 0;
    return set;
}
void peer_set_commit(Ctx* c, int set, int kind, void* const* ptrs, int count, int rows, int n, long long ld) {
    std::lock_guard<std::mutex> lk(c->mu);
    Ctx::PeerMapKey& k = c->peer_key[set];
    k.kind = kind; k.count = count; k.rows = rows; k.n = n; k.ld = ld;
    std::memcpy(k.ptr, ptrs, sizeof(void*) * count);
}

}  // namespace cf

using namespace cf;

extern "C" {

const char* cf_last_error(void) { return t_error; }
int cf_abi_version(void) { return 3; }
uint64_t cf_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int cf_ctx_create(cf_ctx** out, size_t act8_bytes) {
    CF_REQUIRE(out != nullptr, "cf_ctx_create: null out pointer");
    *out = nullptr;
    const int rc = require_sm100();
    if (rc != CF_OK) return rc;
    Ctx* c = new (std::nothrow) Ctx();
    CF_REQUIRE(c != nullptr, "cf_ctx_create: out of host memory");
    cudaError_t e = cudaGetDevice(&c->device);
    if (e == cudaSuccess) e = cudaMalloc(&c->d_status, 64);
    if (e == cudaSuccess) e = cudaMemset(c->d_status, 0, 64);
    if (e == cudaSuccess) e = cudaMalloc(&c->d_peer_maps, 4 * kPeerSetBytes);
    if (e == cudaSuccess && act8_bytes) { e = cudaMalloc(&c->act8, act8_bytes); c->act8_bytes = act8_bytes; }
    if (e == cudaSuccess) {
        c->scalar_blocks = kMaxSlots;
        e = cudaMalloc(&c->scalar_pool, sizeof(float) * kSlotFloats * kMaxSlots);
    }
    if (e != cudaSuccess) {
        if (c->d_status) cudaFree(c->d_status);
        if (c->d_peer_maps) cudaFree(c->d_peer_maps);
        if (c->act8) cudaFree(c->act8);
        if (c->scalar_pool) cudaFree(c->scalar_pool);
        delete c;
        return cuda_fail(e, "cf_ctx_create");
    }
    *out = reinterpret_cast<cf_ctx*>(c);
    return CF_OK;
}

int cf_ctx_destroy(cf_ctx* ctx) {
    if (!ctx) return CF_OK;
    Ctx* c = reinterpret_cast<Ctx*>(ctx);
    if (c->d_status) cudaFree(c->d_status);
    if (c->d_peer_maps) cudaFree(c->d_peer_maps);
    if (c->act8) cudaFree(c->act8);
    if (c->scalar_pool) cudaFree(c->scalar_pool);
    if (c->workspace) cudaFree(c->workspace);
    delete c;
    return CF_OK;
}

void* cf_ctx_act8(cf_ctx* ctx) { return ctx ? reinterpret_cast<Ctx*>(ctx)->act8 : nullptr; }

int cf_ctx_reserve_workspace(cf_ctx* ctx, size_t bytes) {
    CF_REQUIRE(ctx != nullptr, "cf_ctx_reserve_workspace: null context");
    Ctx* c = reinterpret_cast<Ctx*>(ctx);
    std::lock_guard<std::mutex> lk(c->mu);
    if (bytes <= c->workspace_bytes) return CF_OK;
    if (c->workspace) { CF_CUDA(cudaFree(c->workspace)); c->workspace = nullptr; c->workspace_bytes = 0; }
    CF_CUDA(cudaMalloc(&c->workspace, bytes));
    c->workspace_bytes = bytes;
    return CF_OK;
}

int cf_ctx_poll_status(cf_ctx* ctx, void* stream) {
    CF_REQUIRE(ctx != nullptr, "cf_ctx_poll_status: null context");
    Ctx* c = reinterpret_cast<Ctx*>(ctx);
    int h = 0;
    CF_CUDA(cudaMemcpyAsync(&h, c->d_status, sizeof(int), cudaMemcpyDeviceToHost, as_stream(stream)));
    CF_CUDA(cudaStreamSynchronize(as_stream(stream)));
    if (h != 0) {
        CF_CUDA(cudaMemsetAsync(c->d_status, 0, sizeof(int), as_stream(stream)));
        if (((h >> 8) & 0xf) == 5) {
            set_error("a planned run of rows left its destination buffer and was not stored (status 0x%x: %s)", h,
                      (h & 0xff) == 2 ? "receive capacity exceeded in the plan" : "run refused by the sender");
            return CF_ERR_DEVICE_RANGE;
        }
        set_error("a tensor-core kernel abandoned a bounded wait (status 0x%x): role %d", h, (h >> 8) & 0xf);
        return CF_ERR_DEVICE_WAIT;
    }
    return CF_OK;
}

int cf_ctx_selftest_bounded_wait(cf_ctx* ctx, int limit_ms, void* stream) {
    CF_REQUIRE(ctx != nullptr, "cf_ctx_selftest_bounded_wait: null context");
    CF_REQUIRE(limit_ms >= 1 && limit_ms <= 1000, "cf_ctx_selftest_bounded_wait: limit must be 1..1000 ms");
    return launch_wait_selftest(reinterpret_cast<Ctx*>(ctx)->d_status, static_cast<unsigned long long>(limit_ms) * 1000000ull,
                                as_stream(stream));
}

// ------------------------------------------------------------------ GEMM entry points
static int check_gemm_common(const char* fn, cf_ctx* ctx, int M, int N, int K, const void* A, const void* B,
                             const void* C, const float* da, const float* db) {
    CF_REQUIRE(ctx != nullptr, "%s: null context", fn);
    CF_REQUIRE(M >= 0 && N >= 0 && K >= 0, "%s: negative shape", fn);
    if (M == 0 || N == 0) return CF_OK;
    CF_REQUIRE(A && B && C, "%s: null matrix pointer", fn);
    CF_REQUIRE(da && db, "%s: null descale pointer", fn);
    return CF_OK;
}

int cf_gemm_fp8_nt(cf_ctx* ctx, int M, int N, int K, const void* d_A, int lda, int a_is_e5m2, const float* d_a_descale,
                   const void* d_B, const float* d_b_descale, void* d_C, int ldc, const cf_gemm_epilogue* epi,
                   void* stream) {
    const int rc = check_gemm_common("cf_gemm_fp8_nt", ctx, M, N, K, d_A, d_B, d_C, d_a_descale, d_b_descale);
    if (rc != CF_OK || M == 0 || N == 0) return rc;
    CF_REQUIRE(lda >= K && ldc >= N, "cf_gemm_fp8_nt: leading dimension smaller than the row length");
    GemmParams p;
    p.M = M; p.N = N; p.K = K;
    p.d_a_descale = d_a_descale; p.d_b_descale = d_b_descale;
    p.C = d_C; p.ldc = ldc; p.out_kind = 0;
    p.a_e5m2 = a_is_e5m2 ? 1 : 0;
    if (epi) {
        CF_REQUIRE(epi->bias_mode >= 0 && epi->bias_mode <= 2, "cf_gemm_fp8_nt: bias_mode out of range");
        p.bias = static_cast<const uint16_t*>(epi->d_bias);
        p.bias_mode = epi->d_bias ? epi->bias_mode : 0;
        p.d_a_row_descale = epi->d_a_row_descale;
        p.d_b_col_descale = epi->d_b_col_descale;
        if (epi->out_fp32) {
            CF_REQUIRE(epi->d_bias == nullptr, "cf_gemm_fp8_nt: out_fp32 takes no bias");
            p.out_kind = 1;
        }
    }
    p.d_status = reinterpret_cast<Ctx*>(ctx)->d_status;
    if (K == 0) {   // empty contraction: the product is zero, the epilogue still applies
        set_error("cf_gemm_fp8_nt: K == 0 is not supported");
        return CF_ERR_UNSUPPORTED;
    }
    const int tiles = ((M + gemm_tile_m() - 1) / gemm_tile_m()) * ((N + gemm_tile_n() - 1) / gemm_tile_n());
    return launch_gemm_fp8_nt(d_A, lda, M, d_B, N, p, tiles, as_stream(stream));
}

int cf_gemm_fp8_nt_reduce_scatter_f32(cf_ctx* ctx, int M, int N, int K, const void* d_A, int lda, int a_is_e5m2,
                                      const float* d_a_descale, const void* d_B, const float* d_b_descale,
                                      const float* d_a_row_descale_or_null, const float* d_b_col_descale_or_null,
                                      void* const* slices, int num_slices, void* stream) {
    CF_REQUIRE(ctx != nullptr, "cf_gemm_fp8_nt_reduce_scatter_f32: null context");
    CF_REQUIRE(M > 0 && N > 0 && K > 0 && lda >= K, "cf_gemm_fp8_nt_reduce_scatter_f32: bad shape");
    CF_REQUIRE(d_A && d_B && d_a_descale && d_b_descale && slices, "cf_gemm_fp8_nt_reduce_scatter_f32: null pointer");
    CF_REQUIRE(num_slices >= 1 && num_slices <= 16 && M % num_slices == 0, "cf_gemm_fp8_nt_reduce_scatter_f32: M must split evenly over 1..16 slices");
    GemmParams p;
    p.M = M; p.N = N; p.K = K;
    p.d_a_descale = d_a_descale; p.d_b_descale = d_b_descale;
    p.C = nullptr; p.ldc = N; p.out_kind = 2;
    p.a_e5m2 = a_is_e5m2 ? 1 : 0;
    p.d_a_row_descale = d_a_row_descale_or_null; p.d_b_col_descale = d_b_col_descale_or_null;
    p.peer_out_host = slices; p.peer_count = num_slices; p.rows_per_peer = M / num_slices;
    Ctx* c = reinterpret_cast<Ctx*>(ctx);
    const int set = peer_set_lookup(c, 0, slices, num_slices, p.rows_per_peer, N, N, &p.peer_maps_ready);
    p.d_peer_maps = static_cast<char*>(c->d_peer_maps) + static_cast<size_t>(set) * kPeerSetBytes;
    p.d_status = c->d_status;
    const int tiles = ((M + gemm_tile_m() - 1) / gemm_tile_m()) * ((N + gemm_tile_n() - 1) / gemm_tile_n());
    const int rc = launch_gemm_fp8_nt(d_A, lda, M, d_B, N, p, tiles, as_stream(stream));
    if (rc == CF_OK && !p.peer_maps_ready) peer_set_commit(c, set, 0, slices, num_slices, p.rows_per_peer, N, N);
    return rc;
}

int cf_gemm_fp8_nt_grouped_return(cf_ctx* ctx, int num_groups, int max_total_rows, int N, int K, const int* d_counts,
                                  const int* d_offsets, const void* d_A, int lda, int a_is_e5m2, const float* d_a_descale,
                                  const void* d_B, const float* d_b_descale, const cf_row_run* d_return_runs,
                                  int runs_per_group, void* const* dst_buffers, int num_dst, int dst_rows, int ldc,
                                  void* stream) {
    CF_REQUIRE(ctx != nullptr, "cf_gemm_fp8_nt_grouped_return: null context");
    CF_REQUIRE(num_groups >= 1 && max_total_rows >= 0 && N > 0 && K > 0 && lda >= K && ldc >= N,
               "cf_gemm_fp8_nt_grouped_return: bad shape");
    if (max_total_rows == 0) return CF_OK;
    CF_REQUIRE(d_counts && d_offsets && d_A && d_B && d_a_descale && d_b_descale && d_return_runs && dst_buffers,
               "cf_gemm_fp8_nt_grouped_return: null pointer");
    CF_REQUIRE(runs_per_group >= 1 && num_dst >= 1 && num_dst <= 16 && dst_rows > 0,
               "cf_gemm_fp8_nt_grouped_return: 1..16 destination buffers");
    GemmParams p;
    p.groups = num_groups;
    p.M = max_total_rows; p.N = N; p.K = K;
    p.d_counts = d_counts; p.d_offsets = d_offsets;
    p.d_a_descale = d_a_descale; p.d_b_descale = d_b_descale;
    p.C = nullptr; p.ldc = ldc; p.out_kind = 0;
    p.a_e5m2 = a_is_e5m2 ? 1 : 0;
    p.d_out_runs = d_return_runs; p.runs_per_group = runs_per_group;
    p.peer_out_host = dst_buffers; p.peer_count = num_dst; p.rows_per_peer = dst_rows;
    Ctx* c = reinterpret_cast<Ctx*>(ctx);
    const int set = peer_set_lookup(c, 1, dst_buffers, num_dst, dst_rows, N, ldc, &p.peer_maps_ready);
    p.d_peer_maps = static_cast<char*>(c->d_peer_maps) + static_cast<size_t>(set) * kPeerSetBytes;
    p.d_status = c->d_status;
    const int n_blocks = (N + gemm_tile_n() - 1) / gemm_tile_n();
    const int m_blocks = (max_total_rows + gemm_tile_m() - 1) / gemm_tile_m() + num_groups;
    const long long b_rows = static_cast<long long>(num_groups) * N;
    const int rc = launch_gemm_fp8_nt(d_A, lda, max_total_rows, d_B, b_rows, p, m_blocks * n_blocks, as_stream(stream));
    if (rc == CF_OK && !p.peer_maps_ready) peer_set_commit(c, set, 1, dst_buffers, num_dst, dst_rows, N, ldc);
    return rc;
}

static int tn_accum(cf_ctx* ctx, int M, int N, int K, const void* Xt, const float* ds_x, const void* dYt,
                    const float* ds_dy, void* dW, int ldc, int out_kind, cudaStream_t st) {
    const int rc = check_gemm_common("cf_gemm_fp8_tn_accum", ctx, M, N, K, Xt, dYt, dW, ds_x, ds_dy);
    if (rc != CF_OK || M == 0 || N == 0 || K == 0) return rc;
    CF_REQUIRE(ldc >= N, "cf_gemm_fp8_tn_accum: ldc < N");
    GemmParams p;
    p.M = M; p.N = N; p.K = K;
    p.d_a_descale = ds_x; p.d_b_descale = ds_dy;
    p.C = dW; p.ldc = ldc; p.out_kind = out_kind;
    p.a_e5m2 = 0; p.b_e5m2 = 1;
    p.d_status = reinterpret_cast<Ctx*>(ctx)->d_status;
    const int tiles = ((M + gemm_tile_m() - 1) / gemm_tile_m()) * ((N + gemm_tile_n() - 1) / gemm_tile_n());
    return launch_gemm_fp8_nt(Xt, K, M, dYt, N, p, tiles, st);
}

int cf_gemm_fp8_tn_accum_f32(cf_ctx* ctx, int M, int N, int K, const void* d_Xt_e4m3, const float* d_ds_x,
                             const void* d_dYt_e5m2, const float* d_ds_dy, float* d_dW, int ldc, void* stream) {
    return tn_accum(ctx, M, N, K, d_Xt_e4m3, d_ds_x, d_dYt_e5m2, d_ds_dy, d_dW, ldc, 2, as_stream(stream));
}
int cf_gemm_fp8_tn_accum_bf16(cf_ctx* ctx, int M, int N, int K, const void* d_Xt_e4m3, const float* d_ds_x,
                              const void* d_dYt_e5m2, const float* d_ds_dy, void* d_dW, int ldc, void* stream) {
    return tn_accum(ctx, M, N, K, d_Xt_e4m3, d_ds_x, d_dYt_e5m2, d_ds_dy, d_dW, ldc, 3, as_stream(stream));
}

static int dw_accum(cf_ctx* ctx, int M, int N, int K, const void* X8, int ldx, const float* ds_x, const void* dY8, int ldy,
                    const float* ds_dy, void* dW, int ldc, int out_kind, cudaStream_t st) {
    const int rc = check_gemm_common("cf_gemm_fp8_dw_accum", ctx, M, N, K, X8, dY8, dW, ds_x, ds_dy);
    if (rc != CF_OK || M == 0 || N == 0 || K == 0) return rc;
    CF_REQUIRE(ldx >= M && ldy >= N && ldc >= N, "cf_gemm_fp8_dw_accum: leading dimension smaller than the row length");
    GemmParams p;
    p.M = M; p.N = N; p.K = K;
    p.mn_major = 1; p.ldb = ldy;
    p.d_a_descale = ds_x; p.d_b_descale = ds_dy;
    p.C = dW; p.ldc = ldc; p.out_kind = out_kind;
    p.a_e5m2 = 0; p.b_e5m2 = 1;
    p.d_status = reinterpret_cast<Ctx*>(ctx)->d_status;
    const int tiles = ((M + gemm_tile_m() - 1) / gemm_tile_m()) * ((N + gemm_tile_n() - 1) / gemm_tile_n());
    return launch_gemm_fp8_nt(X8, ldx, K, dY8, K, p, tiles, st);
}

int cf_gemm_fp8_dw_accum_f32(cf_ctx* ctx, int M, int N, int K, const void* d_X_e4m3, int ldx, const float* d_ds_x,
                             const void* d_dY_e5m2, int ldy, const float* d_ds_dy, float* d_dW, int ldc, void* stream) {
    return dw_accum(ctx, M, N, K, d_X_e4m3, ldx, d_ds_x, d_dY_e5m2, ldy, d_ds_dy, d_dW, ldc, 2, as_stream(stream));
}
int cf_gemm_fp8_dw_accum_bf16(cf_ctx* ctx, int M, int N, int K, const void* d_X_e4m3, int ldx, const float* d_ds_x,
                              const void* d_dY_e5m2, int ldy, const float* d_ds_dy, void* d_dW, int ldc, void* stream) {
    return dw_accum(ctx, M, N, K, d_X_e4m3, ldx, d_ds_x, d_dY_e5m2, ldy, d_ds_dy, d_dW, ldc, 3, as_stream(stream));
}

// C = A . B with the weight read as it lies in the forward cache ([K, N] per block): the dgrad direction without a
// second, transposed weight cache.
static int gemm_nn(cf_ctx* ctx, int groups, int rows, int N, int K, const int* d_counts, const int* d_offsets, const void* d_A,
                   int lda, int a_is_e5m2, const float* d_a_descale, const void* d_B, int ldb, const float* d_b_descale,
                   void* d_C, int ldc, int accumulate, cudaStream_t st) {
    CF_REQUIRE(ctx != nullptr, "cf_gemm_fp8_nn: null context");
    CF_REQUIRE(groups >= 1 && groups <= 1024 && rows >= 0 && N >= 0 && K > 0, "cf_gemm_fp8_nn: bad shape");
    if (rows == 0 || N == 0) return CF_OK;
    CF_REQUIRE(d_A && d_B && d_C && d_a_descale && d_b_descale, "cf_gemm_fp8_nn: null pointer");
    CF_REQUIRE(lda >= K && ldb >= N && ldc >= N, "cf_gemm_fp8_nn: leading dimension smaller than the row length");
    GemmParams p;
    p.groups = groups;
    p.M = rows; p.N = N; p.K = K;
    p.d_counts = d_counts; p.d_offsets = d_offsets;
    p.b_mn_major = 1; p.ldb = ldb;
    p.d_a_descale = d_a_descale; p.d_b_descale = d_b_descale;
    p.C = d_C; p.ldc = ldc; p.out_kind = accumulate ? 3 : 0;
    p.a_e5m2 = a_is_e5m2 ? 1 : 0;
    p.d_status = reinterpret_cast<Ctx*>(ctx)->d_status;
    const int m_blocks = (rows + gemm_tile_m() - 1) / gemm_tile_m() + (d_counts ? groups : 0);
    const int tiles = m_blocks * ((N + gemm_tile_n() - 1) / gemm_tile_n());
    return launch_gemm_fp8_nt(d_A, lda, rows, d_B, static_cast<long long>(groups) * K, p, tiles, st);
}

int cf_gemm_fp8_nn(cf_ctx* ctx, int M, int N, int K, const void* d_A, int lda, int a_is_e5m2, const float* d_a_descale,
                   const void* d_B_kn, int ldb, const float* d_b_descale, void* d_C, int ldc, int accumulate, void* stream) {
    return gemm_nn(ctx, 1, M, N, K, nullptr, nullptr, d_A, lda, a_is_e5m2, d_a_descale, d_B_kn, ldb, d_b_descale, d_C, ldc,
                   accumulate, as_stream(stream));
}

int cf_gemm_fp8_nn_grouped(cf_ctx* ctx, int num_groups, int max_total_rows, int N, int K, const int* d_counts,
                           const int* d_offsets, const void* d_A, int lda, int a_is_e5m2, const float* d_a_descale,
                           const void* d_B_stacked_kn, const float* d_b_descale, void* d_C, int ldc, int accumulate,
                           void* stream) {
    CF_REQUIRE(d_counts && d_offsets, "cf_gemm_fp8_nn_grouped: null counts or offsets");
    return gemm_nn(ctx, num_groups, max_total_rows, N, K, d_counts, d_offsets, d_A, lda, a_is_e5m2, d_a_descale,
                   d_B_stacked_kn, N, d_b_descale, d_C, ldc, accumulate, as_stream(stream));
}

int cf_gemm_fp8_nt_grouped(cf_ctx* ctx, int num_experts, int max_total_rows, int N, int K, const int* d_counts,
                           const int* d_offsets, const void* d_A, int lda, int a_is_e5m2, const float* d_a_descale,
                           int per_expert_a_descale, const void* d_B, const float* d_b_descale, void* d_C, int ldc,
                           void* stream) {
    return cf_gemm_fp8_nt_segments(ctx, num_experts, num_experts, nullptr, max_total_rows, N, K, d_counts, d_offsets, d_A,
                                   lda, a_is_e5m2, d_a_descale, per_expert_a_descale, d_B, d_b_descale, d_C, ldc, stream);
}

int cf_gemm_fp8_nt_segments(cf_ctx* ctx, int num_segments, int num_weights, const int* d_segment_weight,
                            int max_total_rows, int N, int K, const int* d_counts, const int* d_offsets, const void* d_A,
                            int lda, int a_is_e5m2, const float* d_a_descale, int per_segment_a_descale, const void* d_B,
                            const float* d_b_descale, void* d_C, int ldc, void* stream) {
    return cf_gemm_fp8_nt_segments_scatter(ctx, num_segments, num_weights, d_segment_weight, max_total_rows, N, K, d_counts,
                                           d_offsets, d_A, lda, a_is_e5m2, d_a_descale, per_segment_a_descale, d_B,
                                           d_b_descale, d_C, nullptr, nullptr, ldc, stream);
}

int cf_gemm_fp8_nt_segments_scatter(cf_ctx* ctx, int num_segments, int num_weights, const int* d_segment_weight,
                                    int max_total_rows, int N, int K, const int* d_counts, const int* d_offsets,
                                    const void* d_A, int lda, int a_is_e5m2, const float* d_a_descale,
                                    int per_segment_a_descale, const void* d_B, const float* d_b_descale, void* d_C,
                                    void* const* d_segment_out, const long long* d_segment_out_row0, int ldc,
                                    void* stream) {
    CF_REQUIRE((d_segment_out == nullptr) == (d_segment_out_row0 == nullptr),
               "cf_gemm_fp8_nt_segments_scatter: d_segment_out and d_segment_out_row0 go together");
    if (d_segment_out && d_C == nullptr) d_C = const_cast<void*>(static_cast<const void*>(d_segment_out));   // unused placeholder
    const int num_experts = num_segments;
    const int per_expert_a_descale = per_segment_a_descale;
    CF_REQUIRE(num_weights >= 1, "cf_gemm_fp8_nt_segments: num_weights must be positive");
    CF_REQUIRE(ctx != nullptr, "cf_gemm_fp8_nt_grouped: null context");
    CF_REQUIRE(num_experts >= 1 && num_experts <= 1024, "cf_gemm_fp8_nt_grouped: num_experts out of range");
    CF_REQUIRE(max_total_rows >= 0 && N >= 0 && K > 0, "cf_gemm_fp8_nt_grouped: bad shape");
    if (max_total_rows == 0 || N == 0) return CF_OK;
    CF_REQUIRE(d_counts && d_offsets && d_A && d_B && d_C && d_a_descale && d_b_descale,
               "cf_gemm_fp8_nt_grouped: null pointer");
    CF_REQUIRE(lda >= K && ldc >= N, "cf_gemm_fp8_nt_grouped: leading dimension smaller than the row length");
    GemmParams p;
    p.groups = num_experts;
    p.N = N; p.K = K;
    p.d_counts = d_counts; p.d_offsets = d_offsets;
    p.d_group_weight = d_segment_weight;
    p.d_group_out = d_segment_out;
    p.d_group_out_row0 = d_segment_out_row0;
    p.d_a_descale = d_a_descale; p.a_descale_per_group = per_expert_a_descale ? 1 : 0;
    p.d_b_descale = d_b_descale;
    p.C = d_C; p.ldc = ldc; p.out_kind = 0;
    p.a_e5m2 = a_is_e5m2 ? 1 : 0;
    p.d_status = reinterpret_cast<Ctx*>(ctx)->d_status;
    const int m_blocks = (max_total_rows + gemm_tile_m() - 1) / gemm_tile_m() + num_experts;
    const int tiles = m_blocks * ((N + gemm_tile_n() - 1) / gemm_tile_n());
    return launch_gemm_fp8_nt(d_A, lda, max_total_rows, d_B, static_cast<long long>(num_weights) * N, p, tiles,
                              as_stream(stream));
}

// ------------------------------------------------------------------ ActSlot
int cf_act_slot_init(cf_ctx* ctx, cf_act_slot* slot, float fp8_max, int calib_calls, void* stream) {
    CF_REQUIRE(ctx && slot, "cf_act_slot_init: null pointer");
    CF_REQUIRE(fp8_max == CF_E4M3_MAX || fp8_max == CF_E5M2_MAX, "cf_act_slot_init: fp8_max must be 448 or 57344");
    Ctx* c = reinterpret_cast<Ctx*>(ctx);
    float* base;
    {
        std::lock_guard<std::mutex> lk(c->mu);
        if (c->scalar_used >= c->scalar_blocks) { set_error("cf_act_slot_init: slot pool exhausted (%d)", kMaxSlots); return CF_ERR_LIMIT; }
        base = c->scalar_pool + static_cast<size_t>(c->scalar_used++) * kSlotFloats;
    }
    // 16-byte aligned scalars (the GEMM reads descale through 16-byte aligned pointers, src/trainer.cu:4239-4242)
    std::memset(slot, 0, sizeof(*slot));
    slot->amax = base + 0;
    slot->scale = base + 4;
    slot->descale = base + 8;
    slot->scale_snapshot = base + 12;
    slot->descale_snapshot = base + 16;   // floats 17..19: cursor, count, calib_min ; 20: calib_max
    slot->history_cursor = reinterpret_cast<int*>(base + 17);
    slot->history_count = reinterpret_cast<int*>(base + 18);
    slot->calib_min = base + 19;
    slot->calib_max = base + 20;
    slot->ticket = reinterpret_cast<unsigned*>(base + 21);
    slot->history = nullptr;
    slot->fp8_max = fp8_max;
    slot->init = 0;
    slot->calib_remaining = calib_calls > 0 ? calib_calls : 0;
    slot->calib_commit_pending = 0;
    // history ring lives in a second block
    {
        std::lock_guard<std::mutex> lk(c->mu);
        if (c->scalar_used >= c->scalar_blocks) { set_error("cf_act_slot_init: slot pool exhausted (%d)", kMaxSlots); return CF_ERR_LIMIT; }
        slot->history = c->scalar_pool + static_cast<size_t>(c->scalar_used++) * kSlotFloats;
    }
    cudaStream_t st = as_stream(stream);
    CF_CUDA(cudaMemsetAsync(base, 0, sizeof(float) * kSlotFloats, st));
    CF_CUDA(cudaMemsetAsync(slot->history, 0, sizeof(float) * kSlotFloats, st));
    // running min starts at the byte pattern 0x7f7f7f7f (~3.39e38), running max at 0 (src/trainer.cu:4198-4199)
    CF_CUDA(cudaMemsetAsync(slot->calib_min, 0x7F, sizeof(float), st));
    return CF_OK;
}

static int quant_plain(const cf_act_slot* s, const void* x, void* out, const float* scale, size_t n, void* st) {
    return s->fp8_max == CF_E5M2_MAX ? cf_fp8_quantize_e5m2(x, out, scale, n, st) : cf_fp8_quantize_e4m3(x, out, scale, n, st);
}

#define CF_TRY(call)              \
    do {                          \
        const int rc__ = (call);  \
        if (rc__ != CF_OK) return rc__; \
    } while (0)

int cf_fp8_quant_act(cf_ctx* ctx, cf_act_slot* slot, const void* d_x, size_t n, void* d_out8, void* stream,
                     int is_recompute) {
    CF_REQUIRE(ctx && slot && slot->amax, "cf_fp8_quant_act: null or uninitialised slot");
    CF_REQUIRE(n == 0 || (d_x && d_out8), "cf_fp8_quant_act: null tensor pointer");
    cudaStream_t st = as_stream(stream);
    if (is_recompute) return quant_plain(slot, d_x, d_out8, slot->scale_snapshot, n, stream);

    if (slot->calib_commit_pending) {
        slot->calib_commit_pending = 0;
        float mn = 0.0f, mx = 0.0f;
        CF_CUDA(cudaStreamSynchronize(st));
        CF_CUDA(cudaMemcpy(&mn, slot->calib_min, sizeof(float), cudaMemcpyDeviceToHost));
        CF_CUDA(cudaMemcpy(&mx, slot->calib_max, sizeof(float), cudaMemcpyDeviceToHost));
        const float spread = (mn > 0.0f) ? (mx / mn) : 0.0f;
        if (slot->fp8_max == CF_E4M3_MAX && spread > 4.0f) {    // IDA_FP8_TYPE_SPREAD default, src/trainer.cu:3778
            slot->fp8_max = CF_E5M2_MAX;
            CF_CUDA(cudaMemcpyAsync(slot->amax, slot->calib_max, sizeof(float), cudaMemcpyDeviceToDevice, st));
            CF_CUDA(cudaMemsetAsync(slot->history_cursor, 0, sizeof(int), st));
            CF_CUDA(cudaMemsetAsync(slot->history_count, 0, sizeof(int), st));
            CF_TRY(cf_fp8_scale_from_amax(slot->amax, slot->fp8_max, slot->scale, slot->descale, stream));
            CF_TRY(cf_fp8_update_delayed_scale(slot->amax, slot->fp8_max, slot->scale, slot->descale, slot->history,
                                               kHistoryLen, slot->history_cursor, slot->history_count, stream));
        }
    }

    if (slot->calib_remaining > 0 || !slot->init) {
        // exact per-call amax: amax pass, scale, snapshot, quantise, [spread record], ring update
        const bool calib = slot->calib_remaining > 0;
        CF_TRY(cf_fp8_amax_bf16(d_x, n, slot->amax, stream));
        CF_TRY(cf_fp8_scale_from_amax(slot->amax, slot->fp8_max, slot->scale, slot->descale, stream));
        CF_CUDA(cudaMemcpyAsync(slot->scale_snapshot, slot->scale, sizeof(float), cudaMemcpyDeviceToDevice, st));
        CF_CUDA(cudaMemcpyAsync(slot->descale_snapshot, slot->descale, sizeof(float), cudaMemcpyDeviceToDevice, st));
        CF_TRY(quant_plain(slot, d_x, d_out8, slot->scale, n, stream));
        if (calib) CF_TRY(cf_fp8_calib_minmax_update(slot->amax, slot->calib_min, slot->calib_max, stream));
        CF_TRY(cf_fp8_update_delayed_scale(slot->amax, slot->fp8_max, slot->scale, slot->descale, slot->history,
                                           kHistoryLen, slot->history_cursor, slot->history_count, stream));
        slot->init = 1;
        if (calib && --slot->calib_remaining == 0) slot->calib_commit_pending = 1;
        return CF_OK;
    }

    // steady state: snapshot, record-quantise with the previous scale, advance the ring
    if (slot->ticket) {
        // ONE launch: block 0 snapshots the pair, every block accumulates its amax into the work word next to
        // the ticket, the last block publishes the amax and runs the ring update (src/trainer.cu:4823-4850 takes
        // two scalar copies, a memset and two kernels for the same effect)
        RingTail tail;
        tail.fp8_max = slot->fp8_max; tail.scale = slot->scale; tail.descale = slot->descale;
        tail.history = slot->history; tail.history_len = kHistoryLen;
        tail.history_cursor = slot->history_cursor; tail.history_count = slot->history_count;
        tail.ticket = slot->ticket;
        tail.work_amax = reinterpret_cast<float*>(slot->ticket + 1);
        tail.snap_scale = slot->scale_snapshot; tail.snap_descale = slot->descale_snapshot;
        return quantize_record_fused(d_x, d_out8, slot->scale, slot->amax, n, slot->fp8_max == CF_E5M2_MAX, tail, st);
    }
    CF_TRY(slot_begin(slot->scale, slot->descale, slot->scale_snapshot, slot->descale_snapshot, slot->amax, st));
    if (slot->fp8_max == CF_E5M2_MAX)
        CF_TRY(cf_fp8_quantize_e5m2_record(d_x, d_out8, slot->scale, slot->amax, n, stream));
    else
        CF_TRY(cf_fp8_quantize_e4m3_record(d_x, d_out8, slot->scale, slot->amax, n, stream));
    CF_TRY(cf_fp8_update_delayed_scale(slot->amax, slot->fp8_max, slot->scale, slot->descale, slot->history, kHistoryLen,
                                       slot->history_cursor, slot->history_count, stream));
    return CF_OK;
}

int cf_fp8_swiglu_quant_act(cf_ctx* ctx, cf_act_slot* slot, const void* d_gate, const void* d_up, int ld_in, int rows,
                            int cols, void* d_out8, void* stream) {
    CF_REQUIRE(ctx && slot && slot->amax, "cf_fp8_swiglu_quant_act: null or uninitialised slot");
    CF_REQUIRE(rows >= 0 && cols >= 0 && ld_in >= cols, "cf_fp8_swiglu_quant_act: bad shape");
    CF_REQUIRE(slot->fp8_max == CF_E4M3_MAX, "cf_fp8_swiglu_quant_act: E4M3 slots only");
    CF_REQUIRE(rows == 0 || cols == 0 || (d_gate && d_up && d_out8), "cf_fp8_swiglu_quant_act: null tensor pointer");
    cudaStream_t st = as_stream(stream);
    if (!slot->init) {
        // first use: exact amax of the product (a record pass whose codes are overwritten below), then the
        // same sequence as fp8_quant_act's first call (src/trainer.cu:4793-4815)
        CF_CUDA(cudaMemsetAsync(slot->amax, 0, sizeof(float), st));
        CF_CUDA(cudaMemsetAsync(slot->scale, 0, sizeof(float), st));
        CF_TRY(swiglu_record_launch(d_gate, d_up, ld_in, d_out8, cols, slot->scale, slot->amax, rows, cols, RingTail(), st));
        CF_TRY(cf_fp8_scale_from_amax(slot->amax, slot->fp8_max, slot->scale, slot->descale, stream));
        CF_CUDA(cudaMemcpyAsync(slot->scale_snapshot, slot->scale, sizeof(float), cudaMemcpyDeviceToDevice, st));
        CF_CUDA(cudaMemcpyAsync(slot->descale_snapshot, slot->descale, sizeof(float), cudaMemcpyDeviceToDevice, st));
        CF_TRY(swiglu_record_launch(d_gate, d_up, ld_in, d_out8, cols, slot->scale, slot->amax, rows, cols, RingTail(), st));
        CF_TRY(cf_fp8_update_delayed_scale(slot->amax, slot->fp8_max, slot->scale, slot->descale, slot->history,
                                           kHistoryLen, slot->history_cursor, slot->history_count, stream));
        slot->init = 1;
        return CF_OK;
    }
    CF_TRY(slot_begin(slot->scale, slot->descale, slot->scale_snapshot, slot->descale_snapshot, slot->amax, st));
    RingTail tail;
    if (slot->ticket) {
        tail.fp8_max = slot->fp8_max; tail.scale = slot->scale; tail.descale = slot->descale;
        tail.history = slot->history; tail.history_len = kHistoryLen;
        tail.history_cursor = slot->history_cursor; tail.history_count = slot->history_count;
        tail.ticket = slot->ticket;
    }
    CF_TRY(swiglu_record_launch(d_gate, d_up, ld_in, d_out8, cols, slot->scale, slot->amax, rows, cols, tail, st));
    if (!slot->ticket)
        CF_TRY(cf_fp8_update_delayed_scale(slot->amax, slot->fp8_max, slot->scale, slot->descale, slot->history,
                                           kHistoryLen, slot->history_cursor, slot->history_count, stream));
    return CF_OK;
}

int cf_fp8_rmsnorm_clip_quant_act(cf_ctx* ctx, cf_act_slot* slot, const void* d_x, const void* d_norm_scale,
                                  void* d_normed_or_null, float* d_rms_or_null, int rows, int H, float eps,
                                  float clip_ceiling, void* d_out8, void* stream) {
    CF_REQUIRE(ctx && slot && slot->amax, "cf_fp8_rmsnorm_clip_quant_act: null or uninitialised slot");
    CF_REQUIRE(slot->fp8_max == CF_E4M3_MAX, "cf_fp8_rmsnorm_clip_quant_act: E4M3 slots only");
    cudaStream_t st = as_stream(stream);
    if (!slot->init) {
        // first use: exact amax of the normalised rows (a record pass whose codes are overwritten below), then the
        // sequence of fp8_quant_act's first call (src/trainer.cu:4793-4815)
        CF_CUDA(cudaMemsetAsync(slot->amax, 0, sizeof(float), st));
        CF_CUDA(cudaMemsetAsync(slot->scale, 0, sizeof(float), st));
        CF_TRY(rmsnorm_launch(1, d_x, d_norm_scale, d_normed_or_null, d_rms_or_null, d_out8, slot->scale, slot->amax, nullptr,
                              nullptr, rows, H, eps, RingTail(), st, clip_ceiling));
        CF_TRY(cf_fp8_scale_from_amax(slot->amax, slot->fp8_max, slot->scale, slot->descale, stream));
        CF_CUDA(cudaMemcpyAsync(slot->scale_snapshot, slot->scale, sizeof(float), cudaMemcpyDeviceToDevice, st));
        CF_CUDA(cudaMemcpyAsync(slot->descale_snapshot, slot->descale, sizeof(float), cudaMemcpyDeviceToDevice, st));
        CF_TRY(rmsnorm_launch(1, d_x, d_norm_scale, d_normed_or_null, d_rms_or_null, d_out8, slot->scale, slot->amax, nullptr,
                              nullptr, rows, H, eps, RingTail(), st, clip_ceiling));
        CF_TRY(cf_fp8_update_delayed_scale(slot->amax, slot->fp8_max, slot->scale, slot->descale, slot->history,
                                           kHistoryLen, slot->history_cursor, slot->history_count, stream));
        slot->init = 1;
        return CF_OK;
    }
    CF_TRY(slot_begin(slot->scale, slot->descale, slot->scale_snapshot, slot->descale_snapshot, slot->amax, st));
    RingTail tail;
    if (slot->ticket) {
        tail.fp8_max = slot->fp8_max; tail.scale = slot->scale; tail.descale = slot->descale;
        tail.history = slot->history; tail.history_len = kHistoryLen;
        tail.history_cursor = slot->history_cursor; tail.history_count = slot->history_count;
        tail.ticket = slot->ticket;
    }
    // the kernel reads the scale it quantises with from the snapshot: the tail may rewrite slot->scale while
    // other blocks are still running
    CF_TRY(rmsnorm_launch(1, d_x, d_norm_scale, d_normed_or_null, d_rms_or_null, d_out8, slot->scale_snapshot, slot->amax,
                          nullptr, nullptr, rows, H, eps, tail, st, clip_ceiling));
    if (!slot->ticket)
        CF_TRY(cf_fp8_update_delayed_scale(slot->amax, slot->fp8_max, slot->scale, slot->descale, slot->history,
                                           kHistoryLen, slot->history_cursor, slot->history_count, stream));
    return CF_OK;
}

int cf_fp8_rmsnorm_quant_act(cf_ctx* ctx, cf_act_slot* slot, const void* d_x, const void* d_norm_scale, void* d_normed_or_null,
                             float* d_rms_or_null, int rows, int H, float eps, void* d_out8, void* stream) {
    return cf_fp8_rmsnorm_clip_quant_act(ctx, slot, d_x, d_norm_scale, d_normed_or_null, d_rms_or_null, rows, H, eps, 0.0f,
                                         d_out8, stream);
}

int cf_gemm_fp8_swiglu_quant_act(cf_ctx* ctx, cf_act_slot* slot, int num_segments, int num_weights,
                                 const int* d_segment_weight, int max_total_rows, int F, int K, const int* d_counts,
                                 const int* d_offsets, const void* d_A, int lda, int a_is_e5m2, const float* d_a_descale,
                                 int per_segment_a_descale, const void* d_W_interleaved, const float* d_w_descale,
                                 void* d_h8, int ldh, void* stream) {
    CF_REQUIRE(ctx && slot && slot->amax, "cf_gemm_fp8_swiglu_quant_act: null context or uninitialised slot");
    CF_REQUIRE(slot->fp8_max == CF_E4M3_MAX, "cf_gemm_fp8_swiglu_quant_act: E4M3 slots only");
    CF_REQUIRE(max_total_rows >= 0 && F > 0 && K > 0 && num_segments >= 1 && num_weights >= 1, "cf_gemm_fp8_swiglu_quant_act: bad shape");
    CF_REQUIRE(F % 32 == 0, "cf_gemm_fp8_swiglu_quant_act: F must be a multiple of 32 (gate/up rows interleave in groups of 32)");
    CF_REQUIRE((d_counts == nullptr) == (d_offsets == nullptr), "cf_gemm_fp8_swiglu_quant_act: counts and offsets go together");
    CF_REQUIRE(d_counts != nullptr || num_segments == 1, "cf_gemm_fp8_swiglu_quant_act: the dense form has one segment");
    CF_REQUIRE(lda >= K && ldh >= F, "cf_gemm_fp8_swiglu_quant_act: leading dimension smaller than the row length");
    if (max_total_rows == 0) return CF_OK;
    CF_REQUIRE(d_A && d_a_descale && d_W_interleaved && d_w_descale && d_h8, "cf_gemm_fp8_swiglu_quant_act: null pointer");
    cudaStream_t st = as_stream(stream);
    GemmParams p;
    p.groups = num_segments;
    p.M = max_total_rows;
    p.N = 2 * F; p.K = K;
    p.d_counts = d_counts; p.d_offsets = d_offsets; p.d_group_weight = d_segment_weight;
    p.d_a_descale = d_a_descale; p.a_descale_per_group = per_segment_a_descale == 1 ? 1 : 0;
    if (per_segment_a_descale == 2) p.d_a_row_descale = d_a_descale;      // one descale per row of A
    p.d_b_descale = d_w_descale;
    p.C = d_h8; p.ldc = ldh; p.out_kind = 4;
    p.a_e5m2 = a_is_e5m2 ? 1 : 0;
    p.d_quant_scale = slot->scale; p.d_amax_out = slot->amax;
    p.d_status = reinterpret_cast<Ctx*>(ctx)->d_status;
    const int n_blocks = (2 * F + gemm_tile_n() - 1) / gemm_tile_n();
    const int m_blocks = (max_total_rows + gemm_tile_m() - 1) / gemm_tile_m() + (d_counts ? num_segments : 0);
    const long long b_rows = static_cast<long long>(num_weights) * 2 * F;
    auto run = [&]() { return launch_gemm_fp8_nt(d_A, lda, max_total_rows, d_W_interleaved, b_rows, p, m_blocks * n_blocks, st); };
    if (!slot->init) {
        // first use: one pass with scale 0 only records the exact amax, the second pass quantises with it
        // (the sequence of fp8_quant_act's first call, src/trainer.cu:4793-4815, around a producer that is a GEMM)
        CF_CUDA(cudaMemsetAsync(slot->amax, 0, sizeof(float), st));
        CF_CUDA(cudaMemsetAsync(slot->scale, 0, sizeof(float), st));
        CF_TRY(run());
        CF_TRY(cf_fp8_scale_from_amax(slot->amax, slot->fp8_max, slot->scale, slot->descale, stream));
        CF_CUDA(cudaMemcpyAsync(slot->scale_snapshot, slot->scale, sizeof(float), cudaMemcpyDeviceToDevice, st));
        CF_CUDA(cudaMemcpyAsync(slot->descale_snapshot, slot->descale, sizeof(float), cudaMemcpyDeviceToDevice, st));
        CF_CUDA(cudaMemsetAsync(slot->amax, 0, sizeof(float), st));
        CF_TRY(run());
        slot->init = 1;
    } else {
        CF_TRY(slot_begin(slot->scale, slot->descale, slot->scale_snapshot, slot->descale_snapshot, slot->amax, st));
        CF_TRY(run());
    }
    return cf_fp8_update_delayed_scale(slot->amax, slot->fp8_max, slot->scale, slot->descale, slot->history, kHistoryLen,
                                       slot->history_cursor, slot->history_count, stream);
}

int cf_gemm_fp8_swiglu_bf16_rowamax(cf_ctx* ctx, int M, int F, int K, const void* d_A, int lda, int a_is_e5m2,
                                    const float* d_a_descale, const float* d_a_row_descale_or_null,
                                    const void* d_W_interleaved, const float* d_w_descale,
                                    const float* d_w_col_descale_interleaved_or_null, void* d_h, int ldh, float* d_row_amax,
                                    void* stream) {
    CF_REQUIRE(ctx != nullptr, "cf_gemm_fp8_swiglu_bf16_rowamax: null context");
    CF_REQUIRE(M >= 0 && F > 0 && K > 0 && lda >= K && ldh >= F, "cf_gemm_fp8_swiglu_bf16_rowamax: bad shape");
    CF_REQUIRE(F % 32 == 0, "cf_gemm_fp8_swiglu_bf16_rowamax: F must be a multiple of 32 (gate/up rows interleave in groups of 32)");
    if (M == 0) return CF_OK;
    CF_REQUIRE(d_A && d_W_interleaved && d_h && d_row_amax, "cf_gemm_fp8_swiglu_bf16_rowamax: null pointer");
    CF_REQUIRE(d_a_descale || d_a_row_descale_or_null, "cf_gemm_fp8_swiglu_bf16_rowamax: no activation descale");
    CF_REQUIRE(d_w_descale || d_w_col_descale_interleaved_or_null, "cf_gemm_fp8_swiglu_bf16_rowamax: no weight descale");
    GemmParams p;
    p.M = M; p.N = 2 * F; p.K = K;
    p.d_a_descale = d_a_descale ? d_a_descale : d_a_row_descale_or_null;
    p.d_b_descale = d_w_descale ? d_w_descale : d_w_col_descale_interleaved_or_null;
    p.d_a_row_descale = d_a_row_descale_or_null;
    p.d_b_col_descale = d_w_col_descale_interleaved_or_null;
    p.C = d_h; p.ldc = ldh; p.out_kind = 5;
    p.a_e5m2 = a_is_e5m2 ? 1 : 0;
    p.d_row_amax_out = d_row_amax;
    p.d_status = reinterpret_cast<Ctx*>(ctx)->d_status;
    const int tiles = ((M + gemm_tile_m() - 1) / gemm_tile_m()) * ((2 * F + gemm_tile_n() - 1) / gemm_tile_n());
    return launch_gemm_fp8_nt(d_A, lda, M, d_W_interleaved, 2ll * F, p, tiles, as_stream(stream));
}

int cf_refresh_fp8_weight(const cf_fp8_weight* w, int recompute_amax, void* stream) {
    CF_REQUIRE(w && w->w && w->fwd8 && w->bwd8 && w->amax && w->scale && w->descale, "cf_refresh_fp8_weight: null pointer");
    CF_REQUIRE(w->in_dim > 0 && w->out_dim > 0, "cf_refresh_fp8_weight: bad dims");
    const size_t n = static_cast<size_t>(w->in_dim) * w->out_dim;
    if (recompute_amax) CF_TRY(cf_fp8_amax_bf16(w->w, n, w->amax, stream));
    // One launch: the scale is derived from the amax inside the kernel (and published), and one read of the
    // bf16 master produces both layouts (the reference runs scale + two quantise passes: :4700-4709).
    ScaleFromAmax sfa;
    sfa.amax = w->amax; sfa.fp8_max = CF_E4M3_MAX; sfa.scale_out = w->scale; sfa.descale_out = w->descale;
    if (w->stored_out_major)
        return quant_dual_from_amax(w->w, w->fwd8, w->bwd8, sfa, w->out_dim, w->in_dim, as_stream(stream));
    return quant_dual_from_amax(w->w, w->bwd8, w->fwd8, sfa, w->in_dim, w->out_dim, as_stream(stream));
}

int cf_fp8_linear_forward(cf_ctx* ctx, cf_act_slot* slot, const void* d_x, int M, int K, const void* d_w8,
                          const float* d_w_descale, int N, const void* d_bias, int bias_mode, void* d_y, int ldy,
                          void* stream) {
    CF_REQUIRE(ctx && slot, "cf_fp8_linear_forward: null context or slot");
    CF_REQUIRE(M >= 0 && N >= 0 && K > 0, "cf_fp8_linear_forward: bad shape");
    Ctx* c = reinterpret_cast<Ctx*>(ctx);
    const size_t n = static_cast<size_t>(M) * K;
    if (n > c->act8_bytes) {
        set_error("cf_fp8_linear_forward: activation of %zu bytes exceeds the context's act8 scratch (%zu)", n, c->act8_bytes);
        return CF_ERR_LIMIT;
    }
    CF_TRY(cf_fp8_quant_act(ctx, slot, d_x, n, c->act8, stream, 0));
    cf_gemm_epilogue epi;
    std::memset(&epi, 0, sizeof(epi));
    epi.d_bias = d_bias;
    epi.bias_mode = bias_mode;
    return cf_gemm_fp8_nt(ctx, M, N, K, c->act8, K, slot->fp8_max == CF_E5M2_MAX, slot->descale_snapshot, d_w8,
                          d_w_descale, d_y, ldy, &epi, stream);
}

}  // extern "C"
