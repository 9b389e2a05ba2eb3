// Barrier between the ranks of one box, done by the GPUs themselves: every rank stores an epoch number into its word of
// every peer's flag array (plain stores over NVLink into peer-mapped memory) and then waits until all words of its own
// array have reached that epoch. One tiny kernel per rank per barrier, stream-ordered like any other launch, so the
// work enqueued behind it starts as soon as the last peer has arrived: no host round trip, no collective launch. It
// orders the expert-parallel layer's "all rows have arrived" and "all results are back" points, where a library
// all-reduce of one float costs several times the kernel's few microseconds.
//
// The ranks run on different GPUs (one process per GPU), so the kernels that wait on one another are resident at the
// same time by construction. Every wait is bounded: after `limit_ns` the kernel records a status code in the context
// (CF_ERR_DEVICE_WAIT at the next cf_ctx_poll_status) and returns, so a rank that never arrives cannot hang a GPU.
#include "cf_common.cuh"

namespace cf {
int* ctx_status(cf_ctx* c);

namespace {

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// flags[r] = rank r's array of `world` words, as mapped in this process. Thread t talks to peer t.
__global__ void k_peer_barrier(unsigned* const* __restrict__ flags, int world, int rank, unsigned epoch,
                               unsigned long long limit_ns, int* __restrict__ status) {
    const int t = threadIdx.x;
    if (t >= world) return;
    // everything this rank's earlier kernels wrote (also into peers' buffers) is ordered before the announcement
    __threadfence_system();
    st_release_sys(flags[t] + rank, epoch);
    const unsigned* mine = flags[rank] + t;
    const unsigned long long t0 = now_ns();
    unsigned spins = 0;
    while (static_cast<int>(ld_acquire_sys(mine) - epoch) < 0) {
        if ((++spins & 63u) == 0u && now_ns() - t0 > limit_ns) {
            atomicExch(status, 0x600 | 1);
            return;
        }
        __nanosleep(100);
    }
}

// Small all-gather by stores: this rank's n words go to row `rank` of every rank's [world, n] table, followed by the
// barrier above in the same launch, so when the kernel ends every rank's row is in this rank's table.
__global__ void __launch_bounds__(256) k_peer_share(const int* __restrict__ src, int n, int* const* __restrict__ tables,
                                                    unsigned* const* __restrict__ flags, int world, int rank, unsigned epoch,
                                                    unsigned long long limit_ns, int* __restrict__ status) {
    for (int i = threadIdx.x; i < world * n; i += blockDim.x) {
        const int p = i / n, v = i - p * n;
        tables[p][rank * n + v] = src[v];
    }
    __syncthreads();                       // the stores of all threads happen before the announcements below
    const int t = threadIdx.x;
    if (t >= world) return;
    __threadfence_system();
    st_release_sys(flags[t] + rank, epoch);
    const unsigned* mine = flags[rank] + t;
    const unsigned long long t0 = now_ns();
    unsigned spins = 0;
    while (static_cast<int>(ld_acquire_sys(mine) - epoch) < 0) {
        if ((++spins & 63u) == 0u && now_ns() - t0 > limit_ns) {
            atomicExch(status, 0x600 | 2);
            return;
        }
        __nanosleep(100);
    }
}

}  // namespace
}  // namespace cf

using namespace cf;

extern "C" int cf_peer_share_i32(cf_ctx* ctx, const int* d_src, int n, int* const* d_tables, unsigned* const* d_flag_arrays,
                                 int world, int rank, unsigned epoch, int limit_ms, void* stream) {
    CF_REQUIRE(ctx && d_src && d_tables && d_flag_arrays, "cf_peer_share_i32: null pointer");
    CF_REQUIRE(n >= 1 && n <= 4096, "cf_peer_share_i32: 1..4096 words");
    CF_REQUIRE(world >= 1 && world <= 64 && rank >= 0 && rank < world, "cf_peer_share_i32: 1..64 ranks");
    CF_REQUIRE(limit_ms >= 1 && limit_ms <= 60000, "cf_peer_share_i32: limit must be 1..60000 ms");
    const int rc = require_sm100();
    if (rc != CF_OK) return rc;
    k_peer_share<<<1, 256, 0, as_stream(stream)>>>(d_src, n, d_tables, d_flag_arrays, world, rank, epoch,
                                                    static_cast<unsigned long long>(limit_ms) * 1000000ull, ctx_status(ctx));
    CF_LAUNCH_CHECK("peer_share_i32");
    return CF_OK;
}

extern "C" int cf_peer_barrier(cf_ctx* ctx, unsigned* const* d_flag_arrays, int world, int rank, unsigned epoch, int limit_ms,
                               void* stream) {
    CF_REQUIRE(ctx && d_flag_arrays, "cf_peer_barrier: null pointer");
    CF_REQUIRE(world >= 1 && world <= 64 && rank >= 0 && rank < world, "cf_peer_barrier: 1..64 ranks");
    CF_REQUIRE(limit_ms >= 1 && limit_ms <= 60000, "cf_peer_barrier: limit must be 1..60000 ms");
    const int rc = require_sm100();
    if (rc != CF_OK) return rc;
    k_peer_barrier<<<1, 64, 0, as_stream(stream)>>>(d_flag_arrays, world, rank, epoch,
                                                     static_cast<unsigned long long>(limit_ms) * 1000000ull, ctx_status(ctx));
    CF_LAUNCH_CHECK("peer_barrier");
    return CF_OK;
}
