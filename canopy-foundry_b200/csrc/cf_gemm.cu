// FP8 NT GEMM for sm_100a: TMA -> 128B-swizzled shared-memory ring -> tcgen05.mma
// (kind::f8f6f4, fp32 accumulators in TMEM, double-buffered) -> fused dequant / bias epilogue.
//
//   C[m,n] = (dA * dB) * sum_k A8[m,k] * B8[n,k]          (src/trainer.cu:4498-4534)
//
// One persistent CTA per SM, 320 threads:
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocator + MMA issuer (one elected lane)
//   warps 2..9  epilogue: tcgen05.ld the accumulator, scale, bias / SwiGLU, convert, store (two warps per TMEM
//               lane quarter, each draining 128 of the tile's 256 columns)
// The same kernel serves the dense call, the beta=1 weight-gradient forms and the ragged
// per-expert (grouped) schedule: a tile is (expert, 128-row block of that expert, 256-column block).
//
// Every wait on an mbarrier is bounded by a wall-clock deadline; a wait that gives up raises an
// abort flag, records a code in the context's status word, drains the CTA's own copies and MMAs,
// frees TMEM and returns, so a faulty launch cannot hang the GPU.
#include <cuda.h>

#include <mutex>

#include "cf_common.cuh"
#include "cf_gemm.cuh"

namespace cf {
namespace {

constexpr int BM = 128;                 // rows of A / C per CTA (TMEM lanes)
constexpr int BN = 256;                 // output columns per tile
constexpr int BK = 128;                 // bytes == FP8 elements per k-block (one 128B swizzle row)
constexpr int UMMA_K = 32;              // FP8 elements per tcgen05.mma
constexpr int NUM_THREADS = 320;        // warp 0 producer, warp 1 MMA issuer, warps 2..9 epilogue
constexpr int EPI_WARPS = 8;            // two per TMEM lane quarter: each handles 128 of the tile's 256 columns
constexpr int TMEM_COLS = 512;          // two 128x256 fp32 accumulators per CTA
constexpr unsigned long long WAIT_NS = 1500ull * 1000ull * 1000ull;   // per-wait deadline
constexpr unsigned long long DRAIN_NS = 20ull * 1000ull * 1000ull;

// Output staging for the TMA-store epilogue: per epilogue warp one 32-row x 128-byte (64 bf16) box.
constexpr int C_BOX_COLS = 64;
constexpr int C_BOX_BYTES = 32 * C_BOX_COLS * 2;           // 4 KiB
constexpr int C_STAGING = EPI_WARPS * C_BOX_BYTES;         // 32 KiB

// Shape of the shared-memory ring. Single CTA: the CTA loads all 256 rows of the B tile. CTA pair
// (cta_group::2, one 256x256 tile per pair): each CTA loads its own 128 rows of A and HALF of the B tile,
// which halves the L2 -> shared-memory traffic per SM; the smaller stage buys two more stages.
template <bool PAIR>
struct Cfg {
    static constexpr int B_ROWS = PAIR ? 128 : 256;       // rows of B this CTA loads per stage
    static constexpr int STAGES = PAIR ? 6 : 4;
    static constexpr int A_STAGE = BM * BK;               // 16 KiB
    static constexpr int B_STAGE = B_ROWS * BK;           // 16 / 32 KiB
    static constexpr int TILE_M = PAIR ? 256 : 128;       // rows of C per tile (pair: 128 per CTA)
    static constexpr int RING = STAGES * (A_STAGE + B_STAGE);
    static constexpr int SMEM_BYTES = RING + C_STAGING + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ unsigned long long gtime_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait. Returns false when the deadline passed or another role of this CTA aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* s_abort,
                                          unsigned long long limit_ns = WAIT_NS) {
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = gtime_ns();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*s_abort) return false;
        if (gtime_ns() - t0 > limit_ns) return false;
        __nanosleep(64);
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
// The output is written once and not read again by this kernel: evict-first keeps it from pushing the operand
// slabs (which every tile re-reads) out of L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;"
                 ::"l"(map), "r"(src), "r"(x), "r"(y), "l"(policy) : "memory");
}
// fp32 accumulate (beta = 1) as a TMA reduction: the staged tile is added to global memory in L2, one addition per
// element like a read-modify-write epilogue, but with whole 128-byte lines.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Pair form: the arrive is delivered to the barrier at the same offset in both CTAs of the pair.
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `local_addr` in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Pair form of the TMA load: the data lands in this CTA's shared memory, the byte count is credited to a
// barrier that may live in the other CTA of the pair (no multicast: every CTA fetches its own box).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void umma_f8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile in shared memory, rows of 128 bytes, 128B swizzle (what the TMA box writes):
// start address >> 4 in bits [0,14), leading byte offset (unused for swizzled K-major) = 1 in [16,30),
// stride byte offset = 8 rows * 128 B = 1024 B >> 4 in [32,46), descriptor version 1 in [46,48),
// layout type 2 (SWIZZLE_128B) in [61,64).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// kind::f8f6f4 instruction descriptor: D fp32 (bits 4-5 = 1), A format bits 7-9, B format bits 10-12
// (0 = E4M3, 1 = E5M2), both operands K-major (bits 15,16 = 0), N>>3 in bits 17-22, M>>4 in bits 24-28.
// An MN-major operand lies in shared memory with the rows of the tile running along K and 128 contiguous bytes along
// M / N: bit 15 for A, bit 16 for B.
__device__ __forceinline__ uint32_t make_idesc(int a_e5m2, int b_e5m2, int mma_m, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (static_cast<uint32_t>(a_e5m2) << 7) | (static_cast<uint32_t>(b_e5m2) << 10) |
           (a_mn_major ? (1u << 15) : 0u) | (b_mn_major ? (1u << 16) : 0u) |
           (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(mma_m >> 4) << 24);
}


struct TileCoord {
    int row0;        // first global row of A / C for this tile
    int valid_rows;  // rows of the tile that belong to the expert (<= tile rows)
    int n0;          // first output column
    int b_row0;      // first row of the stacked [E*N, K] weight block
    int weight;      // index of the weight block (0 for a dense problem)
    int group;
    void* out_base;  // where this tile's rows are written (p.C, or a per-segment buffer that may live on a peer GPU)
    long long out_row0;  // output row of the tile's first row inside out_base
};

// Maps a linear tile index to coordinates. Dense: one group of p.M rows. Grouped: the m-blocks of
// all experts are concatenated in expert order; counts/offsets are read from device memory.
// The group table of a ragged problem as the tile mapping reads it: a shared-memory copy made once per CTA (the
// mapping walks the counts for every tile, in each of the three roles; from global memory that walk costs the TMA
// producer a chain of L2 round trips at every tile start, long enough to drain its stage ring), or the arrays in
// global memory when there are more groups than the copy holds.
constexpr int kGroupsInSmem = 96;
struct GroupView {
    const int* counts;
    const int* offsets;
    const int* weight;      // null = group index
};
__device__ __forceinline__ int total_m_blocks(const GemmParams& p, const GroupView& gv, int TM) {
    if (p.groups <= 1 && p.d_counts == nullptr) return (p.M + TM - 1) / TM;
    int t = 0;
    for (int e = 0; e < p.groups; ++e) t += (max(gv.counts[e], 0) + TM - 1) / TM;
    return t;
}
__device__ __forceinline__ TileCoord tile_coord(const GemmParams& p, const GroupView& gv, int tile, int m_blocks, int TM) {
    TileCoord c;
    // Band rasterisation: consecutive tile indices walk RASTER_M row blocks down, then one column block
    // right, so the tiles in flight at any time share few A and B slabs (L2 reuse).
    const int n_blocks = (p.N + BN - 1) / BN;
    const int RASTER_M = p.raster_m;
    const int band_tiles = RASTER_M * n_blocks;
    const int band = tile / band_tiles;
    const int first_m = band * RASTER_M;
    const int band_m = min(RASTER_M, m_blocks - first_m);
    const int r = tile - band * band_tiles;
    const int nb = r / band_m;
    int mb = first_m + (r - nb * band_m);
    c.n0 = nb * BN;
    if (p.groups <= 1 && p.d_counts == nullptr) {
        c.group = 0;
        c.weight = 0;
        c.row0 = mb * TM;
        c.valid_rows = min(TM, p.M - c.row0);
        c.b_row0 = c.n0;
        c.out_base = p.C;
        c.out_row0 = c.row0;
        return c;
    }
    int e = 0, cnt = 0;
    for (; e < p.groups; ++e) {
        cnt = max(gv.counts[e], 0);
        const int blocks = (cnt + TM - 1) / TM;
        if (mb < blocks) break;
        mb -= blocks;
    }
    c.group = e;
    c.row0 = gv.offsets[e] + mb * TM;
    c.valid_rows = min(TM, cnt - mb * TM);
    c.weight = gv.weight ? gv.weight[e] : e;
    c.b_row0 = c.weight * p.N + c.n0;
    if (p.d_group_out) {
        c.out_base = p.d_group_out[e];
        c.out_row0 = p.d_group_out_row0[e] + static_cast<long long>(mb) * TM;
    } else {
        c.out_base = p.C;
        c.out_row0 = c.row0;
    }
    return c;
}

// kernels/activations.cu:11-17
__device__ __forceinline__ float swiglu_sigmoid(float x) {
    // Both branches of the reference (1/(1+exp(-x)) for x >= 0, exp(x)/(1+exp(x)) otherwise) share e = exp(-|x|);
    // one IEEE division with the matching numerator gives the same bits without a divergent branch.
    const float e = expf(-fabsf(x));
    return __fdiv_rn(x >= 0.0f ? 1.0f : e, 1.0f + e);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// max(a, |b|) on two packed bf16 values (a holds non-negative values); a NaN in b leaves a unchanged, like fmaxf.
__device__ __forceinline__ uint32_t bf16x2_absmax(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b & 0x7fff7fffu));
    return r;
}
__device__ __forceinline__ uint16_t to_bf16_bits(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }

// One output value through the epilogue contract (used by the scalar store paths and by the SIMT kernel).
__device__ __forceinline__ void store_one(const GemmParams& p, void* cbase, long long grow, int col, float acc, float da, float db) {
    float v = __fmul_rn(acc, da * db);
    if (p.out_kind == 0) {
        uint16_t* c = static_cast<uint16_t*>(cbase) + grow * p.ldc + col;
        if (p.bias && p.bias_mode == 1) v += bf16_bits_to_f32(p.bias[col]);
        uint16_t r = to_bf16_bits(v);
        if (p.bias && p.bias_mode == 2) r = to_bf16_bits(bf16_bits_to_f32(r) + bf16_bits_to_f32(p.bias[col]));
        *c = r;
    } else if (p.out_kind == 1) {
        static_cast<float*>(cbase)[grow * p.ldc + col] = v;
    } else if (p.out_kind == 2) {
        float* c = static_cast<float*>(cbase) + grow * p.ldc + col;
        *c = __fadd_rn(*c, v);                   // the product is rounded before the addition (beta = 1 of a library GEMM)
    } else {
        uint16_t* c = static_cast<uint16_t*>(cbase) + grow * p.ldc + col;
        *c = to_bf16_bits(__fadd_rn(bf16_bits_to_f32(*c), v));
    }
}

// WIDE = true adds the fp32-output and accumulate epilogues (out_kind 1, 2, 3); the bf16-store and SwiGLU forms run the
// WIDE = false instantiation, whose epilogue stays small.
template <bool PAIR, bool WIDE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
k_gemm_fp8_nt(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
              const __grid_constant__ CUtensorMap map_c, const GemmParams p) {
    using C = Cfg<PAIR>;
    constexpr int STAGES = C::STAGES, A_STAGE = C::A_STAGE, B_STAGE = C::B_STAGE, TM = C::TILE_M;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;           // swizzle atoms need 1024-byte alignment
    const uint32_t smem_a = base;
    const uint32_t smem_b = base + STAGES * A_STAGE;
    const uint32_t smem_c = smem_b + STAGES * B_STAGE;       // output staging (1024-byte aligned)
    const uint32_t bars = smem_c + C_STAGING;                // 8-byte mbarriers
    const uint32_t full_bar = bars, empty_bar = bars + 8 * STAGES;
    const uint32_t tfull_bar = bars + 16 * STAGES, tempty_bar = tfull_bar + 16, drain_bar = tempty_bar + 16;
    uint8_t* gen = smem_raw + (base - raw);
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(gen + C::RING + C_STAGING + 16 * STAGES + 48);
    volatile int* s_abort = reinterpret_cast<volatile int*>(const_cast<uint32_t*>(s_tmem) + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;       // 0 = leader of the pair
    const bool leader = cta_rank == 0;
    const int unit = PAIR ? (blockIdx.x >> 1) : blockIdx.x;        // persistent scheduling unit (CTA or pair)
    const int n_units = PAIR ? (gridDim.x >> 1) : gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);                  // one arrive.expect_tx by the (leader's) producer
            mbar_init(empty_bar + 8 * s, 1);                 // one tcgen05.commit
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar + 8 * a, 1);                 // one tcgen05.commit
            mbar_init(tempty_bar + 8 * a, PAIR ? 2 * EPI_WARPS : EPI_WARPS);   // one arrive per epilogue warp (of both CTAs)
        }
        mbar_init(drain_bar, 1);
        s_abort[0] = 0;
        s_abort[1] = 0;                                      // stays 0: abort source for the drain waits
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
        if (p.tma_store || (p.tma_reduce && p.d_peer_maps == nullptr)) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c) : "memory");
    }
    if (warp == 1) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t*>(s_tmem))), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t*>(s_tmem))), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();                            // peer barriers are initialised before any remote signal
    tcgen05_fence_after();
    const uint32_t tmem_base = *s_tmem;
    // Everything above touched only this CTA's shared memory, TMEM and kernel parameters; from here on the kernel
    // reads what earlier kernels of the stream wrote (operands, scales, counts).
    pdl_wait();

    __shared__ int s_groups[3 * kGroupsInSmem];
    GroupView gv = {p.d_counts, p.d_offsets, p.d_group_weight};
    if (p.d_counts != nullptr && p.groups <= kGroupsInSmem) {          // kernel-uniform
        for (int e = threadIdx.x; e < p.groups; e += NUM_THREADS) {
            s_groups[e] = p.d_counts[e];
            s_groups[kGroupsInSmem + e] = p.d_offsets[e];
            if (p.d_group_weight) s_groups[2 * kGroupsInSmem + e] = p.d_group_weight[e];
        }
        __syncthreads();
        gv.counts = s_groups;
        gv.offsets = s_groups + kGroupsInSmem;
        gv.weight = p.d_group_weight ? s_groups + 2 * kGroupsInSmem : nullptr;
    }
    const int m_blocks = total_m_blocks(p, gv, TM);
    const int n_blocks = (p.N + BN - 1) / BN;
    const int total_tiles = m_blocks * n_blocks;
    const int k_iters = (p.K + BK - 1) / BK;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs of a pair)
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            // the byte count of a stage is credited to the leader's barrier
            const uint32_t full_dst = PAIR ? mapa(full_bar, 0) : full_bar;
            for (int tile = unit; ok && tile < total_tiles; tile += n_units) {
                const TileCoord tc = tile_coord(p, gv, tile, m_blocks, TM);
                const int a_row = tc.row0 + static_cast<int>(cta_rank) * BM;
                const int b_row = tc.b_row0 + static_cast<int>(cta_rank) * C::B_ROWS;
                for (int kb = 0; kb < k_iters; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(empty_bar + 8 * s, ph ^ 1, s_abort)) { ok = false; break; }
                    if (PAIR) {
                        if (leader) mbar_expect_tx(full_bar + 8 * s, 2 * (A_STAGE + B_STAGE));
                        // K-major operands: x runs along K; MN-major operands ([K, M] / [K, N] in memory): x runs
                        // along M / N and the box rows are K
                        const bool mn = WIDE && p.mn_major;
                        const bool bmn = WIDE && (p.mn_major || p.b_mn_major);
                        const int ax = mn ? a_row : kb * BK, ay = mn ? kb * BK : a_row;
                        // MN-major B: the weight block lies as [K, N] (stacked blocks: [weights * K, N]); this CTA's half
                        // of the tile's columns is one 128-byte box row, the box rows run along K
                        const int bx = bmn ? tc.n0 + static_cast<int>(cta_rank) * C::B_ROWS : kb * BK;
                        const int by = bmn ? tc.weight * p.K + kb * BK : b_row;
                        tma_load_2d_pair(smem_a + s * A_STAGE, &map_a, full_dst + 8 * s, ax, ay);
                        tma_load_2d_pair(smem_b + s * B_STAGE, &map_b, full_dst + 8 * s, bx, by);
                    } else {
                        mbar_expect_tx(full_bar + 8 * s, A_STAGE + B_STAGE);
                        tma_load_2d(smem_a + s * A_STAGE, &map_a, full_bar + 8 * s, kb * BK, a_row);
                        tma_load_2d(smem_b + s * B_STAGE, &map_b, full_bar + 8 * s, kb * BK, b_row);
                    }
                }
            }
            if (!ok && !*s_abort) { *s_abort = 1; atomicExch(p.d_status, 0x100 | 1); }
            if ((*s_abort || !ok) && leader) {
                // wait (bounded) for the copies still in flight into this stage ring (for a pair the leader's
                // barriers also count the peer's copies; the peer meets the leader at the closing cluster barrier)
                for (int j = max(0, it - STAGES); j < it; ++j)
                    mbar_wait(full_bar + 8 * (j % STAGES), (j / STAGES) & 1, s_abort + 1 /*never set*/, DRAIN_NS);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            const bool mn = WIDE && p.mn_major;
            const bool bmn = WIDE && (p.mn_major || p.b_mn_major);
            const uint32_t idesc = make_idesc(p.a_e5m2, p.b_e5m2, TM, mn, bmn);
            int it = 0, local_tile = 0;
            bool ok = true;
            for (int tile = unit; ok && tile < total_tiles; tile += n_units, ++local_tile) {
                const int acc = local_tile & 1;
                if (!mbar_wait(tempty_bar + 8 * acc, ((local_tile >> 1) & 1) ^ 1, s_abort)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (int kb = 0; kb < k_iters; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(full_bar + 8 * s, (it / STAGES) & 1, s_abort)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint64_t adesc = make_smem_desc(smem_a + s * A_STAGE);
                    const uint64_t bdesc = make_smem_desc(smem_b + s * B_STAGE);
                    // One MMA covers 32 elements of K. K-major operand: 32 bytes further inside the 128B swizzle atom = +2
                    // in the descriptor's (address >> 4) field; MN-major operand: 32 rows of 128 bytes further = +256.
                    const uint32_t a_step = (WIDE && mn) ? 256u : 2u, b_step = (WIDE && bmn) ? 256u : 2u;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        if (PAIR) umma_f8_pair(tmem_d, adesc + a_step * kk, bdesc + b_step * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
                        else umma_f8(tmem_d, adesc + a_step * kk, bdesc + b_step * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
                    }
                    // frees the stage (in both CTAs of a pair) once these MMAs have read it
                    if (PAIR) tcgen05_commit_pair(empty_bar + 8 * s); else tcgen05_commit(empty_bar + 8 * s);
                }
                if (!ok) break;
                if (PAIR) tcgen05_commit_pair(tfull_bar + 8 * acc); else tcgen05_commit(tfull_bar + 8 * acc);
            }
            if (!ok && !*s_abort) { *s_abort = 1; atomicExch(p.d_status, 0x200 | 1); }
            if (*s_abort || !ok) {
                // all MMAs issued so far
                if (PAIR) asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(drain_bar) : "memory");
                else tcgen05_commit(drain_bar);
                mbar_wait(drain_bar, 0, s_abort + 1, DRAIN_NS);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps (both CTAs of a pair)
        const int quarter = warp & 3;                      // TMEM lanes this warp may read
        const int col_half = (warp - 2) >> 2;              // which 128 columns of the tile this warp drains
        const int trow = quarter * 32 + lane;
        const uint32_t tempty_dst = PAIR ? mapa(tempty_bar, 0) : tempty_bar;
        int local_tile = 0;
        const uint64_t store_policy = l2_policy_evict_first();
        bool ok = true;
        for (int tile = unit; ok && tile < total_tiles; tile += n_units, ++local_tile) {
            const int acc = local_tile & 1;
            const TileCoord tc = tile_coord(p, gv, tile, m_blocks, TM);
            if (!mbar_wait(tfull_bar + 8 * acc, (local_tile >> 1) & 1, s_abort)) { ok = false; break; }
            tcgen05_fence_after();
            const int row_in_tile = static_cast<int>(cta_rank) * BM + trow;
            const long long grow = tc.out_row0 + row_in_tile;             // output row
            const bool row_ok = row_in_tile < tc.valid_rows;
            float da = 1.0f;
            if (row_ok) {
                if (p.d_a_row_descale) da = p.d_a_row_descale[static_cast<long long>(tc.row0) + row_in_tile];
                else da = p.d_a_descale[p.a_descale_per_group ? tc.group : 0];
            }
            const float db_t = p.d_b_col_descale ? 1.0f : *p.d_b_descale;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
            if (p.out_kind == 4) {
                // SwiGLU -> E4M3 epilogue. B's rows are interleaved in groups of 64 = 32 gate rows followed by the 32 up
                // rows of the same features, so chunk 2c holds gate and chunk 2c+1 holds up for features
                // n0/2 + 32c .. +31. Rounding points are those of the unfused sequence: GEMM output to bf16
                // (src/trainer.cu:6310-6313), silu(g)*u to bf16 (kernels/activations.cu:39), then the record-quantise
                // of kernels/fp8.cu:67-84 with the slot's scale; the amax of the bf16 product goes to p.d_amax_out.
                const float hs = *p.d_quant_scale;
                const float dab = da * db_t;
                uint32_t amax2 = 0u;                       // two running maxima of |h| as bf16
                uint8_t* orow = static_cast<uint8_t*>(tc.out_base) + grow * p.ldc + (tc.n0 >> 1);
                // Every lane stores the 32 codes of a chunk as two 16-byte words (one whole sector of its row); staging the
                // warp's rows for a TMA store, as the bf16 form below does, measured no faster here.
#pragma unroll 1
                for (int c = col_half * 2; c < col_half * 2 + 2; ++c) {
                    const int col0 = tc.n0 + c * 64;
                    if (col0 >= p.N) break;                // warp-uniform
                    uint32_t vg[32], vu[32];
                    tmem_ld32(taddr + c * 64, vg);
                    tmem_ld32(taddr + c * 64 + 32, vu);
                    tmem_ld_wait();
                    if (!row_ok) continue;
                    uint32_t q[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float h[4];
#pragma unroll
                        for (int e = 0; e < 4; e += 2) {
                            // every bf16 rounding of the unfused sequence is done on a pair (cvt.rn.bf16x2); the amax is
                            // taken on the packed product
                            const uint32_t g2 = pack_bf16x2(__uint_as_float(vg[4 * j + e]) * dab, __uint_as_float(vg[4 * j + e + 1]) * dab);
                            const uint32_t u2 = pack_bf16x2(__uint_as_float(vu[4 * j + e]) * dab, __uint_as_float(vu[4 * j + e + 1]) * dab);
                            const float g0 = __uint_as_float(g2 << 16), g1 = __uint_as_float(g2 & 0xffff0000u);
                            const uint32_t h2 = pack_bf16x2(g0 * swiglu_sigmoid(g0) * __uint_as_float(u2 << 16),
                                                            g1 * swiglu_sigmoid(g1) * __uint_as_float(u2 & 0xffff0000u));
                            amax2 = bf16x2_absmax(amax2, h2);
                            h[e] = __uint_as_float(h2 << 16);
                            h[e + 1] = __uint_as_float(h2 & 0xffff0000u);
                        }
                        q[j] = cvt_fp8x4<false>(h[0] * hs, h[1] * hs, h[2] * hs, h[3] * hs);
                    }
                    uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
                    dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
                    dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
                }
                float local_amax = fmaxf(__uint_as_float(amax2 << 16), __uint_as_float(amax2 & 0xffff0000u));
                local_amax = warp_max(local_amax);
                if (lane == 0 && local_amax > 0.0f) atomicMax(reinterpret_cast<int*>(p.d_amax_out), __float_as_int(local_amax));
            } else if (p.out_kind == 5) {
                // SwiGLU -> bf16 epilogue with a per-row amax, for per-token re-quantisation: same interleaved weight layout
                // and rounding points as above (GEMM output to bf16 with the row's and the column's descale, silu(g)*u to
                // bf16), but the product is stored as bf16 [., N/2] and max|h| of every row is accumulated into
                // p.d_row_amax_out (integer atomicMax on the float bits; the caller zeroes it). The row-wise quantiser
                // then reads h once: the [., N] gate/up intermediate never reaches HBM.
                // The warp's 32 rows x 64 features (its two chunks) leave as ONE box of whole 128-byte lines through the
                // staging buffer and a TMA store (rows and features outside the tensor are clipped by the tensor map).
                // Four 16-byte stores from every lane to its own row measured 5 % slower on the 16384 x 28672 x 4096
                // gate/up GEMM (tensor pipe 82 % busy against 86 %) at unchanged DRAM traffic: fewer store
                // instructions and L2 write requests per tile, not fewer bytes.
                uint32_t amax2 = 0u;                       // two running maxima of |h| as bf16
                const uint32_t buf = smem_c + static_cast<uint32_t>(warp - 2) * C_BOX_BYTES;
                const uint32_t row_off = static_cast<uint32_t>(lane) * 128u;
                const uint32_t sw = static_cast<uint32_t>(lane & 7);
                if (lane == 0) bulk_wait_read_0();         // the store that last read this warp's box has drained it
                __syncwarp();
                bool any = false;
#pragma unroll 1
                for (int c = col_half * 2; c < col_half * 2 + 2; ++c) {
                    const int col0 = tc.n0 + c * 64;
                    if (col0 >= p.N) break;                // warp-uniform
                    any = true;
                    uint32_t vg[32], vu[32];
                    tmem_ld32(taddr + c * 64, vg);
                    tmem_ld32(taddr + c * 64 + 32, vu);
                    tmem_ld_wait();
                    uint32_t w[16];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float4 cg = make_float4(db_t, db_t, db_t, db_t), cu = cg;
                        if (p.d_b_col_descale) {
                            cg = __ldg(reinterpret_cast<const float4*>(p.d_b_col_descale + col0) + j);
                            cu = __ldg(reinterpret_cast<const float4*>(p.d_b_col_descale + col0 + 32) + j);
                        }
                        const float sg[4] = {cg.x, cg.y, cg.z, cg.w}, su[4] = {cu.x, cu.y, cu.z, cu.w};
                        float h[4];
#pragma unroll
                        for (int e = 0; e < 4; e += 2) {
                            // gate and up as the bf16 values the unfused GEMM would have stored: rounded two at a time
                            const uint32_t g2 = pack_bf16x2(__uint_as_float(vg[4 * j + e]) * (da * sg[e]),
                                                            __uint_as_float(vg[4 * j + e + 1]) * (da * sg[e + 1]));
                            const uint32_t u2 = pack_bf16x2(__uint_as_float(vu[4 * j + e]) * (da * su[e]),
                                                            __uint_as_float(vu[4 * j + e + 1]) * (da * su[e + 1]));
                            const float g0 = __uint_as_float(g2 << 16), g1 = __uint_as_float(g2 & 0xffff0000u);
                            h[e] = g0 * swiglu_sigmoid(g0) * __uint_as_float(u2 << 16);
                            h[e + 1] = g1 * swiglu_sigmoid(g1) * __uint_as_float(u2 & 0xffff0000u);
                        }
                        // the pack is the bf16 rounding of the product; the row amax is taken on the packed pairs
                        // (max of |bf16| values, NaN ignored like fmaxf: committed for rows of the matrix only)
                        w[2 * j] = pack_bf16x2(h[0], h[1]);
                        w[2 * j + 1] = pack_bf16x2(h[2], h[3]);
                        amax2 = bf16x2_absmax(amax2, w[2 * j]);
                        amax2 = bf16x2_absmax(amax2, w[2 * j + 1]);
                    }
                    const uint32_t half = static_cast<uint32_t>(c & 1) * 4u;       // which 64 bytes of the 128-byte box row
#pragma unroll
                    for (uint32_t q = 0; q < 4; ++q)       // 16-byte chunk q of this row sits at (q ^ row % 8): 128B swizzle
                        st_shared_v4(buf + row_off + (((half + q) ^ sw) << 4), w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
                }
                if (any) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&map_c, buf, (tc.n0 >> 1) + col_half * C_BOX_COLS,
                                     tc.row0 + static_cast<int>(cta_rank) * BM + quarter * 32, store_policy);
                        bulk_commit();
                    }
                }
                const float local_amax = fmaxf(__uint_as_float(amax2 << 16), __uint_as_float(amax2 & 0xffff0000u));
                if (row_ok && local_amax > 0.0f)
                    atomicMax(reinterpret_cast<int*>(p.d_row_amax_out + static_cast<long long>(tc.row0) + row_in_tile),
                              __float_as_int(local_amax));
            } else {
            // Full boxes of bf16 output go through shared memory and TMA stores (whole 128-byte lines per row);
            // ragged rows of a grouped tile, column tails and the fp32 / accumulate forms use direct stores.
            const int warp_row0 = static_cast<int>(cta_rank) * BM + quarter * 32;
            const bool warp_rows_full = (p.d_counts == nullptr) || (warp_row0 + 32 <= tc.valid_rows);
            // Where this lane's row and this warp's 32-row box go. Normally the tile's own output; in the return form
            // every run of rows inside the group has its own destination buffer (possibly on a peer GPU).
            const CUtensorMap* cmap = &map_c;
            int ystore = tc.row0 + warp_row0;
            void* out_base_l = tc.out_base;
            long long grow_l = grow;
            bool box_tma = p.tma_store && warp_rows_full && warp_row0 < tc.valid_rows;
            if (WIDE && p.d_out_runs != nullptr) {
                const cf_row_run* runs = p.d_out_runs + static_cast<long long>(tc.group) * p.runs_per_group;
                const long long r_l = static_cast<long long>(tc.row0) + row_in_tile;
                int s_l = 0;
                for (int s = 1; s < p.runs_per_group; ++s)
                    if (r_l >= runs[s].src_row) s_l = s;          // runs ascend; empty ones share their successor's start
                out_base_l = p.d_peer_bases[runs[s_l].dst];
                grow_l = runs[s_l].dst_row + (r_l - runs[s_l].src_row);
                const int s_first = __shfl_sync(0xffffffffu, s_l, 0), s_last = __shfl_sync(0xffffffffu, s_l, 31);
                box_tma = box_tma && s_first == s_last;           // the whole box belongs to one run
                cmap = static_cast<const CUtensorMap*>(p.d_peer_maps) + runs[s_first].dst;
                ystore = static_cast<int>(runs[s_first].dst_row + (tc.row0 + warp_row0 - runs[s_first].src_row));
            }
            if (WIDE && p.tma_reduce && warp_rows_full && warp_row0 < tc.valid_rows) {
                // fp32 output, added (dW += ...) or stored (partial products): 32 columns = one 128-byte line per box row
                const uint32_t buf = smem_c + static_cast<uint32_t>(warp - 2) * C_BOX_BYTES;
                const uint32_t row_off = static_cast<uint32_t>(lane) * 128u;
                const uint32_t sw = static_cast<uint32_t>(lane & 7);
                const float dab = da * db_t;
                int ch = col_half * 4;
#pragma unroll 1
                for (; ch < col_half * 4 + 4; ++ch) {
                    const int col0 = tc.n0 + ch * 32;
                    if (col0 + 32 > p.N) break;            // warp-uniform; the tail takes the direct path below
                    uint32_t v[32];
                    tmem_ld32(taddr + ch * 32, v);
                    tmem_ld_wait();
                    if (lane == 0) bulk_wait_read_0();
                    __syncwarp();
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        float4 m4 = make_float4(dab, dab, dab, dab);
                        if (p.d_b_col_descale) {       // the same address in every lane: one broadcast load per four columns
                            const float4 cq = __ldg(reinterpret_cast<const float4*>(p.d_b_col_descale + col0) + q);
                            m4 = make_float4(da * cq.x, da * cq.y, da * cq.z, da * cq.w);
                        }
                        st_shared_v4(buf + row_off + ((static_cast<uint32_t>(q) ^ sw) << 4),
                                     __float_as_uint(__uint_as_float(v[4 * q]) * m4.x), __float_as_uint(__uint_as_float(v[4 * q + 1]) * m4.y),
                                     __float_as_uint(__uint_as_float(v[4 * q + 2]) * m4.z), __float_as_uint(__uint_as_float(v[4 * q + 3]) * m4.w));
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        if (p.tma_reduce == 2) {
                            tma_store_2d(&map_c, buf, col0, tc.row0 + warp_row0, store_policy);
                        } else if (p.d_peer_maps != nullptr) {
                            // reduce-scatter: the slice that owns these rows, wherever it lives (NVLink for a peer's)
                            const int grow0 = tc.row0 + warp_row0;
                            const int owner = grow0 / p.rows_per_peer;
                            tma_reduce_add_2d(static_cast<const CUtensorMap*>(p.d_peer_maps) + owner, buf, col0,
                                              grow0 - owner * p.rows_per_peer);
                        } else {
                            tma_reduce_add_2d(&map_c, buf, col0, tc.row0 + warp_row0);
                        }
                        bulk_commit();
                    }
                }
                for (; ch < col_half * 4 + 4; ++ch) {      // column tail: direct read-modify-write
                    const int col0 = tc.n0 + ch * 32;
                    if (col0 >= p.N) break;
                    uint32_t v[32];
                    tmem_ld32(taddr + ch * 32, v);
                    tmem_ld_wait();
                    if (!row_ok) continue;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (col0 + j < p.N)
                            store_one(p, tc.out_base, grow, col0 + j, __uint_as_float(v[j]), da,
                                      p.d_b_col_descale ? p.d_b_col_descale[col0 + j] : db_t);
                }
            } else if (box_tma) {
                const uint32_t buf = smem_c + static_cast<uint32_t>(warp - 2) * C_BOX_BYTES;
                const uint32_t row_off = static_cast<uint32_t>(lane) * 128u;
                const uint32_t sw = static_cast<uint32_t>(lane & 7);
                int ch64 = col_half * 2;
#pragma unroll 1
                for (; ch64 < col_half * 2 + 2; ++ch64) {
                    const int col0 = tc.n0 + ch64 * C_BOX_COLS;
                    if (col0 + C_BOX_COLS > p.N) break;    // warp-uniform; the tail takes the direct path below
                    if (lane == 0) bulk_wait_read_0();     // the store that last read this warp's box has drained it
                    __syncwarp();
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const int col = col0 + half * 32;
                        // bias and per-column scales of these 32 columns: a few 16-byte loads of addresses that are
                        // the same in every lane (L1 broadcast), issued before the accumulator read-out
                        uint4 bq[4];
                        float4 cq[8];
                        if (p.bias_mode != 0) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) bq[q] = __ldg(reinterpret_cast<const uint4*>(p.bias + col) + q);
                        }
                        if (p.d_b_col_descale) {
#pragma unroll
                            for (int q = 0; q < 8; ++q) cq[q] = __ldg(reinterpret_cast<const float4*>(p.d_b_col_descale + col) + q);
                        }
                        uint32_t v[32];
                        tmem_ld32(taddr + ch64 * C_BOX_COLS + half * 32, v);
                        tmem_ld_wait();
                        uint32_t w[16];
                        const float dab = da * db_t;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            float x0 = __uint_as_float(v[2 * j]), x1 = __uint_as_float(v[2 * j + 1]);
                            if (p.d_b_col_descale) {
                                const float4 c4 = cq[j >> 1];
                                x0 *= da * ((j & 1) ? c4.z : c4.x);
                                x1 *= da * ((j & 1) ? c4.w : c4.y);
                            } else {
                                x0 *= dab;
                                x1 *= dab;
                            }
                            if (p.bias_mode != 0) {
                                const uint4 b4 = bq[j >> 2];
                                const uint32_t bb = (j & 3) == 0 ? b4.x : (j & 3) == 1 ? b4.y : (j & 3) == 2 ? b4.z : b4.w;
                                const float b0 = __uint_as_float(bb << 16), b1 = __uint_as_float(bb & 0xffff0000u);
                                if (p.bias_mode == 1) {
                                    w[j] = pack_bf16x2(x0 + b0, x1 + b1);
                                } else {
                                    const uint32_t r = pack_bf16x2(x0, x1);
                                    w[j] = pack_bf16x2(__uint_as_float(r << 16) + b0, __uint_as_float(r & 0xffff0000u) + b1);
                                }
                            } else {
                                w[j] = pack_bf16x2(x0, x1);
                            }
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q)        // 16-byte chunk c of this row sits at (c ^ row%8): 128B swizzle
                            st_shared_v4(buf + row_off + ((static_cast<uint32_t>(half * 4 + q) ^ sw) << 4), w[4 * q],
                                         w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(cmap, buf, col0, ystore, store_policy);
                        bulk_commit();
                    }
                }
                // column tail (N not a multiple of 64): direct stores
                for (int ch = ch64 * 2; ch < col_half * 4 + 4; ++ch) {
                    const int col0 = tc.n0 + ch * 32;
                    if (col0 >= p.N) break;
                    uint32_t v[32];
                    tmem_ld32(taddr + ch * 32, v);
                    tmem_ld_wait();
                    if (!row_ok) continue;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int col = col0 + j;
                        if (col < p.N) {
                            const float db = p.d_b_col_descale ? p.d_b_col_descale[col] : db_t;
                            store_one(p, out_base_l, grow_l, col, __uint_as_float(v[j]), da, db);
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int ch = col_half * 4; ch < col_half * 4 + 4; ++ch) {
                    const int col0 = tc.n0 + ch * 32;
                    if (col0 >= p.N) break;                    // warp-uniform
                    uint32_t v[32];
                    tmem_ld32(taddr + ch * 32, v);
                    tmem_ld_wait();
                    if (!row_ok) continue;
                    const bool full = col0 + 32 <= p.N;
                    if (p.out_kind == 0 && p.c_vec && full) {
                        uint16_t* crow = static_cast<uint16_t*>(out_base_l) + grow_l * p.ldc + col0;
                        uint32_t w[16];
    #pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            float x0 = __uint_as_float(v[2 * j]), x1 = __uint_as_float(v[2 * j + 1]);
                            const float db0 = p.d_b_col_descale ? p.d_b_col_descale[col0 + 2 * j] : db_t;
                            const float db1 = p.d_b_col_descale ? p.d_b_col_descale[col0 + 2 * j + 1] : db_t;
                            x0 *= da * db0;
                            x1 *= da * db1;
                            if (p.bias_mode == 1) {
                                const uint32_t bb = *reinterpret_cast<const uint32_t*>(p.bias + col0 + 2 * j);
                                x0 += __uint_as_float(bb << 16);
                                x1 += __uint_as_float(bb & 0xffff0000u);
                                w[j] = pack_bf16x2(x0, x1);
                            } else if (p.bias_mode == 2) {
                                const uint32_t bb = *reinterpret_cast<const uint32_t*>(p.bias + col0 + 2 * j);
                                const uint32_t r = pack_bf16x2(x0, x1);
                                w[j] = pack_bf16x2(__uint_as_float(r << 16) + __uint_as_float(bb << 16),
                                                   __uint_as_float(r & 0xffff0000u) + __uint_as_float(bb & 0xffff0000u));
                            } else {
                                w[j] = pack_bf16x2(x0, x1);
                            }
                        }
                        uint4* dst = reinterpret_cast<uint4*>(crow);
    #pragma unroll
                        for (int q = 0; q < 4; ++q) dst[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
                    } else if (WIDE && p.out_kind == 3 && p.c_vec && full && !p.d_b_col_descale) {
                        // bf16 accumulate: 64 bytes of the row in, one fp32 addition and one rounding per element, 64 bytes out
                        uint4* crow = reinterpret_cast<uint4*>(static_cast<uint16_t*>(tc.out_base) + grow * p.ldc + col0);
                        const float dab = da * db_t;
                        uint4 old4[4];
    #pragma unroll
                        for (int q = 0; q < 4; ++q) old4[q] = crow[q];
    #pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint32_t o[4] = {old4[q].x, old4[q].y, old4[q].z, old4[q].w};
                            uint32_t w4[4];
    #pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                const int j = 8 * q + 2 * t;
                                w4[t] = pack_bf16x2(__fadd_rn(__uint_as_float(o[t] << 16), __fmul_rn(__uint_as_float(v[j]), dab)),
                                                    __fadd_rn(__uint_as_float(o[t] & 0xffff0000u), __fmul_rn(__uint_as_float(v[j + 1]), dab)));
                            }
                            crow[q] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                        }
                    } else {
    #pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int col = col0 + j;
                            if (col < p.N) {
                                const float db = p.d_b_col_descale ? p.d_b_col_descale[col] : db_t;
                                store_one(p, out_base_l, grow_l, col, __uint_as_float(v[j]), da, db);
                            }
                        }
                    }
                }
    }
            }   // out_kind != 4
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(tempty_dst + 8 * acc); else mbar_arrive(tempty_bar + 8 * acc);
            }
        }
        if (lane == 0) bulk_wait_all();                    // this warp's TMA stores have completed
        if (!ok && lane == 0 && !*s_abort) { *s_abort = 1; atomicExch(p.d_status, 0x300 | 1); }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();          // the peer may still read this CTA's operands / signal its barriers
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after();
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ bounded-wait self-test
// Exercises the failure path of the waits above without any fault: one CTA arms nothing and waits on an
// mbarrier that nobody signals; the wait gives up after `limit_ns`, the kernel records the same status code a
// starved producer would and returns normally. The host then sees CF_ERR_DEVICE_WAIT from cf_ctx_poll_status.
__global__ void k_wait_selftest(int* d_status, unsigned long long limit_ns) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int s_abort[2];
    if (threadIdx.x == 0) {
        s_abort[0] = s_abort[1] = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!mbar_wait(smem_u32(&bar), 0, s_abort, limit_ns)) atomicExch(d_status, 0x400 | 1);
    }
    __syncthreads();
}

// ------------------------------------------------------------------ SIMT form
// Serves shapes the TMA path cannot address (K or lda not a multiple of 16, operands not 16-byte
// aligned) with identical epilogue semantics. One thread per output element; correctness path only.
__global__ void __launch_bounds__(256) k_gemm_fp8_nt_simt(const uint8_t* __restrict__ A, long long lda,
                                                          const uint8_t* __restrict__ B, const GemmParams p) {
    const int groups = (p.d_counts == nullptr) ? 1 : p.groups;
    for (int g = 0; g < groups; ++g) {
        const int rows = p.d_counts ? max(p.d_counts[g], 0) : p.M;
        const long long row_base = p.d_counts ? p.d_offsets[g] : 0;
        const long long total = static_cast<long long>(rows) * p.N;
        for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
             idx += static_cast<long long>(gridDim.x) * blockDim.x) {
            const long long m = idx / p.N;
            const int n = static_cast<int>(idx - m * p.N);
            const uint8_t* a = A + (row_base + m) * lda;
            const uint8_t* b = B + (static_cast<long long>(p.d_group_weight ? p.d_group_weight[g] : g) * p.N + n) * p.K;
            float acc = 0.0f;
            for (int k = 0; k < p.K; ++k) {
                const float av = p.a_e5m2 ? fp8_to_f32<true>(a[k]) : fp8_to_f32<false>(a[k]);
                const float bv = p.b_e5m2 ? fp8_to_f32<true>(b[k]) : fp8_to_f32<false>(b[k]);
                acc = fmaf(av, bv, acc);
            }
            const long long grow = row_base + m;
            const float da = p.d_a_row_descale ? p.d_a_row_descale[grow] : p.d_a_descale[p.a_descale_per_group ? g : 0];
            const float db = p.d_b_col_descale ? p.d_b_col_descale[n] : *p.d_b_descale;
            if (p.d_group_out) store_one(p, p.d_group_out[g], p.d_group_out_row0[g] + m, n, acc, da, db);
            else store_one(p, p.C, grow, n, acc, da, db);
        }
    }
}

// ------------------------------------------------------------------ host side
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// 2-D byte tensor [rows, K] with row pitch `pitch`, box {BK, box_rows}, 128B swizzle, zero fill out of bounds.
int make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, long long pitch, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled entry point not available"); return CF_ERR_CUDA; }
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r)); return CF_ERR_CUDA; }
    return CF_OK;
}

// Number of CTA pairs the device can keep resident at once (cached per device); 0 = pairs unusable.
int max_resident_pairs() {
    static int cached[64];
    static std::once_flag once[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    std::call_once(once[dev & 63], [&] {
        int n = 0;
        if (cudaFuncSetAttribute(k_gemm_fp8_nt<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<true>::SMEM_BYTES) == cudaSuccess &&
            cudaFuncSetAttribute(k_gemm_fp8_nt<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<true>::SMEM_BYTES) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2 * sm_count());
            cfg.blockDim = dim3(NUM_THREADS);
            cfg.dynamicSmemBytes = Cfg<true>::SMEM_BYTES;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
            cfg.attrs = at;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n, k_gemm_fp8_nt<true, true>, &cfg) != cudaSuccess) n = 0;
        }
        (void)cudaGetLastError();
        cached[dev & 63] = n;
    });
    return cached[dev & 63];
}

// bf16 output tensor [rows, N] with row pitch ldc elements, box {64 columns, 32 rows}, 128B swizzle.
int make_map_c(CUtensorMap* map, const void* ptr, long long rows, long long N, long long ldc) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled entry point not available"); return CF_ERR_CUDA; }
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldc) * 2};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(C_BOX_COLS), 32};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (output) failed with CUresult %d", static_cast<int>(r)); return CF_ERR_CUDA; }
    return CF_OK;
}

// fp32 accumulator tensor [rows, N] with row pitch ldc elements, box {32 columns, 32 rows}, 128B swizzle.
int make_map_c_f32(CUtensorMap* map, const void* ptr, long long rows, long long N, long long ldc) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled entry point not available"); return CF_ERR_CUDA; }
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldc) * 4};
    const cuuint32_t box[2] = {32, 32};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (fp32 output) failed with CUresult %d", static_cast<int>(r)); return CF_ERR_CUDA; }
    return CF_OK;
}

}  // namespace

int launch_gemm_fp8_nt(const void* d_A, long long lda, long long a_rows, const void* d_B, long long b_rows,
                       GemmParams p, int tile_upper_bound, cudaStream_t st) {
    if (p.N <= 0 || p.K <= 0 || tile_upper_bound <= 0) return CF_OK;
    const int rc = require_sm100();
    if (rc != CF_OK) return rc;
    const uintptr_t aa = reinterpret_cast<uintptr_t>(d_A), ba = reinterpret_cast<uintptr_t>(d_B);
    const bool tma_ok = p.mn_major ? ((aa % 16 == 0) && (ba % 16 == 0) && (lda % 16 == 0) && (p.ldb % 16 == 0))
                      : p.b_mn_major ? ((aa % 16 == 0) && (ba % 16 == 0) && (lda % 16 == 0) && (p.K % 16 == 0) && (p.ldb % 16 == 0) && (p.N % 16 == 0))
                                     : ((aa % 16 == 0) && (ba % 16 == 0) && (lda % 16 == 0) && (p.K % 16 == 0));
    if ((p.mn_major || p.b_mn_major) && !tma_ok) { set_error("MN-major operands need 16-byte aligned bases and row pitches (and K, N multiples of 16)"); return CF_ERR_UNSUPPORTED; }
    if (p.b_mn_major && p.groups > 1 && p.K % BK != 0) {
        // a k-block that runs past one weight block would read the next block's rows
        set_error("grouped GEMM over [K, N] weight blocks: K must be a multiple of %d", BK);
        return CF_ERR_UNSUPPORTED;
    }
    const uintptr_t ca = reinterpret_cast<uintptr_t>(p.C);
    // per-segment output buffers: the caller guarantees 16-byte aligned bases (checked at the API boundary)
    p.c_vec = (p.out_kind == 0 || p.out_kind == 3) && (p.d_group_out != nullptr || ca % 16 == 0) && (p.ldc % 8 == 0) &&
              (p.bias == nullptr || reinterpret_cast<uintptr_t>(p.bias) % 4 == 0);
    if (!p.bias) p.bias_mode = 0;
    if (p.out_kind == 4) {
        // E4M3 output of width N/2: 16-byte stores need an aligned base and row pitch; whole 64-column groups only
        if (!tma_ok || ca % 16 != 0 || p.ldc % 16 != 0 || p.N % 64 != 0 || !p.d_quant_scale || !p.d_amax_out ||
            p.d_b_col_descale || p.d_group_out) {
            set_error("swiglu epilogue: needs TMA-aligned operands, N %% 64 == 0, a 16-byte aligned E4M3 output, no per-column scales");
            return CF_ERR_UNSUPPORTED;
        }
        p.c_vec = 0;
    }
    if (p.out_kind == 5) {
        // bf16 SwiGLU product of width N/2 with per-row amax: 16-byte stores, whole 64-column groups, dense rows only
        if (!tma_ok || ca % 16 != 0 || p.ldc % 8 != 0 || p.N % 64 != 0 || !p.d_row_amax_out || p.d_group_out || p.bias ||
            (p.d_b_col_descale && reinterpret_cast<uintptr_t>(p.d_b_col_descale) % 16 != 0)) {
            set_error("swiglu bf16 epilogue: needs TMA-aligned operands, N %% 64 == 0, a 16-byte aligned bf16 output with ldc %% 8 == 0, a row amax array, 16-byte aligned column scales");
            return CF_ERR_UNSUPPORTED;
        }
        p.c_vec = 0;
    }
    // Row blocks per rasterisation band. Eight keeps the operand slabs of the ~74 tiles in flight smallest (8 + 74/8 row
    // and column blocks). When the weight operand is larger than L2 (N x K > 64 MB) it is re-streamed from HBM once per
    // band, and a taller band pays as long as the band's own A rows (band x 256 x K bytes) stay within about 32 MB:
    // measured over seconds under the power cap (shorter timings follow the power controller's history, not the
    // rasterisation), dense bf16-output GEMMs: 16384 x 28672 x 4096: 1.472 / 1.429 / 1.419 ms with 8 / 16 / 32;
    // 32768 x 28672 x 8192: 5.63 / 5.52 / 6.01 ms; 32768 x 14336 x 8192: 2.82 / 2.76 / 3.02 ms; 32768 x 8192 x 28672
    // (A band 58 MB at 8): 5.61 / 5.54 / 5.96 ms with 4 / 8 / 16. The SwiGLU forms (gate/up projections, 28672 x 4096) take
    // 16, ragged ones included: a taller band would span several experts' weight blocks.
    if (static_cast<long long>(p.N) * p.K > (64ll << 20)) {
        if (p.out_kind == 4 || p.out_kind == 5) {
            if (p.K <= 4096) p.raster_m = 16;
        } else if (p.d_counts == nullptr && !p.mn_major) {
            if (p.K <= 4096) p.raster_m = 32;
            else if (p.K <= 8192) p.raster_m = 16;
        }
    }
    if (p.peer_out_host != nullptr && !tma_ok) {
        set_error("reduce-scatter GEMM: operands must be 16-byte aligned with K %% 16 == 0");
        return CF_ERR_UNSUPPORTED;
    }
    if (!tma_ok) {
        const int grid = sm_count() * 4;
        k_gemm_fp8_nt_simt<<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(d_A), lda, static_cast<const uint8_t*>(d_B), p);
        CF_LAUNCH_CHECK("gemm_fp8_nt_simt");
        return CF_OK;
    }
    // Paired CTAs (256-row tiles) pay off when the row blocks are mostly full; small or very ragged problems
    // keep the 128-row single-CTA tiles.
    const long long rows_per_group = (p.d_counts ? a_rows / (p.groups > 0 ? p.groups : 1) : p.M);
    bool pair = p.mn_major || p.b_mn_major || rows_per_group >= 512;
    const int pairs = pair ? max_resident_pairs() : 0;
    if (pairs <= 0) pair = false;

    CUtensorMap map_a, map_b, map_c;
    int r;
    if (p.mn_major) {
        // A is [K, M] with pitch lda, B is [K, N] with pitch p.ldb: boxes of 128 bytes along M / N by BK rows of K.
        // Only the pair form is built for this layout (each CTA's share of both operands is one 128-byte swizzle atom).
        if (!pair) { set_error("MN-major operands need the CTA-pair form (at least 512 rows, clusters available)"); return CF_ERR_UNSUPPORTED; }
        r = make_map(&map_a, d_A, p.K, p.M, lda, BK);
        if (r != CF_OK) return r;
        r = make_map(&map_b, d_B, p.K, p.N, p.ldb, BK);
        if (r != CF_OK) return r;
    } else if (p.b_mn_major) {
        // A is [rows, K] as usual; B is the stacked [weights * K, N] tensor with pitch p.ldb (b_rows counts its rows)
        if (!pair) { set_error("[K, N] weight operands need the CTA-pair form (clusters available)"); return CF_ERR_UNSUPPORTED; }
        r = make_map(&map_a, d_A, a_rows, p.K, lda, BM);
        if (r != CF_OK) return r;
        r = make_map(&map_b, d_B, b_rows, p.N, p.ldb, BK);
        if (r != CF_OK) return r;
    } else {
        r = make_map(&map_a, d_A, a_rows, p.K, lda, BM);
        if (r != CF_OK) return r;
        r = make_map(&map_b, d_B, b_rows, p.K, p.K, pair ? Cfg<true>::B_ROWS : Cfg<false>::B_ROWS);
        if (r != CF_OK) return r;
    }
    p.c_rows = p.d_counts ? a_rows : p.M;
    p.tma_store = (p.c_vec && p.out_kind == 0 && p.d_group_out == nullptr && p.N >= C_BOX_COLS &&
                   (p.bias == nullptr || reinterpret_cast<uintptr_t>(p.bias) % 16 == 0) &&
                   (p.d_b_col_descale == nullptr || reinterpret_cast<uintptr_t>(p.d_b_col_descale) % 16 == 0)) ? 1 : 0;
    const bool return_form = p.d_out_runs != nullptr;
    if (return_form) {
        // grouped bf16 output whose runs of rows go to per-run destination buffers
        if (p.out_kind != 0 || p.d_counts == nullptr || p.peer_out_host == nullptr || p.peer_count < 1 || p.peer_count > 16 ||
            p.d_peer_maps == nullptr || p.rows_per_peer <= 0 || p.runs_per_group < 1 || p.N % 64 != 0 || p.ldc % 8 != 0 ||
            p.bias || p.d_group_out || !tma_ok) {
            set_error("return-form GEMM: needs a grouped bf16 product, TMA-aligned operands, N %% 64 == 0, 1..16 destination buffers");
            return CF_ERR_UNSUPPORTED;
        }
        if (!p.peer_maps_ready) {
            struct { CUtensorMap maps[16]; void* bases[16]; } host;
            for (int i = 0; i < 16; ++i) host.bases[i] = nullptr;
            for (int i = 0; i < p.peer_count; ++i) {
                if (p.peer_out_host[i] == nullptr || reinterpret_cast<uintptr_t>(p.peer_out_host[i]) % 16 != 0) {
                    set_error("return-form GEMM: destination %d is null or not 16-byte aligned", i);
                    return CF_ERR_INVALID_ARG;
                }
                r = make_map_c(&host.maps[i], p.peer_out_host[i], p.rows_per_peer, p.N, p.ldc);
                if (r != CF_OK) return r;
                host.bases[i] = p.peer_out_host[i];
            }
            CF_CUDA(cudaMemcpyAsync(p.d_peer_maps, &host, sizeof(host), cudaMemcpyHostToDevice, st));
        }
        p.d_peer_bases = reinterpret_cast<void* const*>(static_cast<char*>(p.d_peer_maps) + 16 * sizeof(CUtensorMap));
        p.peer_out_host = nullptr;
    } else if (p.peer_out_host != nullptr) {
        // every tile must lie inside one slice and take the TMA path as a whole (no ragged rows, no column tail)
        if (p.out_kind != 2 || p.d_counts != nullptr || p.peer_count < 1 || p.peer_count > 16 || p.d_peer_maps == nullptr ||
            p.rows_per_peer <= 0 || p.rows_per_peer % 256 != 0 || p.M != p.rows_per_peer * p.peer_count || p.N % 32 != 0 ||
            !tma_ok || (p.d_b_col_descale && reinterpret_cast<uintptr_t>(p.d_b_col_descale) % 16 != 0)) {
            set_error("reduce-scatter GEMM: needs TMA-aligned operands, N %% 32 == 0, M = peers x rows_per_peer with rows_per_peer %% 256 == 0, 16-byte aligned column scales");
            return CF_ERR_UNSUPPORTED;
        }
        if (!p.peer_maps_ready) {
            CUtensorMap hmaps[16];
            for (int i = 0; i < p.peer_count; ++i) {
                if (p.peer_out_host[i] == nullptr || reinterpret_cast<uintptr_t>(p.peer_out_host[i]) % 16 != 0) {
                    set_error("reduce-scatter GEMM: slice %d is null or not 16-byte aligned", i);
                    return CF_ERR_INVALID_ARG;
                }
                r = make_map_c_f32(&hmaps[i], p.peer_out_host[i], p.rows_per_peer, p.N, p.N);
                if (r != CF_OK) return r;
            }
            // pageable source: the runtime stages the bytes before the call returns, so the stack array may go (the
            // copy waits for the stream's earlier work first, which is why the caller caches the maps)
            CF_CUDA(cudaMemcpyAsync(p.d_peer_maps, hmaps, sizeof(CUtensorMap) * p.peer_count, cudaMemcpyHostToDevice, st));
        }
        p.peer_out_host = nullptr;          // host pointer: of no use to the kernel
    } else {
        p.d_peer_maps = nullptr;
    }
    const bool f32_tma = (p.out_kind == 2 || p.out_kind == 1) && ca % 16 == 0 && p.ldc % 4 == 0 && p.N >= 32 &&
                         p.d_group_out == nullptr &&
                         (p.d_b_col_descale == nullptr || reinterpret_cast<uintptr_t>(p.d_b_col_descale) % 16 == 0);
    p.tma_reduce = return_form ? 0 : p.d_peer_maps ? 1 : (f32_tma ? (p.out_kind == 2 ? 1 : 2) : 0);
    if (return_form) p.tma_store = 1;
    if (p.out_kind == 5) {
        // bf16 SwiGLU product [rows, N/2]: boxes of 64 features x 32 rows, clipped at the tensor's edges
        p.tma_store = 1;
        r = make_map_c(&map_c, p.C, p.c_rows, p.N / 2, p.ldc);
        if (r != CF_OK) return r;
    } else if (p.d_peer_maps) {
        map_c = map_a;   // the kernel takes its output maps from d_peer_maps
    } else if (p.tma_store) {
        r = make_map_c(&map_c, p.C, p.c_rows, p.N, p.ldc);
        if (r != CF_OK) return r;
    } else if (p.tma_reduce) {
        r = make_map_c_f32(&map_c, p.C, p.c_rows, p.N, p.ldc);
        if (r != CF_OK) return r;
    } else {
        map_c = map_a;   // never dereferenced by the kernel when tma_store == 0
    }
    int dev = 0;
    CF_CUDA(cudaGetDevice(&dev));
    const bool wide = (p.out_kind >= 1 && p.out_kind <= 3) || p.d_out_runs != nullptr || p.b_mn_major;
    if (pair) {
        // tile_upper_bound counts 128-row blocks; a pair tile covers two of them
        const int n_blocks = (p.N + BN - 1) / BN;
        const int m128 = tile_upper_bound / (n_blocks > 0 ? n_blocks : 1);
        const int pair_tiles = ((m128 + 1) / 2 + (p.d_counts ? p.groups : 0)) * n_blocks;
        const int units = pair_tiles < pairs ? pair_tiles : pairs;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * units);
        cfg.blockDim = dim3(NUM_THREADS);
        cfg.dynamicSmemBytes = Cfg<true>::SMEM_BYTES;
        cfg.stream = st;
        cudaLaunchAttribute at[2];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = 2;
        if (wide) CF_CUDA(cudaLaunchKernelEx(&cfg, k_gemm_fp8_nt<true, true>, map_a, map_b, map_c, p));
        else CF_CUDA(cudaLaunchKernelEx(&cfg, k_gemm_fp8_nt<true, false>, map_a, map_b, map_c, p));
        CF_LAUNCH_CHECK("gemm_fp8_nt<pair>");
        return CF_OK;
    }
    static std::once_flag attr_once[64];
    cudaError_t attr_err = cudaSuccess;
    std::call_once(attr_once[dev & 63], [&] {
        attr_err = cudaFuncSetAttribute(k_gemm_fp8_nt<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<false>::SMEM_BYTES);
        if (attr_err == cudaSuccess)
            attr_err = cudaFuncSetAttribute(k_gemm_fp8_nt<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<false>::SMEM_BYTES);
    });
    if (attr_err != cudaSuccess) return cuda_fail(attr_err, "cudaFuncSetAttribute(k_gemm_fp8_nt)");
    const int sms = sm_count();
    const int grid = tile_upper_bound < sms ? tile_upper_bound : sms;
    if (wide) CF_CUDA(launch_pdl(k_gemm_fp8_nt<false, true>, dim3(grid), dim3(NUM_THREADS), Cfg<false>::SMEM_BYTES, st, map_a, map_b, map_c, p));
    else CF_CUDA(launch_pdl(k_gemm_fp8_nt<false, false>, dim3(grid), dim3(NUM_THREADS), Cfg<false>::SMEM_BYTES, st, map_a, map_b, map_c, p));
    CF_LAUNCH_CHECK("gemm_fp8_nt");
    return CF_OK;
}

int launch_wait_selftest(int* d_status, unsigned long long limit_ns, cudaStream_t st) {
    const int rc = require_sm100();
    if (rc != CF_OK) return rc;
    k_wait_selftest<<<1, 32, 0, st>>>(d_status, limit_ns);
    CF_LAUNCH_CHECK("wait_selftest");
    return CF_OK;
}

int gemm_tile_m() { return BM; }
int gemm_tile_n() { return BN; }

}  // namespace cf
