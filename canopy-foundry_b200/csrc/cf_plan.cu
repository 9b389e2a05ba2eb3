// Host-side sharding glue of the FP8 path: where the experts of an expert-parallel MoE layer live and how a dimension
// is split over the ranks. Pure host code (no device work): the counterpart of what the reference keeps in
// src/parallel/plan.cpp and include/canopy_foundry/parallel/plan.hpp, whose ParallelMode::ExpertSharded is a name
// without a layout behind it. The device side of the same plan is cf_moe_ep_plan (cf_moe.cu).
#include <cstring>

#include "cf_common.cuh"

extern "C" {

int cf_shard_range(long long n, int world, int rank, int multiple, long long* lo, long long* hi) {
    CF_REQUIRE(n >= 0 && world >= 1 && rank >= 0 && rank < world && multiple >= 1 && lo && hi, "cf_shard_range: bad argument");
    const long long units = (n + multiple - 1) / multiple;
    const long long base = units / world, extra = units % world;
    const long long start_u = rank * base + (rank < extra ? rank : extra);
    const long long stop_u = start_u + base + (rank < extra ? 1 : 0);
    const long long a = start_u * multiple, b = stop_u * multiple;
    *lo = a < n ? a : n;
    *hi = b < n ? b : n;
    return CF_OK;
}

int cf_ep_placement_build(const double* popularity, int num_experts, int world, double min_share, cf_ep_placement* out) {
    CF_REQUIRE(popularity && out, "cf_ep_placement_build: null pointer");
    CF_REQUIRE(num_experts >= 1 && num_experts <= CF_EP_MAX_EXPERTS, "cf_ep_placement_build: 1..%d experts", CF_EP_MAX_EXPERTS);
    CF_REQUIRE(world >= 1 && world <= CF_EP_MAX_RANKS, "cf_ep_placement_build: 1..%d ranks", CF_EP_MAX_RANKS);
    CF_REQUIRE(min_share >= 0.0 && min_share < 1.0, "cf_ep_placement_build: min_share must be in [0, 1)");
    double tot = 0.0;
    for (int e = 0; e < num_experts; ++e) {
        CF_REQUIRE(popularity[e] >= 0.0, "cf_ep_placement_build: negative popularity");
        tot += popularity[e];
    }
    CF_REQUIRE(tot > 0.0, "cf_ep_placement_build: all popularities are zero");
    std::memset(out, 0, sizeof(*out));
    out->world = world;
    out->num_experts = num_experts;
    const double piece = 1.0 / world;
    static thread_local double rep_len[CF_EP_MAX_REPLICAS];
    static thread_local double p[CF_EP_MAX_EXPERTS];
    for (int e = 0; e < num_experts; ++e) p[e] = popularity[e] / tot;
    // The experts lie end to end on a line, each as long as its share of the rows; the line is cut into `world` equal
    // pieces. Every (expert, rank) overlap is a replica; overlaps below min_share of a piece are not worth a weight copy
    // and go to the expert's largest replica.
    int v = 0;
    double pos = 0.0;
    for (int e = 0; e < num_experts; ++e) {
        const double lo = pos, hi = pos + p[e];
        pos = hi;
        int g0 = static_cast<int>(lo / piece + 1e-12);
        if (g0 > world - 1) g0 = world - 1;
        int g1 = g0;
        if (hi > lo) {
            g1 = static_cast<int>((hi - 1e-12) / piece);
            if (g1 > world - 1) g1 = world - 1;
        }
        if (g1 < g0) g1 = g0;
        double part[CF_EP_MAX_RANKS];
        double sum_parts = 0.0;
        for (int g = g0; g <= g1; ++g) {
            const double top = hi < (g + 1) * piece ? hi : (g + 1) * piece;
            const double bot = lo > g * piece ? lo : g * piece;
            part[g - g0] = top - bot > 0.0 ? top - bot : 0.0;
            sum_parts += part[g - g0];
        }
        const int first = v;
        double sum_keep = 0.0;
        for (int g = g0; g <= g1; ++g) {
            if (part[g - g0] >= min_share * piece) {
                if (v >= CF_EP_MAX_REPLICAS) { cf::set_error("cf_ep_placement_build: more than %d replicas", CF_EP_MAX_REPLICAS); return CF_ERR_LIMIT; }
                out->replica_expert[v] = e; out->replica_rank[v] = g; rep_len[v] = part[g - g0];
                sum_keep += part[g - g0];
                ++v;
            }
        }
        if (v == first) {               // nothing survived: keep the largest overlap (the first one on ties)
            int best = g0;
            for (int g = g0; g <= g1; ++g) if (part[g - g0] > part[best - g0]) best = g;
            if (v >= CF_EP_MAX_REPLICAS) { cf::set_error("cf_ep_placement_build: more than %d replicas", CF_EP_MAX_REPLICAS); return CF_ERR_LIMIT; }
            out->replica_expert[v] = e; out->replica_rank[v] = best; rep_len[v] = part[best - g0];
            sum_keep = part[best - g0];
            ++v;
        }
        int big = first;
        for (int i = first; i < v; ++i) if (rep_len[i] > rep_len[big]) big = i;
        rep_len[big] += sum_parts - sum_keep;
    }
    out->num_replicas = v;
    // per expert: first replica id, every replica's share of the expert's rows and the cumulative share
    int id = 0;
    for (int e = 0; e < num_experts; ++e) {
        out->replica_start[e] = id;
        int n_e = 0;
        double tot_e = 0.0;
        for (int i = id; i < v && out->replica_expert[i] == e; ++i) { ++n_e; tot_e += rep_len[i]; }
        if (tot_e == 0.0) tot_e = 1.0;
        double run = 0.0;
        for (int k = 0; k < n_e; ++k) {
            const double sh = p[e] > 0.0 ? rep_len[id + k] / tot_e : 1.0 / n_e;
            run += sh;
            out->replica_share[id + k] = sh;
            out->replica_cum_share[id + k] = (k == n_e - 1) ? 1.0 : run;
        }
        id += n_e;
    }
    out->replica_start[num_experts] = v;
    // ranks along the line are non-decreasing, so every rank's replica ids are contiguous; a rank without replicas gets
    // an empty range placed where it belongs in the order
    int prev_hi = 0;
    for (int g = 0; g < world; ++g) {
        int lo_id = -1, hi_id = -1;
        for (int i = 0; i < v; ++i)
            if (out->replica_rank[i] == g) { if (lo_id < 0) lo_id = i; hi_id = i + 1; }
        if (lo_id < 0) { out->rank_lo[g] = prev_hi; out->rank_hi[g] = prev_hi; }
        else { out->rank_lo[g] = lo_id; out->rank_hi[g] = hi_id; prev_hi = hi_id; }
    }
    return CF_OK;
}

}  // extern "C"

namespace {

// The placement for arbitrary cut points cut[0] = 0 < ... < cut[world] = 1 of the line (rank g owns [cut[g], cut[g+1])).
// rep_len receives every replica's length on the line. Same merging rule as the uniform form.
int place_with_cuts(const double* p, int num_experts, int world, double min_share, const double* cut, cf_ep_placement* out,
                    double* rep_len) {
    std::memset(out, 0, sizeof(*out));
    out->world = world;
    out->num_experts = num_experts;
    int v = 0;
    double pos = 0.0;
    for (int e = 0; e < num_experts; ++e) {
        const double lo = pos, hi = pos + p[e];
        pos = hi;
        int g0 = 0;
        while (g0 < world - 1 && cut[g0 + 1] <= lo + 1e-12) ++g0;
        int g1 = g0;
        if (hi > lo) while (g1 < world - 1 && cut[g1 + 1] < hi - 1e-12) ++g1;
        double part[CF_EP_MAX_RANKS];
        double sum_parts = 0.0, sum_keep = 0.0;
        for (int g = g0; g <= g1; ++g) {
            const double top = hi < cut[g + 1] ? hi : cut[g + 1];
            const double bot = lo > cut[g] ? lo : cut[g];
            part[g - g0] = top - bot > 0.0 ? top - bot : 0.0;
            sum_parts += part[g - g0];
        }
        const int first = v;
        for (int g = g0; g <= g1; ++g) {
            if (part[g - g0] >= min_share * (cut[g + 1] - cut[g])) {
                if (v >= CF_EP_MAX_REPLICAS) return CF_ERR_LIMIT;
                out->replica_expert[v] = e; out->replica_rank[v] = g; rep_len[v] = part[g - g0];
                sum_keep += part[g - g0];
                ++v;
            }
        }
        if (v == first) {
            int best = g0;
            for (int g = g0; g <= g1; ++g) if (part[g - g0] > part[best - g0]) best = g;
            if (v >= CF_EP_MAX_REPLICAS) return CF_ERR_LIMIT;
            out->replica_expert[v] = e; out->replica_rank[v] = best; rep_len[v] = part[best - g0];
            sum_keep = part[best - g0];
            ++v;
        }
        int big = first;
        for (int i = first; i < v; ++i) if (rep_len[i] > rep_len[big]) big = i;
        rep_len[big] += sum_parts - sum_keep;
    }
    out->num_replicas = v;
    int id = 0;
    for (int e = 0; e < num_experts; ++e) {
        out->replica_start[e] = id;
        int n_e = 0;
        double tot_e = 0.0;
        for (int i = id; i < v && out->replica_expert[i] == e; ++i) { ++n_e; tot_e += rep_len[i]; }
        if (tot_e == 0.0) tot_e = 1.0;
        double run = 0.0;
        for (int k = 0; k < n_e; ++k) {
            const double sh = p[e] > 0.0 ? rep_len[id + k] / tot_e : 1.0 / n_e;
            run += sh;
            out->replica_share[id + k] = sh;
            out->replica_cum_share[id + k] = (k == n_e - 1) ? 1.0 : run;
        }
        id += n_e;
    }
    out->replica_start[num_experts] = v;
    int prev_hi = 0;
    for (int g = 0; g < world; ++g) {
        int lo_id = -1, hi_id = -1;
        for (int i = 0; i < v; ++i)
            if (out->replica_rank[i] == g) { if (lo_id < 0) lo_id = i; hi_id = i + 1; }
        if (lo_id < 0) { out->rank_lo[g] = prev_hi; out->rank_hi[g] = prev_hi; }
        else { out->rank_lo[g] = lo_id; out->rank_hi[g] = hi_id; prev_hi = hi_id; }
    }
    return CF_OK;
}

// Expected tile work of the busiest rank, as a fraction of all rows: a replica with r rows costs the tiles it fills,
// ceil(r / tile) * tile; with r only known in expectation that is r + tile / 2.
double worst_rank_cost(const cf_ep_placement& pl, const double* rep_len, double half_tile, const double* speed) {
    double worst = 0.0;
    for (int g = 0; g < pl.world; ++g) {
        double c = 0.0;
        for (int v = pl.rank_lo[g]; v < pl.rank_hi[g]; ++v) c += rep_len[v] + half_tile;
        c /= speed[g];                                   // time, in units of the mean rank's time per row
        if (c > worst) worst = c;
    }
    return worst;
}

}  // namespace

extern "C" int cf_ep_placement_build_balanced(const double* popularity, int num_experts, int world, double min_share,
                                              double expected_total_rows, int tile_rows, cf_ep_placement* out) {
    return cf_ep_placement_build_weighted(popularity, num_experts, world, min_share, expected_total_rows, tile_rows, nullptr, out);
}

extern "C" int cf_ep_placement_build_weighted(const double* popularity, int num_experts, int world, double min_share,
                                              double expected_total_rows, int tile_rows, const double* rank_speed_or_null,
                                              cf_ep_placement* out) {
    CF_REQUIRE(popularity && out, "cf_ep_placement_build_balanced: null pointer");
    CF_REQUIRE(num_experts >= 1 && num_experts <= CF_EP_MAX_EXPERTS, "cf_ep_placement_build_balanced: 1..%d experts", CF_EP_MAX_EXPERTS);
    CF_REQUIRE(world >= 1 && world <= CF_EP_MAX_RANKS, "cf_ep_placement_build_balanced: 1..%d ranks", CF_EP_MAX_RANKS);
    CF_REQUIRE(min_share >= 0.0 && min_share < 1.0, "cf_ep_placement_build_balanced: min_share must be in [0, 1)");
    CF_REQUIRE(expected_total_rows > 0.0 && tile_rows >= 1, "cf_ep_placement_build_balanced: needs the expected row total and the tile height");
    double tot = 0.0;
    for (int e = 0; e < num_experts; ++e) {
        CF_REQUIRE(popularity[e] >= 0.0, "cf_ep_placement_build_balanced: negative popularity");
        tot += popularity[e];
    }
    CF_REQUIRE(tot > 0.0, "cf_ep_placement_build_balanced: all popularities are zero");
    static thread_local double p[CF_EP_MAX_EXPERTS], rep_len[CF_EP_MAX_REPLICAS], best_len[CF_EP_MAX_REPLICAS];
    for (int e = 0; e < num_experts; ++e) p[e] = popularity[e] / tot;
    const double half_tile = 0.5 * tile_rows / expected_total_rows;      // expected padding of one replica, as a share of all rows
    // relative speed of every rank (mean 1): a rank that needs less time per row takes a longer piece of the line
    double speed[CF_EP_MAX_RANKS], speed_sum = 0.0;
    for (int g = 0; g < world; ++g) {
        speed[g] = rank_speed_or_null ? rank_speed_or_null[g] : 1.0;
        CF_REQUIRE(speed[g] > 0.0, "cf_ep_placement_build_weighted: rank speeds must be positive");
        speed_sum += speed[g];
    }
    for (int g = 0; g < world; ++g) speed[g] *= world / speed_sum;
    double cut[CF_EP_MAX_RANKS + 1];
    cut[0] = 0.0;
    for (int g = 0; g < world; ++g) cut[g + 1] = cut[g] + speed[g] / world;
    cut[world] = 1.0;
    cf_ep_placement cand;
    double best = -1.0;
    // Fixed-point iteration on the cut points: a rank that holds n replicas gives up n half-tiles of rows, so that rows +
    // expected padding, the tile work, is what the ranks have in common. The replica count changes as the cuts move; the
    // best of a few passes is kept (the first pass is the equal-rows placement, so the result is never worse than that).
    for (int pass = 0; pass < 6; ++pass) {
        const int rc = place_with_cuts(p, num_experts, world, min_share, cut, &cand, rep_len);
        if (rc != CF_OK) { cf::set_error("cf_ep_placement_build_balanced: more than %d replicas", CF_EP_MAX_REPLICAS); return rc; }
        const double cost = worst_rank_cost(cand, rep_len, half_tile, speed);
        if (best < 0.0 || cost < best) {
            best = cost;
            *out = cand;
            std::memcpy(best_len, rep_len, sizeof(double) * cand.num_replicas);
        }
        const double level = (1.0 + half_tile * cand.num_replicas) / world;       // tile work a rank of mean speed should end up with
        double piece[CF_EP_MAX_RANKS], sum = 0.0;
        for (int g = 0; g < world; ++g) {
            piece[g] = level * speed[g] - half_tile * (cand.rank_hi[g] - cand.rank_lo[g]);
            if (piece[g] < 0.25 / world) piece[g] = 0.25 / world;
            sum += piece[g];
        }
        double acc = 0.0;
        for (int g = 0; g < world; ++g) { cut[g] = acc; acc += piece[g] / sum; }
        cut[0] = 0.0;
        cut[world] = 1.0;
    }
    return CF_OK;
}
