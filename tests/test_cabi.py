"""CPU-side checks of the boundary: the shared library loads without a GPU and exports every symbol
include/canopy_fp8.h declares; argument validation that needs no device works."""
import ctypes as C
import os
import re

from gpu_util import ROOT, package


def test_library_exports_every_declared_symbol():
    cfb = package()
    lib = cfb._capi.lib()
    hdr = open(os.path.join(ROOT, "include", "canopy_fp8.h")).read()
    declared = set(re.findall(r"\b(cf_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations parsed"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/canopy_fp8.h but not exported"
    assert declared == set(cfb._capi.SIGNATURES), "ctypes table and header disagree"
    assert lib.cf_abi_version() == cfb._capi.ABI_VERSION


def test_struct_layouts_match_the_header():
    cfb = package()
    # pointer-sized and 4-byte members only; sizes follow the C layout rules on LP64
    assert C.sizeof(cfb._capi.GemmEpilogue) == 40
    assert C.sizeof(cfb._capi.ActSlotStruct) == 8 * 8 + 4 * 4 + 3 * 8
    assert C.sizeof(cfb._capi.Fp8WeightStruct) == 6 * 8 + 3 * 4 + 4


def test_argument_validation_without_a_device():
    cfb = package()
    lib = cfb._capi.lib()
    assert lib.cf_fp8_quantize_e4m3(None, None, None, 16, None) == cfb._capi.CF_ERR_INVALID_ARG
    assert b"null pointer" in lib.cf_last_error()
    assert lib.cf_swiglu_forward(None, None, None, -1, None) == cfb._capi.CF_ERR_INVALID_ARG
    assert lib.cf_fp8_quantize_e4m3(None, None, C.c_void_p(16), 0, None) == cfb._capi.CF_OK     # n == 0 is a no-op
    assert lib.cf_moe_topk_route_f32(None, 4, 100, 2, None, None, None, 1) == cfb._capi.CF_ERR_INVALID_ARG
    # dispatch front end: scratch sizing (one int per 256-row chunk and list) and argument checks
    assert lib.cf_moe_route_dispatch_scratch_ints(0, 8) == 0
    assert lib.cf_moe_route_dispatch_scratch_ints(256, 8) == 8
    assert lib.cf_moe_route_dispatch_scratch_ints(257, 15) == 30
    assert lib.cf_moe_route_dispatch_lists(None, 4, 100, 2, 1, None, None, None, 0, None, None, 0, None, None, None, None, 0,
                                           None) == cfb._capi.CF_ERR_INVALID_ARG
    assert lib.cf_moe_route_dispatch_lists(None, 4, 8, 2, 1, None, None, None, 0, None, None, 0, None, None, None, None, 0,
                                           None) == cfb._capi.CF_ERR_INVALID_ARG      # counts / offsets missing


def test_shim_compiles_against_the_reference_headers(tmp_path):
    """The C++ drop-in (namespace ida_native definitions) must match the reference's declarations: compile it
    against include/ida_native/kernels.hpp where the reference tree is available (this container only)."""
    import shutil
    import subprocess

    import pytest
    ref = os.environ.get("CANOPY_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.isdir(os.path.join(ref, "include", "ida_native")) or shutil.which("nvcc") is None:
        pytest.skip("reference tree or nvcc not present")
    src = os.path.join(ROOT, "canopy-foundry_b200", "shim", "ida_native_kernels.cu")
    out = tmp_path / "shim.o"
    r = subprocess.run(["nvcc", "-std=c++20", "-gencode", "arch=compute_100a,code=sm_100a", f"-I{ref}/include",
                        f"-I{ref}/include-public", f"-I{ROOT}/include", "-c", src, "-o", str(out)],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, r.stdout[-3000:]


def test_expert_sharded_plan_glue_compiles_and_runs_against_the_reference_headers(tmp_path):
    """cf_parallel_shim.hpp gives the reference's ParallelMode::ExpertSharded a layout: compile a small program
    against include/canopy_foundry/parallel/plan.hpp (where the reference tree is available), link the library and
    run it on the CPU: an 8-expert Zipf load over 4 devices gives contiguous replica ranges and equal expected rows."""
    import shutil
    import subprocess

    import pytest
    ref = os.environ.get("CANOPY_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.isdir(os.path.join(ref, "include", "canopy_foundry")) or shutil.which("g++") is None:
        pytest.skip("reference tree or g++ not present")
    src = tmp_path / "plan_glue.cpp"
    src.write_text(r"""
#include <cmath>
#include <cstdio>
#include "cf_parallel_shim.hpp"
int main() {
    canopy_foundry::ParallelPlan plan;
    plan.mode = canopy_foundry::ParallelMode::ExpertSharded;
    plan.transport = canopy_foundry::TransportKind::CudaP2P;
    plan.devices = {0, 1, 2, 3};
    std::vector<double> load;
    for (int e = 0; e < 8; ++e) load.push_back(std::pow(e + 1.0, -1.1));
    cf_shim::ExpertShardedLayout lay = cf_shim::expert_sharded_layout(plan, load);
    double tot = 0; for (double x : load) tot += x;
    for (int r = 0; r < lay.world(); ++r) {
        double rows = 0;
        for (int v = lay.placement.rank_lo[r]; v < lay.placement.rank_hi[r]; ++v)
            rows += load[lay.placement.replica_expert[v]] / tot * lay.placement.replica_share[v];
        std::printf("rank %d replicas [%d,%d) share %.4f\n", r, lay.placement.rank_lo[r], lay.placement.rank_hi[r], rows);
        if (std::fabs(rows - 0.25) > 0.02) return 2;
    }
    // pieces by tile work, the second device 10 % slower: it expects clearly fewer rows than the others
    cf_shim::ExpertShardedLayout w = cf_shim::expert_sharded_layout(plan, load, 0.02, 65536.0, {1.0, 0.9, 1.0, 1.0});
    double rows_w[4] = {0, 0, 0, 0};
    for (int r = 0; r < 4; ++r)
        for (int v = w.placement.rank_lo[r]; v < w.placement.rank_hi[r]; ++v)
            rows_w[r] += load[w.placement.replica_expert[v]] / tot * w.placement.replica_share[v];
    if (!(rows_w[1] < 0.95 * rows_w[0] && rows_w[1] < 0.95 * rows_w[2])) return 5;
    try { cf_shim::expert_sharded_layout(plan, load, 0.02, 0.0, {1.0, 1.0, 1.0, 1.0}); return 6; } catch (const std::invalid_argument&) {}
    plan.transport = canopy_foundry::TransportKind::HostStaged;
    try { cf_shim::expert_sharded_layout(plan, load); return 3; } catch (const std::invalid_argument&) {}
    plan.mode = canopy_foundry::ParallelMode::LayerPipeline;
    try { cf_shim::expert_sharded_layout(plan, load); return 4; } catch (const std::invalid_argument&) {}
    return 0;
}
""")
    exe = tmp_path / "plan_glue"
    libdir = os.path.join(ROOT, "canopy-foundry_b200", "lib")
    r = subprocess.run(["g++", "-std=c++20", f"-I{ref}/include", f"-I{ROOT}/include", f"-I{ROOT}/canopy-foundry_b200/shim",
                        str(src), os.path.join(ref, "src", "parallel", "plan.cpp"), f"-L{libdir}", "-lcanopy_fp8",
                        f"-Wl,-rpath,{libdir}", "-o", str(exe)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, r.stdout[-3000:]
    run = subprocess.run([str(exe)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert run.returncode == 0, run.stdout


def test_route_plan_glue_compiles_and_runs_against_the_reference_contracts(tmp_path):
    """cf_contracts_shim.hpp publishes the dispatch front end's buffers through the reference's RoutePlanStore and
    SchedulerWorkspaceCache and the FP8 weight caches through its ExecutionViewCache: compile a small program against the
    reference's headers and its own src/moe/route_plan.cpp, scheduler.cpp and src/precision/execution_view.cpp (where the
    reference tree is available) and run it on the CPU: publish, backward reuse by generation, duplicate and stale
    rejections, schedule build and reuse, one weight refresh per tensor generation whatever the number of roles."""
    import shutil
    import subprocess

    import pytest
    ref = os.environ.get("CANOPY_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.isfile(os.path.join(ref, "src", "moe", "route_plan.cpp")) or shutil.which("g++") is None:
        pytest.skip("reference tree or g++ not present")
    src = tmp_path / "route_glue.cpp"
    src.write_text(r"""
#include <cstdio>
#include "cf_contracts_shim.hpp"
int main() {
    using namespace canopy_foundry;
    static int counts[8], offsets[8], idx[8 * 64];
    static float rw[64 * 8];
    cf_shim::DispatchBuffers b;
    b.d_counts = counts; b.d_offsets = offsets; b.d_row_indices = idx; b.d_route_weights = rw;
    b.lists = 8; b.rows = 64; b.top_k = 2;
    RoutePlanStore store;
    const RoutePlanKey key{7, 3};
    const RoutePlan& p = cf_shim::publish_dispatch(store, key, RouteGeneration{1}, b);
    if (!p.valid() || p.routes != 128 || p.experts != 8 || p.actual_rows != -1) return 2;
    const RoutePlan& again = store.require_for_backward(key, RouteGeneration{1});
    const cf_shim::DispatchBuffers back = cf_shim::buffers_of(again);
    if (back.d_counts != counts || back.d_row_indices != idx || back.d_route_weights != rw || back.rows != 64) return 3;
    try { store.require_for_backward(key, RouteGeneration{2}); return 4; } catch (const RoutePlanError&) {}
    try { cf_shim::publish_dispatch(store, key, RouteGeneration{2}, b); return 5; } catch (const RoutePlanError&) {}
    try { cf_shim::publish_dispatch(store, RoutePlanKey{8, 3}, RouteGeneration{1}, b); return 6; } catch (const RoutePlanError&) {}
    cf_shim::DispatchBuffers other = b; other.top_k = 1;
    if (cf_shim::dispatch_fingerprint(other) == cf_shim::dispatch_fingerprint(b)) return 7;
    SchedulerWorkspaceCache cache;
    const SchedulerWorkspace& w = cf_shim::require_schedule(cache, RouteGeneration{1}, b, 28672, 4096, 0);
    if (!w.schedule_valid || w.key.n_tiles != 112 || w.key.k_chunks != 32 || w.tile_capacity != (1 + 8) * 112u) return 8;
    cf_shim::require_schedule(cache, RouteGeneration{1}, b, 28672, 4096, 0);
    cf_shim::require_schedule(cache, RouteGeneration{1}, b, 4096, 14336, 0);
    if (cache.stats().builds != 2 || cache.stats().reuses != 1) return 9;
    cache.invalidate_route(RouteGeneration{2});
    try { cf_shim::require_schedule(cache, RouteGeneration{1}, b, 28672, 4096, 0); return 10; } catch (const SchedulerWorkspaceError&) {}
    // weights: one refresh per tensor generation, shared by the roles
    static unsigned char fwd[16], bwd[16];
    cf_fp8_weight wt{};
    wt.fwd8 = fwd; wt.bwd8 = bwd; wt.in_dim = 4; wt.out_dim = 4;
    int refreshes = 0;
    auto fake = [&refreshes](const cf_fp8_weight&, void*) { ++refreshes; return 0; };
    ExecutionViewCache views;
    const PackedExecutionView& f1 = cf_shim::require_weight_view(views, 42, TensorGeneration{1}, ExecutionRole::Forward, wt, nullptr, fake);
    if (refreshes != 1 || f1.storage_token != cf_shim::token_of(fwd) || f1.key.layout.orientation != PackedOrientation::RowMajor) return 11;
    const PackedExecutionView& d1 = cf_shim::require_weight_view(views, 42, TensorGeneration{1}, ExecutionRole::BackwardDx, wt, nullptr, fake);
    if (refreshes != 1 || d1.storage_token != cf_shim::token_of(bwd) || d1.key.layout.orientation != PackedOrientation::Transposed) return 12;
    cf_shim::require_weight_view(views, 42, TensorGeneration{1}, ExecutionRole::Forward, wt, nullptr, fake);
    if (refreshes != 1 || views.stats().reuses != 1) return 13;
    views.invalidate(42, TensorGeneration{2});                   // the optimiser stepped
    cf_shim::require_weight_view(views, 42, TensorGeneration{2}, ExecutionRole::ExpertForward, wt, nullptr, fake);
    if (refreshes != 2) return 14;
    try { cf_shim::require_weight_view(views, 42, TensorGeneration{1}, ExecutionRole::Forward, wt, nullptr, fake); return 15; }
    catch (const ExecutionViewError&) {}
    cf_fp8_weight single = wt;
    single.bwd8 = nullptr;                                       // dgrad reads the forward cache MN-major
    const PackedExecutionView& d2 = cf_shim::require_weight_view(views, 43, TensorGeneration{1}, ExecutionRole::ExpertDx, single, nullptr, fake);
    if (d2.storage_token != cf_shim::token_of(fwd) || d2.key.layout.orientation != PackedOrientation::ColumnMajor) return 16;
    auto failing = [](const cf_fp8_weight&, void*) { return 3; };
    try { cf_shim::require_weight_view(views, 44, TensorGeneration{1}, ExecutionRole::Forward, wt, nullptr, failing); return 17; }
    catch (const ExecutionViewError&) {}
    std::puts("route plan glue: ok");
    return 0;
}
""")
    exe = tmp_path / "route_glue"
    libdir = os.path.join(ROOT, "canopy-foundry_b200", "lib")
    r = subprocess.run(["g++", "-std=c++20", f"-I{ref}/include", f"-I{ROOT}/include", f"-I{ROOT}/canopy-foundry_b200/shim", str(src),
                        os.path.join(ref, "src", "moe", "route_plan.cpp"), os.path.join(ref, "src", "moe", "scheduler.cpp"),
                        os.path.join(ref, "src", "precision", "execution_view.cpp"), f"-L{libdir}", "-lcanopy_fp8",
                        f"-Wl,-rpath,{libdir}", "-o", str(exe)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, r.stdout[-3000:]
    r = subprocess.run([str(exe)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0 and "route plan glue: ok" in r.stdout, (r.returncode, r.stdout)


def test_bench_line_contract_without_a_gpu():
    """bench.py imports without a GPU, offers the legs the default line carries, and the reference arm prints the
    same `config` keys as the GPU arm (the driver compares the two)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert set(bench.LEGS) == {"moe", "mlp", "sweep"}
    cfg = bench.linear_config(2, 1)
    assert {"workload", "M", "N", "K", "step", "bias_mode", "sharding", "l2"} <= set(cfg)
    assert cfg["M"] * cfg["N"] * cfg["K"] * 2.0 == bench.FLOP_PER_STEP
    assert bench.load_peaks()["hbm_gbs"] > 0
