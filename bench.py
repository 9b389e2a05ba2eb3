#!/usr/bin/env python
"""Benchmark of the FP8 quantize-and-GEMM hot path (BASELINE configuration 2, the single-GPU FP8 linear).

One step = one pass of the path over one batch resident in HBM:
    weight refresh   bf16 W[4096x4096] -> E4M3 in both layouts with the amax the optimiser left (delayed amax)
    fp8_quant_act    bf16 X[8192x4096] -> E4M3 with the previous step's scale, recording this step's amax,
                     then the delayed-scale ring update
    FP8 GEMM         tcgen05, fp32 accumulate, fused dequant + bf16 bias epilogue, bf16 Y[8192x4096]
`value` is 2*M*N*K per step over the device time of the whole step (all ranks); `roofline` isolates the GEMM
kernel with CUDA events inside the same timed region; `e2e` repeats the step with pinned HOST input and output
buffers and the copies inside the timed region; `cpu_baseline` times the CPU oracle on a bounded row sample.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
With N > 1 (torchrun, one rank per GPU) every rank runs the same workload on its own token shard against a
replicated weight: no data-path collective, weak scaling. `--impl reference` times the CPU restatement of the
reference's path on the host cores (the reference has no runnable CPU FP8 GEMM of its own).
"""
import argparse
import importlib
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, K, N = 8192, 4096, 4096
FLOP_PER_STEP = 2.0 * M * N * K
METRIC = "fp8_scaled_gemm_tflops"
UNIT = "TFLOP/s"
WORKLOAD = "fp8_linear_X8192x4096_W4096x4096_bf16_in_bf16_out (BASELINE config 2)"
N_ROTATE = 3            # activation buffers rotated between steps: 3 x 67 MB > 126 MB of L2


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d.get("hbm_gbs"), "bf16_tflops": d.get("bf16_tflops"),
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "sw_power_cap": 0x4, "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr:
            self._thr.join()
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def oracle():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_bindings import Oracle
    return Oracle()


def synth_host(seed):
    """Configuration-2 inputs as numpy bf16 bit patterns: X ~ N(0,1) with 0.1 % of elements x20, W ~ N(0,0.02),
    bias ~ N(0,0.01)."""
    import numpy as np
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K), dtype=np.float32)
    mask = rng.random((M, K), dtype=np.float32) < 1e-3
    x[mask] *= 20.0
    w = rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)
    b = rng.standard_normal(N, dtype=np.float32) * np.float32(0.01)
    return x, w, b


_CPU_CACHE = {}


def cpu_sample(orc, target_seconds, threads):
    """Times the oracle's record-quantise + FP8 GEMM + bias on a row slab of the same workload; the slab is
    sized from a short pilot so that the measurement takes about `target_seconds`."""
    import ctypes as C

    import numpy as np
    if "inputs" not in _CPU_CACHE:
        x, w, b = synth_host(0)
        xs, ws, bs = orc.to_bf16(x), orc.to_bf16(w), orc.to_bf16(b)
        sw, dw = orc.scale_from_amax(orc.amax_bf16(ws), 448.0)
        w8 = orc.quantize_bf16(ws, sw)
        sx, dx = orc.scale_from_amax(orc.amax_bf16(xs), 448.0)
        _CPU_CACHE["inputs"] = (xs, bs, w8, sx, dx, dw)
    xs, bs, w8, sx, dx, dw = _CPU_CACHE["inputs"]

    def run(rows):
        out = np.empty((rows, N), dtype=np.uint16)
        t0 = time.perf_counter()
        orc.lib.orc_linear_bf16_sample(xs.ctypes.data_as(C.c_void_p), w8.ctypes.data_as(C.c_void_p),
                                       bs.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), C.c_int(rows),
                                       C.c_int(N), C.c_int(K), C.c_float(sx), C.c_float(dx), C.c_float(dw),
                                       C.c_int(threads))
        return time.perf_counter() - t0

    pilot_rows = 64
    t_pilot = run(pilot_rows)
    rows = int(min(M, max(pilot_rows, pilot_rows * target_seconds / max(t_pilot, 1e-6))))
    rows = max(threads, rows - rows % max(threads, 1))
    # when the whole batch takes less than the target, repeat it until about target_seconds of CPU work are timed
    t, passes = 0.0, 0
    while passes == 0 or (rows == M and t < target_seconds and passes < 16):
        t += run(rows)
        passes += 1
    return rows * passes, t, 2.0 * rows * passes * N * K / t / 1e12


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    orc = oracle()
    threads = orc.lib.orc_hw_threads()
    per_step = max(1.0, min(20.0, 120.0 / max(args.steps + args.warmup, 1)))
    vals, rows = [], 0
    for i in range(args.warmup + args.steps):
        rows, t, tf = cpu_sample(orc, per_step, threads)
        if i >= args.warmup:
            vals.append((t, tf))
    ms = 1e3 * sum(t for t, _ in vals) / len(vals)
    tf = sum(v for _, v in vals) / len(vals)
    sample = f"{rows} rows ({rows / M:.2f} passes over the {M}-row batch) of X against the full W[{N}x{K}] per step (record-quantise + GEMM + bias), scaled by flops"
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "host run"},
        "cpu_baseline": {"value": tf, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_moe(args):
    """BASELINE configuration 4: 32768 tokens, hidden 4096, 8 SwiGLU experts of ffn 14336, top-2 routing with a
    Zipf(1.1)-skewed load. One step = route + dispatch lists + quantise + permute + ragged gate/up GEMM + SwiGLU
    re-quantise + ragged down GEMM + unpermute/combine. N > 1: expert parallel (E/N experts and 32768/N tokens per
    rank, E4M3 all-to-all out, bf16 all-to-all back): strong scaling, value = tokens of all ranks per second."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    cfb = importlib.import_module("canopy-foundry_b200")
    par = cfb.parallel
    TOK, H, F, E, TOPK = 32768, 4096, 14336, 8, 2
    rows = TOK // world
    use_ep = world > 1 and args.moe_mode == "ep"
    e_lo, e_hi = par.EpPlan.expert_range(E, world, rank) if use_ep else (0, E)
    ctx = cfb.Fp8Ctx(act8_bytes=0)
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    x = torch.randn((rows, H), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    pz = [(e + 1) ** -1.1 for e in range(E)]
    # Expert placement by expected load (longest-processing-time greedy over the Zipf popularity): expert ids are
    # renamed so that every rank owns a contiguous range of about equal total popularity. Renaming experts changes
    # nothing in the maths; with one expert per rank (N = 8) no placement can balance a skewed load.
    order = sorted(range(E), key=lambda e: -pz[e])
    bins = [[] for _ in range(world if use_ep else 1)]
    per = E // len(bins)
    for e in order:
        cand = [b for b in range(len(bins)) if len(bins[b]) < per]
        tgt = min(cand, key=lambda b: sum(pz[i] for i in bins[b]))
        bins[tgt].append(e)
    perm = [e for b in bins for e in b]                  # new id -> popularity rank
    p = torch.tensor([pz[e] for e in perm], device=dev, dtype=torch.float32)
    logits = (torch.randn((rows, E), generator=g, device=dev) + torch.log(p / p.sum())).contiguous()

    # Expert parallelism under the skewed load: popular experts are replicated so that every rank expects the same
    # number of rows (ReplicaPlacement). The expected load is the observed one of a calibration routing of this batch
    # (summed over the ranks), as a trainer would take it from the previous steps.
    placement = None
    if use_ep and not args.moe_no_replicas:
        rw0 = logits.clone()
        cfb.moe_topk_route_f32(rw0, rows, E, TOPK)
        load = (rw0 > 0).sum(dim=0).to(torch.float32)
        dist.all_reduce(load)
        placement = par.ReplicaPlacement.build(load.cpu().tolist(), world)
        local_ids = placement.local_experts(rank)
    else:
        local_ids = list(range(e_lo, e_hi))

    def quant_experts(shape, std, seed):
        amax = torch.zeros(4, dtype=torch.float32, device=dev)
        sc, de = torch.zeros_like(amax), torch.zeros_like(amax)
        w8 = torch.empty(shape, dtype=torch.uint8, device=dev)
        ws = []
        for e in local_ids:                             # replicas of one expert hold the same weights on every rank
            gw = torch.Generator(device=dev).manual_seed(seed + perm[e])
            ws.append((torch.randn(shape[1:], generator=gw, device=dev, dtype=torch.float32) * std).to(torch.bfloat16))
        wall = torch.stack(ws)
        cfb.fp8_amax_bf16(wall, amax)
        par.allreduce_max_(amax)                        # one per-tensor scale over all experts of all ranks
        cfb.fp8_scale_from_amax(amax, cfb.E4M3_MAX, sc, de)
        cfb.fp8_quantize_e4m3(wall, w8, sc)
        return w8, de

    n_local = len(local_ids)
    wgu8, dgu = quant_experts((n_local, 2 * F, H), 0.02, 50)
    wd8, dd = quant_experts((n_local, H, F), 0.02, 70)
    mixed = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
    fused_swiglu = (not args.moe_unfused_swiglu) or (use_ep and not args.moe_a2a)    # the device-planned form is fused only
    if fused_swiglu:
        wgu8 = cfb.fp8_interleave_gate_up(wgu8)       # one-time weight layout for the fused SwiGLU epilogue
    if use_ep and (not args.moe_a2a):
        layer = par.EpMoeSwigluFp8Direct(cfb, ctx, rows, H, F, E, TOPK, placement=placement, device=dev,
                                         fused_return=not args.moe_copy_return)
    elif use_ep:
        layer = par.EpMoeSwigluFp8(cfb, ctx, rows, H, F, E, TOPK, device=dev, fused_return=args.moe_fused_return,
                                   fused_swiglu=fused_swiglu, placement=placement)
    else:
        layer = cfb.MoeSwigluFp8(ctx, rows, H, F, E, TOPK, device=dev, fused_swiglu=fused_swiglu)

    def step():
        rw = logits.clone()
        layer.forward(x, rw, wgu8, dgu, wd8, dd, mixed, accumulate=False)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    ctx.poll_status()
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    l0 = cfb.launch_count()
    sampler.start()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    clocks = sampler.stop()
    launches = cfb.launch_count() - l0
    ctx.poll_status()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    loads = torch.tensor([float(layer.grp_counts.sum().item()) if (use_ep and (not args.moe_a2a)) else float(layer.plan.total_recv) if use_ep else float(rows * TOPK)], dtype=torch.float64, device=dev)
    lmax = loads.clone()
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(lmax, op=dist.ReduceOp.MAX)
    ms = t.item() / args.steps
    if rank == 0:
        flop = 2.0 * TOK * TOPK * 3 * H * F
        print(json.dumps({
            "metric": "moe_fp8_tokens_per_s", "value": TOK / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": "moe_swiglu_fp8_32768tok_H4096_E8_F14336_top2_zipf1.1 (BASELINE config 4)",
                       "parallelism": (f"ep{world} ({'device-planned dispatch, rows stored into the serving ranks over NVLink' if (not args.moe_a2a) else 'all-to-all'}, {'popular experts replicated: ' + str(placement.num_replicas) + ' replicas of ' + str(E) + ' experts' if placement else 'experts placed by load'}{', GEMM-fused return leg' if args.moe_fused_return else ''})" if use_ep else
                                       f"dp{world} (experts replicated, tokens sharded, no collective)") if world > 1 else "single GPU",
                       "swiglu": "fused into the gate/up GEMM epilogue" if fused_swiglu else "separate pass over the bf16 intermediate",
                       "max_rows_on_one_rank": int(lmax.item()), "mean_rows_per_rank": TOK * TOPK / world,
                       "l2": "inputs larger than L2 (1.4 GB of expert weights per step)"},
            "tflops": flop / (ms * 1e-3) / 1e12, "gpu_launches": int(launches), "clocks": clocks}), flush=True)
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def run_rowparallel(args):
    """Configuration-3 down projection (M 16384, N 4096, K 14336) with K sharded over the ranks: the strong-scaling
    form whose exchange is a reduce-scatter of the fp32 partial products. Two arms in one run: GEMM to fp32 + NCCL
    all-reduce + rounding, and the GEMM whose epilogue adds its tiles straight into the owners' slices (NVLink
    reduce-adds), followed by the bf16 read-out of this rank's rows."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    cfb = importlib.import_module("canopy-foundry_b200")
    par = cfb.parallel
    M, N, K = 16384, 4096, 14336
    k0, k1 = par.shard_range(K, world, rank, 128)
    Kl = k1 - k0
    ctx = cfb.Fp8Ctx(act8_bytes=0)
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    a8 = [torch.randint(0, 0x60, (M, Kl), generator=g, dtype=torch.uint8, device=dev) for _ in range(2)]
    w8 = torch.randint(0, 0x60, (N, Kl), generator=g, dtype=torch.uint8, device=dev)
    d = torch.full((4,), 2.0 ** -8, dtype=torch.float32, device=dev)
    y_full = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    partial = torch.empty((M, N), dtype=torch.float32, device=dev)
    y_slice = torch.empty((M // world, N), dtype=torch.bfloat16, device=dev)
    rs = par.RowParallelReduceScatterGemm(cfb, ctx, M, N, device=dev)
    it = [0]

    def step_nccl():
        it[0] += 1
        par.row_parallel_gemm_fp8(cfb, ctx, M, N, Kl, a8[it[0] & 1], d, w8, d, y_full, partial=partial)

    def step_fused():
        it[0] += 1
        rs.forward(a8[it[0] & 1], d, w8, d, y_slice)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() / args.steps

    sampler = ClockSampler(local)
    sampler.start()
    l0 = cfb.launch_count()
    ms_nccl = timed(step_nccl)
    ms_fused = timed(step_fused)
    launches = cfb.launch_count() - l0
    clocks = sampler.stop()
    ctx.poll_status()
    if rank == 0:
        flop = 2.0 * M * N * K
        print(json.dumps({
            "metric": "fp8_row_parallel_gemm_tflops", "value": flop / (ms_fused * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_fused, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": "fp8_down_projection_M16384_N4096_K14336 (BASELINE config 3), K sharded over the ranks",
                       "exchange": "reduce-scatter fused into the GEMM epilogue (bulk reduce-adds into the owners' slices)",
                       "l2": "two rotating activation shards, operands and output larger than L2"},
            "gemm_plus_nccl_allreduce": {"ms_per_step": ms_nccl, "tflops": flop / (ms_nccl * 1e-3) / 1e12,
                                         "note": "fp32 partial product + NCCL all-reduce + rounding; every rank ends with all rows"},
            "gpu_launches": int(launches), "clocks": clocks}), flush=True)
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def run_quantize(args):
    """HBM-bound side of the path on one GPU: the quantise family and the RMSNorm -> E4M3 fusion on 32768 x 4096 bf16
    activations (268 MB, three rotating inputs, all larger than L2). One step = one launch of each kernel; the line's
    value is the bandwidth of the steady-state activation kernel (record-quantise, 3 B/element)."""
    import torch

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    cfb = importlib.import_module("canopy-foundry_b200")
    peaks = load_peaks()
    rows, H = 32768, 4096
    n = rows * H
    g = torch.Generator(device=dev).manual_seed(3)
    xs = [torch.randn((rows, H), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16) for _ in range(3)]
    gamma = torch.ones(H, dtype=torch.bfloat16, device=dev)
    out8 = torch.empty((rows, H), dtype=torch.uint8, device=dev)
    out8t = torch.empty((H, rows), dtype=torch.uint8, device=dev)
    normed = torch.empty((rows, H), dtype=torch.bfloat16, device=dev)
    rms = torch.empty(rows, dtype=torch.float32, device=dev)
    rowd = torch.empty(rows, dtype=torch.float32, device=dev)
    scale = torch.full((4,), 20.0, dtype=torch.float32, device=dev)
    amax = torch.zeros(4, dtype=torch.float32, device=dev)
    it = [0]

    def nx():
        it[0] += 1
        return xs[it[0] % 3]

    kernels = [
        ("record_quantise_e4m3", 3, lambda: cfb.fp8_quantize_e4m3_record(nx(), out8, scale, amax)),
        ("amax_only", 2, lambda: cfb.fp8_amax_bf16(nx(), amax)),
        ("quantise_both_layouts", 4, lambda: cfb.fp8_quant_and_transpose_e4m3(nx(), out8, out8t, scale, rows, H)),
        ("rowwise_quantise_e4m3", 3, lambda: cfb.fp8_quantize_rowwise_e4m3(nx(), out8, rowd)),
        ("rmsnorm", 4, lambda: cfb.rmsnorm_forward(nx(), gamma, normed, rms, rows, H)),
        ("rmsnorm_record_quantise_keep_bf16", 5, lambda: cfb.rmsnorm_quantize_e4m3_record(nx(), gamma, normed, rms, out8, scale, amax, rows, H)),
        ("rmsnorm_record_quantise_e4m3_only", 3, lambda: cfb.rmsnorm_quantize_e4m3_record(nx(), gamma, None, rms, out8, scale, amax, rows, H)),
    ]
    sampler = ClockSampler(0)
    sampler.start()
    l0 = cfb.launch_count()
    res = {}
    for name, bpe, fn in kernels:
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        res[name] = {"ms": ms, "bytes_per_element": bpe, "GBps": bpe * n / (ms * 1e-3) / 1e9,
                     "frac_of_measured_hbm": bpe * n / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    launches = cfb.launch_count() - l0
    clocks = sampler.stop()
    head = res["record_quantise_e4m3"]
    print(json.dumps({
        "metric": "fp8_quantize_GBps", "value": head["GBps"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 -> fp8_e4m3", "data": "synthetic",
        "config": {"workload": "quantize_family_32768x4096_bf16 (BASELINE configuration 3/4 activation size)",
                   "l2": "three rotating 268 MB inputs, larger than L2"},
        "roofline": {"bound": "hbm", "kernel": "k_stream<e4m3, quantise, record>", "achieved": head["GBps"],
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": head["frac_of_measured_hbm"], "traffic": None,
                     "peak_source": f"STREAM-style copy figure of MEASURED_PEAKS.json ({peaks['source']})",
                     "frac_of_nominal_8000": head["GBps"] / 8000.0},
        "kernels": res, "gpu_launches": int(launches), "clocks": clocks}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the host-buffer leg (default min(steps, 20))")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--bias-mode", type=int, default=2, help="2 = reference rounding order, 1 = single rounding")
    ap.add_argument("--moe-unfused-swiglu", action="store_true", help="keep the [T,2F] bf16 intermediate (separate SwiGLU pass)")
    ap.add_argument("--moe-fused-return", action="store_true",
                    help="ep mode: the down GEMM stores its rows straight into the owners' buffers over NVLink (no return all-to-all)")
    ap.add_argument("--moe-copy-return", action="store_true",
                    help="device-planned form: write the results locally and copy them to their owners after the down GEMM "
                         "(default: the GEMM epilogue stores them straight into the owners' buffers)")
    ap.add_argument("--moe-a2a", action="store_true",
                    help="expert parallel through NCCL all-to-all with a host-side plan (default: plan, dispatch and return on "
                         "the device, rows stored straight into the serving ranks' buffers)")
    ap.add_argument("--moe-no-replicas", action="store_true",
                    help="expert parallel without replicas of the popular experts (one owner per expert, placed by load)")
    ap.add_argument("--moe-mode", default="ep", choices=["ep", "dp"],
                    help="N > 1: ep = expert parallel with all-to-all (experts placed by load), dp = experts replicated, tokens sharded")
    ap.add_argument("--workload", default="linear", choices=["linear", "moe", "rowparallel", "quantize"],
                    help="linear = BASELINE configuration 2 (the headline line); moe = configuration 4 tokens/s")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload == "rowparallel":
        return run_rowparallel(args)
    if args.workload == "quantize":
        return run_quantize(args)
    if args.workload == "moe":
        run_moe(args)
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfb = importlib.import_module("canopy-foundry_b200")

    dev = torch.device("cuda", local)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    xs = []
    for _ in range(N_ROTATE):
        x = torch.randn((M, K), generator=g, device=dev, dtype=torch.float32)
        x = torch.where(torch.rand((M, K), generator=g, device=dev) < 1e-3, x * 20.0, x)
        xs.append(x.to(torch.bfloat16))
        del x
    gw = torch.Generator(device=dev).manual_seed(99)       # the weight is replicated: same on every rank
    w = (torch.randn((N, K), generator=gw, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    bias = (torch.randn((N,), generator=gw, device=dev, dtype=torch.float32) * 0.01).to(torch.bfloat16)
    y = torch.empty((M, N), dtype=torch.bfloat16, device=dev)

    ctx = cfb.Fp8Ctx(act8_bytes=M * K)
    fw = cfb.Fp8Weight(w, stored_out_major=True)
    cfb.refresh_fp8_weight(fw, recompute_amax=True)          # initial amax; later steps reuse it (optimiser-provided)
    slot = cfb.ActSlot(ctx, cfb.E4M3_MAX, calib_calls=0)
    act8 = ctx.act8_ptr()
    import ctypes as C
    L = cfb._capi.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    epi = cfb._capi.GemmEpilogue(bias.data_ptr(), args.bias_mode, None, None)

    GEMM_EVENT_EVERY = 4     # CUDA events around the GEMM on every 4th step only: an event between two kernels
                             # keeps the second one from being scheduled behind the first (it serialises the stream)

    def step(i, ev=None):
        x = xs[i % N_ROTATE]
        cfb.refresh_fp8_weight(fw, recompute_amax=False)
        cfb._capi.check(L.cf_fp8_quant_act(ctx.handle, C.byref(slot.c), C.c_void_p(x.data_ptr()), M * K,
                                           C.c_void_p(act8), stream, 0))
        if ev is not None:
            ev[0].record()
        cfb._capi.check(L.cf_gemm_fp8_nt(ctx.handle, M, N, K, C.c_void_p(act8), K, 0, slot.c.descale_snapshot,
                                         C.c_void_p(fw.fwd8.data_ptr()), C.c_void_p(fw.descale.data_ptr()),
                                         C.c_void_p(y.data_ptr()), N, C.byref(epi), stream))
        if ev is not None:
            ev[1].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    ctx.poll_status()

    gemm_events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    barrier()
    launches0 = cfb.launch_count()
    sampler.start()
    e0.record()
    t_host0 = time.perf_counter()
    for i in range(args.steps):
        step(args.warmup + i, gemm_events[i] if i % GEMM_EVENT_EVERY == 0 else None)
    host_enqueue_ms = (time.perf_counter() - t_host0) * 1e3 / args.steps
    e1.record()
    barrier()
    clocks = sampler.stop()
    launches = cfb.launch_count() - launches0
    ctx.poll_status()
    ms_total = e0.elapsed_time(e1)
    timed = [gemm_events[i] for i in range(0, args.steps, GEMM_EVENT_EVERY)]
    gemm_ms = sum(a.elapsed_time(b) for a, b in timed) / len(timed)
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = t.item() / args.steps
    value = world * FLOP_PER_STEP / (ms_per_step * 1e-3) / 1e12

    # ---- host-buffer leg: pinned X in, pinned Y out, copies inside the timed region ----------------
    e2e_steps = args.e2e_steps or min(args.steps, 40)
    if args.no_e2e:
        e2e_steps = 0
    e2e_ms = e2e_val = None
    if e2e_steps > 0:
        # Three streams, double-buffered device X and Y: the H2D copy of step i+1 and the D2H copy of step i-1
        # run while step i computes (PCIe is full duplex). Every step still copies its own 67 MB in and its own
        # 67 MB result out inside the timed region; the delayed scale makes the steps independent of the copy order.
        hx = [torch.empty((M, K), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        for i in range(2):
            hx[i].copy_(xs[i])
        hy = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        xd = [torch.empty((M, K), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        yd = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        s_cmp = torch.cuda.current_stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_cmp = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def e2e_step(i):
            b = i % 2
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_cmp[b])                 # the step that last read xd[b] has finished
                xd[b].copy_(hx[b], non_blocking=True)
                ev_in[b].record(s_in)
            s_cmp.wait_event(ev_in[b])
            s_cmp.wait_event(ev_out[b])                    # the copy that last read yd[b] has finished
            cfb.refresh_fp8_weight(fw, recompute_amax=False)
            cfb.fp8_linear_forward(ctx, slot, xd[b], fw.fwd8, fw.descale, yd[b], bias=bias, bias_mode=args.bias_mode)
            ev_cmp[b].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[b])
                hy[b].copy_(yd[b], non_blocking=True)
                ev_out[b].record(s_out)

        for i in range(4):
            e2e_step(i)
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for i in range(e2e_steps):
            e2e_step(i)
        s_cmp.wait_event(ev_out[0])
        s_cmp.wait_event(ev_out[1])
        f1.record()
        barrier()
        t2 = torch.tensor([f0.elapsed_time(f1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        e2e_ms = t2.item() / e2e_steps
        e2e_val = world * FLOP_PER_STEP / (e2e_ms * 1e-3) / 1e12
        ctx.poll_status()
        # the result that reached the host is the result the device computed
        assert torch.equal(hy[(e2e_steps - 1) % 2], yd[(e2e_steps - 1) % 2].cpu()), "host copy of Y differs"

    if rank == 0:
        peaks = load_peaks()
        fp8_peak = 2.0 * peaks["bf16_tflops"]
        achieved = FLOP_PER_STEP / (gemm_ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": WORKLOAD, "M": M, "N": N, "K": K,
                       "step": "weight refresh (both layouts) + delayed-scale record-quantise of X + tcgen05 GEMM with fused dequant/bias",
                       "bias_mode": args.bias_mode, "sharding": "token shards per rank, replicated W, no collective" if world > 1 else "single GPU",
                       "l2": f"inputs larger than L2: {N_ROTATE} rotating activation buffers (201 MB) + 67 MB output per step"},
            "roofline": {"bound": "tensor", "kernel": "k_gemm_fp8_nt", "achieved": achieved, "peak": fp8_peak, "unit": UNIT,
                         "frac": achieved / fp8_peak, "traffic": 75.0e6,
                         "traffic_note": "dram__bytes_read+write per launch from the ncu capture in profiles/gemm_fp8_nt_pair_config2_8192x4096x4096.md",
                         "peak_source": f"2 x bf16 burst GEMM figure of MEASURED_PEAKS.json ({peaks['source']}); no FP8 figure is measured there",
                         "frac_of_nominal_4500": achieved / 4500.0, "gemm_ms": gemm_ms},
            "e2e": {"value": e2e_val, "unit": UNIT, "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2,
                    "how": "pinned host X in, pinned host Y out every step; copies double-buffered on two copy streams around the compute stream"},
            "gpu_launches": int(launches),
            "host_enqueue_ms_per_step": host_enqueue_ms,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            orc = oracle()
            threads = orc.lib.orc_hw_threads()
            rows, tsec, tf = cpu_sample(orc, 12.0, threads)
            line["cpu_baseline"] = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"{rows} rows ({rows / M:.2f} passes over the {M}-row batch) against the full W: record-quantise + GEMM + bias, {tsec:.1f} s"}
        print(json.dumps(line), flush=True)
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
