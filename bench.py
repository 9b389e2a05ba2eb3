#!/usr/bin/env python
"""Benchmark of the FP8 quantize-and-GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--legs linear,moe,mlp,sweep]

The headline line is the single-GPU FP8 linear (bf16 X[8192x4096], W[4096x4096]). One step = one pass of the path over
one batch resident in HBM:
    weight refresh   bf16 W -> E4M3 in both layouts with the amax the optimiser left (delayed amax)
    fp8_quant_act    bf16 X -> E4M3 with the previous step's scale, recording this step's amax, ring update
    FP8 GEMM         tcgen05, fp32 accumulate, fused dequant + bf16 bias epilogue, bf16 Y[8192x4096]
`value` is 2*M*N*K per step over the device time of the whole step (all ranks); `roofline` isolates the GEMM kernel with
CUDA events (burst), adds a seconds-long sustained loop and times the incumbent library GEMM (cuBLASLt through
torch._scaled_mm) on the same bytes; `e2e` repeats the step with pinned HOST input and output buffers and the copies
inside the timed region; `cpu_baseline` times the CPU oracle on a bounded row sample.

The same JSON line carries three more objects, one per remaining workload of the metric, each measured over the N ranks
of the run with its own parity check outside the timed region:
    "moe"    32768 tokens, hidden 4096, 8 SwiGLU experts of ffn 14336, top-2, Zipf(1.1) load: tokens/s, expert parallel
             over the N ranks (device-planned dispatch, rows stored into the serving ranks over NVLink), with the
             single-GPU layer timed on rank 0 of the same box beside it
    "mlp"    SwiGLU MLP 16384 x 4096 x 14336 with per-token x per-channel scales, gate/up sharded by output features and
             the down projection by its contraction dimension
    "sweep"  32768 x 8192 x 28672 E4M3 forward GEMM and the E5M2 x E4M3 dgrad of the same shape, N-sharded, the dgrad
             with and without its all-reduce
With N > 1 (torchrun, one rank per GPU) the headline leg runs on token shards against a replicated weight (weak scaling,
no collective); the other three legs are strong-scaling workloads with real exchanges. `--workload X` runs one leg (or
one of the side benches `rowparallel`, `quantize`) as its own line. `--impl reference` times the CPU restatement of the
reference's path on the host cores (the reference has no runnable CPU FP8 GEMM of its own).
"""
import argparse
import importlib
import json
import math
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
WORKLOAD = "fp8_linear_X8192x4096_W4096x4096_bf16_in_bf16_out"
STEP_TEXT = "weight refresh (both layouts) + delayed-scale record-quantise of X + tcgen05 GEMM with fused dequant/bias"
N_ROTATE = 3            # activation buffers rotated between steps: 3 x 67 MB > 126 MB of L2
PKG = "canopy-foundry_b200"


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d.get("hbm_gbs"), "bf16_tflops": d.get("bf16_tflops"),
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a timed region runs."""

    def __init__(self, index, interval_s=0.0005):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.interval = interval_s
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
            time.sleep(self.interval)

    def start(self):
        if self.nv:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thr:
            self._thr.join()
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


class NearGpuCpus:
    """Context manager: inside it this process runs on the CPUs NVML lists as local to the GPU, so that pinned host
    buffers allocated there are placed on the GPU's own NUMA node (the host<->device copies of the end-to-end leg then
    stay off the inter-socket link). The previous CPU set is restored on exit. A process attribute only; nothing about
    the GPU changes. `cpus` is the number of CPUs bound to, or None where NVML or the affinity call is unavailable."""

    def __init__(self, index):
        self.index, self.cpus, self._orig = index, None, None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
            near = {64 * w + b for w, mask in enumerate(words) for b in range(64) if (mask >> b) & 1}
            orig = os.sched_getaffinity(0)
            near &= orig
            if near and near != orig:
                os.sched_setaffinity(0, near)
                self._orig = orig
            self.cpus = len(near) if near else None
        except Exception:
            self.cpus = None
        return self

    def __exit__(self, *exc):
        if self._orig is not None:
            try:
                os.sched_setaffinity(0, self._orig)
            except Exception:
                pass
        return False


def oracle():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_bindings import Oracle
    return Oracle()


def synth_host(seed):
    """Inputs of the headline workload as numpy arrays: X ~ N(0,1) with 0.1 % of elements x20, W ~ N(0,0.02),
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


def linear_config(bias_mode, world):
    """The `config` object of the headline leg; the reference arm prints the same keys."""
    return {"workload": WORKLOAD, "M": M, "N": N, "K": K, "step": STEP_TEXT, "bias_mode": bias_mode,
            "sharding": "token shards per rank, replicated W, no collective" if world > 1 else "single GPU",
            "l2": f"inputs larger than L2: {N_ROTATE} rotating activation buffers (201 MB) + 67 MB output per step"}


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
        "config": linear_config(args.bias_mode, int(os.environ.get("WORLD_SIZE", "1"))),
        "cpu_baseline": {"value": tf, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ shared plumbing of the GPU legs
class Env:
    """One process per GPU: ranks, device, the package, and the barrier / timing helpers every leg uses."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)
        self.cfb = importlib.import_module(PKG)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, value):
        t = self.torch.tensor([float(value)], dtype=self.torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.item()

    def timed(self, fn, steps, warmup, sampler=None):
        """W untimed calls, then `steps` calls between two events, bracketed by barrier + synchronize on both sides;
        returns ms per call, the maximum over the ranks."""
        torch = self.torch
        for i in range(warmup):
            fn(i)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler:
            sampler.start()
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        e1.record()
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1)) / steps

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def median(xs):
    s = sorted(xs)
    return s[len(s) // 2] if s else None


def time_alone(torch, fn, iters, warmup=5):
    """ms per call of `fn` launched back to back on the current stream (CUDA events, after warm-up)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


# ------------------------------------------------------------------ headline leg: the FP8 linear
def leg_linear(args, env):
    import ctypes as C
    torch, cfb, dev, world = env.torch, env.cfb, env.dev, env.world

    g = torch.Generator(device=dev).manual_seed(1234 + env.rank)
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
    L = cfb._capi.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    epi = cfb._capi.GemmEpilogue(bias.data_ptr(), args.bias_mode, None, None)

    GEMM_EVENT_EVERY = 4     # inside the timed region CUDA events bracket the GEMM on every 4th step only: an event
                             # between two kernels keeps the second from being scheduled behind the first

    def gemm():
        cfb._capi.check(L.cf_gemm_fp8_nt(ctx.handle, M, N, K, C.c_void_p(act8), K, 0, slot.c.descale_snapshot,
                                         C.c_void_p(fw.fwd8.data_ptr()), C.c_void_p(fw.descale.data_ptr()),
                                         C.c_void_p(y.data_ptr()), N, C.byref(epi), stream))

    def step(i, ev=None):
        x = xs[i % N_ROTATE]
        cfb.refresh_fp8_weight(fw, recompute_amax=False)
        cfb._capi.check(L.cf_fp8_quant_act(ctx.handle, C.byref(slot.c), C.c_void_p(x.data_ptr()), M * K,
                                           C.c_void_p(act8), stream, 0))
        if ev is not None:
            ev[0].record()
        gemm()
        if ev is not None:
            ev[1].record()

    for i in range(args.warmup):
        step(i)
    ctx.poll_status()

    def ev_pair():
        return (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))

    gemm_events = [ev_pair() if i % GEMM_EVENT_EVERY == 0 else None for i in range(args.steps)]
    e0, e1 = ev_pair()
    sampler = ClockSampler(env.local)
    env.barrier()
    launches0 = cfb.launch_count()
    sampler.start()
    e0.record()
    t_host0 = time.perf_counter()
    for i in range(args.steps):
        step(args.warmup + i, gemm_events[i])
    host_enqueue_ms = (time.perf_counter() - t_host0) * 1e3 / args.steps
    e1.record()
    env.barrier()
    clocks = sampler.stop()
    launches = cfb.launch_count() - launches0
    ctx.poll_status()
    ms_per_step = env.max_over_ranks(e0.elapsed_time(e1)) / args.steps
    value = world * FLOP_PER_STEP / (ms_per_step * 1e-3) / 1e12
    in_region = [a.elapsed_time(b) for a, b in (p for p in gemm_events if p is not None)]
    # More GEMM samples than a short --steps gives: the same three-launch step repeated right after the timed region
    # with the events on every step (at least 32), so that the median does not rest on a handful of launches.
    extra = [ev_pair() for _ in range(max(32, args.steps))]
    for i, ev in enumerate(extra):
        step(args.warmup + args.steps + i, ev)
    torch.cuda.synchronize()
    samples = in_region + [a.elapsed_time(b) for a, b in extra]
    gemm_ms = median(samples)
    out = {"value": value, "ms_per_step": ms_per_step, "gemm_ms": gemm_ms, "gemm_samples": len(samples),
           "gemm_ms_in_timed_region": median(in_region), "launches": int(launches), "clocks": clocks,
           "host_enqueue_ms": host_enqueue_ms}

    state = dict(ctx=ctx, fw=fw, slot=slot, act8=act8, xs=xs, y=y, bias=bias, step=step, gemm=gemm)
    out["incumbent"] = linear_incumbent(args, env, state) if (env.rank == 0 and not args.no_incumbent) else None
    out["sustained"] = linear_sustained(args, env, state)
    out["e2e"] = None if args.no_e2e else linear_e2e(args, env, state)
    ctx.poll_status()
    ctx.close()
    return out


def linear_incumbent(args, env, st):
    """The library kernel the reference calls for this GEMM (cuBLASLt, src/trainer.cu:4516-4533), reached here through
    torch._scaled_mm, timed in the same process on the same FP8 bytes as this library's kernel, both launched back to
    back on their own (operands L2-warm for both). Two shapes: the headline 8192 x 4096 x 4096 and 8192^3."""
    torch, cfb, dev = env.torch, env.cfb, env.dev
    ctx, fw, slot, bias = st["ctx"], st["fw"], st["slot"], st["bias"]
    res = {"library": "cuBLASLt via torch._scaled_mm", "timing": "each kernel alone, back to back, same bytes, CUDA events"}
    f8 = torch.float8_e4m3fn
    iters = 40
    try:
        # headline shape: the E4M3 bytes of one activation buffer under the slot's snapshot scale
        x8 = torch.empty((M, K), dtype=torch.uint8, device=dev)
        cfb.fp8_quant_act(ctx, slot, st["xs"][0], x8, is_recompute=True)
        sa = torch.tensor(slot.scalars()["descale_snapshot"], dtype=torch.float32, device=dev)
        sb = fw.descale.reshape(()).clone()
        y_own = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        keep = {}

        def lib_gemm():
            keep["y"] = torch._scaled_mm(x8.view(f8), fw.fwd8.view(f8).t(), scale_a=sa, scale_b=sb, bias=bias,
                                         out_dtype=torch.bfloat16)

        def own_gemm():
            cfb.lt_gemm_fp8_nt(ctx, M, N, K, x8, K, False, cfb.ops._DevPtr(slot.c.descale_snapshot), fw.fwd8, fw.descale,
                               y_own, N, bias=bias, bias_mode=1)

        ms_lib = time_alone(torch, lib_gemm, iters)
        ms_own = time_alone(torch, own_gemm, iters)
        y_lib = keep.pop("y")
        diff = (y_lib.float() - y_own.float())
        res["8192x4096x4096"] = {
            "incumbent_cublaslt_tflops": FLOP_PER_STEP / (ms_lib * 1e-3) / 1e12, "incumbent_ms": ms_lib,
            "this_library_tflops": FLOP_PER_STEP / (ms_own * 1e-3) / 1e12, "this_library_ms": ms_own,
            "rel_fro_between_them": (diff.norm() / y_lib.float().norm()).item(),
            "bit_identical": bool(torch.equal(y_lib.view(torch.int16), y_own.view(torch.int16)))}
        # the same two kernels looped for about a second each (library first, then this one, then the library again): what
        # each holds under the power cap, with the SM clock it ran at
        if args.sustain_seconds > 0:
            def held(fn, ms_est):
                n = max(50, int(math.ceil(0.5 * args.sustain_seconds * 1e3 / max(ms_est, 1e-3))))
                sampler = ClockSampler(env.local, 0.0005)
                torch.cuda.synchronize()
                sampler.start()
                ms = time_alone(torch, fn, n, warmup=2)
                clk = sampler.stop()
                return {"tflops": FLOP_PER_STEP / (ms * 1e-3) / 1e12, "ms": ms, "seconds": ms * n * 1e-3,
                        "sm_mhz_median": clk["sm_mhz"], "reasons": clk["reasons"]}
            lib1 = held(lib_gemm, ms_lib)
            own1 = held(own_gemm, ms_own)
            lib2 = held(lib_gemm, ms_lib)
            res["8192x4096x4096"]["sustained"] = {"incumbent_cublaslt_first": lib1, "this_library": own1,
                                                  "incumbent_cublaslt_again": lib2}
            keep.pop("y", None)
        del x8, y_lib, y_own, diff
        # 8192^3 on seeded random E4M3 codes
        S = 8192
        g = torch.Generator(device=dev).manual_seed(77)
        a8 = torch.randint(0, 0x60, (S, S), generator=g, dtype=torch.uint8, device=dev)
        b8 = torch.randint(0, 0x60, (S, S), generator=g, dtype=torch.uint8, device=dev)
        d = torch.full((4,), 2.0 ** -10, dtype=torch.float32, device=dev)
        ds = d[0].reshape(()).clone()
        c_own = torch.empty((S, S), dtype=torch.bfloat16, device=dev)

        def lib_gemm2():
            keep["c"] = torch._scaled_mm(a8.view(f8), b8.view(f8).t(), scale_a=ds, scale_b=ds, out_dtype=torch.bfloat16)

        ms_lib = time_alone(torch, lib_gemm2, iters)
        c_lib = keep.pop("c")
        ms_own = time_alone(torch, lambda: cfb.lt_gemm_fp8_nt(ctx, S, S, S, a8, S, False, d, b8, d, c_own, S), iters)
        fl = 2.0 * S * S * S
        res["8192x8192x8192"] = {
            "incumbent_cublaslt_tflops": fl / (ms_lib * 1e-3) / 1e12, "incumbent_ms": ms_lib,
            "this_library_tflops": fl / (ms_own * 1e-3) / 1e12, "this_library_ms": ms_own,
            "rel_fro_between_them": ((c_lib.float() - c_own.float()).norm() / c_lib.float().norm()).item()}
    except Exception as e:  # noqa: BLE001  (an older torch without this signature: report, do not fail the bench)
        res["unavailable"] = f"{type(e).__name__}: {e}"[:300]
    return res


def linear_sustained(args, env, st):
    """Burst numbers of a 3 ms timed region run at the maximum clock; this loop runs the same three-launch step for at
    least `--sustain-seconds` (default 2 s), then the GEMM alone for a second, with the SM clock sampled every 0.5 ms,
    which is what the part holds under its power cap."""
    torch = env.torch
    if args.sustain_seconds <= 0:
        return None
    step, gemm = st["step"], st["gemm"]
    est = time_alone(torch, lambda: step(0), 20, warmup=2)
    n = max(50, int(math.ceil(args.sustain_seconds * 1e3 / est)))
    sampler = ClockSampler(env.local, 0.0005)
    env.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    e0.record()
    for i in range(n):
        step(i)
    e1.record()
    env.barrier()
    clk = sampler.stop()
    ms = env.max_over_ranks(e0.elapsed_time(e1)) / n
    out = {"seconds": ms * n * 1e-3, "steps": n, "ms_per_step": ms,
           "tflops": env.world * FLOP_PER_STEP / (ms * 1e-3) / 1e12, "sm_mhz_median": clk["sm_mhz"],
           "reasons": clk["reasons"], "clock_samples": clk["samples"],
           "ms_times_mhz": ms * clk["sm_mhz"] if clk["sm_mhz"] else None}
    ng = max(50, int(math.ceil(0.5 * args.sustain_seconds * 1e3 / max(est * 0.7, 1e-3))))
    sampler = ClockSampler(env.local, 0.0005)
    torch.cuda.synchronize()
    sampler.start()
    ms_g = time_alone(torch, gemm, ng, warmup=2)
    clk = sampler.stop()
    out["gemm_alone"] = {"seconds": ms_g * ng * 1e-3, "launches": ng, "ms": ms_g,
                         "tflops": FLOP_PER_STEP / (ms_g * 1e-3) / 1e12, "sm_mhz_median": clk["sm_mhz"],
                         "reasons": clk["reasons"], "ms_times_mhz": ms_g * clk["sm_mhz"] if clk["sm_mhz"] else None}
    return out


def linear_e2e(args, env, st):
    """Host-buffer leg: pinned X in, pinned Y out, copies inside the timed region. Three streams, double-buffered device
    X and Y: the H2D copy of step i+1 and the D2H copy of step i-1 run while step i computes (PCIe is full duplex).
    Every step still copies its own 67 MB in and its own 67 MB result out inside the timed region; the delayed scale
    makes the steps independent of the copy order. The pinned buffers are allocated while the process is bound to the
    GPU's own NUMA node; the bandwidth of each direction alone is measured beside the overlapped figure, so the limiter
    can be read from the line."""
    torch, cfb, dev = env.torch, env.cfb, env.dev
    ctx, fw, slot, bias, xs = st["ctx"], st["fw"], st["slot"], st["bias"], st["xs"]
    e2e_steps = args.e2e_steps or min(max(args.steps, 20), 40)
    with NearGpuCpus(env.local) as near:
        hx = [torch.empty((M, K), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        hy = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        for i in range(2):
            hx[i].copy_(xs[i])
            hy[i].zero_()
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
    env.barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    s_cmp.wait_event(ev_out[0])
    s_cmp.wait_event(ev_out[1])
    f1.record()
    env.barrier()
    e2e_ms = env.max_over_ranks(f0.elapsed_time(f1)) / e2e_steps
    ctx.poll_status()
    # the result that reached the host is the result the device computed
    assert torch.equal(hy[(e2e_steps - 1) % 2], yd[(e2e_steps - 1) % 2].cpu()), "host copy of Y differs"
    # each direction alone (all ranks copying at once, as in the leg above)
    env.barrier()
    h2d_ms = env.max_over_ranks(time_alone(torch, lambda: xd[0].copy_(hx[0], non_blocking=True), 8, warmup=2))
    env.barrier()
    d2h_ms = env.max_over_ranks(time_alone(torch, lambda: hy[0].copy_(yd[0], non_blocking=True), 8, warmup=2))
    # both directions at once (what the pipelined leg needs): PCIe is full duplex, but not at twice the one-way rate

    def duplex():
        with torch.cuda.stream(s_in):
            xd[0].copy_(hx[0], non_blocking=True)
        with torch.cuda.stream(s_out):
            hy[0].copy_(yd[0], non_blocking=True)

    def duplex_ms(iters=8):
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        s_in.wait_event(g0)
        s_out.wait_event(g0)
        for _ in range(iters):
            duplex()
        a, b = torch.cuda.Event(), torch.cuda.Event()
        a.record(s_in)
        b.record(s_out)
        s_cmp.wait_event(a)
        s_cmp.wait_event(b)
        g1.record()
        torch.cuda.synchronize()
        return g0.elapsed_time(g1) / iters

    duplex_ms(2)
    env.barrier()
    both_ms = env.max_over_ranks(duplex_ms())
    return {"value": env.world * FLOP_PER_STEP / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
            "steps": e2e_steps, "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * N * 2,
            "how": "pinned host X in, pinned host Y out every step; copies double-buffered on two copy streams around the compute stream",
            "h2d_GBps_per_rank_alone": M * K * 2 / (h2d_ms * 1e-3) / 1e9,
            "d2h_GBps_per_rank_alone": M * N * 2 / (d2h_ms * 1e-3) / 1e9,
            "copy_bound_ms_per_step": both_ms,
            "copy_bound_note": "one 67 MB copy in each direction at the same time, all ranks at once: the floor of a step of this leg",
            "copy_ms_one_direction_alone": max(h2d_ms, d2h_ms),
            "pinned_buffers_numa": f"allocated on the {near.cpus} CPUs NVML lists as local to the GPU" if near.cpus else "default placement (no NVML CPU affinity)"}


# ------------------------------------------------------------------ MoE leg: tokens/s, expert parallel over the ranks
MOE_TOK, MOE_H, MOE_F, MOE_E, MOE_TOPK = 32768, 4096, 14336, 8, 2
MOE_FLOP = 2.0 * MOE_TOK * MOE_TOPK * 3 * MOE_H * MOE_F


def moe_inputs(env, part, parts):
    """Tokens and router logits of shard `part` of `parts` (seeded per shard, so a run over fewer ranks sees the same
    tokens): x ~ N(0,1) bf16, logits ~ N(0,1) + log p_e with p_e ~ (e+1)^-1.1 (Zipf-skewed expert load)."""
    torch, dev = env.torch, env.dev
    rows = MOE_TOK // parts
    g = torch.Generator(device=dev).manual_seed(1000 + part)
    x = torch.randn((rows, MOE_H), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    p = torch.tensor([(e + 1) ** -1.1 for e in range(MOE_E)], device=dev, dtype=torch.float32)
    logits = (torch.randn((rows, MOE_E), generator=g, device=dev) + torch.log(p / p.sum())).contiguous()
    return x, logits


def moe_weights(env, expert_ids, allreduce):
    """E4M3 expert weights for `expert_ids` (seeded per expert: a replica holds the same bytes on every rank) with ONE
    per-tensor scale over all experts, as the reference keeps for a multi-expert block (src/trainer.cu:4284-4289)."""
    torch, cfb, dev = env.torch, env.cfb, env.dev

    def quant(shape, seed):
        amax = torch.zeros(4, dtype=torch.float32, device=dev)
        sc, de = torch.zeros_like(amax), torch.zeros_like(amax)
        w8 = torch.empty((len(expert_ids),) + shape, dtype=torch.uint8, device=dev)
        ws = []
        for e in expert_ids:
            gw = torch.Generator(device=dev).manual_seed(seed + e)
            ws.append((torch.randn(shape, generator=gw, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16))
        wall = torch.stack(ws)
        del ws
        cfb.fp8_amax_bf16(wall, amax)
        if allreduce:
            cfb.parallel.allreduce_max_(amax)
        cfb.fp8_scale_from_amax(amax, cfb.E4M3_MAX, sc, de)
        cfb.fp8_quantize_e4m3(wall, w8, sc)
        return w8, de

    wgu8, dgu = quant((2 * MOE_F, MOE_H), 50)
    wd8, dd = quant((MOE_H, MOE_F), 70)
    return wgu8, dgu, wd8, dd


def moe_oracle_check(env, x8_rows, weights_rows, sample, replica_expert, replica_scales, dx, wgu8_of, dgu, wd8_of, dd, got):
    """Host oracle on sampled tokens with the very scales the layer used. weights_rows [len(sample), V]: the sparse
    weights the layer combined with; replica v is expert replica_expert[v], re-quantised with replica_scales[v] =
    (scale, descale) of the SwiGLU slot of the rank that served it. Returns the relative Frobenius error."""
    import numpy as np
    orc = oracle()
    F = MOE_F
    want = np.zeros((len(sample), MOE_H), dtype=np.uint16)
    for v in range(weights_rows.shape[1]):
        hit = [i for i in range(len(sample)) if weights_rows[i, v] > 0]
        if not hit:
            continue
        e = replica_expert[v]
        sh, dh = (np.float32(q) for q in replica_scales[v])
        gu = orc.gemm_fp8_nt(np.ascontiguousarray(x8_rows[hit]), wgu8_of(e), np.float32(dx), np.float32(dgu))
        h = orc.swiglu_forward(np.ascontiguousarray(gu[:, :F]), np.ascontiguousarray(gu[:, F:]))
        ye = orc.gemm_fp8_nt(orc.quantize_bf16(h, sh), wd8_of(e), dh, np.float32(dd))
        for j, i in enumerate(hit):       # replicas ascend with the expert id: the single-GPU order of the bf16 additions
            want[i] = orc.to_bf16(orc.bf16_to_f32(want[i:i + 1]) + np.float32(weights_rows[i, v]) * orc.bf16_to_f32(ye[j:j + 1]))[0]
    wf = orc.bf16_to_f32(want)
    return float(np.linalg.norm(got.astype(np.float64) - wf) / max(np.linalg.norm(wf), 1e-30))


def leg_moe(args, env):
    """One step = route + dispatch lists + quantise + permute/dispatch + ragged gate/up GEMM with the SwiGLU re-quantise
    in its epilogue + ragged down GEMM (return leg in its epilogue) + unpermute/combine, for 32768 tokens in total.
    N > 1: expert parallel, device-planned (EpMoeSwigluFp8Direct), popular experts replicated by observed load; strong
    scaling. Rank 0 first runs the single-GPU layer over all tokens alone on the same box (`n1_ms_same_box`)."""
    import numpy as np
    torch, dist, cfb, dev, world, rank = env.torch, env.dist, env.cfb, env.dev, env.world, env.rank
    par = cfb.parallel
    TOK, H, F, E, TOPK = MOE_TOK, MOE_H, MOE_F, MOE_E, MOE_TOPK
    steps, warmup = args.steps, max(args.warmup, 3)
    ctx = cfb.Fp8Ctx(act8_bytes=0)
    res = {"workload": "moe_swiglu_fp8_32768tok_H4096_E8_F14336_top2_zipf1.1", "n_gpus": world, "steps": steps,
           "warmup": warmup, "scaling": "strong", "unit": "tokens/s"}

    # ---- single-GPU layer over all tokens (rank 0; the other ranks wait): the N = 1 point of the same box
    single = {}
    if rank == 0:
        xs, ls = zip(*[moe_inputs(env, r, world) for r in range(world)])
        x_all, logits_all = torch.cat(xs).contiguous(), torch.cat(ls).contiguous()
        del xs, ls
        wgu8_all, dgu, wd8_all, dd = moe_weights(env, list(range(E)), allreduce=False)
        wgu8_il = cfb.fp8_interleave_gate_up(wgu8_all)
        layer1 = cfb.MoeSwigluFp8(ctx, TOK, H, F, E, TOPK, device=dev, fused_swiglu=True)
        mixed1 = torch.zeros((TOK, H), dtype=torch.bfloat16, device=dev)
        rw1 = [None]

        def step1(i):
            rw1[0] = logits_all.clone()
            layer1.forward(x_all, rw1[0], wgu8_il, dgu, wd8_all, dd, mixed1, accumulate=False)

        for i in range(warmup):
            step1(i)
        sampler = ClockSampler(env.local, 0.002).start()
        l0 = cfb.launch_count()
        ms1 = time_alone(torch, lambda: step1(0), steps, warmup=0)
        single = {"ms": ms1, "clocks": sampler.stop(), "launches": int(cfb.launch_count() - l0)}
        ctx.poll_status()
        sample = [0, 1, TOK // world // 3, TOK // world - 1] if world > 1 else [0, 1, TOK // 3, TOK // 2, TOK - 1]
        hs = layer1.slot_h.scalars()
        err1 = moe_oracle_check(
            env, layer1.x8[sample].cpu().numpy(), rw1[0][sample].cpu().numpy(), sample, list(range(E)),
            [(hs["scale_snapshot"], hs["descale_snapshot"])] * E, layer1.slot_x.scalars()["descale_snapshot"],
            lambda e: wgu8_all[e].cpu().numpy(), dgu[0].item(), lambda e: wd8_all[e].cpu().numpy(), dd[0].item(),
            mixed1[sample].float().cpu().numpy())
        single["rel_fro_vs_oracle"] = err1
        del wgu8_il, layer1
    if world == 1:
        ms = single["ms"]
        res.update({"value": TOK / (ms * 1e-3), "ms_per_step": ms, "tflops": MOE_FLOP / (ms * 1e-3) / 1e12,
                    "parallelism": "single GPU", "n1_ms_same_box": ms, "max_rows_on_one_rank": TOK * TOPK,
                    "mean_rows_per_rank": TOK * TOPK, "clocks": single["clocks"], "gpu_launches": single["launches"],
                    "moe_parity": {"rel_fro": single["rel_fro_vs_oracle"], "ok": bool(single["rel_fro_vs_oracle"] < 1e-2),
                                   "tolerance": 1e-2, "against": "CPU oracle on sampled tokens with the layer's own scales"}})
        ctx.close()
        return res
    env.barrier()

    # ---- expert parallel over the ranks
    rows = TOK // world
    x, logits = moe_inputs(env, rank, world)
    rw0 = logits.clone()
    cfb.moe_topk_route_f32(rw0, rows, E, TOPK)
    load = (rw0 > 0).sum(dim=0).to(torch.float32)          # observed load of a calibration routing, summed over ranks
    dist.all_reduce(load)
    # pieces sized for equal tile work (rows + expected padding of each replica's last 256-row tile), not equal rows
    placement = par.ReplicaPlacement.build(load.cpu().tolist(), world, total_rows=TOK * TOPK, tile_rows=256)
    local_ids = placement.local_experts(rank)
    wgu8, dgu_l, wd8, dd_l = moe_weights(env, local_ids, allreduce=True)
    wgu8 = cfb.fp8_interleave_gate_up(wgu8)
    layer = par.EpMoeSwigluFp8Direct(cfb, ctx, rows, H, F, E, TOPK, placement=placement, device=dev)
    mixed = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)

    def step(i):
        layer.forward(x, logits.clone(), wgu8, dgu_l, wd8, dd_l, mixed, accumulate=False)

    sampler = ClockSampler(env.local, 0.002)
    l0 = cfb.launch_count()
    ms = env.timed(step, steps, warmup, sampler)
    clocks = sampler.stop()
    launches = int((cfb.launch_count() - l0) * steps / (steps + warmup))
    ctx.poll_status()
    lmax = env.max_over_ranks(float(layer.grp_counts.sum().item()))
    # where the time of one layer goes on this rank: CUDA events between the stages of one extra call (not timed above;
    # the events serialise the launches a little, so the stages add up to slightly more than a step)
    step(0)                       # keeps the GPU busy while the marked call is being queued (no launch gaps in it)
    layer.stage_marks = []
    step(0)
    torch.cuda.synchronize()
    marks, layer.stage_marks = layer.stage_marks, None
    stages = {marks[i][0]: round(marks[i - 1][1].elapsed_time(marks[i][1]), 4) for i in range(1, len(marks))}
    # the two GEMM stages and the rows served, of every rank (what the closing barrier of a layer waits for)
    mine_g = torch.tensor([stages.get("gate/up GEMM + SwiGLU + re-quantise", 0.0), stages.get("down GEMM with the return leg", 0.0),
                           float(layer.grp_counts.sum().item()), float((layer.grp_counts > 0).sum().item())],
                          dtype=torch.float32, device=dev)
    all_g = [torch.empty_like(mine_g) for _ in range(world)]
    dist.all_gather(all_g, mine_g)
    gemm_by_rank = [{"gate_up_ms": round(t[0].item(), 4), "down_ms": round(t[1].item(), 4), "rows": int(t[2].item()),
                     "groups": int(t[3].item())} for t in all_g]
    # ---- parity, outside the timed region: sampled tokens of rank 0 against the host oracle with the scales the ranks
    # used, and rank 0's rows against the single-GPU layer (other scale granularity: FP8 noise, reported, not gated)
    hs = layer.slot_h.scalars()
    mine = torch.tensor([hs["scale_snapshot"], hs["descale_snapshot"]], dtype=torch.float32, device=dev)
    allh = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(allh, mine)
    if rank == 0:
        scales = [tuple(allh[placement.replica_rank[v]].cpu().tolist()) for v in range(placement.num_replicas)]
        err = moe_oracle_check(
            env, layer.x8[sample].cpu().numpy(), layer.rwv[sample].cpu().numpy(), sample, placement.replica_expert, scales,
            layer.slot_x.scalars()["descale_snapshot"], lambda e: wgu8_all[e].cpu().numpy(), dgu[0].item(),
            lambda e: wd8_all[e].cpu().numpy(), dd[0].item(), mixed[sample].float().cpu().numpy())
        a, b = mixed.float(), mixed1[:rows].float()
        vs_single = ((a - b).norm() / b.norm()).item()
        res.update({
            "value": TOK / (ms * 1e-3), "ms_per_step": ms, "tflops": MOE_FLOP / (ms * 1e-3) / 1e12,
            "parallelism": f"ep{world}: device-planned dispatch, rows stored into the serving ranks over NVLink, return leg in the down GEMM's epilogue, {placement.num_replicas} replicas of {E} experts placed by observed load",
            "n1_ms_same_box": single["ms"], "n1_clocks": single["clocks"],
            "efficiency_vs_n1_same_box": single["ms"] / (world * ms),
            "max_rows_on_one_rank": int(lmax), "mean_rows_per_rank": TOK * TOPK / world, "clocks": clocks,
            "gpu_launches": launches, "stage_ms_rank0": stages, "gemm_stages_by_rank": gemm_by_rank,
            "moe_parity": {"rel_fro": err, "ok": bool(err < 1e-2 and single["rel_fro_vs_oracle"] < 1e-2), "tolerance": 1e-2,
                           "against": "CPU oracle on sampled tokens of rank 0 with the scales the serving ranks used",
                           "n1_layer_rel_fro_vs_oracle": single["rel_fro_vs_oracle"],
                           "rel_fro_vs_n1_layer_rows_of_rank0": vs_single,
                           "note": "the N=1 layer scales all tokens with one activation scale, a rank with its own: the two differ by FP8 quantisation noise"}})
    ctx.close()
    return res


# ------------------------------------------------------------------ SwiGLU MLP leg: per-token x per-channel scales, sharded
MLP_M, MLP_H, MLP_F = 16384, 4096, 14336
MLP_FLOP = 2.0 * MLP_M * 3 * MLP_H * MLP_F


def leg_mlp(args, env):
    """Llama-style SwiGLU MLP in FP8, tokens 16384, hidden 4096, ffn 14336, per-token activation scales and
    per-output-channel weight scales. One step = row-wise quantise of X, gate/up GEMM with SwiGLU and the per-row amax in
    its epilogue, [max-all-reduce of the row amax over the feature shards], row-wise quantise of h, down GEMM
    [+ reduce-scatter of the fp32 partial products]. Rank r holds features [r F/N, (r+1) F/N) of gate/up and the same
    slice of the down projection's contraction dimension; X is replicated; rank r ends with rows [r M/N, (r+1) M/N) of Y."""
    import numpy as np
    torch, dist, cfb, dev, world, rank = env.torch, env.dist, env.cfb, env.dev, env.world, env.rank
    par = cfb.parallel
    Mm, H, F = MLP_M, MLP_H, MLP_F
    Fl = F // world
    assert F % world == 0 and Fl % 128 == 0 and (Mm // world) % 256 == 0
    steps, warmup = args.steps, max(args.warmup, 3)
    ctx = cfb.Fp8Ctx(act8_bytes=0)
    g = torch.Generator(device=dev).manual_seed(31)            # X and the weights are the same on every rank
    xs = [torch.randn((Mm, H), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16) for _ in range(2)]

    def rowquant(w):
        w8 = torch.empty(w.shape, dtype=torch.uint8, device=dev)
        d = torch.empty(w.shape[0], dtype=torch.float32, device=dev)
        cfb.fp8_quantize_rowwise_e4m3(w, w8, d)
        return w8, d

    wgu8, dgu = rowquant((torch.randn((2 * F, H), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16))
    wd8, dd = rowquant((torch.randn((H, F), generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16))
    f0, f1 = rank * Fl, (rank + 1) * Fl
    il = cfb.fp8_interleave_gate_up(torch.cat([wgu8[f0:f1], wgu8[F + f0:F + f1]]).view(1, 2 * Fl, H)).view(2 * Fl, H)
    dil = cfb.interleave_gate_up_vector(torch.cat([dgu[f0:f1], dgu[F + f0:F + f1]]), Fl)
    wd8_l = wd8[:, f0:f1].contiguous()
    x8 = torch.empty((Mm, H), dtype=torch.uint8, device=dev)
    dx = torch.empty(Mm, dtype=torch.float32, device=dev)
    h = torch.empty((Mm, Fl), dtype=torch.bfloat16, device=dev)
    h8 = torch.empty((Mm, Fl), dtype=torch.uint8, device=dev)
    hmax = torch.empty(Mm, dtype=torch.float32, device=dev)
    dh = torch.empty(Mm, dtype=torch.float32, device=dev)
    one = torch.ones(4, dtype=torch.float32, device=dev)
    rows_out = Mm // world
    y = torch.empty((rows_out, H), dtype=torch.bfloat16, device=dev)
    partial = torch.empty((Mm, H), dtype=torch.float32, device=dev) if world > 1 else None
    part_rs = torch.empty((rows_out, H), dtype=torch.float32, device=dev) if world > 1 else None
    rs = par.RowParallelReduceScatterGemm(cfb, ctx, Mm, H, device=dev) if world > 1 else None

    def front(i):
        x = xs[i & 1]
        cfb.fp8_quantize_rowwise_e4m3(x, x8, dx)
        hmax.zero_()
        cfb.gemm_fp8_swiglu_bf16_rowamax(ctx, Mm, Fl, H, x8, H, False, None, dx, il, None, dil, h, hmax)
        if world > 1:
            dist.all_reduce(hmax, op=dist.ReduceOp.MAX)
        cfb.fp8_quantize_rowwise_given_amax_e4m3(h, h8, hmax, dh)

    def step_single(i):
        front(i)
        cfb.lt_gemm_fp8_nt(ctx, Mm, H, Fl, h8, Fl, False, one, wd8_l, one, y, H, a_row_descale=dh, b_col_descale=dd)

    def step_fused(i):
        front(i)
        rs.forward(h8, one, wd8_l, one, y, a_row_descale=dh, b_col_descale=dd)

    def step_nccl(i):
        front(i)
        cfb.lt_gemm_fp8_nt(ctx, Mm, H, Fl, h8, Fl, False, one, wd8_l, one, partial, H, a_row_descale=dh, b_col_descale=dd)
        dist.reduce_scatter_tensor(part_rs, partial)
        cfb.f32_to_bf16_and_zero(part_rs, y)

    # Pipelined form: the rows are cut into chunks (per-token scales make row chunks independent); the reduce-scatter of
    # chunk c runs on a second stream while the GEMMs of chunk c + 1 run. The small max-all-reduce of the row amax uses
    # its own communicator so that it does not queue behind the large reduce-scatter of the previous chunk. Rank r ends
    # with rows [r Mc/N, (r + 1) Mc/N) of every chunk.
    CH = 4
    Mc = Mm // CH
    pipelined_ok = world > 1 and Mc % (256 * world) == 0
    if pipelined_ok:
        comm = torch.cuda.Stream(device=dev)
        amax_group = dist.new_group(backend="nccl")
        ev_g = [torch.cuda.Event() for _ in range(CH)]
        ev_r = [torch.cuda.Event() for _ in range(CH)]
        y_p = torch.empty((rows_out, H), dtype=torch.bfloat16, device=dev)
        rs_out = torch.empty((rows_out, H), dtype=torch.float32, device=dev)
        rc = Mc // world

    def step_pipelined(i):
        x = xs[i & 1]
        main = torch.cuda.current_stream()
        for c in range(CH):
            r0, r1 = c * Mc, (c + 1) * Mc
            cfb.fp8_quantize_rowwise_e4m3(x[r0:r1], x8[r0:r1], dx[r0:r1])
            hmax[r0:r1].zero_()
            cfb.gemm_fp8_swiglu_bf16_rowamax(ctx, Mc, Fl, H, x8[r0:r1], H, False, None, dx[r0:r1], il, None, dil, h[r0:r1],
                                             hmax[r0:r1])
            dist.all_reduce(hmax[r0:r1], op=dist.ReduceOp.MAX, group=amax_group)
            cfb.fp8_quantize_rowwise_given_amax_e4m3(h[r0:r1], h8[r0:r1], hmax[r0:r1], dh[r0:r1])
            cfb.lt_gemm_fp8_nt(ctx, Mc, H, Fl, h8[r0:r1], Fl, False, one, wd8_l, one, partial[r0:r1], H,
                               a_row_descale=dh[r0:r1], b_col_descale=dd)
            ev_g[c].record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(ev_g[c])
                dist.reduce_scatter_tensor(rs_out[c * rc:(c + 1) * rc], partial[r0:r1])
                cfb.f32_to_bf16_and_zero(rs_out[c * rc:(c + 1) * rc], y_p[c * rc:(c + 1) * rc])
                ev_r[c].record(comm)
        for c in range(CH):
            main.wait_event(ev_r[c])

    partial_b = torch.empty((Mm, H), dtype=torch.bfloat16, device=dev) if world > 1 else None

    def step_nccl_bf16(i):
        # partial products rounded to bf16 before the exchange: half the bytes on the wire, one extra rounding per rank
        front(i)
        cfb.lt_gemm_fp8_nt(ctx, Mm, H, Fl, h8, Fl, False, one, wd8_l, one, partial_b, H, a_row_descale=dh, b_col_descale=dd)
        dist.reduce_scatter_tensor(y, partial_b)

    res = {"workload": "swiglu_mlp_fp8_M16384_H4096_F14336_per_token_x_per_channel_scales", "n_gpus": world,
           "steps": steps, "warmup": warmup, "scaling": "strong", "unit": UNIT,
           "sharding": "single GPU" if world == 1 else f"gate/up by output features ({Fl} per rank), down by its contraction dimension, X replicated, Y rows scattered"}
    l0 = cfb.launch_count()
    sampler = ClockSampler(env.local, 0.002)
    arms = {}
    if world == 1:
        arms["single"] = env.timed(step_single, steps, warmup, sampler)
        used = "single"
    else:
        arms["nccl_reduce_scatter"] = env.timed(step_nccl, steps, warmup, sampler)
        arms["gemm_fused_reduce_scatter"] = env.timed(step_fused, steps, warmup)
        if pipelined_ok:
            arms["nccl_reduce_scatter_pipelined_4_row_chunks"] = env.timed(step_pipelined, steps, warmup)
        used = min(arms, key=arms.get)          # among the forms that sum the partial products in fp32
        t_bf16 = env.timed(step_nccl_bf16, steps, warmup)
    clocks = sampler.stop()
    ctx.poll_status()
    ms = arms[used]
    # parity outside the timed region: sampled rows of this rank's slice against the host oracle on the full weights
    piped = used.startswith("nccl_reduce_scatter_pipelined")
    (step_single if world == 1 else step_pipelined if piped else step_fused if used == "gemm_fused_reduce_scatter" else step_nccl)(0)
    torch.cuda.synchronize()
    err = None
    if rank == 0:
        orc = oracle()
        local = [0, 255, 256, rows_out - 1]
        # rank 0's local row j is global row j, or (chunk, row in the chunk's share) in the pipelined form
        sample = [(j // rc) * Mc + j % rc for j in local] if piped else local
        if piped:
            y = y_p
        xr = xs[0][sample].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        q8, _, qd = orc.quantize_rowwise_e4m3(xr)
        gu = orc.gemm_fp8_nt(q8, wgu8.cpu().numpy(), qd, dgu.cpu().numpy())
        hq, _, hd = orc.quantize_rowwise_e4m3(np.ascontiguousarray(gu[:, :F]), np.ascontiguousarray(gu[:, F:]))
        want = orc.bf16_to_f32(orc.gemm_fp8_nt(hq, wd8.cpu().numpy(), hd, dd.cpu().numpy()))
        got = y[local].float().cpu().numpy()
        err = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    bf16_arm = None
    if world > 1:
        step_nccl_bf16(0)
        torch.cuda.synchronize()
        if rank == 0:
            got_b = y[[0, 255, 256, rows_out - 1]].float().cpu().numpy()
            want_b = want
            if piped:      # the bf16 arm scatters plain row slices: recompute the oracle rows for those
                xr2 = xs[0][[0, 255, 256, rows_out - 1]].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
                q2, _, qd2 = orc.quantize_rowwise_e4m3(xr2)
                gu2 = orc.gemm_fp8_nt(q2, wgu8.cpu().numpy(), qd2, dgu.cpu().numpy())
                hq2, _, hd2 = orc.quantize_rowwise_e4m3(np.ascontiguousarray(gu2[:, :F]), np.ascontiguousarray(gu2[:, F:]))
                want_b = orc.bf16_to_f32(orc.gemm_fp8_nt(hq2, wd8.cpu().numpy(), hd2, dd.cpu().numpy()))
            bf16_arm = {"ms_per_step": t_bf16, "tflops": MLP_FLOP / (t_bf16 * 1e-3) / 1e12,
                        "rel_fro_vs_oracle": float(np.linalg.norm(got_b - want_b) / np.linalg.norm(want_b)),
                        "note": "partial products rounded to bf16 and summed by NCCL in bf16: half the bytes, not bit-comparable with the fp32 sum"}
    nv_bytes = 0 if world == 1 else (world - 1) / world * Mm * H * 4
    res.update({"value": MLP_FLOP / (ms * 1e-3) / 1e12, "ms_per_step": ms, "exchange_used": used,
                "ms_per_step_by_exchange": arms, "bf16_partials": bf16_arm,
                "exchange": "none" if world == 1 else "max-all-reduce of float[M] row amax + reduce-scatter of the fp32 [M,H] partial products",
                "nvlink_bytes_sent_per_rank_per_step": nv_bytes,
                "nvlink_bound_ms_at_770GBps": nv_bytes / 770e9 * 1e3,
                "gemm_bound_ms_at_measured_peak": MLP_FLOP / world / (2 * load_peaks()["bf16_tflops"] * 1e12) * 1e3,
                "clocks": clocks, "gpu_launches": int(cfb.launch_count() - l0),
                "parity": {"rel_fro": err, "ok": bool(err is not None and err < 1e-2), "tolerance": 1e-2,
                           "against": "CPU oracle (row-wise quantise, GEMM, SwiGLU, re-quantise, GEMM) on sampled rows of rank 0"}})
    ctx.close()
    return res


# ------------------------------------------------------------------ large-shape sweep leg: forward and dgrad, N-sharded
SW_M, SW_K, SW_N, SW_CHUNKS = 32768, 8192, 28672, 8
SW_FLOP = 2.0 * SW_M * SW_K * SW_N


def leg_sweep(args, env):
    """E4M3 forward GEMM Y[32768, 28672] = A[32768, 8192] . W[28672, 8192]^T with W sharded by output columns, and the
    dgrad of the same shape, dX[32768, 8192] = dY[32768, 28672] (E5M2) . W (E4M3), whose contraction dimension is then
    the sharded one: every rank produces a partial dX that an all-reduce sums. Per-tensor scales (the weight's and the
    gradient's amax are max-all-reduced so every rank quantises with the single-GPU scale). Timed: the GEMMs (operands
    already quantised), the dgrad with and without its all-reduce."""
    import numpy as np
    torch, dist, cfb, dev, world, rank = env.torch, env.dist, env.cfb, env.dev, env.world, env.rank
    par = cfb.parallel
    Mm, Kk, Nn = SW_M, SW_K, SW_N
    assert SW_CHUNKS % world == 0
    cw = Nn // SW_CHUNKS                                   # columns per generation chunk (seeded per chunk: the tensors
    c0, c1 = rank * SW_CHUNKS // world, (rank + 1) * SW_CHUNKS // world   # are the same whatever the rank count)
    Nl = (c1 - c0) * cw
    steps, warmup = args.steps, max(args.warmup, 3)
    ctx = cfb.Fp8Ctx(act8_bytes=0)

    def scalars():
        return [torch.zeros(4, dtype=torch.float32, device=dev) for _ in range(3)]

    # A ~ N(0,1) -> E4M3 (replicated)
    g = torch.Generator(device=dev).manual_seed(200)
    a = torch.randn((Mm, Kk), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    am, sa, da = scalars()
    cfb.fp8_amax_bf16(a, am)
    cfb.fp8_scale_from_amax(am, cfb.E4M3_MAX, sa, da)
    a8 = torch.empty((Mm, Kk), dtype=torch.uint8, device=dev)
    cfb.fp8_quantize_e4m3(a, a8, sa)
    del a
    # W ~ N(0,0.02): this rank's column shard [Nl, K]
    w = torch.cat([(torch.randn((cw, Kk), generator=torch.Generator(device=dev).manual_seed(300 + c), device=dev,
                                dtype=torch.float32) * 0.02).to(torch.bfloat16) for c in range(c0, c1)])
    wm, sw, dw = scalars()
    cfb.fp8_amax_bf16(w, wm)
    par.allreduce_max_(wm)
    cfb.fp8_scale_from_amax(wm, cfb.E4M3_MAX, sw, dw)
    w8 = torch.empty((Nl, Kk), dtype=torch.uint8, device=dev)
    cfb.fp8_quantize_e4m3(w, w8, sw)
    del w
    wt8 = torch.empty((Kk, Nl), dtype=torch.uint8, device=dev)          # the dgrad's operand: [K, Nl], contraction-major
    cfb.transpose_u8(w8, wt8, Nl, Kk)
    # dY ~ N(0,1) * 1e-3 -> E5M2: this rank's columns [M, Nl]
    dy = torch.cat([(torch.randn((Mm, cw), generator=torch.Generator(device=dev).manual_seed(400 + c), device=dev,
                                 dtype=torch.float32) * 1e-3).to(torch.bfloat16) for c in range(c0, c1)], dim=1).contiguous()
    gm, sg, dg = scalars()
    cfb.fp8_amax_bf16(dy, gm)
    par.allreduce_max_(gm)
    cfb.fp8_scale_from_amax(gm, cfb.E5M2_MAX, sg, dg)
    dy8 = torch.empty((Mm, Nl), dtype=torch.uint8, device=dev)
    cfb.fp8_quantize_e5m2(dy, dy8, sg)
    del dy
    yout = torch.empty((Mm, Nl), dtype=torch.bfloat16, device=dev)
    dx_b = torch.empty((Mm, Kk), dtype=torch.bfloat16, device=dev)
    dx_f = torch.empty((Mm, Kk), dtype=torch.float32, device=dev) if world > 1 else None

    def fwd(i):
        cfb.lt_gemm_fp8_nt(ctx, Mm, Nl, Kk, a8, Kk, False, da, w8, dw, yout, Nl)

    def dgrad_gemm_bf16(i):
        # the reference's form: NT GEMM against the transposed weight cache (bwd8)
        cfb.lt_gemm_fp8_nt(ctx, Mm, Kk, Nl, dy8, Nl, True, dg, wt8, dw, dx_b, Kk)

    def dgrad_gemm_bf16_nn(i):
        # the same product with the weight read from the forward cache as it lies ([Nl, K] = [contraction, output])
        cfb.gemm_fp8_nn(ctx, Mm, Kk, Nl, dy8, Nl, True, dg, w8, Kk, dw, dx_b, Kk)

    def dgrad_gemm_f32(i):
        cfb.lt_gemm_fp8_nt(ctx, Mm, Kk, Nl, dy8, Nl, True, dg, wt8, dw, dx_f, Kk)

    def dgrad_f32_allreduce(i):
        dgrad_gemm_f32(i)
        dist.all_reduce(dx_f)

    def dgrad_bf16_allreduce(i):
        dgrad_gemm_bf16(i)
        dist.all_reduce(dx_b)

    dx_rs = torch.empty((Mm // world, Kk), dtype=torch.float32, device=dev) if world > 1 else None

    def dgrad_f32_reduce_scatter(i):
        # rank r keeps rows [r M/N, (r+1) M/N) of dX (sequence-parallel consumer): half the bytes of the all-reduce
        dgrad_gemm_f32(i)
        dist.reduce_scatter_tensor(dx_rs, dx_f)

    CH = 4
    Mc = Mm // CH
    if world > 1:
        comm = torch.cuda.Stream(device=dev)
        ev_g = [torch.cuda.Event() for _ in range(CH)]
        ev_r = [torch.cuda.Event() for _ in range(CH)]

    def dgrad_f32_allreduce_pipelined(i):
        # row chunks: the all-reduce of chunk c runs on a second stream while the GEMM of chunk c + 1 runs
        main = torch.cuda.current_stream()
        for c in range(CH):
            r0, r1 = c * Mc, (c + 1) * Mc
            cfb.lt_gemm_fp8_nt(ctx, Mc, Kk, Nl, dy8[r0:r1], Nl, True, dg, wt8, dw, dx_f[r0:r1], Kk)
            ev_g[c].record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(ev_g[c])
                dist.all_reduce(dx_f[r0:r1])
                ev_r[c].record(comm)
        for c in range(CH):
            main.wait_event(ev_r[c])

    l0 = cfb.launch_count()
    sampler = ClockSampler(env.local, 0.002)
    t_fwd = env.timed(fwd, steps, warmup, sampler)
    clocks = sampler.stop()
    t_dg = env.timed(dgrad_gemm_bf16, steps, warmup)
    t_dg_nn = env.timed(dgrad_gemm_bf16_nn, steps, warmup)
    fl = SW_FLOP
    res = {"workload": "fp8_gemm_M32768_K8192_N28672_forward_e4m3_and_dgrad_e5m2xe4m3", "n_gpus": world, "steps": steps,
           "warmup": warmup, "scaling": "strong", "unit": UNIT,
           "sharding": "single GPU" if world == 1 else f"W sharded by output columns ({Nl} per rank): forward needs no exchange, dgrad sums partial dX over the ranks",
           "forward": {"ms": t_fwd, "tflops": fl / (t_fwd * 1e-3) / 1e12},
           "dgrad_without_allreduce": {"ms": t_dg, "tflops": fl / (t_dg * 1e-3) / 1e12, "output": "bf16 (partial dX at N > 1)",
                                       "weight_operand": "transposed E4M3 cache [K, N] (the reference's bwd8), K-major tensor-core operand",
                                       "ms_reading_the_forward_cache_as_it_lies": t_dg_nn}}
    if world > 1:
        t_f32 = env.timed(dgrad_f32_allreduce, steps, warmup)
        t_b16 = env.timed(dgrad_bf16_allreduce, steps, warmup)
        t_pipe = env.timed(dgrad_f32_allreduce_pipelined, steps, warmup)
        t_rs = env.timed(dgrad_f32_reduce_scatter, steps, warmup)
        nbytes = Mm * Kk * 4
        res["dgrad_with_allreduce"] = {"ms": t_f32, "tflops": fl / (t_f32 * 1e-3) / 1e12,
                                       "exchange": "NCCL all-reduce(sum) of the fp32 [32768 x 8192] partial dX (1.07 GB)",
                                       "allreduce_bus_bound_ms_at_725GBps": 2 * (world - 1) / world * nbytes / 725e9 * 1e3}
        res["dgrad_with_allreduce_pipelined"] = {"ms": t_pipe, "tflops": fl / (t_pipe * 1e-3) / 1e12,
                                                 "exchange": "the same fp32 all-reduce in 4 row chunks on a second stream, overlapped with the GEMM of the next chunk"}
        res["dgrad_with_reduce_scatter"] = {"ms": t_rs, "tflops": fl / (t_rs * 1e-3) / 1e12,
                                            "exchange": "NCCL reduce-scatter of the fp32 partial dX: every rank keeps its M/N rows (for a consumer that is sharded by rows)"}
        res["dgrad_with_allreduce_bf16_partials"] = {"ms": t_b16, "tflops": fl / (t_b16 * 1e-3) / 1e12,
                                                     "exchange": "NCCL all-reduce(sum) of bf16 partial dX (0.54 GB); partial sums rounded to bf16 per hop"}
    ctx.poll_status()
    res["value"] = res["forward"]["tflops"]
    res["ms_per_step"] = t_fwd
    res["frac_of_2x_bf16_burst"] = res["value"] / world / (2 * load_peaks()["bf16_tflops"])
    res["clocks"] = clocks
    res["gpu_launches"] = int(cfb.launch_count() - l0)
    # ---- parity outside the timed region: sampled rows against the host oracle
    fwd(0)
    if world > 1:
        dgrad_f32_allreduce(0)
        shards = [torch.empty_like(w8) for _ in range(world)]
        dist.all_gather(shards, w8)
        sample = [0, 4097, Mm - 1]
        rows8 = dy8[sample].contiguous()
        rows_all = [torch.empty_like(rows8) for _ in range(world)]
        dist.all_gather(rows_all, rows8)
    else:
        dgrad_gemm_bf16(0)
        sample = [0, 4097, Mm - 1]
        shards, rows_all = [w8], [dy8[sample].contiguous()]
    torch.cuda.synchronize()
    if rank == 0:
        orc = oracle()
        w_host = w8.cpu().numpy()
        want = orc.bf16_to_f32(orc.gemm_fp8_nt(a8[sample].cpu().numpy(), w_host, da[0].item(), dw[0].item()))
        got = yout[sample].float().cpu().numpy()
        e_f = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        w_full = np.concatenate([s_.cpu().numpy() for s_ in shards], axis=0)               # [N, K]
        dy_rows = np.concatenate([r_.cpu().numpy() for r_ in rows_all], axis=1)            # [len(sample), N]
        wt = np.ascontiguousarray(w_full.T)                                                # [K, N]
        want_dx = orc.gemm_fp8_nt(dy_rows, wt, dg[0].item(), dw[0].item(), a_is_e5m2=True, out_kind=1)
        got_dx = (dx_f if world > 1 else dx_b)[sample].float().cpu().numpy()
        e_d = float(np.linalg.norm(got_dx - want_dx) / np.linalg.norm(want_dx))
        res["parity"] = {"forward_rel_fro": e_f, "dgrad_rel_fro": e_d, "ok": bool(e_f < 1e-2 and e_d < 1e-2),
                         "tolerance": 1e-2, "against": "CPU oracle on sampled rows (dgrad: the summed dX against the full contraction)"}
    ctx.close()
    return res


# ------------------------------------------------------------------ side benches
def run_rowparallel(args):
    """The SwiGLU MLP's down projection alone (M 16384, N 4096, K 14336) with K sharded over the ranks: the strong-scaling
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
    cfb = importlib.import_module(PKG)
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
            "config": {"workload": "fp8_down_projection_M16384_N4096_K14336, K sharded over the ranks",
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
    cfb = importlib.import_module(PKG)
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

    bad = torch.zeros(4, dtype=torch.int32, device=dev)
    sc2, de2 = torch.zeros(4, dtype=torch.float32, device=dev), torch.zeros(4, dtype=torch.float32, device=dev)
    ramax = torch.rand(rows, dtype=torch.float32, device=dev) + 3.0
    H2 = 4100                                            # rows that are not a multiple of 16 bytes: the plain form
    x_odd = torch.randn((rows, H2), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    out_odd = torch.empty((rows, H2), dtype=torch.uint8, device=dev)
    kernels = [
        ("record_quantise_e4m3", 3, n, lambda: cfb.fp8_quantize_e4m3_record(nx(), out8, scale, amax)),
        ("amax_only", 2, n, lambda: cfb.fp8_amax_bf16(nx(), amax)),
        ("quantise_both_layouts", 4, n, lambda: cfb.fp8_quant_and_transpose_e4m3(nx(), out8, out8t, scale, rows, H)),
        ("byte_transpose", 2, n, lambda: cfb.transpose_u8(out8, out8t, rows, H)),
        ("raw_pack_e4m3_two_pass", 5, n, lambda: cfb.fp8_pack_bf16_e4m3_raw(nx(), out8, amax, sc2, de2, bad)),
        ("rowwise_quantise_e4m3", 3, n, lambda: cfb.fp8_quantize_rowwise_e4m3(nx(), out8, rowd)),
        ("rowwise_quantise_given_amax", 3, n, lambda: cfb.fp8_quantize_rowwise_given_amax_e4m3(nx(), out8, ramax, rowd)),
        ("rowwise_quantise_e4m3_4100_columns", 3, rows * H2, lambda: cfb.fp8_quantize_rowwise_e4m3(x_odd, out_odd, rowd)),
        ("rmsnorm", 4, n, lambda: cfb.rmsnorm_forward(nx(), gamma, normed, rms, rows, H)),
        ("rmsnorm_record_quantise_keep_bf16", 5, n, lambda: cfb.rmsnorm_quantize_e4m3_record(nx(), gamma, normed, rms, out8, scale, amax, rows, H)),
        ("rmsnorm_record_quantise_e4m3_only", 3, n, lambda: cfb.rmsnorm_quantize_e4m3_record(nx(), gamma, None, rms, out8, scale, amax, rows, H)),
        ("rmsnorm_clip_record_quantise_e4m3_only", 3, n, lambda: cfb.rmsnorm_clip_quantize_e4m3_record(nx(), gamma, None, rms, out8, scale, amax, rows, H, 1000.0)),
        ("rmsnorm_rowwise_quantise_e4m3_only", 3, n, lambda: cfb.rmsnorm_quantize_rowwise_e4m3(nx(), gamma, None, rms, out8, rowd, rows, H)),
    ]
    # optimiser pass: plain Lion step (fp32 state: 4 B gradient + 8 B momentum + 4 B master per element), Lion step that
    # also writes both E4M3 caches (+ 2 B), and the stand-alone refresh it replaces (2 B read + 2 B written)
    lw = xs[0].clone()
    lm = torch.zeros((rows, H), dtype=torch.float32, device=dev)
    lg = torch.randn((rows, H), generator=g, device=dev, dtype=torch.float32)
    am_a, am_b = torch.ones(4, dtype=torch.float32, device=dev), torch.zeros(4, dtype=torch.float32, device=dev)
    fwl = cfb.Fp8Weight(lw, stored_out_major=True)
    fwl.amax.fill_(4.0)
    hp = (1e-4, 0.9, 0.99, 0.0)
    kernels += [
        ("lion_step_f32_state", 16, n, lambda: cfb.lion_step(lw.view(-1), lm.view(-1), lg.view(-1), *hp, weight_amax=am_b, sr_seed=1)),
        ("lion_step_f32_state_with_both_e4m3_caches", 18, n, lambda: cfb.lion_step_quantize(lw, lm, lg, *hp, am_b, am_a, sc2, de2, out8, out8t, sr_seed=1)),
        ("weight_refresh_both_layouts", 4, n, lambda: cfb.refresh_fp8_weight(fwl, recompute_amax=False)),
    ]
    sampler = ClockSampler(0)
    sampler.start()
    l0 = cfb.launch_count()
    res = {}
    for name, bpe, ne, fn in kernels:
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
        res[name] = {"ms": ms, "bytes_per_element": bpe, "GBps": bpe * ne / (ms * 1e-3) / 1e9,
                     "frac_of_measured_hbm": bpe * ne / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    launches = cfb.launch_count() - l0
    clocks = sampler.stop()
    head = res["record_quantise_e4m3"]
    print(json.dumps({
        "metric": "fp8_quantize_GBps", "value": head["GBps"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": head["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 -> fp8_e4m3", "data": "synthetic",
        "config": {"workload": "quantize_family_32768x4096_bf16",
                   "l2": "three rotating 268 MB inputs, larger than L2"},
        "roofline": {"bound": "hbm", "kernel": "k_stream<e4m3, quantise, record>", "achieved": head["GBps"],
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": head["frac_of_measured_hbm"], "traffic": None,
                     "peak_source": f"STREAM-style copy figure of MEASURED_PEAKS.json ({peaks['source']})",
                     "frac_of_nominal_8000": head["GBps"] / 8000.0},
        "kernels": res, "gpu_launches": int(launches), "clocks": clocks}), flush=True)




LEGS = {"moe": leg_moe, "mlp": leg_mlp, "sweep": leg_sweep}


def run_default(args):
    """The line the driver reads: the headline leg plus one object per remaining workload of the metric."""
    env = Env()
    legs = [x for x in args.legs.split(",") if x]
    lin = leg_linear(args, env)
    extra = {}
    for name in ("moe", "mlp", "sweep"):
        if name in legs:
            env.barrier()
            env.torch.cuda.empty_cache()
            extra[name] = LEGS[name](args, env)
    if env.rank == 0:
        peaks = load_peaks()
        fp8_peak = 2.0 * peaks["bf16_tflops"]
        achieved = FLOP_PER_STEP / (lin["gemm_ms"] * 1e-3) / 1e12
        inc = (lin["incumbent"] or {})
        inc2 = inc.get("8192x4096x4096", {})
        sus = lin["sustained"] or {}
        roofline = {
            "bound": "tensor", "kernel": "k_gemm_fp8_nt", "achieved": achieved, "peak": fp8_peak, "unit": UNIT,
            "frac": achieved / fp8_peak,
            "traffic": 75.0e6, "traffic_measured_in_run": False,
            "traffic_note": "dram__bytes_read + dram__bytes_write of one launch of this kernel at this shape from an ncu capture taken on 2026-11-25 (117.4 MB algorithmic: the operands partly stay in L2 between the quantiser and the GEMM); not re-measured by this run",
            "peak_source": f"2 x bf16 burst GEMM figure of MEASURED_PEAKS.json ({peaks['source']}); that file holds no FP8 figure, the library FP8 GEMM timed in this run is `incumbent_cublaslt_tflops`",
            "frac_of_nominal_4500": achieved / 4500.0, "gemm_ms": lin["gemm_ms"], "gemm_samples": lin["gemm_samples"],
            "gemm_ms_in_timed_region": lin["gemm_ms_in_timed_region"],
            "timing": "CUDA events around the GEMM launch on the launching stream: every 4th step of the timed region plus every step of an identical loop run right after it; median (burst clocks: the region lasts milliseconds)",
            "incumbent_cublaslt_tflops": inc2.get("incumbent_cublaslt_tflops"),
            "frac_of_incumbent": (inc2.get("this_library_tflops") / inc2["incumbent_cublaslt_tflops"]) if inc2.get("incumbent_cublaslt_tflops") else None,
            "incumbent": inc,
            "sustained": dict(sus, **{
                "frac_of_2x_bf16_sustained": (sus.get("gemm_alone", {}).get("tflops") / (2.0 * peaks["bf16_tflops_sustained"])) if sus.get("gemm_alone") and peaks.get("bf16_tflops_sustained") else None,
                "note": "same three-launch step looped for seconds, then the GEMM alone; SM clock sampled every 0.5 ms"}) if sus else None,
        }
        line = {
            "metric": METRIC, "value": lin["value"], "unit": UNIT, "n_gpus": env.world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": lin["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
            "config": linear_config(args.bias_mode, env.world),
            "roofline": roofline,
            "e2e": lin["e2e"],
            "gpu_launches": lin["launches"],
            "host_enqueue_ms_per_step": lin["host_enqueue_ms"],
            "clocks": dict(lin["clocks"], note="sampled during the timed region of the headline leg (milliseconds at a small --steps); roofline.sustained carries thousands of samples over seconds"),
        }
        line.update(extra)
        if env.world == 1 and not args.no_cpu_baseline:
            orc = oracle()
            threads = orc.lib.orc_hw_threads()
            rows, tsec, tf = cpu_sample(orc, 12.0, threads)
            line["cpu_baseline"] = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"{rows} rows ({rows / M:.2f} passes over the {M}-row batch) against the full W: record-quantise + GEMM + bias, {tsec:.1f} s"}
        print(json.dumps(line), flush=True)
    env.close()


def run_one_leg(args, name):
    """`--workload moe|mlp|sweep`: that leg alone as its own JSON line (profiling, sweeps)."""
    env = Env()
    res = LEGS[name](args, env)
    if env.rank == 0:
        metric = {"moe": "moe_fp8_tokens_per_s", "mlp": "fp8_swiglu_mlp_tflops", "sweep": "fp8_large_gemm_tflops"}[name]
        line = {"metric": metric, "value": res.get("value"), "unit": res.get("unit"), "n_gpus": env.world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": res.get("ms_per_step"),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "fp8_e4m3 (fp32 accumulate)", "data": "synthetic",
                "config": {"workload": res.get("workload"), "l2": "operands and outputs larger than L2"},
                "gpu_launches": res.get("gpu_launches"), "clocks": res.get("clocks"), name: res}
        print(json.dumps(line), flush=True)
    env.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the host-buffer leg (default: steps, within 20..40)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-incumbent", action="store_true", help="skip the library-GEMM comparison (profiling runs)")
    ap.add_argument("--bias-mode", type=int, default=2, help="2 = reference rounding order, 1 = single rounding")
    ap.add_argument("--sustain-seconds", type=float, default=2.0, help="length of the sustained loop of the headline leg (0 = skip)")
    ap.add_argument("--legs", default="linear,moe,mlp,sweep",
                    help="objects the default line carries beside the headline leg (comma list of moe, mlp, sweep)")
    ap.add_argument("--workload", default="linear", choices=["linear", "moe", "mlp", "sweep", "rowparallel", "quantize"],
                    help="linear = the headline line with the legs of --legs; any other name = that workload alone")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "rowparallel":
        return run_rowparallel(args)
    if args.workload == "quantize":
        return run_quantize(args)
    if args.workload in LEGS:
        return run_one_leg(args, args.workload)
    return run_default(args)


if __name__ == "__main__":
    main()
