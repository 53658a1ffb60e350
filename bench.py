#!/usr/bin/env python
"""bench.py -- throughput of the B200 path against its roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" is one pass of a workload over its synthetic input. The headline line
is saxpy (y = 2.5*x + y, N = 2^30 elements per GPU, 12 bytes of HBM traffic per
element); the other workloads of the path (vector add, int32/fp32 sum, fp32 GEMM,
Asian-option Monte Carlo) are measured in the same run and reported under
"workloads" in the same JSON line. Multi-GPU runs are one process per GPU: every
rank works on its own contiguous shard (weak scaling), the sum and the pricer end
in one NCCL all-reduce issued by libbooth_sm100 itself; torch.distributed (gloo)
only carries the barrier, the NCCL id and the max-over-ranks of the timings.

All device work goes through the C ABI of libbooth_sm100.so (ctypes); timing is
by CUDA events recorded on the stream that library launches on.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 0xB0070000
LOG2_STREAM = 30            # saxpy / reduce elements per GPU
LOG2_VADD = 24              # BASELINE config 0
LOG2_PATHS = 26             # Monte Carlo paths per GPU
NSTEP = 252
GEMM_SIZES = (4096, 8192)
BYTES_PER_ELEM = {"saxpy": 12, "vadd": 12, "reduce": 4}
# DRAM bytes per element per launch as counted by ncu (dram__bytes_read.sum +
# dram__bytes_write.sum); see the summaries under profiles/. None = not captured.
NCU_TRAFFIC_PER_ELEM = {"saxpy": 11.67, "vadd": 11.77, "reduce_i32": 4.03, "reduce_f32": 4.03}


def measured_peaks():
    """Roofline denominators: the pool's measured copy bandwidth and bf16 GEMM rate."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML (read-only) every
    few milliseconds while a timed region runs; nvidia-smi is the fallback."""
    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))

    def __init__(self, index, period_s=0.004):
        self.index, self.period = index, period_s
        self.rows, self.stop_flag, self.thread, self.nvml = [], threading.Event(), None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None

    def start(self):
        self.rows, self.stop_flag = [], threading.Event()
        if self.nvml is None:
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        n = self.nvml
        while not self.stop_flag.is_set():
            try:
                sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                pw = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                try:
                    rs = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    rs = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.rows.append((sm, pw, rs))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        if self.nvml is None:
            return self._smi_once()
        self.stop_flag.set()
        self.thread.join(timeout=5)
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": float(self.sm_max), "reasons": ["no samples"]}
        reasons = sorted(name for name, bit in self.REASONS if any(r[2] & bit for r in self.rows))
        return {"sm_mhz": float(np.median([r[0] for r in self.rows])), "sm_max_mhz": float(self.sm_max),
                "sm_min_mhz": float(min(r[0] for r in self.rows)), "power_w_max": max(r[1] for r in self.rows),
                "samples": len(self.rows), "reasons": reasons, "source": "nvml"}

    def _smi_once(self):
        fields = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
                  "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                  "clocks_event_reasons.sw_power_cap")
        try:
            out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + fields,
                                  "--format=csv,noheader,nounits"], stdout=subprocess.PIPE, text=True, timeout=20).stdout
            r = [c.strip() for c in out.strip().split(",")]
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            return {"sm_mhz": float(r[0]), "sm_max_mhz": float(r[1]), "power_w_max": float(r[2]), "samples": 1,
                    "reasons": [n for n, v in zip(names, r[3:7]) if v.lower().startswith("active")],
                    "source": "nvidia-smi after the timed region"}
        except Exception as e:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable: %s" % e]}


class Ranks:
    """Process group plumbing: gloo for control, device chosen by LOCAL_RANK."""

    def __init__(self, gpus):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("gloo")
            self.dist = dist
        if gpus != self.world:
            if self.rank == 0:
                sys.stderr.write("bench: --gpus %d but WORLD_SIZE %d; launch through torch.distributed.run "
                                 "for N>1\n" % (gpus, self.world))
            raise SystemExit(2)

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def max(self, v):
        if not self.dist:
            return float(v)
        import torch
        t = torch.tensor([float(v)], dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t[0])

    def bcast_bytes(self, b):
        if not self.dist:
            return b
        box = [b]
        self.dist.broadcast_object_list(box, src=0)
        return box[0]

    def close(self):
        if self.dist:
            self.dist.barrier()
            self.dist.destroy_process_group()


def timed(dev, ranks, warmup, steps, body):
    """W untimed steps, then exactly K steps between two events on the library's
    stream, a barrier and a stream sync on both sides; max over ranks, in ms."""
    for _ in range(warmup):
        body()
    dev.sync()
    ranks.barrier()
    dev.tic()
    for _ in range(steps):
        body()
    ms = dev.toc()
    dev.sync()
    ranks.barrier()
    return ranks.max(ms)


def timed_short(dev, ranks, warmup, steps, body, repeats=3):
    """For kernels that run for tens of microseconds: the median of `repeats` timed
    runs of K steps each, so that one disturbed half-millisecond window (a clock
    sample, a host interrupt) does not decide the figure."""
    runs = sorted(timed(dev, ranks, warmup if r == 0 else 1, steps, body) for r in range(repeats))
    return runs[len(runs) // 2]


def mufu_ceiling(path_steps_per_s, sm_count, clocks):
    """The pricer is bound by the special-function unit, not by HBM or the tensor
    pipe: 3 MUFU operations per path-step on 16 MUFU lanes per SM allow at most
    16/3 path-steps per clock per SM. Reported per GPU at the SM clock sampled
    during the timed region."""
    mhz = clocks.get("sm_mhz") or clocks.get("sm_max_mhz")
    if not mhz:
        return None
    achieved = path_steps_per_s / (sm_count * mhz * 1e6)
    return {"bound": "mufu issue", "achieved": achieved, "peak": 16.0 / 3.0, "unit": "path-steps/clk/SM",
            "frac": achieved / (16.0 / 3.0), "sm_mhz": mhz}


def roofline(bound, achieved, peak, unit, traffic, peaks):
    return {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
            "frac": achieved / peak if peak else None, "traffic": traffic,
            "peak_source": "of " + peaks["source"]}


def run_ours(args):
    import booth_b200 as sm
    ranks = Ranks(args.gpus)
    peaks = measured_peaks()
    dev = sm.Device(ranks.local)
    comm = None
    if ranks.world > 1:
        uid = ranks.bcast_bytes(sm.Comm.unique_id() if ranks.rank == 0 else None)
        comm = sm.Comm(dev, ranks.world, ranks.rank, uid)
    W, K = max(args.warmup, 3), args.steps
    G = ranks.world
    workloads = []
    sampler = ClockSampler(ranks.local)

    n = 1 << args.log2n
    first = ranks.rank * n                      # this rank's contiguous shard of the global vectors
    dx, dy = dev.alloc(n * 4), dev.alloc(n * 4)
    dev.fill(dx, first, n, SEED + 1, 0, sm.FILL_F32_PM1)
    dev.fill(dy, first, n, SEED + 1, 1, sm.FILL_F32_PM1)
    dev.sync()

    # ---- headline: saxpy, inputs resident in HBM ----
    sampler.start()
    l0 = dev.launches
    ms = timed(dev, ranks, W, K, lambda: dev.saxpy(dy, dx, 2.5, n))
    launches = dev.launches - l0 - W
    clocks = sampler.stop()
    saxpy_ms = ms / K
    saxpy_gbs = BYTES_PER_ELEM["saxpy"] * n * G / (saxpy_ms * 1e-3) / 1e9
    per_gpu = saxpy_gbs / G
    t_el = NCU_TRAFFIC_PER_ELEM["saxpy"]
    head_roof = roofline("hbm", per_gpu, peaks["hbm_gbs"], "GB/s", t_el * n if t_el else None, peaks)
    head_roof["frac_of_nominal_8TBs"] = per_gpu / 8000.0

    # ---- e2e: the launcher API with host buffers (the examples/launch_saxpy.c flow) ----
    e2e = None if args.no_e2e else run_e2e_saxpy(sm, dev, ranks, n, max(1, min(K, args.e2e_steps)))
    want = set(args.workloads.split(",")) if args.workloads != "all" else {"sweep", "vadd", "reduce", "asian", "gemm"}
    if args.headline_only:
        want = set()

    # ---- size sweep (config 1) and vector add (config 0) ----
    if "sweep" in want:
        sweep = []
        for lg in range(20, args.log2n + 1, 2):
            m = 1 << lg
            t = (timed_short if lg < 28 else timed)(dev, ranks, W, K, lambda: dev.saxpy(dy, dx, 2.5, m)) / K
            sweep.append({"log2n": lg, "ms": t, "gbs_per_gpu": 12.0 * m / (t * 1e-3) / 1e9})
        workloads.append({"name": "saxpy_sweep", "unit": "GB/s per GPU", "note": "sizes below ~2^25 fit the 126 MB L2; points below 2^28 are the median of 3 runs of K steps",
                          "points": sweep})
    if "vadd" in want:
        for lg in (LOG2_VADD, min(28, args.log2n)):
            m = 1 << lg
            dz = dev.alloc(m * 4)
            t = (timed_short if lg < 28 else timed)(dev, ranks, W, K, lambda: dev.vadd(dx, dy, dz, m)) / K
            gbs = 12.0 * m / (t * 1e-3) / 1e9
            workloads.append({"name": "vadd_2^%d" % lg, "metric": "hbm_gbs", "value": gbs * G, "unit": "GB/s",
                              "ms_per_step": t,
                              "roofline": roofline("hbm", gbs, peaks["hbm_gbs"], "GB/s",
                                                   NCU_TRAFFIC_PER_ELEM["vadd"] * m if lg > 26 else None, peaks),
                              "note": "201 MB working set, partly L2-resident; median of 3 runs of K steps" if lg == LOG2_VADD else "3 GiB working set"})
            dev.free(dz)

    out = dev.alloc(64)
    if "reduce" in want:
        # ---- reduction (config 2): per-GPU sum then one NCCL all-reduce ----
        for name, kind, fn, dt in (("reduce_i32", sm.FILL_I32_1000, dev.reduce_i32, sm.I32),
                                   ("reduce_f32", sm.FILL_F32_01, dev.reduce_f32, sm.F64)):
            dev.fill(dx, first, n, SEED + 2, 0 if dt == sm.I32 else 1, kind)

            def step():
                fn(dx, n, out)
                if comm:
                    comm.allreduce_sum(out, 1, dt)
            t = timed(dev, ranks, W, K, step) / K
            res = dev.download(out, 1, np.int32 if dt == sm.I32 else np.float64)[0]
            gbs = 4.0 * n / (t * 1e-3) / 1e9
            workloads.append({"name": name + "_2^%d" % args.log2n, "metric": "hbm_gbs", "value": gbs * G, "unit": "GB/s",
                              "ms_per_step": t, "result": float(res), "allreduce": bool(comm),
                              "roofline": roofline("hbm", gbs, peaks["hbm_gbs"], "GB/s",
                                                   NCU_TRAFFIC_PER_ELEM[name] * n, peaks)})

    if "asian" in want:
        # ---- Asian-option Monte Carlo (config 4): disjoint Philox subsequences per GPU ----
        npaths = 1 << args.log2paths
        for precise in (0, 1):
            prm = sm.asian_params(k0=SEED + 5, precise=precise)
            ksteps = K if not precise else max(1, K // 4)

            def mc_step():
                dev.asian(prm, ranks.rank * npaths, npaths, out)
                if comm:
                    comm.allreduce_sum(out, 4, sm.F64)
            mc_sampler = ClockSampler(ranks.local)
            mc_sampler.start()
            t = timed(dev, ranks, W, ksteps, mc_step) / ksteps
            mc_clocks = mc_sampler.stop()
            s = dev.download(out, 4, np.float64)
            tot = npaths * G
            disc = math.exp(-0.05)
            workloads.append({"name": "asian_mc_%s_2^%d_paths_per_gpu" % ("precise" if precise else "fast", args.log2paths),
                              "metric": "paths_per_s", "value": tot / (t * 1e-3), "unit": "paths/s",
                              "path_steps_per_s": tot * NSTEP / (t * 1e-3), "ms_per_step": t,
                              "price_arith": disc * s[0] / tot, "price_geom": disc * s[1] / tot,
                              "stderr_geom": disc * math.sqrt(max(s[3] / tot - (s[1] / tot) ** 2, 0.0) / tot),
                              "allreduce": bool(comm), "clocks": mc_clocks,
                              "mufu_ceiling": mufu_ceiling(npaths * NSTEP / (t * 1e-3), dev.sm_count, mc_clocks)})

    if "gemm" in want:
        # ---- fp32 GEMM (config 3): row blocks of A per GPU, B replicated ----
        sizes = [int(v) for v in args.gemm_sizes.split(",")]
        workloads.extend(run_gemm(sm, dev, ranks, peaks, W, K, sizes))

    line = {
        "metric": "saxpy_hbm_gbs", "value": saxpy_gbs, "unit": "GB/s", "n_gpus": G, "steps": K, "warmup": W,
        "ms_per_step": saxpy_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "saxpy y=2.5*x+y, N=2^%d fp32 per GPU, unfused mul+add, x,y~U[-1,1) Philox-seeded"
                               % args.log2n,
                   "bytes_per_element": 12, "sharding": "contiguous ranges, no data-path collective",
                   "cache": ("inputs (%.3g GiB per GPU) exceed the 126 MB L2; no flush needed" % (8.0 * n / 2 ** 30)
                             if 8 * n > (256 << 20) else
                             "inputs (%.3g MiB per GPU) fit the 126 MB L2: not an HBM figure" % (8.0 * n / 2 ** 20))},
        "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        "roofline": head_roof,
        "workloads": workloads,
        "device": dev.name,
    }
    if ranks.rank == 0 and G == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_saxpy(args.cpu_seconds)
        if workloads:
            others = cpu_baselines_other()
            for wl in workloads:
                for fam, base in others.items():
                    if wl["name"].startswith(fam if fam != "asian" else "asian_mc") and "value" in wl:
                        wl["cpu_baseline"] = base
    dev.free(dx); dev.free(dy)
    if comm:
        comm.close()
    dev.close()
    if ranks.rank == 0:
        emit(line)
    ranks.close()


def run_e2e_saxpy(sm, dev, ranks, n, steps):
    """The bc_* launcher API end to end: pinned host x and y go to the device,
    the saxpy kernel is dispatched by name, y comes back. Every byte counted."""
    import ctypes as C
    L = sm.lib()
    os.environ["BOOTH_DEVICE"] = str(ranks.local)
    bcd = sm.BcDevice()
    if L.bc_device_init(C.byref(bcd)) != 0:
        raise RuntimeError("bc_device_init failed")
    k = sm.BcKernel()
    if L.bc_load_kernel(C.byref(bcd), sm.CUBIN_PATH.encode(), b"saxpy", C.byref(k)) != 0:
        raise RuntimeError("bc_load_kernel failed")
    nbytes = n * 4
    hx, hy = dev.hostalloc(nbytes), dev.hostalloc(nbytes)
    dx, dy = L.bc_alloc(C.byref(bcd), nbytes), L.bc_alloc(C.byref(bcd), nbytes)
    sm.lib().booth_sm100_fill_host(hx, ranks.rank * n, n, SEED + 1, 0, sm.FILL_F32_PM1, 16)
    sm.lib().booth_sm100_fill_host(hy, ranks.rank * n, n, SEED + 1, 1, sm.FILL_F32_PM1, 16)

    class Args(C.Structure):
        _fields_ = [("y", C.c_void_p), ("x", C.c_void_p), ("a", C.c_float), ("n", C.c_uint32)]
    a = Args(dy, dx, 2.5, n)
    blocks = 148 * 8

    def step():
        L.bc_copy_h2d(C.byref(bcd), dx, hx, nbytes)
        L.bc_copy_h2d(C.byref(bcd), dy, hy, nbytes)
        if L.bc_dispatch(C.byref(bcd), C.byref(k), blocks, 1, 1, 256, 1, 1, C.byref(a), C.sizeof(a)) != 0:
            raise RuntimeError("bc_dispatch failed")
        L.bc_copy_d2h(C.byref(bcd), hy, dy, nbytes)
    step()
    ranks.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    ranks.barrier()
    dt = ranks.max(dt)
    L.bc_free(C.byref(bcd), dx); L.bc_free(C.byref(bcd), dy)
    L.bc_unload_kernel(C.byref(bcd), C.byref(k))
    L.bc_device_shutdown(C.byref(bcd))
    launcher = {"value": 12.0 * n * ranks.world * steps / dt / 1e9, "unit": "GB/s",
                "api": "bc_copy_h2d x2 + bc_dispatch(saxpy) + bc_copy_d2h (the examples/launch_saxpy.c flow), synchronous"}

    # The pipelined host-vector call: same pinned buffers, same bytes, both link directions busy at once.
    dev.saxpy_host(hy, hx, 2.5, n)
    ranks.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        dev.saxpy_host(hy, hx, 2.5, n)
    dt = ranks.max(time.perf_counter() - t0)
    ranks.barrier()
    dev.hostfree(hx); dev.hostfree(hy)
    return {"value": 12.0 * n * ranks.world * steps / dt / 1e9, "unit": "GB/s", "steps": steps,
            "h2d_bytes_per_step": 2 * nbytes * ranks.world, "d2h_bytes_per_step": nbytes * ranks.world,
            "bytes_scope": "whole job (all GPUs), like value",
            "api": "booth_sm100_saxpy_host on pinned host vectors: 16 Mi-element chunks, H2D / saxpy / D2H pipelined "
                   "on two streams; returns with y in host memory",
            "launcher_api": launcher}


def run_gemm(sm, dev, ranks, peaks, W, K, sizes):
    out = []
    G = ranks.world
    # 3xTF32: three TF32 MMAs per fp32 product; TF32 dense rate is half the bf16 rate.
    peak = peaks["bf16_tflops"] / 2.0 / 3.0
    for size in sizes:
        M = size // G
        a, b, c = dev.alloc(M * size * 4), dev.alloc(size * size * 4), dev.alloc(M * size * 4)
        dev.fill(a, ranks.rank * M * size, M * size, SEED + 3, 0, sm.FILL_F32_PM1)
        dev.fill(b, 0, size * size, SEED + 3, 1, sm.FILL_F32_PM1)
        try:
            t = timed(dev, ranks, W, K, lambda: dev.gemm(c, a, b, M, size, size)) / K
        except sm.Sm100Error as e:
            out.append({"name": "gemm_%d" % size, "unavailable": str(e)})
            for p in (a, b, c):
                dev.free(p)
            continue
        tf = 2.0 * size * size * size / (t * 1e-3) / 1e12
        # The same step with the caller stating that B has not changed since the last
        # call: the split, transposed copy of B in the workspace is reused. Reported
        # beside the full figure, never in its place.
        t_kept = timed(dev, ranks, W, K, lambda: dev.gemm(c, a, b, M, size, size, b_unchanged=True)) / K
        out.append({"name": "gemm_fp32_3xtf32_%d" % size, "metric": "tflops", "value": tf, "unit": "TFLOP/s",
                    "ms_per_step": t, "sharding": "A/C row blocks of %d rows per GPU, B replicated" % M,
                    "b_unchanged": {"value": 2.0 * size * size * size / (t_kept * 1e-3) / 1e12, "unit": "TFLOP/s",
                                    "ms_per_step": t_kept,
                                    "note": "booth_sm100_gemm_ex(BOOTH_GEMM_B_UNCHANGED): B's planes kept from the previous call"},
                    "roofline": dict(roofline("tensor", tf / G, peak, "TFLOP/s", None, peaks),
                                     frac_of_sustained_peak=tf / G / (peaks["bf16_tflops_sustained"] / 6.0)),
                    "hbm_bytes": 4.0 * (M * size + size * size + M * size)})
        for p in (a, b, c):
            dev.free(p)
    return out


def cpu_baselines_other(seconds_each=3.0):
    """The CPU checker timed on bounded samples of the other four workloads, all
    host threads over disjoint ranges (the reference compiler's x86-64 objects when
    they are built here). Returned keyed by workload family."""
    import oracle
    import booth_b200 as sm
    orc = oracle.load()
    out = {}

    def run(fn, units, unit, sample):
        fn()
        reps, t0 = 0, time.perf_counter()
        while True:
            fn()
            reps += 1
            dt = time.perf_counter() - t0
            if dt >= seconds_each or reps >= 50:
                break
        return {"value": units * reps / dt, "unit": unit, "cores": orc.cores, "kind": orc.kind,
                "sample": "%s x %d repetitions, %d threads" % (sample, reps, orc.cores)}

    m = 1 << 26
    x = sm.fill_host(m, SEED, 0, sm.FILL_F32_PM1, threads=orc.cores)
    y = sm.fill_host(m, SEED, 1, sm.FILL_F32_PM1, threads=orc.cores)
    out["vadd"] = run(lambda: orc.vadd(x, y), 12.0 * m / 1e9, "GB/s", "vector add on 2^26 elements")
    vi = sm.fill_host(m, SEED + 2, 0, sm.FILL_I32_1000, threads=orc.cores)
    out["reduce_i32"] = run(lambda: orc.reduce_i32(vi), 4.0 * m / 1e9, "GB/s", "int32 sum of 2^26 elements")
    vf = sm.fill_host(m, SEED + 2, 1, sm.FILL_F32_01, threads=orc.cores)
    out["reduce_f32"] = run(lambda: orc.reduce_f32(vf), 4.0 * m / 1e9, "GB/s", "fp32 sum of 2^26 elements")
    g = 1024
    a = sm.fill_host(g * g, SEED + 3, 0, sm.FILL_F32_PM1).reshape(g, g)
    b = sm.fill_host(g * g, SEED + 3, 1, sm.FILL_F32_PM1).reshape(g, g)
    out["gemm"] = run(lambda: orc.matmul(a, b), 2.0 * g ** 3 / 1e12, "TFLOP/s", "1024^3 GEMM by 4x4x2 tiles")
    prm = sm.asian_params(k0=SEED + 5)
    npth = 1 << 20
    out["asian"] = run(lambda: orc.asian(prm, 0, npth), float(npth), "paths/s", "2^20 paths x 252 steps")
    return out


def cpu_baseline_saxpy(seconds):
    """The CPU checker (the reference compiler's x86-64 objects when built) timed
    on this machine's cores on a bounded sample of the same workload."""
    import oracle
    import booth_b200 as sm
    orc = oracle.load()
    m = 1 << 28
    x = sm.fill_host(m, SEED + 1, 0, sm.FILL_F32_PM1, threads=orc.cores)
    y = sm.fill_host(m, SEED + 1, 1, sm.FILL_F32_PM1, threads=orc.cores)
    orc.saxpy_inplace(y, x, 2.5)
    reps, t0 = 0, time.perf_counter()
    while True:
        orc.saxpy_inplace(y, x, 2.5)
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= seconds or reps >= 200:
            break
    return {"value": 12.0 * m * reps / dt / 1e9, "unit": "GB/s", "cores": orc.cores, "kind": orc.kind,
            "sample": "saxpy on 2^28 elements x %d repetitions, %d threads over disjoint ranges" % (reps, orc.cores)}


def run_reference(args):
    """--impl reference: the reference's own CPU implementation of the headline
    workload (its x86-64 backend's saxpy through the CPU launcher), all host
    threads, each step a 2^28-element sample of the 2^30-element workload."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    import booth_b200 as sm
    orc = oracle.load()
    m = 1 << 28
    x = sm.fill_host(m, SEED + 1, 0, sm.FILL_F32_PM1, threads=orc.cores)
    y = sm.fill_host(m, SEED + 1, 1, sm.FILL_F32_PM1, threads=orc.cores)
    W, K = max(args.warmup, 1), args.steps
    for _ in range(W):
        orc.saxpy_inplace(y, x, 2.5)
    t0 = time.perf_counter()
    for _ in range(K):
        orc.saxpy_inplace(y, x, 2.5)
    dt = time.perf_counter() - t0
    gbs = 12.0 * m * K / dt / 1e9
    line = {"impl": "reference", "metric": "saxpy_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": dt / K * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "saxpy y=2.5*x+y, N=2^30 fp32 per GPU, unfused mul+add, x,y~U[-1,1) Philox-seeded",
                       "sample": "each step is 2^28 elements of it on the host cores"},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": orc.cores, "kind": orc.kind,
                             "sample": "2^28 elements per step, %d threads over disjoint ranges" % orc.cores},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


def emit(line):
    """The one JSON line, on the process's real stdout."""
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


# Libraries (NCCL prints its version) may write to stdout; the contract is ONE JSON
# line there. File descriptor 1 is pointed at stderr for the whole run and the
# line goes to a saved copy of the original stdout.
sys.stdout.flush()
_REAL_STDOUT = os.dup(1)
os.dup2(2, 1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--log2n", type=int, default=LOG2_STREAM, help="saxpy/reduce elements per GPU (log2)")
    ap.add_argument("--log2paths", type=int, default=LOG2_PATHS, help="Monte Carlo paths per GPU (log2)")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--headline-only", action="store_true", help="skip the other workloads")
    ap.add_argument("--workloads", default="all",
                    help="comma list of the extra workloads to run: sweep,vadd,reduce,asian,gemm (default all)")
    ap.add_argument("--gemm-sizes", default=",".join(str(v) for v in GEMM_SIZES))
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
