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
CHECK_PIECE = 1 << 26       # elements the CPU checker generates and sums at a time
CHECK_WINDOW = 1 << 20      # elements per saxpy window / Monte Carlo paths per rank checked
TOL = {"fp32_sum": 1e-6, "mc": 1e-5, "gemm": 1e-5}     # the workloads' stated tolerances


def ncu_traffic():
    """DRAM bytes per unit per launch as counted by ncu (dram__bytes_read.sum +
    dram__bytes_write.sum): the one table profiles/dram_traffic_per_unit.md holds,
    keyed by its first column. A key that is not there has not been captured."""
    table = {}
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic_per_unit.md")) as f:
            for ln in f:
                cells = [c.strip() for c in ln.strip().strip("|").split("|")]
                if len(cells) >= 4 and ln.lstrip().startswith("|"):
                    try:
                        table[cells[0]] = float(cells[3])
                    except ValueError:
                        pass
    except OSError:
        pass
    return table


NCU_TRAFFIC = ncu_traffic()


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

    def sum(self, values, integer=False):
        """Element-wise sum over ranks of a short list (float64, or int64 when integer)."""
        if not self.dist:
            return list(values)
        import torch
        t = torch.tensor(list(values), dtype=torch.int64 if integer else torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return [int(v) if integer else float(v) for v in t]

    def gather(self, v):
        """One float per rank, on every rank."""
        if not self.dist:
            return [float(v)]
        box = [None] * self.world
        self.dist.all_gather_object(box, float(v))
        return box

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


def mc_rooflines(path_steps_per_s, sm_count, clocks):
    """The pricer is bound by neither HBM nor the tensor pipe. Two issue limits
    apply per SM and clock: the special-function unit (3 MUFU operations per
    path-step on 16 lanes: 16/3 path-steps) and the warp schedulers (17.1 warp
    instructions per warp-step as counted by ncu, 4 schedulers x 32 lanes:
    128/17.1 path-steps). Reported per GPU at the SM clock sampled during the
    timed region; the lower of the two ceilings is the `roofline`."""
    mhz = clocks.get("sm_mhz") or clocks.get("sm_max_mhz")
    clock_source = "sampled during the timed region"
    if not mhz:
        mhz, clock_source = 1965.0, "no clock sample available: the B200's maximum SM clock assumed"
    achieved = path_steps_per_s / (sm_count * mhz * 1e6)
    mufu = {"bound": "mufu issue", "achieved": achieved, "peak": 16.0 / 3.0, "unit": "path-steps/clk/SM",
            "frac": achieved / (16.0 / 3.0), "traffic": None, "sm_mhz": mhz, "sm_mhz_source": clock_source,
            "peak_source": "derived: 16 MUFU lanes per SM / 3 MUFU operations per path-step"}
    issue = {"bound": "warp instruction issue", "achieved": achieved, "peak": 128.0 / 17.1, "unit": "path-steps/clk/SM",
             "frac": achieved / (128.0 / 17.1),
             "peak_source": "derived: 4 schedulers x 32 lanes / 17.1 warp instructions per warp-step (ncu, profiles/asian_mc_2p22.md)"}
    return mufu, issue


def pipe_probe(sm, dev, mhz, achieved):
    """Times the image's three probe kernels (kernels/pipe_probe.cu): the two
    instruction groups the pricer cannot do without, per Philox call 12 MUFU and
    20 IMAD.WIDE with their 20 xors, on independent register chains, alone and
    together. A trip stands for four path-steps, so the pace of the two together
    is a ceiling in the roofline's own unit (the pricer issues these and 16 more
    instructions per call); `frac` is the pricer against it."""
    import ctypes as C
    L = sm.lib()
    trips, blocks = 2048, dev.sm_count * 8
    scratch = dev.alloc(64)
    res = {"bound": "MUFU and IMAD.WIDE together (probe kernels, measured in this run)",
           "unit": "path-steps/clk/SM", "trips": trips, "grid": [blocks, 256], "sm_mhz": mhz}
    for name in ("probe_mufu", "probe_imad_wide", "probe_mufu_imad_wide"):
        k = sm.Kern()
        rc = L.sm100_rt_load_builtin(dev.handle, name.encode(), C.byref(k))
        if rc != 0:
            raise sm.Sm100Error("sm100_rt_load_builtin(%s)" % name, rc)
        vals = [C.c_uint64(scratch), C.c_int(trips), C.c_float(0.999), C.c_uint32(12345)]
        argv = (C.c_void_p * len(vals))(*[C.cast(C.byref(v), C.c_void_p) for v in vals])

        def go():
            rc = L.sm100_rt_launch(dev.handle, C.byref(k), blocks, 1, 1, 256, 1, 1, 0, argv)
            if rc != 0:
                raise sm.Sm100Error("sm100_rt_launch(%s)" % name, rc)
        for _ in range(3):
            go()
        dev.sync()
        dev.tic()
        for _ in range(5):
            go()
        ms = dev.toc() / 5
        # trips per warp scheduler (8 warps a block, 4 schedulers an SM) against the cycles the launch took
        warp_trips = blocks * 8 * trips / (dev.sm_count * 4.0)
        cyc = ms * 1e-3 * mhz * 1e6 / warp_trips
        res[name] = {"ms": ms, "cycles_per_warp_trip_per_scheduler": cyc,
                     "path_steps_per_clk_sm": 4 * 32 * 4.0 / cyc if cyc else None}
        L.sm100_rt_unload(dev.handle, C.byref(k))
    dev.free(scratch)
    res["peak"] = res["probe_mufu_imad_wide"]["path_steps_per_clk_sm"]
    res["achieved"] = achieved
    res["frac"] = achieved / res["peak"] if res["peak"] else None
    return res


def roofline(bound, achieved, peak, unit, traffic, peaks):
    r = {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
         "frac": achieved / peak if peak else None, "traffic": traffic,
         "peak_source": "of " + peaks["source"]}
    if bound == "hbm":
        r["frac_of_nominal_8TBs"] = achieved / 8000.0
    if peak and achieved > peak:
        r["warning"] = ("above the denominator: the measured peak is a plain copy (half reads, half writes) / a cuBLAS "
                        "bf16 GEMM scaled to 3xTF32, neither is a hard ceiling for this kernel; read the nominal "
                        "fraction beside it")
    return r


def host_placement(index):
    """Where this rank's GPU hangs off the host, read from sysfs (nothing is changed
    except this process's own CPU affinity): when the GPU's PCI device names a NUMA
    node and a CPU list, the process (and with it the threads that fill and touch
    the page-locked buffers) is kept on those CPUs, so that staging memory is
    allocated next to the GPU. Returns what was found for the JSON line."""
    info = {"numa_node": None, "bound_to_local_cpus": False}
    try:
        import pynvml
        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(index)).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        if len(bus.split(":")[0]) == 8:
            bus = bus[4:]
        base = os.path.join("/sys/bus/pci/devices", bus)
        with open(os.path.join(base, "numa_node")) as f:
            info["numa_node"] = int(f.read().strip())
        with open(os.path.join(base, "local_cpulist")) as f:
            text = f.read().strip()
        info["local_cpulist"] = text
        cpus = set()
        for part in text.split(","):
            if "-" in part:
                lo, hi = part.split("-")
                cpus.update(range(int(lo), int(hi) + 1))
            elif part:
                cpus.add(int(part))
        allowed = os.sched_getaffinity(0)
        if info["numa_node"] is not None and info["numa_node"] >= 0 and cpus and cpus & allowed and (cpus & allowed) != allowed:
            os.sched_setaffinity(0, cpus & allowed)
            info["bound_to_local_cpus"] = True
    except Exception as e:
        info["note"] = "not available: %s" % type(e).__name__
    return info


def wall(ranks, steps, body):
    """End-to-end timing of a host-buffer call: one untimed call, then `steps`
    calls on the wall clock between barriers (each call returns with its result in
    host memory); max over ranks, seconds, plus every rank's own time."""
    body()
    ranks.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        body()
    mine = time.perf_counter() - t0
    ranks.barrier()
    return ranks.max(mine), ranks.gather(mine)


def wrap32(v):
    v &= 0xFFFFFFFF
    return v - (1 << 32) if v & 0x80000000 else v


def run_ours(args):
    import booth_b200 as sm
    ranks = Ranks(args.gpus)
    peaks = measured_peaks()
    # With several ranks on one host, keep each next to its own GPU before any staging
    # memory is allocated. A 1-GPU run keeps all cores (they time the CPU baseline).
    placement = host_placement(ranks.local) if ranks.world > 1 else {"bound_to_local_cpus": False, "note": "single rank: all cores kept"}
    dev = sm.Device(ranks.local)
    comm = None
    if ranks.world > 1:
        uid = ranks.bcast_bytes(sm.Comm.unique_id() if ranks.rank == 0 else None)
        comm = sm.Comm(dev, ranks.world, ranks.rank, uid)
    W, K = max(args.warmup, 3), args.steps
    G = ranks.world
    workloads = []
    sampler = ClockSampler(ranks.local)
    # The CPU checker: used outside every timed region to check results (all ranks)
    # and, on rank 0 of a 1-GPU run, as the timed CPU baseline. Never the product path.
    orc = None
    if not args.no_parity or (ranks.rank == 0 and G == 1 and not args.no_cpu_baseline):
        import oracle
        orc = oracle.load()
    parity, misses = {}, []
    Ke = max(1, min(K, args.e2e_steps))

    def check(name, ok, detail):
        parity[name] = detail
        if not ok:
            misses.append(name)

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
    t_el = NCU_TRAFFIC.get("saxpy")
    head_roof = roofline("hbm", per_gpu, peaks["hbm_gbs"], "GB/s", t_el * n if t_el else None, peaks)

    if not args.no_parity:
        # saxpy parity at the benchmark's own size and shard: fresh inputs, one launch over
        # all n elements, three windows of this rank's shard against the CPU checker on the
        # same elements of the global stream, bit for bit.
        dev.fill(dy, first, n, SEED + 1, 1, sm.FILL_F32_PM1)
        dev.saxpy(dy, dx, 2.5, n)
        wlen = min(CHECK_WINDOW, n)
        bad = 0
        for off in sorted({0, (n // 2 - wlen // 2 + 5) if n > wlen else 0, n - wlen}):
            hx = orc.fill(wlen, SEED + 1, 0, sm.FILL_F32_PM1, first=first + off)
            hy = orc.fill(wlen, SEED + 1, 1, sm.FILL_F32_PM1, first=first + off)
            got = dev.download(dy + 4 * off, wlen, np.float32)
            bad += int(np.count_nonzero(got.view(np.uint32) != orc.saxpy(hy, hx, 2.5).view(np.uint32)))
        bad = int(ranks.sum([bad], integer=True)[0])
        check("saxpy_mismatches", bad == 0, bad)
        dev.fill(dy, first, n, SEED + 1, 1, sm.FILL_F32_PM1)

    # ---- e2e: host buffers in, result back in host memory, through the library's calls ----
    e2e = None if args.no_e2e else run_e2e_saxpy(sm, dev, ranks, n, Ke, placement)
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
            t_el = NCU_TRAFFIC.get("vadd")
            workloads.append({"name": "vadd_2^%d" % lg, "metric": "hbm_gbs", "value": gbs * G, "unit": "GB/s",
                              "ms_per_step": t,
                              "roofline": roofline("hbm", gbs, peaks["hbm_gbs"], "GB/s",
                                                   t_el * m if (t_el and lg > 26) else None, peaks),
                              "note": "201 MB working set, partly L2-resident; median of 3 runs of K steps" if lg == LOG2_VADD else "3 GiB working set"})
            dev.free(dz)
            if not args.no_e2e:
                # end to end: the host-vector call behind the CPU-launcher symbol vector_add
                hv = [dev.hostalloc(m * 4) for _ in range(3)]
                for i in (0, 1):
                    sm.lib().booth_sm100_fill_host(hv[i], first, m, SEED + 1, i, sm.FILL_F32_PM1, 16)
                dt_s, per_rank = wall(ranks, Ke, lambda: dev.vadd_host(hv[0], hv[1], hv[2], m))
                workloads[-1]["e2e"] = {"value": 12.0 * m * G * Ke / dt_s / 1e9, "unit": "GB/s", "steps": Ke,
                                        "h2d_bytes_per_step": 8 * m * G, "d2h_bytes_per_step": 4 * m * G,
                                        "per_rank_s": per_rank, "api": "booth_sm100_vadd_host on pinned host vectors"}
                for hp in hv:
                    dev.hostfree(hp)

    out = dev.alloc(64)
    if "reduce" in want:
        # ---- reduction (config 2): per-GPU sum then one NCCL all-reduce ----
        hostv = None if args.no_e2e else dev.hostalloc(n * 4)
        for name, kind, fn, dt in (("reduce_i32", sm.FILL_I32_1000, dev.reduce_i32, sm.I32),
                                   ("reduce_f32", sm.FILL_F32_01, dev.reduce_f32, sm.F64)):
            stream_id = 0 if dt == sm.I32 else 1
            dev.fill(dx, first, n, SEED + 2, stream_id, kind)

            def step():
                fn(dx, n, out)
                if comm:
                    comm.allreduce_sum(out, 1, dt)
            t = timed(dev, ranks, W, K, step) / K
            res = dev.download(out, 1, np.int32 if dt == sm.I32 else np.float64)[0]
            gbs = 4.0 * n / (t * 1e-3) / 1e9
            entry = {"name": name + "_2^%d" % args.log2n, "metric": "hbm_gbs", "value": gbs * G, "unit": "GB/s",
                     "ms_per_step": t, "result": float(res), "allreduce": bool(comm),
                     "roofline": roofline("hbm", gbs, peaks["hbm_gbs"], "GB/s",
                                          NCU_TRAFFIC[name] * n if name in NCU_TRAFFIC else None, peaks)}
            if not args.no_parity:
                # the all-reduced sum against the CPU checker's sum of the same global stream:
                # every rank sums its own shard on the host cores, generated piece by piece,
                # and the partial sums are added over the process group
                acc_i, acc_f = 0, 0.0
                for off in range(0, n, CHECK_PIECE):
                    m = min(CHECK_PIECE, n - off)
                    piece = orc.fill(m, SEED + 2, stream_id, kind, first=first + off)
                    if dt == sm.I32:
                        acc_i = wrap32(acc_i + orc.reduce_i32(piece))
                    else:
                        acc_f += orc.reduce_f32(piece)
                if dt == sm.I32:
                    ref = wrap32(int(ranks.sum([acc_i], integer=True)[0]))
                    check("int32", int(res) == ref, "bit-exact" if int(res) == ref else "device %d != checker %d" % (int(res), ref))
                else:
                    ref = ranks.sum([acc_f])[0]
                    rel = abs(float(res) - ref) / abs(ref)
                    check("fp32_rel", rel <= TOL["fp32_sum"], rel)
            if hostv:
                # end to end: the vector starts in page-locked host memory, one scalar comes back
                sm.lib().booth_sm100_fill_host(hostv, first, n, SEED + 2, stream_id, kind, 16)

                def host_step():
                    dev.h2d_async(dx, hostv, n * 4)
                    step()
                    dev.download(out, 1, np.int32 if dt == sm.I32 else np.float64)
                dt_s, per_rank = wall(ranks, Ke, host_step)
                entry["e2e"] = {"value": 4.0 * n * G * Ke / dt_s / 1e9, "unit": "GB/s", "steps": Ke,
                                "h2d_bytes_per_step": 4 * n * G, "d2h_bytes_per_step": (4 if dt == sm.I32 else 8) * G,
                                "api": "sm100_rt_h2d_async + booth_sm100_%s%s + sm100_rt_d2h" % (name, " + sm100_comm_allreduce_sum" if comm else ""),
                                "per_rank_s": per_rank}
            workloads.append(entry)
        if hostv:
            dev.hostfree(hostv)

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
            mufu, issue = mc_rooflines(npaths * NSTEP / (t * 1e-3), dev.sm_count, mc_clocks)
            entry = {"name": "asian_mc_%s_2^%d_paths_per_gpu" % ("precise" if precise else "fast", args.log2paths),
                     "metric": "paths_per_s", "value": tot / (t * 1e-3), "unit": "paths/s",
                     "path_steps_per_s": tot * NSTEP / (t * 1e-3), "ms_per_step": t,
                     "price_arith": disc * s[0] / tot, "price_geom": disc * s[1] / tot,
                     "stderr_geom": disc * math.sqrt(max(s[3] / tot - (s[1] / tot) ** 2, 0.0) / tot),
                     "allreduce": bool(comm), "clocks": mc_clocks, "roofline": mufu, "second_bound": issue}
            if not precise:
                entry["pipe_probe"] = pipe_probe(sm, dev, mufu["sm_mhz"], mufu["achieved"])
            if not args.no_e2e:
                # end to end: parameters in (a 32-byte struct by value), four doubles back
                def mc_host_step():
                    mc_step()
                    dev.download(out, 4, np.float64)
                dt_s, per_rank = wall(ranks, max(1, min(Ke, ksteps)), mc_host_step)
                ke = max(1, min(Ke, ksteps))
                entry["e2e"] = {"value": tot * ke / dt_s, "unit": "paths/s", "steps": ke, "h2d_bytes_per_step": 32 * G,
                                "d2h_bytes_per_step": 32 * G, "per_rank_s": per_rank,
                                "api": "booth_sm100_asian%s + sm100_rt_d2h" % (" + sm100_comm_allreduce_sum" if comm else "")}
            if not args.no_parity:
                # a check-sized run of the same kernel on this rank's own subsequence, all-reduced,
                # against the CPU checker over the union of the ranks' ranges
                cp = min(CHECK_WINDOW, npaths)
                dev.asian(prm, ranks.rank * cp, cp, out)
                if comm:
                    comm.allreduce_sum(out, 4, sm.F64)
                got = dev.download(out, 4, np.float64)
                ref = ranks.sum(list(orc.asian(prm, ranks.rank * cp, cp)))
                rels = [abs(got[i] - ref[i]) / abs(ref[i]) for i in range(2)]
                check("mc_rel_%s" % ("precise" if precise else "fast"), max(rels) <= TOL["mc"], rels)
            workloads.append(entry)

    if "gemm" in want:
        # ---- fp32 GEMM (config 3): row blocks of A per GPU, B replicated ----
        sizes = [int(v) for v in args.gemm_sizes.split(",")]
        workloads.extend(run_gemm(sm, dev, ranks, peaks, W, K, sizes, orc if not args.no_parity else None, check,
                                  0 if args.no_e2e else Ke, args.gemm_shard_of))

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
        "parity": dict(parity, checker=orc.kind, tolerances=TOL, checked_on="all %d rank(s), outside the timed regions" % G,
                       status="green" if not misses else "MISS: " + ", ".join(misses)) if not args.no_parity else None,
        "workloads": workloads,
        "device": dev.name,
    }
    if ranks.rank == 0 and G == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_saxpy(orc, args.cpu_seconds)
        if workloads:
            others = cpu_baselines_other(orc)
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
    if misses:
        sys.stderr.write("bench: PARITY MISS on %s\n" % ", ".join(misses))
        raise SystemExit(3)


def run_e2e_saxpy(sm, dev, ranks, n, steps, placement):
    """The headline workload end to end: pinned host x and y go to the device, y
    comes back, every byte counted. Two forms: the pipelined host-vector call
    (booth_sm100_saxpy_host, the figure), and the synchronous bc_* flow of the
    reference's example program beside it. The link itself is measured in the same
    run so the figure reads as a fraction of something measured."""
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
    dt, _ = wall(ranks, steps, step)
    L.bc_free(C.byref(bcd), dx); L.bc_free(C.byref(bcd), dy)
    L.bc_unload_kernel(C.byref(bcd), C.byref(k))
    L.bc_device_shutdown(C.byref(bcd))
    launcher = {"value": 12.0 * n * ranks.world * steps / dt / 1e9, "unit": "GB/s",
                "api": "bc_copy_h2d x2 + bc_dispatch(saxpy) + bc_copy_d2h (the examples/launch_saxpy.c flow), synchronous"}

    # The pipelined host-vector call: same pinned buffers, same bytes, both link directions busy at once.
    dt, per_rank = wall(ranks, steps, lambda: dev.saxpy_host(hy, hx, 2.5, n))
    dev.hostfree(hx); dev.hostfree(hy)
    value = 12.0 * n * ranks.world * steps / dt / 1e9
    # The link, measured alone on this rank while the others do the same (so at N > 1 the
    # ranks share the host's memory and root complexes as they do in the timed calls).
    ranks.barrier()
    up, down, up2, down2 = dev.link_probe(min(1 << 30, max(nbytes, 1 << 16)), 3)
    ranks.barrier()
    # 2 bytes go up for every byte that comes down, so the call cannot end before the
    # upload alone would: 8N bytes at the host-to-device rate this link reaches when it
    # has the link to itself (the ceiling), nor, more tightly, before the slower of the
    # two directions at the rates they reach while BOTH stream flat out (a 1:1 mix,
    # harder on the link than this call's 2:1, so that second figure can be beaten).
    bound_s = max(2.0 * nbytes / (up * 1e9), 1.0 * nbytes / (down * 1e9)) if up > 0 and down > 0 else None
    duplex_s = max(2.0 * nbytes / (up2 * 1e9), 1.0 * nbytes / (down2 * 1e9)) if up2 > 0 and down2 > 0 else None
    peak = 12.0 * n / bound_s / 1e9 if bound_s else None
    mine = 12.0 * n * steps / per_rank[ranks.rank] / 1e9
    fracs = ranks.gather(mine / peak if peak else 0.0)
    return {"value": value, "unit": "GB/s", "steps": steps,
            "h2d_bytes_per_step": 2 * nbytes * ranks.world, "d2h_bytes_per_step": nbytes * ranks.world,
            "bytes_scope": "whole job (all GPUs), like value",
            "api": "booth_sm100_saxpy_host on pinned host vectors: 16 Mi-element chunks, H2D / saxpy / D2H pipelined "
                   "on three streams; returns with y in host memory",
            "roofline": {"bound": "pcie", "unit": "GB/s", "achieved": mine, "peak": peak,
                         "frac": mine / peak if peak else None,
                         "peak_source": "measured in this run on this rank's GPU while every rank measures its own "
                                        "(booth_sm100_link_probe, 3 x 1 GiB pinned copies): H2D %.1f, D2H %.1f GB/s alone; "
                                        "%.1f and %.1f with both directions flat out; peak = 12 B x N / max(8N/H2D, 4N/D2H) "
                                        "from the rates alone" % (up, down, up2, down2),
                         "peak_both_directions_flat_out": 12.0 * n / duplex_s / 1e9 if duplex_s else None,
                         "link_gbs": {"h2d": up, "d2h": down, "h2d_duplex": up2, "d2h_duplex": down2},
                         "frac_per_rank": fracs},
            "host": placement,
            "per_rank_s": per_rank,
            "launcher_api": launcher}


def run_gemm(sm, dev, ranks, peaks, W, K, sizes, orc, check, e2e_steps, shard_of=0):
    out = []
    G = ranks.world
    # 3xTF32: three TF32 MMAs per fp32 product; TF32 dense rate is half the bf16 rate.
    peak = peaks["bf16_tflops"] / 2.0 / 3.0
    for size in sizes:
        # shard_of: on one GPU, time (and check) the row block one of `shard_of` GPUs would hold
        M = size // (shard_of if shard_of and G == 1 else G)
        a, b, c = dev.alloc(M * size * 4), dev.alloc(size * size * 4), dev.alloc(M * size * 4)
        dev.fill(a, ranks.rank * M * size, M * size, SEED + 3, 0, sm.FILL_F32_PM1)
        dev.fill(b, 0, size * size, SEED + 3, 1, sm.FILL_F32_PM1)
        gemm_sampler = ClockSampler(ranks.local)
        gemm_sampler.start()
        try:
            t = timed(dev, ranks, W, K, lambda: dev.gemm(c, a, b, M, size, size)) / K
        except sm.Sm100Error as e:
            gemm_sampler.stop()
            out.append({"name": "gemm_%d" % size, "unavailable": str(e)})
            for p in (a, b, c):
                dev.free(p)
            continue
        gemm_clocks = gemm_sampler.stop()
        flop = 2.0 * M * G * size * size
        tf = flop / (t * 1e-3) / 1e12
        # The same step with the caller stating that B has not changed since the last
        # call: the split, transposed copy of B in the workspace is reused. Reported
        # beside the full figure, never in its place.
        t_kept = timed(dev, ranks, W, K, lambda: dev.gemm(c, a, b, M, size, size, b_unchanged=True)) / K
        traffic = NCU_TRAFFIC.get("gemm_%d" % size) if G == 1 and not shard_of else None
        entry = {"name": "gemm_fp32_3xtf32_%d" % size, "metric": "tflops", "value": tf, "unit": "TFLOP/s",
                 "ms_per_step": t, "sharding": "A/C row blocks of %d rows per GPU, B replicated" % M if not (shard_of and G == 1)
                 else "the %d-row block one of %d GPUs holds, alone on this GPU" % (M, shard_of),
                 "b_unchanged": {"value": flop / (t_kept * 1e-3) / 1e12, "unit": "TFLOP/s",
                                 "ms_per_step": t_kept,
                                 "note": "booth_sm100_gemm_ex(BOOTH_GEMM_B_UNCHANGED): B's planes kept from the previous call"},
                 "roofline": dict(roofline("tensor", tf / G, peak, "TFLOP/s", traffic, peaks),
                                  frac_of_sustained_peak=tf / G / (peaks["bf16_tflops_sustained"] / 6.0),
                                  traffic_note="DRAM bytes of the contraction kernel per launch (ncu); above the algorithmic "
                                               "hbm_bytes because it reads the split planes (2x) and re-reads panels: "
                                               "harmless, the kernel is bound by the tensor pipe" if traffic else
                                               "not captured for this shape"),
                 "hbm_bytes": 4.0 * (M * size + size * size + M * size), "clocks": gemm_clocks}
        if orc is not None:
            # 16 four-row blocks of this rank's rows of C against the CPU checker's 4x4x2 tiles
            # on the same seeded inputs (only the sampled rows of A are generated on the host)
            dev.gemm(c, a, b, M, size, size)
            dev.sync()
            rng = np.random.default_rng(size * 131 + ranks.rank)
            nblk = min(16, M // 4)
            rows4 = np.sort(rng.choice(M // 4, size=nblk, replace=False))
            hb = orc.fill(size * size, SEED + 3, 1, sm.FILL_F32_PM1).reshape(size, size)
            ha = np.concatenate([orc.fill(4 * size, SEED + 3, 0, sm.FILL_F32_PM1,
                                          first=(ranks.rank * M + 4 * int(r)) * size) for r in rows4]).reshape(4 * nblk, size)
            want = orc.matmul(ha, hb).astype(np.float64)
            got = np.concatenate([dev.download(c + 4 * int(r) * size * 4, (4, size), np.float32) for r in rows4]).astype(np.float64)
            num2, den2 = ranks.sum([float(((got - want) ** 2).sum()), float((want ** 2).sum())])
            rel = math.sqrt(num2 / den2)
            check("gemm_rel_fro_%d" % size, rel <= 1e-5, rel)
            del hb, ha
        if e2e_steps:
            # end to end: A's row block and B in page-locked host memory, C back to the host
            na, nb = M * size * 4, size * size * 4
            ha_p, hb_p, hc_p = dev.hostalloc(na), dev.hostalloc(nb), dev.hostalloc(na)
            sm.lib().booth_sm100_fill_host(ha_p, ranks.rank * M * size, M * size, SEED + 3, 0, sm.FILL_F32_PM1, 16)
            sm.lib().booth_sm100_fill_host(hb_p, 0, size * size, SEED + 3, 1, sm.FILL_F32_PM1, 16)

            def host_step():
                dev.h2d_async(a, ha_p, na)
                dev.h2d_async(b, hb_p, nb)
                dev.gemm(c, a, b, M, size, size)
                dev.d2h_async(hc_p, c, na)
                dev.sync()
            dt_s, per_rank = wall(ranks, e2e_steps, host_step)
            entry["e2e"] = {"value": flop * e2e_steps / dt_s / 1e12, "unit": "TFLOP/s", "steps": e2e_steps,
                            "h2d_bytes_per_step": (na + nb) * G, "d2h_bytes_per_step": na * G, "per_rank_s": per_rank,
                            "api": "sm100_rt_h2d_async(A, B) + booth_sm100_gemm + sm100_rt_d2h_async(C) + sm100_rt_sync"}
            for hp in (ha_p, hb_p, hc_p):
                dev.hostfree(hp)
        out.append(entry)
        for p in (a, b, c):
            dev.free(p)
    return out


def cpu_baselines_other(orc, seconds_each=3.0):
    """The CPU checker timed on bounded samples of the other four workloads, all
    host threads over disjoint ranges (the reference compiler's x86-64 objects when
    they are built here). Returned keyed by workload family."""
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
    x = orc.fill(m, SEED, 0, 0)
    y = orc.fill(m, SEED, 1, 0)
    out["vadd"] = run(lambda: orc.vadd(x, y), 12.0 * m / 1e9, "GB/s", "vector add on 2^26 elements")
    vi = orc.fill(m, SEED + 2, 0, 2)
    out["reduce_i32"] = run(lambda: orc.reduce_i32(vi), 4.0 * m / 1e9, "GB/s", "int32 sum of 2^26 elements")
    vf = orc.fill(m, SEED + 2, 1, 1)
    out["reduce_f32"] = run(lambda: orc.reduce_f32(vf), 4.0 * m / 1e9, "GB/s", "fp32 sum of 2^26 elements")
    g = 1024
    a = orc.fill(g * g, SEED + 3, 0, 0).reshape(g, g)
    b = orc.fill(g * g, SEED + 3, 1, 0).reshape(g, g)
    out["gemm"] = run(lambda: orc.matmul(a, b), 2.0 * g ** 3 / 1e12, "TFLOP/s", "1024^3 GEMM by 4x4x2 tiles")
    prm = asian_params_host()
    npth = 1 << 20
    out["asian"] = run(lambda: orc.asian(prm, 0, npth), float(npth), "paths/s", "2^20 paths x 252 steps")
    return out


class _AsianParams:
    pass


def asian_params_host(k0=SEED + 5):
    """The pricer's parameters for the CPU checker, computed in fp32 as the workload
    states them (drift = (r - sigma^2/2) dt, vol = sigma sqrt(dt)); no product code."""
    p = _AsianParams()
    dt = np.float32(1.0) / np.float32(NSTEP)
    p.s0, p.strike, p.nstep, p.k0, p.k1 = 100.0, 100.0, NSTEP, k0, 0
    p.drift = float((np.float32(0.05) - np.float32(0.5) * np.float32(0.2) * np.float32(0.2)) * dt)
    p.vol = float(np.float32(0.2) * np.sqrt(dt, dtype=np.float32))
    return p


def cpu_baseline_saxpy(orc, seconds):
    """The CPU checker (the reference compiler's x86-64 objects when built) timed
    on this machine's cores on a bounded sample of the same workload."""
    m = 1 << 28
    x = orc.fill(m, SEED + 1, 0, 0)
    y = orc.fill(m, SEED + 1, 1, 0)
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
    threads, each step the whole 2^log2n-element vector pair of one GPU's shard.
    Nothing of the product is loaded here: inputs come from the checker harness's
    own generator."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    orc = oracle.load()
    m = 1 << args.log2n
    x = orc.fill(m, SEED + 1, 0, 0)
    y = orc.fill(m, SEED + 1, 1, 0)
    W, K = max(args.warmup, 1), args.steps
    for _ in range(W):
        orc.saxpy_inplace(y, x, 2.5)
    t0 = time.perf_counter()
    for _ in range(K):
        orc.saxpy_inplace(y, x, 2.5)
    dt = time.perf_counter() - t0
    gbs = 12.0 * m * K / dt / 1e9
    sample = ("each step is one GPU's whole shard, 2^%d elements, on the host cores (%d threads over disjoint ranges)"
              % (args.log2n, orc.cores))
    line = {"impl": "reference", "metric": "saxpy_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": dt / K * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "saxpy y=2.5*x+y, N=2^%d fp32 per GPU, unfused mul+add, x,y~U[-1,1) Philox-seeded"
                                   % args.log2n,
                       "bytes_per_element": 12, "sample": sample},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": orc.cores, "kind": orc.kind, "sample": sample},
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
    ap.add_argument("--gemm-shard-of", type=int, default=0,
                    help="with one GPU: run the GEMM on the row block one of this many GPUs holds (M = size / this)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true",
                    help="skip the checks of the results against the CPU checker (they run outside the timed regions)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
