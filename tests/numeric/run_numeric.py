#!/usr/bin/env python
"""Numeric cross-check of the five workloads: sm100 against the x86-64 path.

Modelled on the reference's tests/numeric/run_numeric.py:309-395: every case is
judged on two axes, accuracy (against the known-good result) and regression
(against the committed baseline for the same backend), and like its differential
harness (tests/diff/run_diff.sh:32-33) a run with --inject corrupts one output
element and must then FAIL.

    python tests/numeric/run_numeric.py --backends cpu            (no GPU needed)
    python tests/numeric/run_numeric.py --backends cpu,sm100 [--full] [--inject] [--update-baseline]

Backends: "cpu" = the CPU checker (oracle/), "sm100" = libbooth_sm100 through its
C ABI, "nvptx" = the PTX the reference compiler's own NVIDIA back end emits for the
same kernel sources (oracle/_ref/ptx, built by oracle/Makefile), run on the GPU
through the library's nv_rt_* entry points: the counterpart of the reference
runner's "nvidia" backend (tests/numeric/run_numeric.py:230-296). It covers vadd,
saxpy and the chunked sums; for the pricer and the Triton matmul tile the reference
emits PTX that ptxas rejects, those lines are skipped. Exit status 0 when every
gating line is ok.
"""
import argparse
import json
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import booth_b200 as sm      # noqa: E402
import oracle                # noqa: E402

DISC = math.exp(-0.05)


def key_of(w, case):
    return w["name"] + "/" + ",".join("%s=%s" % (k, case[k]) for k in sorted(case) if k != "full")


class Cpu:
    name = "cpu"

    def __init__(self):
        self.o = oracle.load()

    def run(self, w, case, seed):
        n = case.get("n", 0)
        name = w["name"]
        if name == "vadd":
            return self.o.vadd(sm.fill_host(n, seed, 0, 0), sm.fill_host(n, seed, 1, 0))
        if name == "saxpy":
            return self.o.saxpy(sm.fill_host(n, seed + 1, 1, 0), sm.fill_host(n, seed + 1, 0, 0), w["alpha"])
        if name == "reduce_i32":
            return np.array([self.o.reduce_i32(sm.fill_host(n, seed + 2, 0, 2))], np.int64)
        if name == "reduce_f32":
            return np.array([self.o.reduce_f32(sm.fill_host(n, seed + 2, 1, 1))], np.float64)
        if name == "gemm":
            M, N, K = case["m"], case["n"], case["k"]
            a = sm.fill_host(M * K, seed + 3, 0, 0).reshape(M, K)
            b = sm.fill_host(K * N, seed + 3, 1, 0).reshape(K, N)
            rows4 = gemm_rows4(case)
            c = self.o.matmul(a, b, rows4=rows4)
            return c if rows4 is None else c[gemm_rows(rows4)]
        if name in ("asian", "asian_precise"):
            prm = sm.asian_params(k0=(seed + 5) & 0xFFFFFFFF)
            sa, sg = self.o.asian(prm, 0, case["paths"])
            return np.array([DISC * sa / case["paths"], DISC * sg / case["paths"]], np.float64)
        raise ValueError(name)


class Sm100:
    name = "sm100"

    def __init__(self):
        self.d = sm.Device(0)

    def run(self, w, case, seed):
        d, n, name = self.d, case.get("n", 0), w["name"]
        if name in ("vadd", "saxpy"):
            s = seed if name == "vadd" else seed + 1
            x, y = d.alloc(n * 4), d.alloc(n * 4)
            d.fill(x, 0, n, s, 0, 0); d.fill(y, 0, n, s, 1, 0)
            if name == "vadd":
                out = d.alloc(n * 4); d.vadd(x, y, out, n)
            else:
                out = y; d.saxpy(y, x, w["alpha"], n)
            res = d.download(out, n, np.float32)
            for p in {x, y, out}:
                d.free(p)
            return res
        if name in ("reduce_i32", "reduce_f32"):
            p, out = d.alloc(n * 4), d.alloc(8)
            if name == "reduce_i32":
                d.fill(p, 0, n, seed + 2, 0, 2); d.reduce_i32(p, n, out)
                res = d.download(out, 1, np.int32).astype(np.int64)
            else:
                d.fill(p, 0, n, seed + 2, 1, 1); d.reduce_f32(p, n, out)
                res = d.download(out, 1, np.float64)
            d.free(p); d.free(out)
            return res
        if name == "gemm":
            M, N, K = case["m"], case["n"], case["k"]
            a, b, c = d.alloc(M * K * 4), d.alloc(K * N * 4), d.alloc(M * N * 4)
            d.fill(a, 0, M * K, seed + 3, 0, 0); d.fill(b, 0, K * N, seed + 3, 1, 0)
            d.gemm(c, a, b, M, N, K); d.sync()
            rows4 = gemm_rows4(case)
            if rows4 is None:
                res = d.download(c, (M, N), np.float32)
            else:
                res = np.stack([d.download(c + int(r) * N * 4, N, np.float32) for r in gemm_rows(rows4)])
            for p in (a, b, c):
                d.free(p)
            return res
        if name in ("asian", "asian_precise"):
            prm = sm.asian_params(k0=(seed + 5) & 0xFFFFFFFF, precise=int(name == "asian_precise"))
            out = d.alloc(32)
            d.asian(prm, 0, case["paths"], out)
            s = d.download(out, 4, np.float64)
            d.free(out)
            return np.array([DISC * s[0] / case["paths"], DISC * s[1] / case["paths"]], np.float64)
        raise ValueError(name)


class NvPtx:
    """The reference compiler's PTX on the GPU, launched the way the reference's host
    programs launch (one thread per element, 256-thread blocks; the chunk-sum kernels
    one block of up to 1024 threads, partial sums combined on the host as the CPU
    checker combines them)."""
    name = "nvptx"

    def __init__(self):
        import ctypes as C
        self.C = C
        self.L = L = sm.lib()
        L.nv_rt_alloc.restype = C.c_uint64
        L.nv_rt_alloc.argtypes = [C.c_void_p, C.c_size_t]
        L.nv_rt_free.argtypes = [C.c_void_p, C.c_uint64]
        L.nv_rt_h2d.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_size_t]
        L.nv_rt_d2h.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_size_t]
        L.nv_rt_load.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p, C.c_void_p]
        L.nv_rt_launch.argtypes = [C.c_void_p, C.c_void_p] + [C.c_uint32] * 7 + [C.c_void_p]
        self.dev = (C.c_char * 320)()
        if L.nv_rt_init(self.dev) != 0:
            raise RuntimeError("nv_rt_init failed")
        self.dir = os.path.join(ROOT, "oracle", "_ref", "ptx")

    def close(self):
        self.L.nv_rt_shut(self.dev)

    def _launch(self, ptx, entry, arrays, scalars, grid, block, out_index):
        C, L = self.C, self.L
        path = os.path.join(self.dir, ptx)
        if not os.path.exists(path):
            return None
        k = (C.c_char * 144)()
        if L.nv_rt_load(self.dev, path.encode(), entry, k) != 0:
            raise RuntimeError("nv_rt_load %s" % ptx)
        ptrs = []
        for arr in arrays:
            p = L.nv_rt_alloc(self.dev, max(arr.nbytes, 4))
            L.nv_rt_h2d(self.dev, p, arr.ctypes.data, arr.nbytes)
            ptrs.append(p)
        vals = [C.c_uint64(p) for p in ptrs] + scalars
        args = (C.c_void_p * len(vals))(*[C.cast(C.pointer(v), C.c_void_p) for v in vals])
        if L.nv_rt_launch(self.dev, k, grid, 1, 1, block, 1, 1, 0, args) != 0 or L.nv_rt_sync(self.dev) != 0:
            raise RuntimeError("launch of %s" % entry)
        out = np.empty_like(arrays[out_index])
        L.nv_rt_d2h(self.dev, out.ctypes.data, ptrs[out_index], out.nbytes)
        for p in ptrs:
            L.nv_rt_free(self.dev, p)
        L.nv_rt_unload(self.dev, k)
        return out

    def run(self, w, case, seed):
        C, n, name = self.C, case.get("n", 0), w["name"]
        if n >= 1 << 28:
            return None                                  # host-side staging of the whole vector: keep it modest
        grid = (n + 255) // 256
        if name == "vadd":
            x, y = sm.fill_host(n, seed, 0, 0), sm.fill_host(n, seed, 1, 0)
            return self._launch("vadd.ptx", b"vadd", [x, y, np.empty(n, np.float32)], [C.c_int(n)], grid, 256, 2)
        if name == "saxpy":
            x, y = sm.fill_host(n, seed + 1, 0, 0), sm.fill_host(n, seed + 1, 1, 0)
            return self._launch("saxpy.ptx", b"saxpy", [y, x], [C.c_float(w["alpha"]), C.c_int(n)], grid, 256, 0)
        if name in ("reduce_i32", "reduce_f32"):
            threads = min(n, 1024)
            chunk = n // threads                         # the tail beyond threads * chunk is added on the host
            kind = name[-3:]
            v = sm.fill_host(n, seed + 2, 0, 2) if kind == "i32" else sm.fill_host(n, seed + 2, 1, 1)
            part = self._launch("reduce_chunk_%s.ptx" % kind, ("reduce_chunk_%s" % kind).encode(),
                                [np.empty(threads, v.dtype), v], [C.c_int(chunk)], 1, threads, 0)
            if part is None:
                return None
            tail = v[threads * chunk:]
            if kind == "i32":
                total = part.sum(dtype=np.int64) + tail.sum(dtype=np.int64)
                return np.array([int(np.int64(total).astype(np.int32))], np.int64)
            return np.array([float(part.astype(np.float64).sum() + tail.astype(np.float64).sum())], np.float64)
        return None


def gemm_rows4(case):
    if "rows4" not in case:
        return None
    rng = np.random.default_rng(case["m"])
    return np.sort(rng.choice(case["m"] // 4, size=case["rows4"], replace=False)).astype(np.int32)


def gemm_rows(rows4):
    return (rows4[:, None] * 4 + np.arange(4)[None, :]).ravel()


def summary(w, res):
    if w["name"] in ("vadd", "saxpy"):
        return float(res.astype(np.float64).mean())
    if w["name"] == "gemm":
        return float(np.linalg.norm(res.astype(np.float64)))
    return [float(v) for v in res] if res.size > 1 else float(res[0])


def accuracy(w, got, want):
    """Error of `got` against the known-good `want` in the workload's own measure."""
    if w["tolerance"] == 0:
        if got.dtype.kind == "f":
            return float(np.count_nonzero(got.view(np.uint32) != want.view(np.uint32)))
        return float(np.count_nonzero(got != want))
    if w["name"] == "gemm":
        g, t = got.astype(np.float64), want.astype(np.float64)
        return float(np.linalg.norm(g - t) / np.linalg.norm(t))
    if w["name"] == "reduce_f32":          # the workload's answer is the fp32 value
        return float(abs(np.float32(got[0]) - np.float32(want[0])) / abs(want[0]))
    return float(np.max(np.abs(got - want) / np.abs(want)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backends", default="cpu")
    ap.add_argument("--full", action="store_true", help="also run the BASELINE-size cases")
    ap.add_argument("--inject", action="store_true", help="corrupt one sm100 output element; the run must FAIL")
    ap.add_argument("--update-baseline", action="store_true")
    ap.add_argument("--workload")
    args = ap.parse_args()
    man = json.load(open(os.path.join(HERE, "manifest.json")))
    gate, seed = man["config"]["regression_gate_rel"], man["config"]["seed"]
    bl_path = os.path.join(HERE, "baseline.json")
    baseline = json.load(open(bl_path)) if os.path.exists(bl_path) else {}
    names = args.backends.split(",")
    cpu = Cpu()
    gpu = Sm100() if "sm100" in names else None
    ptx = NvPtx() if "nvptx" in names else None
    failures, measured = [], {}
    for w in man["workloads"]:
        if args.workload and w["name"] != args.workload:
            continue
        for case in w["cases"]:
            if case.get("full") and not args.full:
                continue
            key = key_of(w, case)
            want = cpu.run(w, case, seed)
            for be in names:
                res = want if be == "cpu" else gpu.run(w, case, seed) if be == "sm100" else ptx.run(w, case, seed)
                if res is None:
                    print("  %-4s %-6s %-40s not produced by this backend" % ("skip", be, key), flush=True)
                    continue
                if be == "sm100" and args.inject:
                    res = res.copy()
                    flat = res.reshape(-1)
                    flat[flat.size // 2] = flat[flat.size // 2] * 1.001 + 1
                verdict, notes = "ok", []
                if be != "cpu":
                    err = accuracy(w, res, want)
                    if err > w["tolerance"]:
                        verdict = "FAIL"
                        notes.append("accuracy %.3g > %g" % (err, w["tolerance"]))
                    else:
                        notes.append("accuracy %.3g" % err)
                s = summary(w, res)
                measured.setdefault(be, {})[key] = s
                prev = baseline.get(be, {}).get(key)
                if prev is None:
                    notes.append("no baseline (recorded)")
                else:
                    pa, sa = np.atleast_1d(prev).astype(np.float64), np.atleast_1d(s).astype(np.float64)
                    drift = float(np.max(np.abs(sa - pa) / np.where(pa != 0, np.abs(pa), 1.0)))
                    if drift > gate:
                        verdict = "FAIL"
                        notes.append("regression %.3g vs baseline" % drift)
                if verdict == "FAIL":
                    failures.append("%s %s" % (be, key))
                print("  %-4s %-6s %-40s %s  [%s]" % (verdict, be, key, s, "; ".join(notes)), flush=True)
    if args.update_baseline:
        for be, dct in measured.items():
            baseline.setdefault(be, {}).update(dct)
        with open(bl_path, "w") as f:
            f.write(json.dumps(baseline, indent=2, sort_keys=True) + "\n")
        print("baseline updated:", bl_path)
    if gpu:
        gpu.d.close()
    if ptx:
        ptx.close()
    if failures:
        print("FAILED: %d line(s): %s" % (len(failures), ", ".join(failures[:8])))
        return 1
    print("all ok (checker: %s)" % cpu.o.kind)
    return 0


if __name__ == "__main__":
    sys.exit(main())
