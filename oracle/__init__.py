"""oracle -- the CPU checker for the B200 path. TEST INFRASTRUCTURE ONLY.

Only the test-suite, ``__graft_entry__.smoke()`` and the benchmark's CPU
baseline / reference arm may import this package, and only to check or to time
the CPU side. The product (booth_b200) never does.

Two interchangeable libraries export the same ``orc_*`` entry points
(oracle/harness.c):

* ``reference``  oracle/_ref/libbooth_ref.so: the kernels as emitted by the
  reference compiler's own x86-64 backend (``kath --cpu``), built from the
  reference's sources by oracle/Makefile. It is a build product (git-ignored)
  and exists wherever ``make -C oracle`` ran with the reference tree present.
* ``port``       oracle/libbooth_port.so: the C restatement in oracle/port.c,
  bit-identical to the above on every case tests/test_oracle.py runs.

``load()`` prefers the reference build and falls back to the port.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_SO = os.path.join(HERE, "_ref", "libbooth_ref.so")
PORT_SO = os.path.join(HERE, "libbooth_port.so")


def build(want_ref=True):
    """(Re)build the checker libraries with oracle/Makefile."""
    target = ["all"] if want_ref else ["libbooth_port.so"]
    res = subprocess.run(["make", "-C", HERE, "-j8"] + target, stdout=subprocess.PIPE,
                         stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + res.stdout)
    return res.stdout


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


class Oracle:
    """One of the two checker libraries behind the orc_* entry points."""

    def __init__(self, path, kind):
        self.kind = kind            # "reference" or "port"
        self.path = path
        L = C.CDLL(path)
        L.orc_cores.restype = C.c_int
        L.orc_now.restype = C.c_double
        L.orc_vadd.argtypes = [C.c_void_p] * 3 + [C.c_longlong, C.c_int]
        L.orc_saxpy.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_longlong, C.c_int]
        L.orc_reduce_i32.argtypes = [C.c_void_p, C.c_longlong, C.c_int, C.c_int]
        L.orc_reduce_i32.restype = C.c_int
        L.orc_reduce_f32.argtypes = [C.c_void_p, C.c_longlong, C.c_int, C.c_int]
        L.orc_reduce_f32.restype = C.c_double
        L.orc_sum_f64.argtypes = [C.c_void_p, C.c_longlong, C.c_int]
        L.orc_sum_f64.restype = C.c_double
        L.orc_matmul.argtypes = [C.c_void_p] * 3 + [C.c_int] * 3 + [C.c_void_p, C.c_int, C.c_int]
        L.orc_matmul_tile.argtypes = [C.c_void_p] * 3 + [C.c_int] * 6
        L.orc_asian.argtypes = [C.c_longlong, C.c_longlong, C.c_uint, C.c_uint] + [C.c_float] * 4 + \
                               [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        self.L = L
        self.cores = L.orc_cores()

    def vadd(self, x, y, threads=None):
        out = np.empty_like(x)
        self.L.orc_vadd(_p(x), _p(y), _p(out), x.size, threads or self.cores)
        return out

    def saxpy(self, y, x, a, threads=None):
        """Returns a*x + y; y is not modified."""
        out = y.copy()
        self.L.orc_saxpy(_p(out), _p(x), a, x.size, threads or self.cores)
        return out

    def saxpy_inplace(self, y, x, a, threads=None):
        self.L.orc_saxpy(_p(y), _p(x), a, x.size, threads or self.cores)

    def reduce_i32(self, v, chunk=4096, threads=None):
        return int(self.L.orc_reduce_i32(_p(v), v.size, chunk, threads or self.cores))

    def reduce_f32(self, v, chunk=4096, threads=None):
        """fp32 chunk sums combined in double; the fp32 answer is np.float32 of it."""
        return float(self.L.orc_reduce_f32(_p(v), v.size, chunk, threads or self.cores))

    def sum_f64(self, v, threads=None):
        return float(self.L.orc_sum_f64(_p(v), v.size, threads or self.cores))

    def matmul(self, a, b, rows4=None, threads=None):
        """C = A.B by 4x4 tiles. With rows4 (int32 array of 4-row block indices)
        only those row blocks of C are computed; the rest stays zero."""
        M, K = a.shape
        K2, N = b.shape
        assert K == K2 and M % 4 == 0 and N % 4 == 0 and K % 2 == 0
        c = np.zeros((M, N), np.float32)
        if rows4 is None:
            self.L.orc_matmul(_p(a), _p(b), _p(c), M, N, K, None, 0, threads or self.cores)
        else:
            rows4 = np.ascontiguousarray(rows4, dtype=np.int32)
            self.L.orc_matmul(_p(a), _p(b), _p(c), M, N, K, _p(rows4), rows4.size, threads or self.cores)
        return c

    def matmul_tile(self, a, b, c, sam, sak, sbk, sbn, scm, scn):
        self.L.orc_matmul_tile(_p(a), _p(b), _p(c), sam, sak, sbk, sbn, scm, scn)

    def asian(self, params, path0, npaths, threads=None, per_path=False):
        """Returns (sum_arith, sum_geom[, arith[], geom[]]) -- undiscounted sums."""
        sums = (C.c_double * 2)()
        pa = np.empty(npaths, np.float32) if per_path else None
        pg = np.empty(npaths, np.float32) if per_path else None
        self.L.orc_asian(path0, npaths, params.k0, params.k1, params.s0, params.strike,
                         params.drift, params.vol, params.nstep, threads or self.cores, sums,
                         _p(pa) if per_path else None, _p(pg) if per_path else None)
        if per_path:
            return sums[0], sums[1], pa, pg
        return sums[0], sums[1]

    def now(self):
        return self.L.orc_now()


def load(kind=None):
    """kind: None (reference if built, else port), "reference" or "port"."""
    if kind in (None, "reference") and os.path.exists(REF_SO):
        return Oracle(REF_SO, "reference")
    if kind == "reference":
        raise FileNotFoundError("oracle/_ref/libbooth_ref.so is not built (run make -C oracle with the reference tree)")
    if not os.path.exists(PORT_SO):
        build(want_ref=False)
    return Oracle(PORT_SO, "port")
