"""booth_b200 -- Python bindings (ctypes) over libbooth_sm100.so.

The product is the C-ABI library: Booth's launcher API (``bc_*``,
src/runtime/bc_runtime.h:43-67 in the reference), the driver shim (``sm100_rt_*``,
the sm_100a twin of src/nvidia/nv_rt.h:96-127), the five workloads
(``booth_sm100_*``) and the NCCL all-reduce (``sm100_comm_*``). This module only
loads that library and gives its entry points Python signatures, for the tests
and the benchmark. Nothing here computes: without the library, or without a
B200 behind it, calls raise.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libbooth_sm100.so")
CUBIN_PATH = os.path.join(_HERE, "lib", "booth_sm100.cubin")
INCLUDE_DIR = os.path.join(os.path.dirname(_HERE), "include")

OK, ERR_DL, ERR_SYM, ERR_CUDA, ERR_NO_GPU, ERR_IO, ERR_KERN, ERR_ARG, ERR_NCCL = 0, -1, -2, -3, -4, -5, -6, -7, -8
FILL_F32_PM1, FILL_F32_01, FILL_I32_1000, FILL_U32_RAW = 0, 1, 2, 3
I32, F32, F64 = 0, 1, 2
GEMM_B_UNCHANGED, GEMM_TEST_SILENT_PRODUCER = 1, 0x80000000
COMM_ID_BYTES = 128

_ptr = C.c_ulonglong
_dev = C.c_void_p


class Sm100Error(RuntimeError):
    """A libbooth_sm100 entry point returned a non-zero status."""

    def __init__(self, what, code, detail=""):
        super().__init__("%s failed with status %d%s" % (what, code, (": " + detail) if detail else ""))
        self.code = code


class AsianParams(C.Structure):
    """booth_asian_t (include/booth_sm100.h)."""
    _fields_ = [("s0", C.c_float), ("strike", C.c_float), ("drift", C.c_float), ("vol", C.c_float),
                ("nstep", C.c_int32), ("k0", C.c_uint32), ("k1", C.c_uint32), ("precise", C.c_int32)]


class Kern(C.Structure):
    """sm100_kern_t (include/booth_sm100.h)."""
    _fields_ = [("mod", C.c_void_p), ("func", C.c_void_p), ("param_bytes", C.c_uint32),
                ("shared_bytes", C.c_uint32), ("local_bytes", C.c_uint32), ("_pad", C.c_uint32),
                ("name", C.c_char * 128)]


class BcKernel(C.Structure):
    """bc_kernel_t (include/bc_runtime.h)."""
    _fields_ = [("kernel_object", C.c_uint64), ("kernarg_size", C.c_uint32), ("group_size", C.c_uint32),
                ("private_size", C.c_uint32), ("_exec", C.c_uint64), ("_reader", C.c_uint64)]


class BcDevice(C.Structure):
    """bc_device_t (include/bc_runtime.h)."""
    _fields_ = [("_data", C.c_uint8 * 384)]


_SIGNATURES = {
    # layer 1
    "sm100_rt_init": (C.c_int, [C.POINTER(_dev), C.c_int]),
    "sm100_rt_shut": (None, [_dev]),
    "sm100_rt_device_count": (C.c_int, []),
    "sm100_rt_name": (C.c_char_p, [_dev]),
    "sm100_rt_sm_count": (C.c_int, [_dev]),
    "sm100_rt_ordinal": (C.c_int, [_dev]),
    "sm100_rt_errs": (C.c_char_p, [_dev]),
    "sm100_rt_load": (C.c_int, [_dev, C.c_char_p, C.c_char_p, C.POINTER(Kern)]),
    "sm100_rt_load_builtin": (C.c_int, [_dev, C.c_char_p, C.POINTER(Kern)]),
    "sm100_rt_unload": (None, [_dev, C.POINTER(Kern)]),
    "sm100_rt_alloc": (_ptr, [_dev, C.c_size_t]),
    "sm100_rt_free": (None, [_dev, _ptr]),
    "sm100_rt_h2d": (C.c_int, [_dev, _ptr, C.c_void_p, C.c_size_t]),
    "sm100_rt_d2h": (C.c_int, [_dev, C.c_void_p, _ptr, C.c_size_t]),
    "sm100_rt_h2d_async": (C.c_int, [_dev, _ptr, C.c_void_p, C.c_size_t]),
    "sm100_rt_d2h_async": (C.c_int, [_dev, C.c_void_p, _ptr, C.c_size_t]),
    "sm100_rt_zero": (C.c_int, [_dev, _ptr, C.c_size_t]),
    "sm100_rt_launch": (C.c_int, [_dev, C.POINTER(Kern)] + [C.c_uint32] * 7 + [C.POINTER(C.c_void_p)]),
    "sm100_rt_launch_packed": (C.c_int, [_dev, C.POINTER(Kern)] + [C.c_uint32] * 7 + [C.c_void_p, C.c_uint32]),
    "sm100_rt_sync": (C.c_int, [_dev]),
    "sm100_rt_hostalloc": (C.c_int, [_dev, C.POINTER(C.c_void_p), C.c_size_t]),
    "sm100_rt_hostmap": (C.c_int, [_dev, C.POINTER(C.c_void_p), C.POINTER(C.c_uint64), C.c_size_t]),
    "sm100_rt_hostfree": (None, [_dev, C.c_void_p]),
    "sm100_rt_tic": (C.c_int, [_dev]),
    "sm100_rt_toc": (C.c_int, [_dev, C.POINTER(C.c_float)]),
    "sm100_rt_launches": (C.c_ulonglong, [_dev]),
    "sm100_rt_stream": (C.c_void_p, [_dev]),
    # layer 2
    "booth_sm100_fill": (C.c_int, [_dev, _ptr, C.c_longlong, C.c_longlong, C.c_uint32, C.c_uint32, C.c_int]),
    "booth_sm100_fill_host": (None, [C.c_void_p, C.c_longlong, C.c_longlong, C.c_uint32, C.c_uint32, C.c_int, C.c_int]),
    "booth_sm100_philox4x32_10": (None, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "booth_sm100_vadd": (C.c_int, [_dev, _ptr, _ptr, _ptr, C.c_longlong]),
    "booth_sm100_saxpy": (C.c_int, [_dev, _ptr, _ptr, C.c_float, C.c_longlong]),
    "booth_sm100_vadd_host": (C.c_int, [_dev, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong]),
    "booth_sm100_saxpy_host": (C.c_int, [_dev, C.c_void_p, C.c_void_p, C.c_float, C.c_longlong]),
    "booth_sm100_link_probe": (C.c_int, [_dev, C.c_size_t, C.c_int, C.POINTER(C.c_double)]),
    "booth_sm100_reduce_i32": (C.c_int, [_dev, _ptr, C.c_longlong, _ptr]),
    "booth_sm100_reduce_f32": (C.c_int, [_dev, _ptr, C.c_longlong, _ptr]),
    "booth_sm100_reduce_f32_noalloc": (C.c_int, [_ptr, C.c_longlong, _ptr, C.c_void_p]),
    "booth_sm100_gemm": (C.c_int, [_dev, _ptr, _ptr, _ptr, C.c_int, C.c_int, C.c_int]),
    "booth_sm100_gemm_ex": (C.c_int, [_dev, _ptr, _ptr, _ptr, C.c_int, C.c_int, C.c_int, C.c_uint]),
    "booth_sm100_gemm_wait_limit": (C.c_int, [_dev, C.c_uint]),
    "booth_sm100_asian": (C.c_int, [_dev, C.POINTER(AsianParams), C.c_longlong, C.c_longlong, _ptr]),
    "booth_sm100_asian_paths": (C.c_int, [_dev, C.POINTER(AsianParams), C.c_longlong, C.c_longlong, _ptr, _ptr]),
    # layer 3
    "sm100_comm_unique_id": (C.c_int, [C.c_void_p]),
    "sm100_comm_init_rank": (C.c_int, [C.POINTER(C.c_void_p), _dev, C.c_int, C.c_int, C.c_void_p]),
    "sm100_comm_init_all": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(_dev), C.c_int]),
    "sm100_comm_allreduce_sum": (C.c_int, [C.c_void_p, _ptr, C.c_size_t, C.c_int]),
    "sm100_comm_allreduce_sum_dev": (C.c_int, [C.c_void_p, C.c_int, _ptr, C.c_size_t, C.c_int]),
    "sm100_comm_group_begin": (C.c_int, []),
    "sm100_comm_group_end": (C.c_int, []),
    "sm100_comm_destroy": (None, [C.c_void_p]),
    # Booth's launcher API
    "bc_device_init": (C.c_int, [C.POINTER(BcDevice)]),
    "bc_device_shutdown": (None, [C.POINTER(BcDevice)]),
    "bc_load_kernel": (C.c_int, [C.POINTER(BcDevice), C.c_char_p, C.c_char_p, C.POINTER(BcKernel)]),
    "bc_unload_kernel": (None, [C.POINTER(BcDevice), C.POINTER(BcKernel)]),
    "bc_alloc": (C.c_void_p, [C.POINTER(BcDevice), C.c_size_t]),
    "bc_free": (None, [C.POINTER(BcDevice), C.c_void_p]),
    "bc_trak": (None, [C.POINTER(BcDevice), C.c_void_p, C.c_size_t, C.c_char_p, C.c_int]),
    "bc_copy_h2d": (C.c_int, [C.POINTER(BcDevice), C.c_void_p, C.c_void_p, C.c_size_t]),
    "bc_copy_d2h": (C.c_int, [C.POINTER(BcDevice), C.c_void_p, C.c_void_p, C.c_size_t]),
    "bc_dispatch": (C.c_int, [C.POINTER(BcDevice), C.POINTER(BcKernel)] + [C.c_uint32] * 6 + [C.c_void_p, C.c_uint32]),
    # CPU-launcher symbols (host pointers)
    "vector_add": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "matmul": (None, [C.c_void_p] * 3 + [C.c_int] * 7),
    "matmul_k": (None, [C.c_void_p] * 3 + [C.c_int] * 8),
    "saxpy": (None, [C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int]),
    "vadd": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
}

_lib = None


def lib():
    """The loaded C-ABI library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("libbooth_sm100.so is missing (%s): run `python -m booth_b200.build`; "
                              "there is no fallback path" % LIB_PATH)
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def exported_symbols():
    """Names this module binds; every one must be exported by the library."""
    return sorted(_SIGNATURES)


def _addr(a):
    return a.ctypes.data_as(C.c_void_p)


class Device:
    """One B200 behind the shim (sm100_dev_t)."""

    def __init__(self, ordinal=-1):
        self._h = _dev()
        rc = lib().sm100_rt_init(C.byref(self._h), ordinal)
        if rc != OK:
            raise Sm100Error("sm100_rt_init", rc, "see the 'sm100_rt:' line on stderr")
        self._owned = []

    # -- plumbing --
    def _ck(self, what, rc):
        if rc != OK:
            raise Sm100Error(what, rc, (lib().sm100_rt_errs(self._h) or b"").decode())

    @property
    def handle(self):
        return self._h

    @property
    def name(self):
        return lib().sm100_rt_name(self._h).decode()

    @property
    def sm_count(self):
        return lib().sm100_rt_sm_count(self._h)

    @property
    def stream(self):
        """The CUstream this device's work runs on, as an integer handle."""
        return lib().sm100_rt_stream(self._h)

    @property
    def launches(self):
        return int(lib().sm100_rt_launches(self._h))

    def close(self):
        if self._h:
            for p in self._owned:
                lib().sm100_rt_free(self._h, p)
            self._owned = []
            lib().sm100_rt_shut(self._h)
            self._h = _dev()

    def alloc(self, nbytes):
        p = lib().sm100_rt_alloc(self._h, nbytes)
        if not p:
            raise Sm100Error("sm100_rt_alloc(%d)" % nbytes, ERR_CUDA, (lib().sm100_rt_errs(self._h) or b"").decode())
        self._owned.append(p)
        return p

    def free(self, p):
        if p in self._owned:
            self._owned.remove(p)
        lib().sm100_rt_free(self._h, p)

    def upload(self, arr):
        arr = np.ascontiguousarray(arr)
        p = self.alloc(max(arr.nbytes, 4))
        self._ck("sm100_rt_h2d", lib().sm100_rt_h2d(self._h, p, _addr(arr), arr.nbytes))
        return p

    def h2d(self, p, arr):
        arr = np.ascontiguousarray(arr)
        self._ck("sm100_rt_h2d", lib().sm100_rt_h2d(self._h, p, _addr(arr), arr.nbytes))

    def download(self, p, shape, dtype):
        out = np.empty(shape, dtype=dtype)
        self._ck("sm100_rt_d2h", lib().sm100_rt_d2h(self._h, _addr(out), p, out.nbytes))
        return out

    def zero(self, p, nbytes):
        self._ck("sm100_rt_zero", lib().sm100_rt_zero(self._h, p, nbytes))

    def sync(self):
        self._ck("sm100_rt_sync", lib().sm100_rt_sync(self._h))

    def tic(self):
        self._ck("sm100_rt_tic", lib().sm100_rt_tic(self._h))

    def toc(self):
        ms = C.c_float()
        self._ck("sm100_rt_toc", lib().sm100_rt_toc(self._h, C.byref(ms)))
        return ms.value

    def hostalloc(self, nbytes):
        hp = C.c_void_p()
        self._ck("sm100_rt_hostalloc", lib().sm100_rt_hostalloc(self._h, C.byref(hp), nbytes))
        return hp.value

    def hostfree(self, hp):
        lib().sm100_rt_hostfree(self._h, hp)

    def h2d_async(self, p, host_addr, nbytes):
        self._ck("sm100_rt_h2d_async", lib().sm100_rt_h2d_async(self._h, p, host_addr, nbytes))

    def d2h_async(self, host_addr, p, nbytes):
        self._ck("sm100_rt_d2h_async", lib().sm100_rt_d2h_async(self._h, host_addr, p, nbytes))

    # -- workloads --
    def fill(self, p, first, n, seed, stream, kind):
        self._ck("booth_sm100_fill", lib().booth_sm100_fill(self._h, p, first, n, seed, stream, kind))

    def vadd(self, x, y, out, n):
        self._ck("booth_sm100_vadd", lib().booth_sm100_vadd(self._h, x, y, out, n))

    def saxpy(self, y, x, a, n):
        self._ck("booth_sm100_saxpy", lib().booth_sm100_saxpy(self._h, y, x, a, n))

    def saxpy_host(self, y_addr, x_addr, a, n):
        """y = a*x + y on host vectors (addresses), pipelined over the link."""
        self._ck("booth_sm100_saxpy_host", lib().booth_sm100_saxpy_host(self._h, y_addr, x_addr, a, n))

    def vadd_host(self, x_addr, y_addr, out_addr, n):
        self._ck("booth_sm100_vadd_host", lib().booth_sm100_vadd_host(self._h, x_addr, y_addr, out_addr, n))

    def link_probe(self, nbytes=1 << 30, reps=3):
        """GB/s of the host link with pinned memory: (up alone, down alone, up and down while both run)."""
        g = (C.c_double * 4)()
        self._ck("booth_sm100_link_probe", lib().booth_sm100_link_probe(self._h, nbytes, reps, g))
        return tuple(g)

    def reduce_i32(self, inp, n, out):
        self._ck("booth_sm100_reduce_i32", lib().booth_sm100_reduce_i32(self._h, inp, n, out))

    def reduce_f32(self, inp, n, out):
        self._ck("booth_sm100_reduce_f32", lib().booth_sm100_reduce_f32(self._h, inp, n, out))

    def gemm(self, c, a, b, M, N, K, b_unchanged=False, flags=0):
        flags |= GEMM_B_UNCHANGED if b_unchanged else 0
        if flags:
            self._ck("booth_sm100_gemm_ex", lib().booth_sm100_gemm_ex(self._h, c, a, b, M, N, K, flags))
        else:
            self._ck("booth_sm100_gemm", lib().booth_sm100_gemm(self._h, c, a, b, M, N, K))

    def gemm_wait_limit(self, ms):
        self._ck("booth_sm100_gemm_wait_limit", lib().booth_sm100_gemm_wait_limit(self._h, ms))

    def asian(self, params, path0, npaths, out):
        self._ck("booth_sm100_asian", lib().booth_sm100_asian(self._h, C.byref(params), path0, npaths, out))

    def asian_paths(self, params, path0, npaths, arith, geom):
        self._ck("booth_sm100_asian_paths",
                 lib().booth_sm100_asian_paths(self._h, C.byref(params), path0, npaths, arith, geom))


class Comm:
    """NCCL communicator for one process per GPU (sm100_comm_init_rank)."""

    def __init__(self, dev, nranks, rank, unique_id):
        self._h = C.c_void_p()
        buf = C.create_string_buffer(bytes(unique_id), COMM_ID_BYTES)
        rc = lib().sm100_comm_init_rank(C.byref(self._h), dev.handle, nranks, rank, buf)
        if rc != OK:
            raise Sm100Error("sm100_comm_init_rank", rc)

    @staticmethod
    def unique_id():
        buf = C.create_string_buffer(COMM_ID_BYTES)
        rc = lib().sm100_comm_unique_id(buf)
        if rc != OK:
            raise Sm100Error("sm100_comm_unique_id", rc)
        return buf.raw

    def allreduce_sum(self, p, count, dtype):
        rc = lib().sm100_comm_allreduce_sum(self._h, p, count, dtype)
        if rc != OK:
            raise Sm100Error("sm100_comm_allreduce_sum", rc)

    def close(self):
        if self._h:
            lib().sm100_comm_destroy(self._h)
            self._h = C.c_void_p()


def fill_host(n, seed, stream, kind, first=0, threads=8):
    """The seeded input stream, generated on the host (same bits as Device.fill)."""
    out = np.empty(n, dtype={FILL_I32_1000: np.int32, FILL_U32_RAW: np.uint32}.get(kind, np.float32))
    lib().booth_sm100_fill_host(_addr(out), first, n, seed, stream, kind, threads)
    return out


def asian_params(s0=100.0, strike=100.0, r=0.05, sigma=0.2, T=1.0, nstep=252, k0=0xB0070005, k1=0, precise=0):
    """drift and vol in fp32, the way the CPU statement of the workload gets them."""
    dt = np.float32(T) / np.float32(nstep)
    drift = (np.float32(r) - np.float32(0.5) * np.float32(sigma) * np.float32(sigma)) * dt
    vol = np.float32(sigma) * np.sqrt(dt, dtype=np.float32)
    return AsianParams(float(np.float32(s0)), float(np.float32(strike)), float(drift), float(vol),
                       int(nstep), int(k0), int(k1), int(precise))


def shard_range(n, rank, world, multiple=4):
    """Contiguous range [lo, hi) of rank `rank` when n elements are cut into
    `world` shards whose bounds are multiples of `multiple` (so 16-byte vector
    accesses stay aligned); the last shard takes the remainder."""
    units = n // multiple
    lo = units * rank // world * multiple
    hi = n if rank == world - 1 else units * (rank + 1) // world * multiple
    return lo, hi
