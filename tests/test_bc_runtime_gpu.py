"""GPU: Booth's launcher API (bc_*) served by the sm_100a runtime, driven the way
examples/launch_saxpy.c drives it, plus its host-detectable failure paths."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


class SaxpyArgs(C.Structure):
    # examples/launch_saxpy.c:71-81: {void *y; void *x; float a; uint32_t n}
    _fields_ = [("y", C.c_void_p), ("x", C.c_void_p), ("a", C.c_float), ("n", C.c_uint32)]


@pytest.fixture()
def bc(sm):
    L = sm.lib()
    d = sm.BcDevice()
    assert L.bc_device_init(C.byref(d)) == 0
    yield L, d
    L.bc_device_shutdown(C.byref(d))


def test_launch_saxpy_flow(sm, bc):
    L, d = bc
    N, BLOCK = 1024, 256
    k = sm.BcKernel()
    assert L.bc_load_kernel(C.byref(d), sm.CUBIN_PATH.encode(), b"saxpy", C.byref(k)) == 0
    assert k.kernarg_size == 24 and k.kernel_object != 0
    x = np.arange(N, dtype=np.float32)                       # launch_saxpy.c:54-58
    y = (N - np.arange(N)).astype(np.float32)
    want = np.float32(2.5) * x + y
    dx, dy = L.bc_alloc(C.byref(d), N * 4), L.bc_alloc(C.byref(d), N * 4)
    assert dx and dy
    L.bc_trak(C.byref(d), dx, N * 4, b"x", 0)
    assert L.bc_copy_h2d(C.byref(d), dx, x.ctypes.data, N * 4) == 0
    assert L.bc_copy_h2d(C.byref(d), dy, y.ctypes.data, N * 4) == 0
    args = SaxpyArgs(dy, dx, 2.5, N)
    assert L.bc_dispatch(C.byref(d), C.byref(k), (N + BLOCK - 1) // BLOCK, 1, 1, BLOCK, 1, 1,
                         C.byref(args), C.sizeof(args)) == 0
    got = np.empty(N, np.float32)
    assert L.bc_copy_d2h(C.byref(d), got.ctypes.data, dy, N * 4) == 0
    assert np.array_equal(got, want)
    L.bc_free(C.byref(d), dx); L.bc_free(C.byref(d), dy); L.bc_free(C.byref(d), None)
    L.bc_unload_kernel(C.byref(d), C.byref(k))
    assert k.kernel_object == 0


@pytest.mark.parametrize("grid,block", [((1, 1, 1), (1, 1, 1)), ((0, 0, 0), (0, 0, 0)), ((7, 3, 2), (33, 3, 1)),
                                        ((40, 1, 1), (256, 1, 1)), ((2, 2, 1), (8, 8, 4)),
                                        # more blocks than the tuned geometry: only the first ones work
                                        ((5000, 1, 1), (256, 1, 1)), ((70, 30, 1), (1024, 1, 1)), ((3000, 1, 1), (33, 3, 1))])
def test_any_launch_geometry_and_oversized_args(sm, bc, oracle_lib, grid, block):
    L, d = bc
    n = 10001
    k = sm.BcKernel()
    assert L.bc_load_kernel(C.byref(d), sm.CUBIN_PATH.encode(), b"saxpy", C.byref(k)) == 0
    x = sm.fill_host(n, 3, 0, 0); y = sm.fill_host(n, 3, 1, 0)
    dx, dy = L.bc_alloc(C.byref(d), n * 4), L.bc_alloc(C.byref(d), n * 4)
    L.bc_copy_h2d(C.byref(d), dx, x.ctypes.data, n * 4)
    L.bc_copy_h2d(C.byref(d), dy, y.ctypes.data, n * 4)

    class Padded(C.Structure):          # a caller that appends hidden bytes (src/runtime/lf_gpu_hsa.c:243-255)
        _fields_ = [("a", SaxpyArgs), ("hidden", C.c_uint8 * 18)]
    args = Padded(SaxpyArgs(dy, dx, 2.5, n))
    assert L.bc_dispatch(C.byref(d), C.byref(k), *grid, *block, C.byref(args), C.sizeof(args)) == 0
    got = np.empty(n, np.float32)
    L.bc_copy_d2h(C.byref(d), got.ctypes.data, dy, n * 4)
    assert np.array_equal(got.view(np.uint32), oracle_lib.saxpy(y, x, 2.5).view(np.uint32))
    L.bc_free(C.byref(d), dx); L.bc_free(C.byref(d), dy)
    L.bc_unload_kernel(C.byref(d), C.byref(k))


def test_host_detectable_failures(sm, bc, tmp_path):
    L, d = bc
    k = sm.BcKernel()
    assert L.bc_load_kernel(C.byref(d), b"/nonexistent/file.cubin", b"saxpy", C.byref(k)) == -6   # BC_RT_ERR_IO
    assert L.bc_load_kernel(C.byref(d), sm.CUBIN_PATH.encode(), b"no_such_kernel", C.byref(k)) == -7  # ERR_SYMBOL
    junk = tmp_path / "junk.cubin"
    junk.write_bytes(b"not a cubin at all")
    assert L.bc_load_kernel(C.byref(d), str(junk).encode(), b"saxpy", C.byref(k)) == -3            # driver refused
    assert L.bc_dispatch(C.byref(d), C.byref(k), 1, 1, 1, 1, 1, 1, None, 0) == -7                   # nothing loaded
    assert L.bc_alloc(C.byref(d), 1 << 50) is None                                                # 1 PiB
    # the device is still usable afterwards
    p = L.bc_alloc(C.byref(d), 1024)
    assert p
    L.bc_free(C.byref(d), p)


def test_vector_add_by_name_through_the_shim(sm, dev, oracle_lib):
    """sm100_rt_load + pointer-per-argument launch, the nv_rt_launch form."""
    L = sm.lib()
    k = sm.Kern()
    assert L.sm100_rt_load(dev.handle, sm.CUBIN_PATH.encode(), b"vector_add", C.byref(k)) == 0
    assert k.param_bytes == 32
    n = 777
    x = sm.fill_host(n, 8, 0, 0); y = sm.fill_host(n, 8, 1, 0)
    dx, dy, do = dev.upload(x), dev.upload(y), dev.alloc(n * 4)
    vals = [C.c_ulonglong(dx), C.c_ulonglong(dy), C.c_ulonglong(do), C.c_int(n), C.c_int(256)]
    argv = (C.c_void_p * 5)(*[C.cast(C.pointer(v), C.c_void_p) for v in vals])
    assert L.sm100_rt_launch(dev.handle, C.byref(k), (n + 255) // 256, 1, 1, 256, 1, 1, 0, argv) == 0
    dev.sync()
    assert np.array_equal(dev.download(do, n, np.float32), oracle_lib.vadd(x, y))
    L.sm100_rt_unload(dev.handle, C.byref(k))


EXAMPLES = os.path.join(ROOT, "build", "examples")


@pytest.mark.parametrize("prog,needs_cubin,expect", [
    ("launch_saxpy", True, "PASS: all 1024 elements correct"),
    ("cpu_launch_vadd", False, "OK: Triton vector_add ran"),
    ("cpu_launch_matmul", False, "OK: Triton matmul ran"),
    ("rt_sm100_run", True, "PASS: descriptor 'sm100' (cubin) ran saxpy"),
    ("rt_sm100_run_refhdr", True, "PASS: descriptor 'sm100' (cubin) ran saxpy"),
    ("launch_workloads", False, "PASS: "),
])
def test_reference_example_programs_relinked(sm, prog, needs_cubin, expect):
    """The reference's own example sources, compiled unchanged where they lie in
    the reference tree and linked against libbooth_sm100 by the build step; and
    this repository's rt_sm100_run, which drives the GPU through the run-side
    descriptor contract (src/exec/exec.h:69-93), built once on the mirror header
    and once on the reference's own exec.h."""
    exe = os.path.join(EXAMPLES, prog)
    if not os.path.exists(exe):
        pytest.skip("build/examples/%s was not built (the reference tree was absent at build time)" % prog)
    cmd = [exe] + ([sm.CUBIN_PATH] if needs_cubin else [])
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120,
                         env=dict(os.environ, LD_LIBRARY_PATH=os.path.dirname(sm.LIB_PATH)))
    assert res.returncode == 0, res.stdout + res.stderr
    assert expect in res.stdout


@pytest.mark.parametrize("target", [["--target", "sm100"], []])
def test_reference_booth_run_launches_saxpy_on_the_b200(sm, oracle_lib, tmp_path, target):
    """Row "rt_desc_t registration": the reference's own command line
    (src/exec/booth_run.c:262-313, compiled unchanged; src/exec/execs.c with
    rt_list = { &rt_sm100, NULL }, its documented one-line edit) loads the cubin,
    stages the files, launches saxpy with the geometry given on the command line,
    and writes y back: bit-identical to the CPU checker. With --target and with the
    probing form (rt_open(NULL) takes the first target that has a device)."""
    exe = os.path.join(EXAMPLES, "booth-run")
    if not os.path.exists(exe):
        pytest.skip("build/examples/booth-run was not built (the reference tree was absent at build time)")
    n = 1024
    x = sm.fill_host(n, 0xB0070001, 0, 0)
    y = sm.fill_host(n, 0xB0070001, 1, 0)
    x.tofile(tmp_path / "x.bin"); y.tofile(tmp_path / "y.bin")
    cmd = [exe, sm.CUBIN_PATH, "saxpy"] + target + ["--grid", "4", "--block", "256", "io:%s" % (tmp_path / "y.bin"),
                                                    "in:%s" % (tmp_path / "x.bin"), "f32:2.5", "u32:%d" % n]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "wrote %s (%d bytes)" % (tmp_path / "y.bin", 4 * n) in res.stdout
    got = np.fromfile(tmp_path / "y.bin", np.float32)
    assert np.array_equal(got.view(np.uint32), oracle_lib.saxpy(y, x, 2.5).view(np.uint32))
    # teeth: the file really changed, and a wrong scalar gives another answer
    assert not np.array_equal(got, y)
    # out: form and a vector add by name, block count chosen by the caller (a ragged size)
    m = 1000
    out = tmp_path / "c.bin"
    x[:m].tofile(tmp_path / "a.bin"); y[:m].tofile(tmp_path / "b.bin")
    cmd = [exe, sm.CUBIN_PATH, "vector_add"] + target + ["--grid", "3", "--block", "128,2", "in:%s" % (tmp_path / "a.bin"),
                                                         "in:%s" % (tmp_path / "b.bin"), "out:%s:%d" % (out, 4 * m),
                                                         "i32:%d" % m, "i32:256"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert np.array_equal(np.fromfile(out, np.float32).view(np.uint32), oracle_lib.vadd(x[:m].copy(), y[:m].copy()).view(np.uint32))


def test_reference_differential_harness_relinked(sm):
    """The reference's own parity program (tests/diff/diff_vadd.c with bc_diff.h and
    vadd_io.h, compiled unchanged, linked against libbooth_sm100 in place of the
    kernel object its compiler emits): clean run PASSes, --inject FAILs, as
    tests/diff/run_diff.sh:32-44 demands of every backend. And tests/build/run_vadd.c,
    the same idea for the BIR kernel vadd(a, b, c, n, nthreads)."""
    exe = os.path.join(EXAMPLES, "diff_vadd")
    if not os.path.exists(exe):
        pytest.skip("build/examples/diff_vadd was not built (the reference tree was absent at build time)")
    clean = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert clean.returncode == 0 and "PASS" in clean.stdout, clean.stdout + clean.stderr
    inject = subprocess.run([exe, "--inject"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert inject.returncode != 0 and "FAIL" in inject.stdout, inject.stdout + inject.stderr
    res = subprocess.run([os.path.join(EXAMPLES, "run_vadd")], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert res.returncode == 0 and "all 16 elements correct" in res.stdout, res.stdout + res.stderr


def test_reference_sysprint_demo_relinked(sm):
    """A second consumer of the bc_* API: the reference's SYSPRINT demo
    (examples/launch_sysprint.c, runtime/sysprint.c) built unchanged against this
    library; its kernel (examples/sysprint_kernel.cu) compiled by nvcc for sm_100a.
    The kernel is a C++ symbol there, found by its bare name "sp_demo"."""
    exe, cubin = os.path.join(EXAMPLES, "launch_sysprint"), os.path.join(EXAMPLES, "sp_demo.cubin")
    if not (os.path.exists(exe) and os.path.exists(cubin)):
        pytest.skip("build/examples/launch_sysprint was not built (the reference tree was absent at build time)")
    res = subprocess.run([exe, cubin], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120,
                         env=dict(os.environ, LD_LIBRARY_PATH=os.path.dirname(sm.LIB_PATH)))
    assert res.returncode == 0, res.stdout + res.stderr
    assert "DEMO.RESULT: sp_demo done" in res.stdout and "dropped: 0" in res.stdout


def test_failed_launch_prints_dispatch_snapshot_and_labels(sm):
    """The launcher's share of the reference's ABEND dump (src/runtime/bc_abend.h:57-71):
    when the driver refuses a launch (a host-detected error: 2048 threads per block
    exceed the limit, nothing reaches the GPU), stderr names the kernel, the
    geometry, the parameter bytes and the buffers labelled with bc_trak."""
    code = r"""
import ctypes as C, booth_b200 as b
L = b.lib(); d = b.BcDevice(); assert L.bc_device_init(C.byref(d)) == 0
k = b.BcKernel(); assert L.bc_load_kernel(C.byref(d), b.CUBIN_PATH.encode(), b"saxpy", C.byref(k)) == 0
p = L.bc_alloc(C.byref(d), 4096); L.bc_trak(C.byref(d), p, 4096, b"ybuf", 0)
class A(C.Structure):
    _fields_ = [("y", C.c_void_p), ("x", C.c_void_p), ("a", C.c_float), ("n", C.c_uint32)]
a = A(p, p, 2.5, 16)
rc = L.bc_dispatch(C.byref(d), C.byref(k), 1, 1, 1, 2048, 1, 1, C.byref(a), C.sizeof(a))
print("rc", rc)
a.n = 16
print("rc_ok", L.bc_dispatch(C.byref(d), C.byref(k), 1, 1, 1, 256, 1, 1, C.byref(a), C.sizeof(a)))   # still usable
L.bc_free(C.byref(d), p); L.bc_device_shutdown(C.byref(d))
"""
    res = subprocess.run([os.sys.executable, "-c", code], cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                         text=True, timeout=120)
    assert "rc -3" in res.stdout and "rc_ok 0" in res.stdout, res.stdout + res.stderr
    assert "last dispatch: kernel 'saxpy' grid 1x1x1 block 2048x1x1" in res.stderr
    assert "24 parameter bytes" in res.stderr and "buffer 'ybuf'" in res.stderr


def test_one_process_many_devices_with_nccl(sm):
    """examples/launch_workloads.c on two GPUs: one C99 process, a communicator over
    both devices (sm100_comm_init_all), all-reduced sums checked against device 0
    alone. Skipped on a single-GPU machine (the CPU coverage of the sharding rules
    is tests/test_sharding_gloo.py)."""
    exe = os.path.join(EXAMPLES, "launch_workloads")
    if not os.path.exists(exe):
        pytest.skip("build/examples/launch_workloads was not built")
    if sm.lib().sm100_rt_device_count() < 2:
        pytest.skip("needs two GPUs")
    res = subprocess.run([exe, "2", "24", "20"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300,
                         env=dict(os.environ, LD_LIBRARY_PATH=os.path.dirname(sm.LIB_PATH), NCCL_NVLS_ENABLE="0"))
    assert res.returncode == 0, res.stdout + res.stderr
    assert "PASS: 2 device(s)" in res.stdout


def test_canonical_kernels_by_name(sm, bc):
    """matmul_general and reduce_sum (tests/canonical.cu:18-50,93-108) loaded by
    name and launched with the reference's geometry and with an unrelated one."""
    L, d = bc
    M, N, K = 37, 53, 29                               # "whatever size the user fancies"
    a = sm.fill_host(M * K, 61, 0, 0).reshape(M, K); b = sm.fill_host(K * N, 61, 1, 0).reshape(K, N)
    want = np.zeros((M, N), np.float32)
    for k in range(K):                                   # k ascending, product and sum rounded separately
        want = (want + (a[:, k:k + 1] * b[k:k + 1, :]).astype(np.float32)).astype(np.float32)

    class MmArgs(C.Structure):
        _fields_ = [("C", C.c_void_p), ("A", C.c_void_p), ("B", C.c_void_p), ("M", C.c_int), ("N", C.c_int), ("K", C.c_int)]
    k = sm.BcKernel()
    assert L.bc_load_kernel(C.byref(d), sm.CUBIN_PATH.encode(), b"matmul_general", C.byref(k)) == 0
    da, db, dc = (L.bc_alloc(C.byref(d), x) for x in (M * K * 4, K * N * 4, M * N * 4))
    L.bc_copy_h2d(C.byref(d), da, a.ctypes.data, M * K * 4); L.bc_copy_h2d(C.byref(d), db, b.ctypes.data, K * N * 4)
    args = MmArgs(dc, da, db, M, N, K)
    for grid, block in ((((N + 15) // 16, (M + 15) // 16, 1), (16, 16, 1)), ((2, 1, 1), (8, 4, 1))):
        got = np.full((M, N), -1, np.float32)
        L.bc_copy_h2d(C.byref(d), dc, got.ctypes.data, M * N * 4)
        assert L.bc_dispatch(C.byref(d), C.byref(k), *grid, *block, C.byref(args), C.sizeof(args)) == 0
        L.bc_copy_d2h(C.byref(d), got.ctypes.data, dc, M * N * 4)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    L.bc_unload_kernel(C.byref(d), C.byref(k))

    class RdArgs(C.Structure):
        _fields_ = [("out", C.c_void_p), ("inp", C.c_void_p), ("n", C.c_int)]
    assert L.bc_load_kernel(C.byref(d), sm.CUBIN_PATH.encode(), b"reduce_sum", C.byref(k)) == 0
    n = 100003
    v = sm.fill_host(n, 62, 0, 1)
    dv, do = L.bc_alloc(C.byref(d), n * 4), L.bc_alloc(C.byref(d), 4)
    L.bc_copy_h2d(C.byref(d), dv, v.ctypes.data, n * 4)
    for grid, block in (((64, 1, 1), (256, 1, 1)), ((3, 2, 1), (33, 1, 1))):
        zero = np.zeros(1, np.float32)
        L.bc_copy_h2d(C.byref(d), do, zero.ctypes.data, 4)
        rargs = RdArgs(do, dv, n)
        assert L.bc_dispatch(C.byref(d), C.byref(k), *grid, *block, C.byref(rargs), C.sizeof(rargs)) == 0
        L.bc_copy_d2h(C.byref(d), zero.ctypes.data, do, 4)
        assert abs(float(zero[0]) - float(v.astype(np.float64).sum())) <= 2e-5 * n * 0.5
    for p in (da, db, dc, dv, do):
        L.bc_free(C.byref(d), p)


def test_dot_product_and_tinygrad_reduction_by_name(sm, bc):
    """dot_product (tests/canonical.cu:149-161) and the tinygrad attention reduction
    r_2_1024_16_64 (tests/tg_reduce.cu:4-26) loaded by name through bc_*."""
    L, d = bc
    k = sm.BcKernel()

    class DotArgs(C.Structure):
        _fields_ = [("out", C.c_void_p), ("a", C.c_void_p), ("b", C.c_void_p), ("n", C.c_int)]
    assert L.bc_load_kernel(C.byref(d), sm.CUBIN_PATH.encode(), b"dot_product", C.byref(k)) == 0
    n = 250007
    a, b = sm.fill_host(n, 63, 0, 0), sm.fill_host(n, 63, 1, 0)
    da, db, do = L.bc_alloc(C.byref(d), n * 4), L.bc_alloc(C.byref(d), n * 4), L.bc_alloc(C.byref(d), 4)
    L.bc_copy_h2d(C.byref(d), da, a.ctypes.data, n * 4); L.bc_copy_h2d(C.byref(d), db, b.ctypes.data, n * 4)
    exact = float((a.astype(np.float64) * b.astype(np.float64)).sum())
    for grid, block in (((128, 1, 1), (256, 1, 1)), ((5, 3, 1), (40, 2, 1))):
        start = np.array([1.5], np.float32)                  # *result is added to, not overwritten
        L.bc_copy_h2d(C.byref(d), do, start.ctypes.data, 4)
        args = DotArgs(do, da, db, n)
        assert L.bc_dispatch(C.byref(d), C.byref(k), *grid, *block, C.byref(args), C.sizeof(args)) == 0
        L.bc_copy_d2h(C.byref(d), start.ctypes.data, do, 4)
        assert abs(float(start[0]) - 1.5 - exact) <= 1e-4 * np.sqrt(n)
    L.bc_unload_kernel(C.byref(d), C.byref(k))
    for p in (da, db, do):
        L.bc_free(C.byref(d), p)

    class TgArgs(C.Structure):
        _fields_ = [("data0", C.c_void_p), ("data1", C.c_void_p), ("data2", C.c_void_p), ("data3", C.c_void_p),
                    ("start_pos", C.c_int)]
    assert L.bc_load_kernel(C.byref(d), sm.CUBIN_PATH.encode(), b"r_2_1024_16_64", C.byref(k)) == 0
    rng = np.random.default_rng(64)
    start_pos = 3
    data1 = rng.integers(0, 4, 16 * 64).astype(np.int32)            # 1024 flags drawn from four keys
    data2 = rng.integers(0, 4, start_pos + 2).astype(np.int32)
    data3 = sm.fill_host(16 * 64 * 1024, 64, 0, 0)
    data3[12345] = np.inf                                            # a masked-out infinity must still poison its sum
    cube = data3.reshape(16, 64, 1024)                               # [l][r][x]
    want = np.zeros((2, 1024), np.float32)
    with np.errstate(invalid="ignore"):
        for y in range(2):
            flag = (data1.reshape(16, 64) == data2[start_pos + y]).astype(np.float32)
            part = np.zeros((16, 1024), np.float32)
            for r in range(64):                                      # r ascending inside a thread
                part = part + flag[:, r:r + 1] * cube[:, r, :]
            tot = np.zeros(1024, np.float32)
            for l in range(16):                                      # then the sixteen partials in order
                tot = tot + part[l]
            want[y] = tot
    bufs = [L.bc_alloc(C.byref(d), x.nbytes) for x in (want, data1, data2, data3)]
    for p, x in zip(bufs[1:], (data1, data2, data3)):
        L.bc_copy_h2d(C.byref(d), p, x.ctypes.data, x.nbytes)
    args = TgArgs(bufs[0], bufs[1], bufs[2], bufs[3], start_pos)
    assert L.bc_dispatch(C.byref(d), C.byref(k), 1024, 2, 1, 16, 1, 1, C.byref(args), C.sizeof(args)) == 0
    got = np.empty((2, 1024), np.float32)
    L.bc_copy_d2h(C.byref(d), got.ctypes.data, bufs[0], got.nbytes)
    nan = np.isnan(want)                                             # NaN payloads differ between x86 and the GPU
    assert nan.sum() + np.isinf(want).sum() >= 1
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))
    # more than the 16 threads the kernel is built for is refused by the launch, not run wrongly
    assert L.bc_dispatch(C.byref(d), C.byref(k), 1024, 2, 1, 32, 1, 1, C.byref(args), C.sizeof(args)) != 0
    L.bc_unload_kernel(C.byref(d), C.byref(k))
    for p in bufs:
        L.bc_free(C.byref(d), p)
