"""GPU: the eight-function offload ABI of LFortran-compiled programs
(src/runtime/lf_gpu.h:21-35) served by the sm_100a runtime, driven by the C99
program examples/lf_offload.c, and its fatal-by-contract failure paths."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu
EXAMPLES = os.path.join(ROOT, "build", "examples")


def _run(cmd, env=None):
    return subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=180,
                          env=dict(os.environ, **(env or {})))


@pytest.mark.parametrize("source", ["builtin", "cubin", "env"])
def test_offload_program_on_the_library_implementation(sm, source):
    exe = os.path.join(EXAMPLES, "lf_offload")
    if not os.path.exists(exe):
        pytest.skip("build/examples/lf_offload was not built")
    cmd, env = [exe], {}
    if source == "cubin":
        cmd += [sm.CUBIN_PATH, "65537"]
    elif source == "env":                       # second place the kernel file is looked for
        env["BOOTH_CUBIN"] = sm.CUBIN_PATH
    res = _run(cmd, env)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "saxpy      n=" in res.stdout and ": 0 mismatches" in res.stdout
    assert "lf_offload: ok" in res.stdout


def test_reference_offload_layer_relinked_over_bc_runtime(sm):
    # src/runtime/lf_gpu_hsa.c, compiled unchanged into the program, packs 8-byte
    # slots plus 18 hidden bytes (lf_gpu_hsa.c:222-255) and dispatches through the
    # library's bc_*: the parameter block is cut to the kernel's own size.
    exe = os.path.join(EXAMPLES, "lf_offload_slots")
    if not os.path.exists(exe):
        pytest.skip("build/examples/lf_offload_slots was not built (the reference tree was absent at build time)")
    res = _run([exe, sm.CUBIN_PATH, "100001"])
    assert res.returncode == 0, res.stdout + res.stderr
    assert "vector_add n=100001: 0 mismatches" in res.stdout and "lf_offload: ok" in res.stdout


def test_offload_abi_from_python_matches_the_workload_entry_point(sm, oracle_lib):
    L = sm.lib()
    L.lfortran_gpu_init.restype = C.c_void_p
    L.lfortran_gpu_load_kernel.restype = C.c_void_p
    L.lfortran_gpu_load_kernel.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p]
    L.lfortran_gpu_set_buffer_arg.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t]
    L.lfortran_gpu_set_scalar_arg.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t]
    L.lfortran_gpu_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    for f in ("lfortran_gpu_release_kernel", "lfortran_gpu_shutdown", "lfortran_gpu_sync"):
        getattr(L, f).argtypes = [C.c_void_p]
    n = (1 << 20) + 5
    x = sm.fill_host(n, 0xB0070009, 0, 0)
    y = sm.fill_host(n, 0xB0070009, 1, 0)
    want = oracle_lib.saxpy(y, x, 2.5)
    ctx = L.lfortran_gpu_init()
    k = L.lfortran_gpu_load_kernel(ctx, None, b"saxpy")
    a, nn = C.c_float(2.5), C.c_int(n)
    grid, block = (C.c_int * 3)(148 * 5, 1, 1), (C.c_int * 3)(128, 1, 1)
    L.lfortran_gpu_set_buffer_arg(k, 0, y.ctypes.data, n * 4)
    L.lfortran_gpu_set_buffer_arg(k, 1, x.ctypes.data, n * 4)
    L.lfortran_gpu_set_buffer_arg(k, 40, x.ctypes.data, n * 4)       # out of range: ignored
    L.lfortran_gpu_set_scalar_arg(k, 2, C.byref(a), 4)
    L.lfortran_gpu_set_scalar_arg(k, 3, C.byref(nn), 4)
    L.lfortran_gpu_launch(ctx, k, grid, block)
    L.lfortran_gpu_sync(ctx)
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
    L.lfortran_gpu_release_kernel(k)
    L.lfortran_gpu_shutdown(ctx)


@pytest.mark.parametrize("case,message", [
    ("gap", "argument gap failed (rc=1)"),
    ("dims", "launch dims non-positive failed"),
    ("wide", "scalar arg too wide failed (rc=17)"),
    ("name", "could not load 'no_such_kernel' from the built-in image"),
])
def test_offload_failures_are_fatal_and_named(sm, case, message):
    # No error channel in the ABI: each of these ends the process with status 1 and
    # one line saying what failed (src/runtime/lf_gpu.c:55-59,199-201,218-229).
    code = """
import ctypes as C, booth_b200 as b
L = b.lib()
L.lfortran_gpu_init.restype = C.c_void_p
L.lfortran_gpu_load_kernel.restype = C.c_void_p
L.lfortran_gpu_load_kernel.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p]
L.lfortran_gpu_set_scalar_arg.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t]
L.lfortran_gpu_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
ctx = L.lfortran_gpu_init()
case = %r
k = L.lfortran_gpu_load_kernel(ctx, None, b"no_such_kernel" if case == "name" else b"saxpy")
v = (C.c_char * 32)()
one, zero = (C.c_int * 3)(1, 1, 1), (C.c_int * 3)(1, 0, 1)
if case == "wide":
    L.lfortran_gpu_set_scalar_arg(k, 0, v, 17)
if case == "gap":
    L.lfortran_gpu_set_scalar_arg(k, 0, v, 8); L.lfortran_gpu_set_scalar_arg(k, 2, v, 4)
    L.lfortran_gpu_launch(ctx, k, one, one)
if case == "dims":
    L.lfortran_gpu_launch(ctx, k, zero, one)
print("survived")
""" % case
    res = _run([os.sys.executable, "-c", code], {"PYTHONPATH": ROOT})
    assert res.returncode == 1, res.stdout + res.stderr
    assert "survived" not in res.stdout
    assert message in res.stderr
