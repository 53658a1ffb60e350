"""Host-side logic of libbooth_sm100 on a machine without a GPU: which kernels a
call launches, in which order and geometry, what is copied, and what a failing
driver call leads to. The driver is tests/fake_driver/fake_cuda.c, a stand-in that
runs no kernel and computes nothing (device memory is host memory, a launch is a
line in a log): results are never looked at here, only the host's behaviour.
Failures are injected on the host, as an error code from the fake of the failing
call."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

FAKE_SRC = os.path.join(ROOT, "tests", "fake_driver", "fake_cuda.c")
CUDA_INC = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")


@pytest.fixture(scope="module")
def fake(tmp_path_factory, sm):
    if not os.path.exists(os.path.join(CUDA_INC, "cuda.h")):
        pytest.skip("cuda.h not found")
    out = tmp_path_factory.mktemp("fake_driver") / "libcuda_fake.so"
    subprocess.run(["gcc", "-std=c99", "-O1", "-shared", "-fPIC", "-I", CUDA_INC, FAKE_SRC, "-o", str(out)], check=True)
    return str(out)


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake_nccl") / "libnccl_fake.so"
    subprocess.run(["gcc", "-std=c99", "-O1", "-shared", "-fPIC", os.path.join(ROOT, "tests", "fake_driver", "fake_nccl.c"),
                    "-o", str(out)], check=True)
    return str(out)


def run(fake, tmp_path, code, **env):
    log = tmp_path / "driver.log"
    log.write_text("")
    full = dict(os.environ, BOOTH_CUDA_LIB=fake, FAKE_CUDA_LOG=str(log), PYTHONPATH=ROOT, **env)
    res = subprocess.run([sys.executable, "-c", "import booth_b200 as sm\n" + code], cwd=ROOT, env=full,
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    lines = log.read_text().splitlines()
    launches = []
    for ln in lines:
        f = ln.split()
        if f[0] == "launch":
            launches.append({"kernel": f[1], "grid": tuple(map(int, f[3:6])), "block": tuple(map(int, f[7:10])),
                             "shmem": int(f[11]), "overlap": int(f[13]), "packed": int(f[15])})
    return res, launches, lines


def test_streaming_launch_geometry(fake, tmp_path):
    res, L, _ = run(fake, tmp_path, """
d = sm.Device(0); x = d.alloc(64); y = d.alloc(64)
for lg in (30, 28, 27, 24, 10):
    d.saxpy(y, x, 2.5, 1 << lg)
d.vadd(x, y, y, 1 << 28); d.vadd(x, y, y, (1 << 24) + 5); d.saxpy(y, x, 1.0, 0)
d.sync(); d.close()
""")
    assert res.returncode == 0, res.stderr
    assert [l["kernel"] for l in L] == ["saxpy_stream"] * 5 + ["vadd_stream"] * 2   # n = 0 launches nothing
    assert all(l["block"] == (128, 1, 1) and l["overlap"] == 1 and l["shmem"] == 0 for l in L)
    # three persistent blocks per SM from 2^28 elements on; below that one 256-chunk tile per block,
    # at most 128 blocks per SM
    assert [l["grid"][0] for l in L] == [444, 444, 128 * 148, 8192, 1, 444, 8192]


def test_reduction_pricer_and_gemm_launch_sequences(fake, tmp_path):
    res, L, lines = run(fake, tmp_path, """
d = sm.Device(0); x = d.alloc(64); y = d.alloc(64); out = d.alloc(64)
d.reduce_i32(x, 1 << 30, out); d.reduce_f32(x, 1 << 30, out); d.reduce_f32(x, 1000, out)
d.asian(sm.asian_params(), 0, 1 << 26, out); d.asian(sm.asian_params(precise=1), 0, 1000, out)
d.gemm(out, x, y, 4096, 4096, 4096)
d.gemm(out, x, y, 4096, 4096, 4096, b_unchanged=True)
d.gemm(out, x, y, 8192, 8192, 8192, b_unchanged=True)        # other shape: the flag must be ignored
d.gemm(out, x, y, 100, 200, 50)
d.sync(); d.close()
""")
    assert res.returncode == 0, res.stderr
    seq = [(l["kernel"], l["grid"], l["block"][0]) for l in L]
    assert seq[:5] == [("reduce_sum_i32", (1184, 1, 1), 256), ("reduce_sum_f32", (444, 1, 1), 256),
                       ("reduce_sum_f32", (1, 1, 1), 256), ("asian_mc", (4736, 1, 1), 256),
                       ("asian_mc_precise", (4, 1, 1), 256)]
    g = seq[5:]
    # 4096^3: ONE launch ahead of the contraction (16384 blocks split A, one 16-byte chunk per thread;
    # 64 x 64 blocks split and transpose B), then the persistent contraction: 74 clusters of two CTAs (one per
    # SM pair), 384 threads, 197,632 bytes of dynamic shared memory; both with programmatic stream serialization
    assert g[:2] == [("gemm_prepass", (16384 + 4096, 1, 1), 256), ("gemm_tf32x3_persist", (148, 1, 1), 384)]
    assert L[5 + 1]["shmem"] == 197632 and L[5]["overlap"] == 1 and L[5 + 1]["overlap"] == 1
    # same B declared unchanged: no B blocks
    assert g[2:4] == [("gemm_prepass", (16384, 1, 1), 256), ("gemm_tf32x3_persist", (148, 1, 1), 384)]
    # 8192^3: B split again despite the flag (other shape)
    assert g[4:6] == [("gemm_prepass", (65536 + 16384, 1, 1), 256), ("gemm_tf32x3_persist", (148, 1, 1), 384)]
    # 100 x 200 x 50 pads to 128 x 256 x 64: the one-CTA form, one tile
    assert g[6:] == [("gemm_prepass", (8 + 4, 1, 1), 256), ("gemm_tf32x3", (1, 1, 1), 320)]
    maps = [ln for ln in lines if ln.startswith("tensormap")]
    assert maps[-4:] == ["tensormap dims 64 128 stride 256 box 32 128"] * 2 + ["tensormap dims 64 256 stride 256 box 32 256"] * 2
    # the maps are encoded once per (workspace, padded shape): the two 4096^3 calls share theirs
    assert len(maps) == 3 * 4


def test_gemm_one_tile_per_cluster_form_and_small_grids(fake, tmp_path):
    """BOOTH_SM100_GEMM_PERSIST=0 selects the one-tile-per-cluster contraction (with its
    zeroed shared tiles); the persistent form launches no more clusters than it has
    tiles when the tail is not divided."""
    res, L, _ = run(fake, tmp_path, """
import os
d = sm.Device(0); x = d.alloc(64); y = d.alloc(64); out = d.alloc(64)
d.gemm(out, x, y, 512, 768, 512)                 # 6 pair tiles, K too short to divide: 6 clusters
d.gemm(out, x, y, 512, 4096, 4096)               # 32 tiles on 74 pairs: the tail is dealt out by K chunks, all 74 clusters
os.environ["BOOTH_SM100_GEMM_PERSIST"] = "0"
d.gemm(out, x, y, 4096, 4096, 4096)
d.sync(); d.close()
""")
    assert res.returncode == 0, res.stderr
    seq = [(l["kernel"], l["grid"], l["block"][0]) for l in L]
    assert seq[1] == ("gemm_tf32x3_persist", (12, 1, 1), 384) and seq[3] == ("gemm_tf32x3_persist", (148, 1, 1), 384)
    assert seq[4:] == [("gemm_prepass", (16384 + 4096 + 34, 1, 1), 256), ("gemm_tf32x3_2cta", (580, 1, 1), 320)]


def test_gemm_outcome_reaches_every_call_that_waits(fake, tmp_path):
    """A GEMM whose bounded wait ran out leaves a code in its status word. The caller
    learns of it from whichever call waits for the stream next, not only from
    sm100_rt_sync: here the fake sets the word at the launch and the copy back
    (what Device.download, bc_copy_d2h and nv_rt_d2h do after a GEMM) reports it."""
    res, L, _ = run(fake, tmp_path, """
import numpy as np
d = sm.Device(0); x = d.alloc(1 << 20); y = d.alloc(1 << 20); out = d.alloc(1 << 20)
for waiter in ("download", "toc", "sync", "h2d"):
    d.tic()
    d.gemm(out, x, y, 256, 256, 64)
    try:
        if waiter == "download": d.download(out, 4, np.float32)
        elif waiter == "toc": d.toc()
        elif waiter == "h2d": d.h2d(x, np.zeros(4, np.float32))
        else: d.sync()
        print(waiter, "no error")
    except sm.Sm100Error as e:
        print(waiter, "reported", e.code, "code 3" in str(e))
    d.sync()                                   # reported once; the device is usable again
d.close()
""", FAKE_CUDA_GEMM_STATUS="3")
    assert res.returncode == 0, res.stderr
    for waiter in ("download", "toc", "sync", "h2d"):
        assert "%s reported -3 True" % waiter in res.stdout
    assert res.stderr.count("gave up waiting on a barrier (code 3") == 4


def test_gemm_wait_limit_arguments(fake, tmp_path):
    res, _, _ = run(fake, tmp_path, """
d = sm.Device(0)
L = sm.lib()
print("zero", L.booth_sm100_gemm_wait_limit(d.handle, 0), "huge", L.booth_sm100_gemm_wait_limit(d.handle, 60001),
      "ok", L.booth_sm100_gemm_wait_limit(d.handle, 50), "null", L.booth_sm100_gemm_wait_limit(None, 50))
d.close()
""")
    assert res.returncode == 0, res.stderr
    assert "zero -7 huge -7 ok 0 null -7" in res.stdout


def test_bad_result_addresses_are_refused_before_any_launch(fake, tmp_path):
    """A misaligned result address would fault on the device; the host refuses it."""
    res, L, _ = run(fake, tmp_path, """
d = sm.Device(0); x = d.alloc(4096); out = d.alloc(64)
def rc(f, *a):
    try: f(*a); return 0
    except sm.Sm100Error as e: return e.code
print("f32 out+4", rc(d.reduce_f32, x, 100, out + 4), "i32 out+4", rc(d.reduce_i32, x, 100, out + 4),
      "i32 out+2", rc(d.reduce_i32, x, 100, out + 2), "null in", rc(d.reduce_f32, 0, 100, out),
      "null in n=0", rc(d.reduce_f32, 0, 0, out), "in+2", rc(d.reduce_i32, x + 2, 100, out),
      "asian out+4", rc(d.asian, sm.asian_params(), 0, 1000, out + 4))
print("vadd x+2", rc(d.vadd, x + 2, x, x, 16), "vadd null out", rc(d.vadd, x, x, 0, 16), "saxpy y+1", rc(d.saxpy, x + 1, x, 2.0, 16),
      "saxpy null x n=0", rc(d.saxpy, x, 0, 2.0, 0))
print("noalloc out+4", sm.lib().booth_sm100_reduce_f32_noalloc(x, 100, out + 4, None),
      "noalloc null in", sm.lib().booth_sm100_reduce_f32_noalloc(0, 100, out, None))
d.close()
""")
    assert res.returncode == 0, res.stderr
    assert "f32 out+4 -7 i32 out+4 0 i32 out+2 -7 null in -7 null in n=0 0 in+2 -7 asian out+4 -7" in res.stdout
    assert "vadd x+2 -7 vadd null out -7 saxpy y+1 -7 saxpy null x n=0 0" in res.stdout
    assert "noalloc out+4 -7 noalloc null in -7" in res.stdout
    assert [l["kernel"] for l in L] == ["reduce_sum_i32", "reduce_sum_f32"]     # only the two valid calls launched


def test_reference_booth_run_drives_the_registered_descriptor(fake, tmp_path):
    """The reference's own command line (src/exec/booth_run.c, with src/exec/execs.c's
    registration list holding &rt_sm100) over the fake driver: target lookup,
    rt_open, rt_load, staging, one launch with the geometry of the command line,
    the copy back and the written file; and its answers for an unknown target and an
    unknown kernel. Results are not looked at here (nothing computes)."""
    exe = os.path.join(ROOT, "build", "examples", "booth-run")
    if not os.path.exists(exe):
        pytest.skip("build/examples/booth-run was not built (the reference tree was absent at build time)")
    import numpy as np
    cubin = os.path.join(ROOT, "booth_b200", "lib", "booth_sm100.cubin")
    np.arange(1024, dtype=np.float32).tofile(tmp_path / "x.bin")
    np.ones(1024, np.float32).tofile(tmp_path / "y.bin")
    log = tmp_path / "driver.log"
    env = dict(os.environ, BOOTH_CUDA_LIB=fake, FAKE_CUDA_LOG=str(log))
    for target in (["--target", "sm100"], []):              # by name, and by probing the list
        log.write_text("")
        res = subprocess.run([exe, cubin, "saxpy"] + target + ["--grid", "4", "--block", "256", "io:" + str(tmp_path / "y.bin"),
                              "in:" + str(tmp_path / "x.bin"), "f32:2.5", "u32:1024"], env=env, stdout=subprocess.PIPE,
                             stderr=subprocess.PIPE, text=True, timeout=60)
        assert res.returncode == 0, res.stderr
        assert "wrote %s (4096 bytes)" % (tmp_path / "y.bin") in res.stdout
        ops = [" ".join(ln.split()[:2]) for ln in log.read_text().splitlines()]
        assert ops == ["h2d 4096", "h2d 4096", "launch saxpy", "d2h 4096"]
        assert "launch saxpy grid 4 1 1 block 256 1 1 shmem 0" in log.read_text()
    res = subprocess.run([exe, cubin, "saxpy", "--target", "nvptx"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    assert res.returncode == 2 and "no target named 'nvptx'. Known: sm100" in res.stderr
    res = subprocess.run([exe, cubin, "no_such_kernel", "--target", "sm100"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    assert res.returncode == 1 and "no kernel of that name in the cubin" in res.stderr
    # too many argument bytes for the kernel's parameter block: refused by the descriptor's run
    res = subprocess.run([exe, cubin, "saxpy", "--target", "sm100", "io:" + str(tmp_path / "y.bin"), "in:" + str(tmp_path / "x.bin"),
                          "f32:2.5", "u32:1024", "u32:7", "u32:8"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    assert res.returncode == 1 and "launch:" in res.stderr


def test_bc_dispatch_cuts_oversized_argument_blocks_and_is_synchronous(fake, tmp_path):
    res, L, lines = run(fake, tmp_path, """
import ctypes as C
lib = sm.lib(); d = sm.BcDevice(); k = sm.BcKernel()
assert lib.bc_device_init(C.byref(d)) == 0
assert lib.bc_load_kernel(C.byref(d), sm.CUBIN_PATH.encode(), b"saxpy", C.byref(k)) == 0
print("kernarg", k.kernarg_size)
args = (C.c_char * 42)()                                       # 24 bytes of parameters + 18 hidden ones
print("rc", lib.bc_dispatch(C.byref(d), C.byref(k), 0, 0, 0, 0, 0, 0, args, 42))
print("rc", lib.bc_dispatch(C.byref(d), C.byref(k), 7, 3, 2, 33, 3, 1, args, 24))
lib.bc_device_shutdown(C.byref(d))
""")
    assert res.returncode == 0, res.stderr
    assert "kernarg 24" in res.stdout and res.stdout.count("rc 0") == 2
    assert L[0]["grid"] == (1, 1, 1) and L[0]["block"] == (1, 1, 1)          # zero dimensions become one
    assert L[0]["packed"] == 24 and L[1]["packed"] == 24                      # cut to the kernel's own block
    assert L[1]["grid"] == (7, 3, 2) and L[1]["block"] == (33, 3, 1) and L[1]["overlap"] == 0


def test_failed_launch_reports_the_dispatch_and_the_labelled_buffers(fake, tmp_path):
    res, L, _ = run(fake, tmp_path, """
import ctypes as C
lib = sm.lib(); d = sm.BcDevice(); k = sm.BcKernel()
lib.bc_alloc.restype = C.c_void_p
lib.bc_trak.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_char_p, C.c_int]
assert lib.bc_device_init(C.byref(d)) == 0
assert lib.bc_load_kernel(C.byref(d), sm.CUBIN_PATH.encode(), b"saxpy", C.byref(k)) == 0
p = lib.bc_alloc(C.byref(d), 4096)
lib.bc_trak(C.byref(d), p, 4096, b"y vector", 0)
args = (C.c_char * 24)()
print("first", lib.bc_dispatch(C.byref(d), C.byref(k), 4, 1, 1, 256, 1, 1, args, 24))
print("second", lib.bc_dispatch(C.byref(d), C.byref(k), 4, 1, 1, 256, 1, 1, args, 24))
print("third", lib.bc_dispatch(C.byref(d), C.byref(k), 4, 1, 1, 256, 1, 1, args, 24))
""", FAKE_CUDA_FAIL="cuLaunchKernel:2")
    assert res.returncode == 0, res.stderr
    assert "first 0" in res.stdout and "second -3" in res.stdout and "third 0" in res.stdout   # BC_RT_ERR_HSA, then usable again
    assert len(L) == 2
    assert "kernel 'saxpy'" in res.stderr and "grid 4x1x1 block 256x1x1" in res.stderr
    assert "y vector" in res.stderr and "too many resources" in res.stderr


def test_allocation_and_wrong_device_failures(fake, tmp_path):
    res, _, _ = run(fake, tmp_path, """
import ctypes as C
lib = sm.lib(); lib.bc_alloc.restype = C.c_void_p
d = sm.BcDevice(); print("init", lib.bc_device_init(C.byref(d)))
print("alloc", lib.bc_alloc(C.byref(d), 1 << 20))
""", FAKE_CUDA_FAIL="cuMemAlloc:2")                    # the first allocation is the library's own scratch
    assert "init 0" in res.stdout and "alloc None" in res.stdout
    assert "out of memory" in res.stderr
    res, _, _ = run(fake, tmp_path, """
import ctypes as C
h = C.c_void_p(); print("rc", sm.lib().sm100_rt_init(C.byref(h), 0)); print("rc3", sm.lib().sm100_rt_init(C.byref(h), 3))
""", FAKE_CUDA_SM_MAJOR="9")
    assert "rc -4" in res.stdout and "rc3 -4" in res.stdout      # not an sm_100 part; no such ordinal
    assert "sm_100a code only" in res.stderr


def test_offload_abi_copies_in_at_set_and_back_after_the_launch(fake, tmp_path):
    res, L, lines = run(fake, tmp_path, """
import ctypes as C, numpy as np
lib = sm.lib()
lib.lfortran_gpu_init.restype = C.c_void_p
lib.lfortran_gpu_load_kernel.restype = C.c_void_p
lib.lfortran_gpu_load_kernel.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p]
lib.lfortran_gpu_set_buffer_arg.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t]
lib.lfortran_gpu_set_scalar_arg.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t]
lib.lfortran_gpu_launch.argtypes = [C.c_void_p] * 4
lib.lfortran_gpu_shutdown.argtypes = [C.c_void_p]
ctx = lib.lfortran_gpu_init()
k = lib.lfortran_gpu_load_kernel(ctx, None, b"saxpy")
x = np.ones(1000, np.float32); y = np.ones(500, np.float32)
a, n = C.c_float(2.0), C.c_int(500)
lib.lfortran_gpu_set_buffer_arg(k, 0, y.ctypes.data, y.nbytes)
lib.lfortran_gpu_set_buffer_arg(k, 1, x.ctypes.data, x.nbytes)
lib.lfortran_gpu_set_scalar_arg(k, 2, C.byref(a), 4); lib.lfortran_gpu_set_scalar_arg(k, 3, C.byref(n), 4)
lib.lfortran_gpu_launch(ctx, k, (C.c_int * 3)(2, 1, 1), (C.c_int * 3)(256, 1, 1))
lib.lfortran_gpu_shutdown(ctx)
print("done")
""")
    assert res.returncode == 0 and "done" in res.stdout, res.stderr
    ops = [ln.split()[0] + " " + ln.split()[1] for ln in lines if not ln.startswith("tensormap")]
    assert ops == ["h2d 2000", "h2d 4000", "launch saxpy", "d2h 2000", "d2h 4000"]
    assert L[0]["grid"] == (2, 1, 1) and L[0]["block"] == (256, 1, 1)


def test_reference_launcher_api_over_the_fake(fake, tmp_path):
    res, L, _ = run(fake, tmp_path, """
import ctypes as C
lib = sm.lib(); lib.nv_rt_alloc.restype = C.c_uint64
d = (C.c_char * 320)(); k = (C.c_char * 144)()
print("init", lib.nv_rt_init(d)); print("load", lib.nv_rt_load(d, sm.CUBIN_PATH.encode(), b"vector_add", k))
print("missing", lib.nv_rt_load(d, sm.CUBIN_PATH.encode(), b"no_such_kernel", k))
print("load", lib.nv_rt_load(d, sm.CUBIN_PATH.encode(), b"vector_add", k))
args = (C.c_void_p * 5)()
print("launch", lib.nv_rt_launch(d, k, 3, 2, 1, 64, 1, 1, 0, args), lib.nv_rt_sync(d))
lib.nv_rt_unload(d, k); lib.nv_rt_shut(d); print("after", lib.nv_rt_sync(d))
""")
    assert res.returncode == 0, res.stderr
    assert "init 0" in res.stdout and "missing -6" in res.stdout and "launch 0 0" in res.stdout and "after -3" in res.stdout
    assert [(l["kernel"], l["grid"], l["block"]) for l in L] == [("vector_add", (3, 2, 1), (64, 1, 1))]


def test_host_vector_call_pipelines_chunks_and_leaves_memory_alone(fake, tmp_path):
    res, L, lines = run(fake, tmp_path, """
import numpy as np
d = sm.Device(0)
n = (20 << 20) + 3                                   # one 16 Mi-element chunk and a ragged second one
x = np.arange(n, dtype=np.float32); y = np.ones(n, np.float32)
d.saxpy_host(y.ctypes.data, x.ctypes.data, 2.5, n)
print("y unchanged by the fake:", bool((y == 1).all()))
d.vadd_host(x.ctypes.data, y.ctypes.data, y.ctypes.data, 1000)
d.close()
""")
    assert res.returncode == 0, res.stderr
    assert "y unchanged by the fake: True" in res.stdout          # nothing computes on the CPU
    ops = [" ".join(ln.split()[:2]) for ln in lines if not ln.startswith("tensormap")]
    big, rest = 64 << 20, ((4 << 20) + 3) * 4
    assert ops == ["h2d %d" % big, "h2d %d" % big, "launch saxpy_stream", "d2h %d" % big,
                   "h2d %d" % rest, "h2d %d" % rest, "launch saxpy_stream", "d2h %d" % rest,
                   "h2d 4000", "h2d 4000", "launch vadd_stream", "d2h 4000"]
    assert [l["grid"][0] for l in L] == [8192, 2048, 1]


def test_device_ordinal_comes_from_the_environment(fake, tmp_path):
    res, _, _ = run(fake, tmp_path, """
import ctypes as C
lib = sm.lib(); lib.sm100_rt_ordinal.argtypes = [C.c_void_p]
h = C.c_void_p(); print("rc", lib.sm100_rt_init(C.byref(h), -1), "ordinal", lib.sm100_rt_ordinal(h))
print("count", lib.sm100_rt_device_count())
d = sm.BcDevice(); print("bc", lib.bc_device_init(C.byref(d)))
h2 = C.c_void_p(); print("rc7", lib.sm100_rt_init(C.byref(h2), 7))
""", FAKE_CUDA_DEVICES="4", BOOTH_DEVICE="2")
    assert "rc 0 ordinal 2" in res.stdout and "count 4" in res.stdout and "bc 0" in res.stdout and "rc7 -4" in res.stdout
    assert res.stderr.count("device 2:") == 2


def test_collective_host_logic_one_process_per_gpu(fake, fake_nccl, tmp_path):
    res, _, lines = run(fake, tmp_path, """
import ctypes as C
d = sm.Device(0); buf = d.alloc(64)
uid = sm.Comm.unique_id()
c = sm.Comm(d, 8, 3, uid)
c.allreduce_sum(buf, 1, 0)                    # SM100_I32
c.allreduce_sum(buf, 4, 2)                    # SM100_F64: the pricer's four sums
c.close(); c.close()
lib = sm.lib(); h = C.c_void_p()
print("bad rank", lib.sm100_comm_init_rank(C.byref(h), d.handle, 2, 2, uid))
d.close()
""", BOOTH_NCCL_LIB=fake_nccl)
    assert res.returncode == 0, res.stderr
    nccl = [ln for ln in lines if ln.startswith("nccl")]
    assert nccl == ["nccl init_rank 3 of 8", "nccl allreduce rank 3 count 1 dtype 2 op 0 inplace 1",
                    "nccl allreduce rank 3 count 4 dtype 8 op 0 inplace 1", "nccl destroy rank 3"]
    assert "bad rank -7" in res.stdout


def test_collective_host_logic_one_process_many_gpus_and_a_failing_peer(fake, fake_nccl, tmp_path):
    code = """
import ctypes as C
lib = sm.lib()
devs = (C.c_void_p * 4)()
for i in range(4):
    h = C.c_void_p(); assert lib.sm100_rt_init(C.byref(h), i) == 0; devs[i] = h
lib.sm100_rt_alloc.restype = C.c_uint64; lib.sm100_rt_alloc.argtypes = [C.c_void_p, C.c_size_t]
lib.sm100_comm_allreduce_sum_dev.argtypes = [C.c_void_p, C.c_int, C.c_uint64, C.c_size_t, C.c_int]
lib.sm100_comm_allreduce_sum.argtypes = [C.c_void_p, C.c_uint64, C.c_size_t, C.c_int]
bufs = [lib.sm100_rt_alloc(devs[i], 64) for i in range(4)]
comm = C.c_void_p(); print("init_all", lib.sm100_comm_init_all(C.byref(comm), devs, 4))
print("wrong form", lib.sm100_comm_allreduce_sum(comm, bufs[0], 1, 1))
for step in range(3):
    print("begin", lib.sm100_comm_group_begin())
    rcs = [lib.sm100_comm_allreduce_sum_dev(comm, i, bufs[i], 1, 1) for i in range(4)]
    print("step", step, rcs, "end", lib.sm100_comm_group_end())
print("bad index", lib.sm100_comm_allreduce_sum_dev(comm, 4, bufs[0], 1, 1))
lib.sm100_comm_destroy(comm)
"""
    res, _, lines = run(fake, tmp_path, code, BOOTH_NCCL_LIB=fake_nccl, FAKE_CUDA_DEVICES="4", FAKE_NCCL_FAIL="ncclAllReduce:6")
    assert res.returncode == 0, res.stderr
    assert "init_all 0" in res.stdout and "wrong form -7" in res.stdout and "bad index -7" in res.stdout
    # the sixth all-reduce (step 1, device 1) fails: reported as the NCCL status, with the library's text,
    # and the process carries on; nothing hangs, nothing is retried behind the caller's back
    assert "step 0 [0, 0, 0, 0] end 0" in res.stdout and "step 1 [0, -8, 0, 0] end 0" in res.stdout
    assert "step 2 [0, 0, 0, 0] end 0" in res.stdout
    assert "ncclAllReduce: fake: unhandled system error" in res.stderr
    nccl = [ln for ln in lines if ln.startswith("nccl")]
    assert nccl[0] == "nccl init_all 4 devices, first ordinal 0"
    assert nccl[1:7] == ["nccl group_start"] + ["nccl allreduce rank %d count 1 dtype 7 op 0 inplace 1" % i for i in range(4)] + ["nccl group_end"]
    assert nccl[-4:] == ["nccl destroy rank %d" % i for i in range(4)]


def test_missing_collective_library_is_an_error(fake, tmp_path):
    res, _, _ = run(fake, tmp_path, """
try:
    sm.Comm.unique_id(); print("got an id")
except sm.Sm100Error as e:
    print("error", e.status if hasattr(e, "status") else e)
""", BOOTH_NCCL_LIB="/nonexistent/libnccl.so.2")
    assert "got an id" not in res.stdout and "error" in res.stdout


def test_bench_line_keeps_its_contract_over_the_fake(fake, fake_nccl, tmp_path):
    """bench.py end to end at toy sizes over the fake driver: the figures mean nothing
    (the fake's clock says 1 ms per timed region), the shape of the one JSON line on
    stdout is what is checked."""
    import json
    env = dict(os.environ, BOOTH_CUDA_LIB=fake, BOOTH_NCCL_LIB=fake_nccl, PYTHONPATH=ROOT)
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--log2n", "16", "--log2paths", "10", "--gemm-sizes", "256",
                          "--steps", "4", "--warmup", "3", "--cpu-seconds", "0.05", "--no-parity"], cwd=ROOT, env=env,
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    out = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(out) == 1, out                                   # exactly one line on stdout
    j = json.loads(out[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "clocks", "roofline", "cpu_baseline"):
        assert key in j, key
    assert j["n_gpus"] == 1 and j["steps"] == 4 and j["warmup"] == 3 and j["gpu_launches"] == 4
    assert j["vs_baseline"] is None and j["dtype"] == "f32" and j["scaling"] == "weak" and j["higher_is_better"] is True
    assert set(j["roofline"]) >= {"bound", "achieved", "peak", "unit", "frac", "traffic"}
    assert set(j["e2e"]) >= {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"}
    assert j["e2e"]["h2d_bytes_per_step"] == 2 * 4 * (1 << 16) and j["e2e"]["d2h_bytes_per_step"] == 4 * (1 << 16)
    assert set(j["cpu_baseline"]) >= {"value", "unit", "cores", "kind", "sample"}
    assert "workload" in j["config"] and "model" not in j["config"]
    names = [w["name"] for w in j["workloads"]]
    assert any(n.startswith("gemm") for n in names) and any(n.startswith("asian") for n in names)
    assert j["parity"] is None                                   # switched off above: the fake computes nothing
    assert j["e2e"]["roofline"]["bound"] == "pcie" and set(j["e2e"]["roofline"]["link_gbs"]) == {"h2d", "d2h", "h2d_duplex", "d2h_duplex"}
    for w in j["workloads"]:                                     # every measured workload carries its own e2e and roofline
        if "value" in w:
            assert "roofline" in w and set(w["e2e"]) >= {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"}, w["name"]
    mc = [w for w in j["workloads"] if w["name"].startswith("asian_mc_fast")][0]
    assert mc["roofline"]["bound"] == "mufu issue" and mc["second_bound"]["bound"] == "warp instruction issue"


def test_bench_parity_block_has_teeth(fake, fake_nccl, tmp_path):
    """bench.py checks every workload's result against the CPU checker outside the
    timed regions and exits non-zero on a miss. Over the fake driver nothing is
    computed, so every check must miss: the line still comes out, says which, and
    the exit status is 3."""
    import json
    env = dict(os.environ, BOOTH_CUDA_LIB=fake, BOOTH_NCCL_LIB=fake_nccl, PYTHONPATH=ROOT)
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--log2n", "16", "--log2paths", "10", "--gemm-sizes", "256",
                          "--steps", "2", "--warmup", "3", "--no-cpu-baseline", "--no-e2e"], cwd=ROOT, env=env,
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600)
    assert res.returncode == 3, res.stderr[-2000:]
    j = json.loads([ln for ln in res.stdout.splitlines() if ln.strip()][0])
    par = j["parity"]
    assert par["status"].startswith("MISS") and par["checker"] in ("reference", "port")
    for key in ("saxpy_mismatches", "int32", "fp32_rel", "mc_rel_fast", "mc_rel_precise", "gemm_rel_fro_256"):
        assert key in par and key in par["status"], key
    assert par["saxpy_mismatches"] > 0 and "PARITY MISS" in res.stderr


def test_reference_arm_line_needs_no_gpu(tmp_path):
    """bench.py --impl reference times the reference compiler's x86-64 objects (or
    their C restatement) on the host cores: same metric and config as the GPU arm,
    one JSON line, no driver touched."""
    import json
    env = dict(os.environ, BOOTH_CUDA_LIB="/nonexistent/libcuda.so.1", PYTHONPATH=ROOT)
    res = subprocess.run([sys.executable, "-X", "importtime", os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "1", "--log2n", "24"],
                         cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    out = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(out) == 1
    j = json.loads(out[0])
    assert j["impl"] == "reference" and j["metric"] == "saxpy_hbm_gbs" and j["unit"] == "GB/s" and j["n_gpus"] == 1
    assert j["higher_is_better"] is True and j["value"] > 0
    assert j["cpu_baseline"]["kind"] in ("reference", "port") and j["cpu_baseline"]["cores"] >= 1
    assert j["cpu_baseline"]["value"] == j["value"] == j["e2e"]["value"]
    assert j["e2e"]["h2d_bytes_per_step"] == 0 and j["e2e"]["d2h_bytes_per_step"] == 0
    assert "N=2^24" in j["config"]["workload"]                   # the default is the GPU arm's 2^30
    # nothing of the product is loaded in this arm: no import of the package, no libbooth_sm100
    assert "booth_b200" not in res.stderr and "oracle" in res.stderr


def test_two_rank_bench_path_over_the_fakes(fake, fake_nccl, tmp_path):
    """The launch the driver uses for N > 1 (torchrun, one rank per GPU), on the CPU:
    two ranks on two fake devices, the NCCL id travelling through the gloo group,
    rank 0 alone printing the line, whole-job figures."""
    import json
    env = dict(os.environ, BOOTH_CUDA_LIB=fake, BOOTH_NCCL_LIB=fake_nccl, FAKE_CUDA_DEVICES="2", PYTHONPATH=ROOT,
               FAKE_CUDA_LOG=str(tmp_path / "driver.log"))
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29541", os.path.join(ROOT, "bench.py"),
                          "--gpus", "2", "--log2n", "16", "--log2paths", "10", "--gemm-sizes", "256", "--steps", "3",
                          "--warmup", "3", "--no-cpu-baseline", "--no-parity"], cwd=ROOT, env=env, stdout=subprocess.PIPE,
                         stderr=subprocess.PIPE, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-3000:]
    out = [ln for ln in res.stdout.splitlines() if ln.strip().startswith("{")]
    assert len(out) == 1
    j = json.loads(out[0])
    assert j["n_gpus"] == 2 and j["scaling"] == "weak" and j["gpu_launches"] == 3
    assert j["e2e"]["h2d_bytes_per_step"] == 2 * 2 * 4 * (1 << 16)            # both ranks' vectors
    log = (tmp_path / "driver.log").read_text()
    assert "nccl init_rank 0 of 2" in log and "nccl init_rank 1 of 2" in log
    assert log.count("nccl allreduce") >= 2 * 2                                # sums and prices, on both ranks


def test_nothing_is_computed_on_the_host(fake, tmp_path):
    """The reference's own example programs, relinked against the library, check
    their results themselves. Over the fake driver, where no kernel runs, they must
    report mismatches: the library has no path that computes on the CPU."""
    ex = os.path.join(ROOT, "build", "examples")
    if not os.path.exists(os.path.join(ex, "launch_saxpy")):
        pytest.skip("build/examples was not built (the reference tree was absent at build time)")
    env = dict(os.environ, BOOTH_CUDA_LIB=fake)
    res = subprocess.run([os.path.join(ex, "launch_saxpy"), os.path.join(ROOT, "booth_b200", "lib", "booth_sm100.cubin")],
                         env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=60)
    assert "FAIL: 1023/1024 mismatches" in res.stdout                 # element 0 is x[0] = 0: y unchanged is right there
    res = subprocess.run([os.path.join(ex, "cpu_launch_vadd")], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                         text=True, timeout=60)
    assert "MISMATCH" in res.stdout and "OK" not in res.stdout.replace("MISMATCH", "")
    # the reference's differential harness and its BIR-kernel check fail the same way
    res = subprocess.run([os.path.join(ex, "diff_vadd")], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=60)
    assert res.returncode != 0 and "FAIL" in res.stdout
    res = subprocess.run([os.path.join(ex, "run_vadd")], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=60)
    assert res.returncode != 0 and "MISMATCH" in res.stdout
