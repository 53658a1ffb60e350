"""The reference's CUDA launcher API (nv_rt_*, src/nvidia/nv_rt.h:102-134) served by
libbooth_sm100: layout and export checks on the CPU; on the GPU the reference's own
host programs relinked, and the PTX its compiler emits run through the API and
compared with its x86-64 build of the same kernels."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

from conftest import ROOT, REFERENCE

EXAMPLES = os.path.join(ROOT, "build", "examples")
PTX = os.path.join(ROOT, "oracle", "_ref", "ptx")
REF_HDR = os.path.join(REFERENCE, "src", "nvidia", "nv_rt.h")
NAMES = ["nv_rt_init", "nv_rt_shut", "nv_rt_load", "nv_rt_unload", "nv_rt_alloc", "nv_rt_free",
         "nv_rt_h2d", "nv_rt_d2h", "nv_rt_launch", "nv_rt_sync", "nv_rt_mmap", "nv_rt_mfre"]


class NvKern(C.Structure):
    _fields_ = [("mod", C.c_void_p), ("func", C.c_void_p), ("name", C.c_char * 128)]


class NvDev(C.Structure):
    _fields_ = [("lib", C.c_void_p), ("ctx", C.c_void_p), ("dev", C.c_int), ("dev_name", C.c_char * 128),
                ("sm_major", C.c_int), ("sm_minor", C.c_int), ("reserved", C.c_void_p * 20)]


def _bind(L):
    L.nv_rt_alloc.restype = C.c_uint64
    L.nv_rt_alloc.argtypes = [C.c_void_p, C.c_size_t]
    L.nv_rt_free.argtypes = [C.c_void_p, C.c_uint64]
    L.nv_rt_h2d.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_size_t]
    L.nv_rt_d2h.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_size_t]
    L.nv_rt_load.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p, C.c_void_p]
    L.nv_rt_launch.argtypes = [C.c_void_p, C.c_void_p] + [C.c_uint32] * 7 + [C.c_void_p]
    L.nv_rt_mmap.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_uint64), C.c_size_t]
    L.nv_rt_mfre.argtypes = [C.c_void_p, C.c_void_p]
    return L


def _args(*vals):
    arr = (C.c_void_p * len(vals))(*[C.cast(C.pointer(v), C.c_void_p) for v in vals])
    arr._keep = vals
    return arr


def test_header_and_exports(sm):
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "nv_rt.h")).read(), flags=re.S)
    assert sorted(set(re.findall(r"\b(nv_rt_[a-z0-9_]+)\s*\(", text))) == sorted(NAMES)
    handle = C.CDLL(sm.LIB_PATH)
    for name in NAMES:
        assert hasattr(handle, name), name
    assert C.sizeof(NvDev) == 320 and C.sizeof(NvKern) == 144      # src/nvidia/nv_rt.h:42-91


def test_layout_equals_the_reference_header(tmp_path):
    if not os.path.exists(REF_HDR):
        pytest.skip("reference tree absent")
    probe = r"""
#include <stdio.h>
#include <stddef.h>
#include HDR
int main(void) {
    printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu", sizeof(nv_dev_t), sizeof(nv_kern_t), offsetof(nv_dev_t, lib),
           offsetof(nv_dev_t, ctx), offsetof(nv_dev_t, dev), offsetof(nv_dev_t, dev_name), offsetof(nv_dev_t, sm_major),
           offsetof(nv_dev_t, sm_minor), offsetof(nv_kern_t, mod), offsetof(nv_kern_t, func), offsetof(nv_kern_t, name));
    printf(" %d %d %d %d %d %d %d %zu\n", NV_RT_OK, NV_RT_ERR_DL, NV_RT_ERR_SYM, NV_RT_ERR_CUDA, NV_RT_ERR_NO_GPU,
           NV_RT_ERR_IO, NV_RT_ERR_KERN, sizeof(CUdevptr));
    return 0;
}
"""
    src = tmp_path / "probe.c"
    src.write_text(probe)
    outs = []
    for tag, hdr in (("own", os.path.join(ROOT, "include", "nv_rt.h")), ("ref", REF_HDR)):
        exe = tmp_path / ("probe_" + tag)
        subprocess.run(["gcc", "-std=c99", '-DHDR="%s"' % hdr, str(src), "-o", str(exe)], check=True)
        outs.append(subprocess.run([str(exe)], stdout=subprocess.PIPE, text=True, check=True).stdout)
    assert outs[0] == outs[1], outs
    assert outs[0].split()[:2] == ["320", "144"]


def test_missing_driver_is_reported_not_emulated(sm):
    code = ("import ctypes as C, booth_b200 as b\n"
            "L=b.lib(); d=(C.c_char*320)(); print('rc', L.nv_rt_init(d)); print('sync', L.nv_rt_sync(d))\n")
    res = subprocess.run([os.sys.executable, "-c", code], cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                         text=True, timeout=120, env=dict(os.environ, BOOTH_CUDA_LIB="/nonexistent/libcuda.so.1"))
    assert res.returncode == 0, res.stderr
    assert "rc -1" in res.stdout and "sync -3" in res.stdout          # NV_RT_ERR_DL, then "not open"
    assert "nv_rt: device init failed (-1)" in res.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("prog,ptx,expect", [
    ("gpu_vadd", "vadd.ptx", "OK"), ("gpu_reduce", "reduce.ptx", "OK: an OCaml loop"),
    ("gpu_scale", "scale.ptx", "OK: float immediates survived")])
def test_reference_gpu_programs_relinked(sm, prog, ptx, expect):
    """tests/build/gpu_*.c of the reference, unchanged, on the library's nv_rt_*,
    loading the PTX the reference compiler emitted for tests/ocaml/*.bir."""
    exe, art = os.path.join(EXAMPLES, prog), os.path.join(PTX, ptx)
    if not (os.path.exists(exe) and os.path.exists(art)):
        pytest.skip("%s or %s was not built (the reference tree was absent at build time)" % (prog, ptx))
    res = subprocess.run([exe, art], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert expect in res.stdout and "FAILED" not in res.stdout
    assert "nv_rt: loaded kernel" in res.stderr


@pytest.mark.gpu
def test_reference_offload_layer_over_nv_rt(sm):
    # src/runtime/lf_gpu.c unchanged, compiled into examples/lf_offload.c, on nv_rt_*.
    exe = os.path.join(EXAMPLES, "lf_offload_nv")
    if not os.path.exists(exe):
        pytest.skip("build/examples/lf_offload_nv was not built (the reference tree was absent at build time)")
    res = subprocess.run([exe, sm.CUBIN_PATH, "70001"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                         timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "saxpy x2   n=70001: 0 mismatches" in res.stdout and "lf_offload: ok" in res.stdout


@pytest.mark.gpu
def test_timing_program_under_both_launch_shapes(sm):
    # examples/nv_rt_time.c: the by-name saxpy under a one-thread-per-element launch
    # (most blocks retire at once) and under a fixed grid; the data must come back intact.
    exe = os.path.join(EXAMPLES, "nv_rt_time")
    if not os.path.exists(exe):
        pytest.skip("build/examples/nv_rt_time was not built")
    for name in ("saxpy", "vector_add", "vadd_stream"):
        res = subprocess.run([exe, sm.CUBIN_PATH, "22", "5", name], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                             text=True, timeout=120)
        assert res.returncode == 0, res.stdout + res.stderr
        assert "one thread per element" in res.stdout and "nv_rt_time: ok" in res.stdout


@pytest.fixture()
def nv(sm):
    L = _bind(sm.lib())
    d = NvDev()
    assert L.nv_rt_init(C.byref(d)) == 0
    assert d.lib and d.sm_major == 10 and b"B200" in d.dev_name
    yield L, d
    L.nv_rt_shut(C.byref(d))
    assert not d.lib
    L.nv_rt_shut(C.byref(d))                                          # second shut is a no-op


@pytest.mark.gpu
def test_reference_compilers_saxpy_ptx_equals_its_x86_64_build(sm, nv, oracle_lib, dev):
    """One kernel source (tests/canonical.cu:168-173), three builds: the reference's
    PTX run here through nv_rt_*, its x86-64 object, and this library's own kernel.
    All three must agree bit for bit."""
    art = os.path.join(PTX, "saxpy.ptx")
    if not os.path.exists(art):
        pytest.skip("oracle/_ref/ptx/saxpy.ptx was not built (the reference tree was absent at build time)")
    L, d = nv
    n = (1 << 20) + 3
    x = sm.fill_host(n, 0xB007000A, 0, 0)
    y = sm.fill_host(n, 0xB007000A, 1, 0)
    want = oracle_lib.saxpy(y, x, 2.5)
    k = NvKern()
    assert L.nv_rt_load(C.byref(d), art.encode(), b"saxpy", C.byref(k)) == 0
    assert k.func and k.name == b"saxpy"
    dx, dy = L.nv_rt_alloc(C.byref(d), n * 4), L.nv_rt_alloc(C.byref(d), n * 4)
    assert dx and dy
    assert L.nv_rt_h2d(C.byref(d), dx, x.ctypes.data, n * 4) == 0
    assert L.nv_rt_h2d(C.byref(d), dy, y.ctypes.data, n * 4) == 0
    args = _args(C.c_uint64(dy), C.c_uint64(dx), C.c_float(2.5), C.c_int(n))
    assert L.nv_rt_launch(C.byref(d), C.byref(k), (n + 255) // 256, 1, 1, 256, 1, 1, 0, args) == 0
    assert L.nv_rt_sync(C.byref(d)) == 0
    got = np.empty(n, np.float32)
    assert L.nv_rt_d2h(C.byref(d), got.ctypes.data, dy, n * 4) == 0
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    ox, oy = dev.upload(x), dev.upload(y)                              # the library's own kernel
    dev.saxpy(oy, ox, 2.5, n)
    assert np.array_equal(dev.download(oy, n, np.float32).view(np.uint32), got.view(np.uint32))
    # mapped host memory as the output (src/nvidia/nv_rt.c:348-375): same launch, y in host RAM
    hp, dp = C.c_void_p(), C.c_uint64()
    assert L.nv_rt_mmap(C.byref(d), C.byref(hp), C.byref(dp), n * 4) == 0
    mapped = np.ctypeslib.as_array(C.cast(hp, C.POINTER(C.c_float)), shape=(n,))
    mapped[:] = y
    args = _args(C.c_uint64(dp.value), C.c_uint64(dx), C.c_float(2.5), C.c_int(n))
    assert L.nv_rt_launch(C.byref(d), C.byref(k), (n + 255) // 256, 1, 1, 256, 1, 1, 0, args) == 0
    assert L.nv_rt_sync(C.byref(d)) == 0
    assert np.array_equal(mapped.view(np.uint32), want.view(np.uint32))
    del mapped
    L.nv_rt_mfre(C.byref(d), hp)
    L.nv_rt_free(C.byref(d), dx); L.nv_rt_free(C.byref(d), dy); L.nv_rt_free(C.byref(d), 0)
    L.nv_rt_unload(C.byref(d), C.byref(k))
    assert not k.func


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["i32", "f32"])
def test_reference_compilers_chunk_sum_ptx_equals_its_x86_64_build(sm, nv, oracle_lib, kind):
    """oracle/kernels/reduce_chunk_*.cu built by the reference compiler for both
    targets: per-chunk sums from its PTX on the GPU equal the serial sums its x86-64
    object forms (int32 wrapping; fp32 in element order, hence bit-exact too)."""
    art = os.path.join(PTX, "reduce_chunk_%s.ptx" % kind)
    if not os.path.exists(art):
        pytest.skip("oracle/_ref/ptx was not built (the reference tree was absent at build time)")
    L, d = nv
    threads, chunk = 1024, 96
    n = threads * chunk
    v = sm.fill_host(n, 0xB007000B, 0, 2 if kind == "i32" else 1)
    if kind == "i32":
        v = (v.astype(np.int64) * 2000003 % (1 << 31)).astype(np.int32)      # large terms: sums wrap
        want = v.reshape(threads, chunk).sum(axis=1, dtype=np.int64).astype(np.int32)
        assert oracle_lib.reduce_i32(v) == int(want.sum(dtype=np.int64).astype(np.int32))
    else:
        want = np.zeros(threads, np.float32)
        for j in range(chunk):
            want = want + v.reshape(threads, chunk)[:, j]
    k = NvKern()
    assert L.nv_rt_load(C.byref(d), art.encode(), ("reduce_chunk_%s" % kind).encode(), C.byref(k)) == 0
    din, dpart = L.nv_rt_alloc(C.byref(d), n * 4), L.nv_rt_alloc(C.byref(d), threads * 4)
    assert L.nv_rt_h2d(C.byref(d), din, v.ctypes.data, n * 4) == 0
    args = _args(C.c_uint64(dpart), C.c_uint64(din), C.c_int(chunk))
    assert L.nv_rt_launch(C.byref(d), C.byref(k), 1, 1, 1, threads, 1, 1, 0, args) == 0
    assert L.nv_rt_sync(C.byref(d)) == 0
    got = np.empty(threads, want.dtype)
    assert L.nv_rt_d2h(C.byref(d), got.ctypes.data, dpart, threads * 4) == 0
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    L.nv_rt_free(C.byref(d), din); L.nv_rt_free(C.byref(d), dpart)
    L.nv_rt_unload(C.byref(d), C.byref(k))


@pytest.mark.gpu
def test_bad_ptx_and_missing_names_fail_with_the_reference_codes(sm, tmp_path):
    bad = tmp_path / "bad.ptx"
    bad.write_text(".version 8.0\n.target sm_89\n.address_size 64\n.entry k ()\n{\n\tbogus.instruction;\n}\n")
    good = os.path.join(PTX, "scale.ptx")
    code = """
import ctypes as C, booth_b200 as b
L = b.lib(); d = (C.c_char * 320)(); k = (C.c_char * 144)()
print('init', L.nv_rt_init(d))
print('bad', L.nv_rt_load(d, %r, b'k', k))
print('nofile', L.nv_rt_load(d, b'/nonexistent/k.ptx', b'k', k))
if %r: print('noname', L.nv_rt_load(d, %r, b'no_such', k))
print('launch', L.nv_rt_launch(d, k, 1, 1, 1, 1, 1, 1, 0, None))
L.nv_rt_shut(d)
""" % (str(bad).encode(), os.path.exists(good), good.encode())
    res = subprocess.run([os.sys.executable, "-c", code], cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                         text=True, timeout=120)
    assert res.returncode == 0, res.stderr
    assert "init 0" in res.stdout and "bad -3" in res.stdout and "nofile -5" in res.stdout   # ERR_CUDA, ERR_IO
    assert "launch -3" in res.stdout
    if os.path.exists(good):
        assert "noname -6" in res.stdout                                                     # ERR_KERN
    assert "compiler log" in res.stderr and "nv_rt: could not load kernel 'k'" in res.stderr
