"""CPU-side checks of the C-ABI boundary: the library loads without a GPU,
exports every symbol the headers declare, keeps the reference's struct sizes
and error codes, and fails loudly (never falls back) when the driver is absent."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np

from conftest import REFERENCE, ROOT, fill_np


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b([a-z_][a-z0-9_]*)\s*\([^;{}]*\)\s*;", text)
    return sorted(set(n for n in names if n not in ("defined",)))


def test_headers_declare_the_reference_api():
    names = _declared("bc_runtime.h")
    # src/runtime/bc_runtime.h:43-67 in the reference
    assert names == sorted(["bc_device_init", "bc_device_shutdown", "bc_load_kernel", "bc_unload_kernel",
                            "bc_alloc", "bc_free", "bc_trak", "bc_copy_h2d", "bc_copy_d2h", "bc_dispatch"])


def test_library_exports_every_declared_symbol(sm):
    handle = C.CDLL(sm.LIB_PATH)
    declared = _declared("bc_runtime.h") + _declared("booth_sm100.h") + _declared("lf_gpu.h")
    assert len(declared) > 40
    for name in declared:
        assert hasattr(handle, name), "libbooth_sm100.so does not export %s" % name
    for name in sm.exported_symbols():
        assert name in declared, "%s is bound in Python but not declared in include/" % name


def test_struct_layouts_match_the_reference(sm):
    # bc_device_t is 384 opaque bytes, bc_kernel_t 40 bytes with these offsets
    # (src/runtime/bc_runtime.h:24-39).
    assert C.sizeof(sm.BcDevice) == 384
    assert C.sizeof(sm.BcKernel) == 40
    assert sm.BcKernel.kernarg_size.offset == 8 and sm.BcKernel._exec.offset == 24
    assert C.sizeof(sm.AsianParams) == 32


def test_error_codes_match_the_reference():
    text = open(os.path.join(ROOT, "include", "bc_runtime.h")).read()
    codes = dict(re.findall(r"#define\s+(BC_RT_\w+)\s+(-?\d+)", text))
    # src/runtime/bc_runtime.h:13-20
    assert codes == {"BC_RT_OK": "0", "BC_RT_ERR_DLOPEN": "-1", "BC_RT_ERR_DLSYM": "-2", "BC_RT_ERR_HSA": "-3",
                     "BC_RT_ERR_NO_GPU": "-4", "BC_RT_ERR_NO_MEM": "-5", "BC_RT_ERR_IO": "-6",
                     "BC_RT_ERR_SYMBOL": "-7"}


def test_host_generator_matches_numpy_philox(sm):
    for kind in (0, 1, 2):
        for first, n in ((0, 1000), (5, 4099), (2 ** 33 + 3, 257)):
            got = sm.fill_host(n, 0xB0070001, 7, kind, first=first, threads=3)
            want = fill_np(first, n, 0xB0070001, 7, kind)
            assert got.dtype == want.dtype and np.array_equal(got, want), (kind, first, n)
    pm1 = sm.fill_host(1 << 16, 1, 0, 0)
    assert pm1.min() >= -1.0 and pm1.max() < 1.0
    i32 = sm.fill_host(1 << 16, 1, 0, 2)
    assert i32.min() >= -1000 and i32.max() <= 1000


def test_host_generator_is_thread_count_independent(sm):
    a = sm.fill_host(1 << 18, 42, 1, 0, threads=1)
    b = sm.fill_host(1 << 18, 42, 1, 0, threads=7)
    assert np.array_equal(a, b)


def _run(code, env_extra):
    env = dict(os.environ, **env_extra)
    return subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=env, stdout=subprocess.PIPE,
                          stderr=subprocess.PIPE, text=True, timeout=120)


def test_missing_driver_is_an_error_not_a_fallback(sm):
    # Host-side failure injection: point the shim at a driver library that does
    # not exist. init must return the DLOPEN code of the reference
    # (src/runtime/bc_runtime.h:14) and print one line; nothing computes.
    code = ("import ctypes as C, booth_b200 as b\n"
            "L=b.lib(); d=b.BcDevice(); rc=L.bc_device_init(C.byref(d)); print('rc',rc)\n"
            "h=C.c_void_p(); print('rc2', L.sm100_rt_init(C.byref(h), 0))\n")
    res = _run(code, {"BOOTH_CUDA_LIB": "/nonexistent/libcuda.so.1"})
    assert res.returncode == 0, res.stderr
    assert "rc -1" in res.stdout and "rc2 -1" in res.stdout
    assert "sm100_rt: cannot open the CUDA driver" in res.stderr
    assert "bc_runtime: device init failed (-1)" in res.stderr


def test_cpu_launcher_symbol_aborts_without_a_gpu(sm):
    # vector_add has no error channel (examples/cpu_launch_vadd.c:23-24); without a
    # GPU it must abort, never add on the CPU.
    code = ("import numpy as np, booth_b200 as b\n"
            "x=np.ones(8,np.float32); o=np.zeros(8,np.float32)\n"
            "b.lib().vector_add(x.ctypes.data, x.ctypes.data, o.ctypes.data, 8, 256, 8); print('sum', o.sum())\n")
    res = _run(code, {"BOOTH_CUDA_LIB": "/nonexistent/libcuda.so.1"})
    assert res.returncode != 0
    assert "sum" not in res.stdout
    assert "there is no CPU fallback" in res.stderr


def test_offload_abi_declares_the_reference_functions_and_dies_loudly(sm):
    # src/runtime/lf_gpu.h:21-35: eight void-returning functions with no error
    # channel, so a device that cannot be opened ends the process with status 1
    # and one line on stderr (src/runtime/lf_gpu.c:55-59), never a CPU run.
    assert _declared("lf_gpu.h") == sorted(
        ["lfortran_gpu_init", "lfortran_gpu_shutdown", "lfortran_gpu_load_kernel", "lfortran_gpu_release_kernel",
         "lfortran_gpu_set_buffer_arg", "lfortran_gpu_set_scalar_arg", "lfortran_gpu_launch", "lfortran_gpu_sync"])
    code = ("import ctypes as C, booth_b200 as b\n"
            "L=b.lib(); L.lfortran_gpu_init.restype=C.c_void_p; L.lfortran_gpu_shutdown(None); print('before')\n"
            "L.lfortran_gpu_init(); print('after')\n")
    res = _run(code, {"BOOTH_CUDA_LIB": "/nonexistent/libcuda.so.1"})
    assert res.returncode == 1
    assert "before" in res.stdout and "after" not in res.stdout
    assert "lf_gpu_sm100: sm100_rt_init failed (rc=-1)" in res.stderr


def test_python_layer_raises_when_library_is_missing(sm, tmp_path):
    code = ("import booth_b200 as b\n"
            "b.LIB_PATH='%s/none.so'\n"
            "try:\n    b.lib(); print('loaded')\nexcept ImportError as e:\n    print('ImportError', 'no fallback' in str(e))\n" % tmp_path)
    res = _run(code, {})
    assert "ImportError True" in res.stdout


def test_shard_range_covers_and_aligns(sm):
    for n in (0, 1, 5, 1 << 20, (1 << 20) + 3, 10 ** 6 + 1):
        for world in (1, 2, 3, 4, 8):
            spans = [sm.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (lo, hi), (lo2, _) in zip(spans, spans[1:]):
                assert hi == lo2 and lo <= hi and lo % 4 == 0 and hi % 4 == 0


def test_run_side_descriptor_mirrors_the_reference_contract(sm, tmp_path):
    """include/rt_sm100.h declares rt_desc_t on its own; its layout and status
    codes must be those of the reference's src/exec/exec.h (checked by compiling a
    probe against each header when the reference tree is present), and the
    library must export a descriptor with every required operation filled in."""
    handle = C.CDLL(sm.LIB_PATH)
    desc = C.c_void_p.in_dll(handle, "rt_sm100")          # the exported object exists
    words = (C.c_uint64 * 18).from_address(C.addressof(desc))
    assert C.string_at(words[0]) == b"sm100" and C.string_at(words[1]) == b"cubin"
    dev_size, kern_size = words[2] & 0xFFFFFFFF, words[2] >> 32
    assert 0 < dev_size <= 1024 and 0 < kern_size <= 192   # RT_DEV_MAX / RT_KERN_MAX (src/exec/exec.h:43-44)
    assert all(words[i] != 0 for i in range(3, 17))        # 10 required + 4 optional operations
    ref_hdr = os.path.join(REFERENCE, "src", "exec", "exec.h")
    if not os.path.exists(ref_hdr):
        return
    probe = r"""
#include <stdio.h>
#include <stddef.h>
#ifdef REF
#include "exec.h"
#else
#include "rt_sm100.h"
#endif
int main(void){
  printf("%zu %zu %zu %zu ", sizeof(rt_desc_t), sizeof(rt_arg_t), sizeof(rt_dim_t), sizeof(rt_ptr));
  printf("%zu %zu %zu %zu %zu %zu ", offsetof(rt_desc_t,dev_size), offsetof(rt_desc_t,open), offsetof(rt_desc_t,run),
         offsetof(rt_desc_t,sync), offsetof(rt_desc_t,hmap), offsetof(rt_desc_t,errs));
  printf("%d %d %d %d %d %d %d %d %d %d %d\n", RT_OK, RT_ENODRV, RT_ESYM, RT_EDRV, RT_ENODEV, RT_EIO, RT_EKERN,
         RT_EUNSUP, RT_EINPUT, RT_DEV_MAX, RT_KERN_MAX);
  return 0; }
"""
    src = tmp_path / "probe.c"
    src.write_text(probe)
    outs = []
    for flags in (["-DREF", "-I", os.path.dirname(ref_hdr)], ["-I", os.path.join(ROOT, "include")]):
        exe = tmp_path / ("probe_" + str(len(outs)))
        subprocess.run(["gcc", "-std=c99"] + flags + [str(src), "-o", str(exe)], check=True)
        outs.append(subprocess.run([str(exe)], stdout=subprocess.PIPE, text=True, check=True).stdout)
    assert outs[0] == outs[1], outs
