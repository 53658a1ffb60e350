"""Philox4x32-10 held against the published Random123 known-answer vectors.

The workloads' inputs and every Monte Carlo path hang on this generator, and the
repository states it several times: the CUDA helper of the kernel image, the
host generator of the library, the CPU checker's kernel source as compiled by
the reference compiler's x86-64 backend, its C restatement, the checker
harness's own input generator and the numpy statement in conftest. Agreeing with
each other is not enough (one transcription slip copied everywhere would pass),
so each is compared with vectors from outside the repository."""
import ctypes as C

import numpy as np
import pytest

from conftest import PHILOX_KAT, fill_np, philox_np


def _u32(v):
    return np.asarray(v, np.uint32)


def test_numpy_statement():
    for ctr, key, want in PHILOX_KAT:
        c01 = np.uint64(ctr[0]) | (np.uint64(ctr[1]) << np.uint64(32))
        got = philox_np(np.array([c01], np.uint64), key[0], key[1], c2=ctr[2], c3=ctr[3])[0]
        assert np.array_equal(got, _u32(want))


@pytest.mark.parametrize("kind", ["reference", "port"])
def test_cpu_checker_kernel_object_and_harness_generator(kind):
    import oracle
    try:
        orc = oracle.load(kind)
    except FileNotFoundError:
        pytest.skip("the reference compiler's objects are not built here")
    for ctr, key, want in PHILOX_KAT:
        assert np.array_equal(orc.philox_kernel(ctr, key)[0], _u32(want))     # kath --cpu object / port.c
        assert np.array_equal(orc.philox_host(ctr, key), _u32(want))          # harness generator (orc_fill)
    # consecutive counters, and the input stream built from them: element i = lane i%4 of block i/4
    blocks = orc.philox_kernel((5, 0, 0, 0), (0xB0070001, 1), nblocks=64)
    assert np.array_equal(blocks, philox_np(np.arange(5, 69, dtype=np.uint64), 0xB0070001, 1))
    assert np.array_equal(orc.fill(256, 0xB0070001, 1, 3, first=20), blocks.ravel())
    for k in (0, 1, 2):
        assert np.array_equal(orc.fill(1003, 7, 2, k, first=13).view(np.uint32), fill_np(13, 1003, 7, 2, k).view(np.uint32))
    # path 0, call 0, key 0 of the pricer is the all-zero vector: its first uniforms
    z = orc.philox_kernel((0, 0, 0, 0), (0, 0))[0]
    assert np.array_equal(z, _u32(PHILOX_KAT[0][2]))


def test_library_host_generator(sm):
    L = sm.lib()
    for ctr, key, want in PHILOX_KAT:
        c, k, out = _u32(ctr), _u32(key), np.zeros(4, np.uint32)
        L.booth_sm100_philox4x32_10(c.ctypes.data, k.ctypes.data, out.ctypes.data)
        assert np.array_equal(out, _u32(want))
    # the raw fill kind is that generator, counter (i/4, 0, 0), key (seed, stream)
    assert np.array_equal(sm.fill_host(4, 0, 0, sm.FILL_U32_RAW), _u32(PHILOX_KAT[0][2]))
    got = sm.fill_host(1 << 12, 0xB0070002, 1, sm.FILL_U32_RAW, first=(1 << 34) + 6)
    assert np.array_equal(got, fill_np((1 << 34) + 6, 1 << 12, 0xB0070002, 1, 3))


@pytest.mark.gpu
def test_device_generator_known_answers(sm, dev):
    """The CUDA helper every kernel of the image uses (kernels/common.cuh), through
    the by-name kernel philox_words and through the fill kernel's raw kind."""
    k = sm.Kern()
    assert sm.lib().sm100_rt_load_builtin(dev.handle, b"philox_words", C.byref(k)) == 0
    out = dev.alloc(4 * 4 * 96)
    for ctr, key, want in PHILOX_KAT:
        vals = [C.c_uint64(out)] + [C.c_uint32(v) for v in ctr + key]
        argv = (C.c_void_p * len(vals))(*[C.cast(C.byref(v), C.c_void_p) for v in vals])
        assert sm.lib().sm100_rt_launch(dev.handle, C.byref(k), 1, 1, 1, 1, 1, 1, 0, argv) == 0
        dev.sync()
        assert np.array_equal(dev.download(out, 4, np.uint32), _u32(want))
    # 96 consecutive counters over 3 blocks of 32 threads
    vals = [C.c_uint64(out)] + [C.c_uint32(v) for v in (9, 1, 2, 3, 0xB0070005, 0)]
    argv = (C.c_void_p * len(vals))(*[C.cast(C.byref(v), C.c_void_p) for v in vals])
    assert sm.lib().sm100_rt_launch(dev.handle, C.byref(k), 3, 1, 1, 32, 1, 1, 0, argv) == 0
    dev.sync()
    want = philox_np(np.arange(9, 105, dtype=np.uint64) | (np.uint64(1) << np.uint64(32)), 0xB0070005, 0, c2=2, c3=3)
    assert np.array_equal(dev.download(out, (96, 4), np.uint32), want)
    # the fill kernel: zero vector at element 0, and a window far into the stream
    dev.fill(out, 0, 4, 0, 0, sm.FILL_U32_RAW)
    assert np.array_equal(dev.download(out, 4, np.uint32), _u32(PHILOX_KAT[0][2]))
    first = (1 << 34) + 6
    dev.fill(out, first, 380, 0xB0070002, 1, sm.FILL_U32_RAW)
    assert np.array_equal(dev.download(out, 380, np.uint32), sm.fill_host(380, 0xB0070002, 1, sm.FILL_U32_RAW, first=first))
    dev.free(out)
