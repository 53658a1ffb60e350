"""GPU parity against the committed golden outputs of the reference compiler's
x86-64 objects (tests/golden/reference_x86_64.npz, made by make_golden.py)."""
import os

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

SEED = 0xB0070000
GOLD = np.load(os.path.join(ROOT, "tests", "golden", "reference_x86_64.npz"))


@pytest.mark.parametrize("n", [8, 257, 4099])
def test_stream_kernels_bit_exact_vs_golden(sm, dev, n):
    x = sm.fill_host(n, SEED, 0, 0); y = sm.fill_host(n, SEED, 1, 0)
    dx, dy, do = dev.upload(x), dev.upload(y), dev.alloc(n * 4)
    dev.vadd(dx, dy, do, n)
    assert np.array_equal(dev.download(do, n, np.uint32), GOLD["vadd_%d" % n])
    dev.saxpy(dy, dx, 2.5, n)
    assert np.array_equal(dev.download(dy, n, np.uint32), GOLD["saxpy_%d" % n])


@pytest.mark.parametrize("n", [1, 4097, 100003, 1 << 20])
def test_sums_vs_golden(sm, dev, n):
    out = dev.alloc(8)
    p = dev.upload(sm.fill_host(n, SEED + 2, 0, 2))
    dev.reduce_i32(p, n, out)
    assert int(dev.download(out, 1, np.int32)[0]) == int(GOLD["reduce_i32_%d" % n][0])      # bit-exact
    q = dev.upload(sm.fill_host(n, SEED + 2, 1, 1))
    dev.reduce_f32(q, n, out)
    want = float(GOLD["reduce_f32_%d" % n][0])
    assert abs(np.float32(dev.download(out, 1, np.float64)[0]) - np.float32(want)) <= 1e-6 * want


def test_gemm_vs_golden(sm, dev):
    M, N, K = 128, 256, 96
    a = sm.fill_host(M * K, SEED + 3, 0, 0); b = sm.fill_host(K * N, SEED + 3, 1, 0)
    da, db, dc = dev.upload(a), dev.upload(b), dev.alloc(M * N * 4)
    dev.gemm(dc, da, db, M, N, K)
    dev.sync()
    got = dev.download(dc, (M, N), np.float32).astype(np.float64)
    want = GOLD["matmul_%dx%dx%d" % (M, N, K)].view(np.float32).astype(np.float64)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-5


def test_tile_matmul_symbols_bit_exact_vs_golden(sm, dev):
    """matmul / matmul_k (host pointers, the CPU-launcher ABI) repeat the reference's
    summation order, so single tiles are bit-identical."""
    L = sm.lib()
    a = ((np.arange(16) * 7) % 11).astype(np.float32) * np.float32(0.25) - np.float32(1.0)
    b = ((np.arange(16) * 5) % 13).astype(np.float32) * np.float32(0.5) - np.float32(2.0)
    c = np.full(16, -123.0, np.float32)
    L.matmul(a.ctypes.data, b.ctypes.data, c.ctypes.data, 4, 1, 4, 1, 4, 1, 1)        # examples/cpu_launch_matmul.c:44
    assert np.array_equal(c.view(np.uint32), GOLD["matmul_tile_example"])
    M, N, K = 8, 12, 6
    A = sm.fill_host(M * K, SEED + 3, 0, 0).reshape(M, K); B = sm.fill_host(K * N, SEED + 3, 1, 0).reshape(K, N)
    C = np.zeros((M, N), np.float32)
    for mb in range(M // 4):
        for nb in range(N // 4):
            L.matmul_k(A[mb * 4:].ctypes.data, B[:, nb * 4:].ctypes.data, C[mb * 4:, nb * 4:].ctypes.data,
                       K, K, 1, N, 1, N, 1, 1)
    assert np.array_equal(C.view(np.uint32), GOLD["matmul_%dx%dx%d" % (M, N, K)])


def test_tile_matmul_symbol_walks_a_matrix_like_the_reference_harness(sm, dev, oracle_lib):
    """A caller of the CPU-launcher ABI multiplies matrices by calling matmul_k once per 4 x 4 tile
    with offset base pointers. The library keeps its device buffers between such calls and regrows
    them when a later call needs more (here: K = 64 first, then a 2 MiB-wide operand): every tile
    bit-identical to the CPU checker's, memory around the strided C tile untouched."""
    import time
    L = sm.lib()
    for M, N, K in ((16, 24, 64), (8, 8, 70000)):
        A = sm.fill_host(M * K, SEED + 4, 0, 0).reshape(M, K); B = sm.fill_host(K * N, SEED + 4, 1, 0).reshape(K, N)
        C = np.full((M, N + 4), -7.0, np.float32)            # four guard columns beside the result
        t0 = time.perf_counter()
        for mb in range(M // 4):
            for nb in range(N // 4):
                L.matmul_k(A[mb * 4:].ctypes.data, B[:, nb * 4:].ctypes.data, C[mb * 4:, nb * 4:].ctypes.data,
                           K, K, 1, N, 1, N + 4, 1, 1)
        per_call = (time.perf_counter() - t0) / ((M // 4) * (N // 4))
        want = oracle_lib.matmul(A, B)
        assert np.array_equal(C[:, :N].view(np.uint32), want.view(np.uint32)), (M, N, K)
        assert np.all(C[:, N:] == np.float32(-7.0))
        assert per_call < 0.05, per_call


@pytest.mark.parametrize("precise", [1, 0])
def test_asian_vs_golden(sm, dev, precise):
    prm = sm.asian_params(k0=SEED + 5, precise=precise)
    out = dev.alloc(32)
    dev.asian(prm, 0, 1 << 16, out)
    s = dev.download(out, 4, np.float64)
    want = GOLD["asian_sums_0_65536"]
    assert abs(s[0] - want[0]) <= 1e-5 * want[0] and abs(s[1] - want[1]) <= 1e-5 * want[1]
    n = 1024
    da, dg = dev.alloc(n * 4), dev.alloc(n * 4)
    dev.asian_paths(prm, 0, n, da, dg)
    ga = dev.download(da, n, np.float32); wa = GOLD["asian_arith_0_1024"].view(np.float32)
    assert np.max(np.abs(ga - wa)) < 2e-3


@pytest.mark.parametrize("precise", [1, 0])
def test_asian_at_the_benchmark_size_vs_golden(sm, dev, precise):
    """2^26 paths x 252 steps, the benchmark's own run: both price sums against the
    sums the reference compiler's x86-64 objects produced for the same Philox
    stream (tests/golden/make_golden.py --full), within the 1e-5 the workload states."""
    key = "asian_sums_0_%d" % (1 << 26)
    if key not in GOLD.files:
        pytest.skip("the full-size sums are not in the fixture file")
    prm = sm.asian_params(k0=SEED + 5, precise=precise)
    out = dev.alloc(32)
    dev.asian(prm, 0, 1 << 26, out)
    s = dev.download(out, 4, np.float64)
    want = GOLD[key]
    rel = [abs(s[i] - want[i]) / want[i] for i in (0, 1)]
    assert max(rel) <= 1e-5, rel
    dev.free(out)
