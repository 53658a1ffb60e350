"""CPU tests of the checker itself. The C restatement (oracle/port.c) must agree
bit for bit with (a) the golden outputs of the reference compiler's x86-64 objects
committed under tests/golden/, (b) those objects themselves when they are built
here, and (c) the reference's own fixtures for this path."""
import math
import os

import numpy as np
import pytest

import oracle
from conftest import ROOT

SEED = 0xB0070000
GOLD = np.load(os.path.join(ROOT, "tests", "golden", "reference_x86_64.npz"))


@pytest.fixture(scope="module")
def port():
    if not os.path.exists(oracle.PORT_SO):
        oracle.build(want_ref=False)
    return oracle.Oracle(oracle.PORT_SO, "port")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(oracle.REF_SO):
        pytest.skip("oracle/_ref is not built on this machine (no reference tree at build time)")
    return oracle.Oracle(oracle.REF_SO, "reference")


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.mark.parametrize("n", [8, 257, 4099])
def test_port_vadd_saxpy_match_golden(sm, port, n):
    x = sm.fill_host(n, SEED, 0, 0); y = sm.fill_host(n, SEED, 1, 0)
    assert np.array_equal(bits(port.vadd(x, y)), GOLD["vadd_%d" % n])
    assert np.array_equal(bits(port.saxpy(y, x, 2.5)), GOLD["saxpy_%d" % n])
    # saxpy is the separately rounded product and sum (src/cpu/cpu_emit.c:538-542)
    assert np.array_equal(bits(np.float32(2.5) * x + y), GOLD["saxpy_%d" % n])


@pytest.mark.parametrize("n", [1, 4097, 100003, 1 << 20])
def test_port_sums_match_golden(sm, port, n):
    vi = sm.fill_host(n, SEED + 2, 0, 2); vf = sm.fill_host(n, SEED + 2, 1, 1)
    assert port.reduce_i32(vi) == int(GOLD["reduce_i32_%d" % n][0]) == int(vi.astype(np.int64).sum())
    got = port.reduce_f32(vf)
    assert got == float(GOLD["reduce_f32_%d" % n][0])
    assert abs(got - port.sum_f64(vf)) <= 1e-6 * port.sum_f64(vf)      # the chunked sum is accurate
    for t in (1, 3):                                                    # and independent of the thread count
        assert port.reduce_f32(vf, threads=t) == got and port.reduce_i32(vi, threads=t) == port.reduce_i32(vi)


def test_serial_fp32_sum_would_not_meet_the_tolerance():
    # why the fp32 oracle is chunked: one serial fp32 accumulator over 2^25 values of 0.75 stalls
    v = np.full(1 << 25, 0.75, np.float32)
    assert np.cumsum(v, dtype=np.float32)[-1] < 0.75 * v.size * 0.7


@pytest.mark.parametrize("M,N,K", [(4, 4, 4), (8, 12, 6), (64, 64, 64), (128, 256, 96)])
def test_port_matmul_matches_golden(sm, port, M, N, K):
    a = sm.fill_host(M * K, SEED + 3, 0, 0).reshape(M, K); b = sm.fill_host(K * N, SEED + 3, 1, 0).reshape(K, N)
    got = port.matmul(a, b)
    assert np.array_equal(bits(got), GOLD["matmul_%dx%dx%d" % (M, N, K)])
    ref64 = a.astype(np.float64) @ b.astype(np.float64)
    assert np.linalg.norm(got - ref64) / np.linalg.norm(ref64) < 1e-6
    rows4 = np.array([M // 4 - 1], np.int32)                              # a sampled row block equals the full result
    part = port.matmul(a, b, rows4=rows4)
    assert np.array_equal(part[-4:], got[-4:]) and not part[:-4].any()


def test_reference_example_fixtures(port):
    # examples/cpu_launch_vadd.c:31-45
    x = np.arange(8, dtype=np.float32); y = 10 * x
    assert np.array_equal(port.vadd(x, y), x + y)
    # examples/cpu_launch_matmul.c:38-58: 4x4x4 tile with signed fractions, exact vs the triple loop
    a = ((np.arange(16) * 7) % 11).astype(np.float32) * np.float32(0.25) - np.float32(1.0)
    b = ((np.arange(16) * 5) % 13).astype(np.float32) * np.float32(0.5) - np.float32(2.0)
    c = np.full(16, -123.0, np.float32)
    port.matmul_tile(a, b, c, 4, 1, 4, 1, 4, 1)
    want = np.zeros((4, 4), np.float32)
    for m in range(4):
        for n in range(4):
            acc = np.float32(0)
            for k in range(4):
                acc = np.float32(acc + np.float32(a[m * 4 + k] * b[k * 4 + n]))
            want[m, n] = acc
    assert np.array_equal(c.reshape(4, 4), want)
    assert np.array_equal(bits(c), GOLD["matmul_tile_example"])
    # examples/launch_saxpy.c:54-58: x=i, y=N-i, a=2.5
    N = 1024
    xs = np.arange(N, dtype=np.float32); ys = (N - np.arange(N)).astype(np.float32)
    assert np.array_equal(port.saxpy(ys, xs, 2.5), np.float32(2.5) * xs + ys)
    # tests/numeric/manifest.json:9-25: x=1, y=3, a=2 -> 5 at n = 256, 200, 255
    for n in (256, 200, 255):
        assert np.array_equal(port.saxpy(np.full(n, 3, np.float32), np.ones(n, np.float32), 2.0), np.full(n, 5, np.float32))
    # tests/build/gpu_reduce.c:33-60: ones sum to N
    assert port.reduce_f32(np.ones(100000, np.float32)) == 100000.0


def test_port_asian_matches_golden(sm, port):
    prm = sm.asian_params(k0=SEED + 5)
    for path0, n in ((0, 1024), ((1 << 32) + 5, 256)):
        sa, sg, pa, pg = port.asian(prm, path0, n, per_path=True)
        assert np.array_equal(bits(pa), GOLD["asian_arith_%d_%d" % (path0, n)])
        assert np.array_equal(bits(pg), GOLD["asian_geom_%d_%d" % (path0, n)])
        assert [sa, sg] == list(GOLD["asian_sums_%d_%d" % (path0, n)])
    sa, sg = port.asian(prm, 0, 1 << 16)
    assert [sa, sg] == list(GOLD["asian_sums_0_65536"])
    assert port.asian(prm, 0, 1 << 16, threads=1) == (sa, sg)            # thread-count independent
    # sanity against the closed form of the geometric price (within 4 standard errors at 2^16 paths)
    mu = (0.05 - 0.02) * 253 / 504.0; var = 0.04 * 253 * 505 / (6.0 * 252 * 252)
    d2 = mu / math.sqrt(var); d1 = d2 + math.sqrt(var)
    Nc = lambda v: 0.5 * (1 + math.erf(v / math.sqrt(2)))
    cf = math.exp(-0.05) * (100 * math.exp(mu + var / 2) * Nc(d1) - 100 * Nc(d2))
    assert abs(cf - 5.5655) < 1e-3
    assert abs(math.exp(-0.05) * sg / 65536 - cf) < 4 * 8.0 / 256


def test_port_equals_reference_objects_on_fresh_inputs(sm, port, ref):
    """Beyond the fixtures: random sizes and seeds, bit for bit, when kath's objects are here."""
    rng = np.random.default_rng(20261125)
    for _ in range(4):
        n = int(rng.integers(1, 200000)); seed = int(rng.integers(1, 2 ** 31))
        x = sm.fill_host(n, seed, 0, 0); y = sm.fill_host(n, seed, 1, 0)
        assert np.array_equal(bits(port.vadd(x, y)), bits(ref.vadd(x, y)))
        assert np.array_equal(bits(port.saxpy(y, x, 2.5)), bits(ref.saxpy(y, x, 2.5)))
        vi = sm.fill_host(n, seed, 2, 2); vf = sm.fill_host(n, seed, 3, 1)
        assert port.reduce_i32(vi) == ref.reduce_i32(vi) and port.reduce_f32(vf) == ref.reduce_f32(vf)
    a = sm.fill_host(96 * 80, 5, 0, 0).reshape(96, 80); b = sm.fill_host(80 * 64, 5, 1, 0).reshape(80, 64)
    assert np.array_equal(bits(port.matmul(a, b)), bits(ref.matmul(a, b)))
    prm = sm.asian_params(k0=12345, k1=678)
    assert port.asian(prm, 777, 5000) == ref.asian(prm, 777, 5000)
