"""GPU parity: vector add and saxpy through the C ABI against the CPU checker
(the reference compiler's x86-64 objects when built, else their C restatement).
Bit-exact, as the reference's own example demands (examples/cpu_launch_vadd.c:37-45)."""
import ctypes as C

import numpy as np
import pytest

from conftest import fill_np

pytestmark = pytest.mark.gpu

SIZES = [1, 3, 4, 5, 255, 256, 257, 1000, 4095, 4096, 4097, (1 << 16) - 1, (1 << 16) + 1, 1 << 20, (1 << 22) + 3]


def mismatches(got, want):
    """Bitwise comparison (so -0.0 vs 0.0 and NaN payloads count)."""
    return int(np.count_nonzero(got.view(np.uint32) != want.view(np.uint32)))


def test_device_generator_matches_host_generator(sm, dev):
    for kind in (0, 1, 2):
        for first, n in ((0, 4096), (3, 1001), (2 ** 32 + 6, 5000)):
            p = dev.alloc(n * 4)
            dev.fill(p, first, n, 0xB0070002, 3, kind)
            got = dev.download(p, n, np.int32 if kind == 2 else np.float32)
            want = sm.fill_host(n, 0xB0070002, 3, kind, first=first)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (kind, first, n)
            assert np.array_equal(want, fill_np(first, n, 0xB0070002, 3, kind))
            dev.free(p)


@pytest.mark.parametrize("n", SIZES)
def test_vadd_bit_exact(sm, dev, oracle_lib, n):
    x = sm.fill_host(n, 0xB0070000, 0, 0)
    y = sm.fill_host(n, 0xB0070000, 1, 0)
    dx, dy, do = dev.upload(x), dev.upload(y), dev.alloc(n * 4)
    dev.vadd(dx, dy, do, n)
    got = dev.download(do, n, np.float32)
    want = oracle_lib.vadd(x, y)
    assert mismatches(got, want) == 0
    # inject-must-fail: the comparison has teeth (tests/diff/diff_vadd.c:45-46)
    bad = got.copy()
    bad[n // 2] = np.nextafter(bad[n // 2], np.float32(10))
    assert mismatches(bad, want) == 1
    for p in (dx, dy, do):
        dev.free(p)


@pytest.mark.parametrize("n", SIZES)
def test_saxpy_bit_exact_unfused(sm, dev, oracle_lib, n):
    x = sm.fill_host(n, 0xB0070001, 0, 0)
    y = sm.fill_host(n, 0xB0070001, 1, 0)
    dx, dy = dev.upload(x), dev.upload(y)
    dev.saxpy(dy, dx, 2.5, n)
    got = dev.download(dy, n, np.float32)
    want = oracle_lib.saxpy(y, x, 2.5)
    assert mismatches(got, want) == 0
    # the fused result differs somewhere on random data, so the test can tell
    if n >= 4096:
        fused = (np.float64(2.5) * x.astype(np.float64) + y.astype(np.float64)).astype(np.float32)
        assert mismatches(fused, want) > 0
    dev.free(dx); dev.free(dy)


def test_unaligned_pointers_take_the_scalar_path(sm, dev, oracle_lib):
    n = 10007
    x = sm.fill_host(n + 3, 5, 0, 0)
    y = sm.fill_host(n + 3, 5, 1, 0)
    dx, dy, do = dev.upload(x), dev.upload(y), dev.alloc((n + 3) * 4)
    for off in (1, 2, 3):
        dev.vadd(dx + 4 * off, dy + 4 * off, do + 4 * off, n)
        got = dev.download(do + 4 * off, n, np.float32)
        assert mismatches(got, oracle_lib.vadd(x[off:off + n].copy(), y[off:off + n].copy())) == 0
        ycopy = dev.upload(y)
        dev.saxpy(ycopy + 4 * off, dx + 4 * off, 2.5, n)
        got = dev.download(ycopy + 4 * off, n, np.float32)
        assert mismatches(got, oracle_lib.saxpy(y[off:off + n].copy(), x[off:off + n].copy(), 2.5)) == 0
        dev.free(ycopy)


def test_reference_fixtures(sm, dev):
    # examples/cpu_launch_vadd.c:31-45: x=i, y=10i, N=8, exact
    x = np.arange(8, dtype=np.float32); y = 10 * x
    dx, dy, do = dev.upload(x), dev.upload(y), dev.alloc(32)
    dev.vadd(dx, dy, do, 8)
    assert np.array_equal(dev.download(do, 8, np.float32), x + y)
    # tests/numeric/manifest.json:9-25: saxpy x=1, y=3, a=2 -> 5.0 at n=256/200/255
    for n in (256, 200, 255):
        dxx, dyy = dev.upload(np.ones(n, np.float32)), dev.upload(np.full(n, 3, np.float32))
        dev.saxpy(dyy, dxx, 2.0, n)
        assert np.array_equal(dev.download(dyy, n, np.float32), np.full(n, 5, np.float32))
    # tests/diff/vadd_io.h:12-22 style: signed fractional inputs, N=64
    i = np.arange(64, dtype=np.float32)
    a = (i - 32) * np.float32(0.37); b = (i * i) * np.float32(-0.013) + np.float32(1.5)
    da, db, dc = dev.upload(a), dev.upload(b), dev.alloc(256)
    dev.vadd(da, db, dc, 64)
    assert mismatches(dev.download(dc, 64, np.float32), a + b) == 0


def test_cpu_launcher_symbols_take_host_pointers(sm, dev, oracle_lib):
    L = sm.lib()
    n = 5000
    x = sm.fill_host(n, 9, 0, 0); y = sm.fill_host(n, 9, 1, 0); out = np.full(n, -1, np.float32)
    L.vector_add(x.ctypes.data, y.ctypes.data, out.ctypes.data, n, 256, n)
    assert mismatches(out, oracle_lib.vadd(x, y)) == 0
    want = oracle_lib.saxpy(y, x, 2.5)
    L.saxpy(y.ctypes.data, x.ctypes.data, 2.5, n, n)
    assert mismatches(y, want) == 0


def test_cpu_launcher_symbols_from_several_host_threads(sm, dev, oracle_lib):
    """The reference's x86-64 kernels are plain functions, so a host may cut a vector
    into ranges and call the symbol from one thread per range (offset pointers);
    the library's symbols must stand that too. ctypes releases the GIL during a call."""
    import threading
    L = sm.lib()
    T, per = 6, 1 << 20
    n = T * per + 12345
    x = sm.fill_host(n, 11, 0, 0); y = sm.fill_host(n, 11, 1, 0)
    want_s = oracle_lib.saxpy(y, x, 2.5)
    want_v = oracle_lib.vadd(x, y)
    out = np.full(n, -1, np.float32)
    bounds = [(t * per, (t + 1) * per if t < T - 1 else n) for t in range(T)]

    def work(lo, hi):
        L.vector_add(x.ctypes.data + 4 * lo, y.ctypes.data + 4 * lo, out.ctypes.data + 4 * lo, hi - lo, 256, hi - lo)
    th = [threading.Thread(target=work, args=b) for b in bounds]
    [t.start() for t in th]; [t.join() for t in th]
    assert mismatches(out, want_v) == 0

    def work2(lo, hi):
        L.saxpy(y.ctypes.data + 4 * lo, x.ctypes.data + 4 * lo, 2.5, hi - lo, hi - lo)
    th = [threading.Thread(target=work2, args=b) for b in bounds]
    [t.start() for t in th]; [t.join() for t in th]
    assert mismatches(y, want_s) == 0


def test_full_size_saxpy_windows(sm, dev, oracle_lib):
    """N = 2^30 (4 GiB per vector): inputs generated in place on the device, the
    result checked bit for bit on windows at the start, an odd middle offset and
    the end against the CPU checker run on the same stream positions."""
    n = 1 << 30
    dx, dy = dev.alloc(n * 4), dev.alloc(n * 4)
    dev.fill(dx, 0, n, 0xB0070001, 0, 0)
    dev.fill(dy, 0, n, 0xB0070001, 1, 0)
    dev.saxpy(dy, dx, 2.5, n)
    w = 1 << 20
    for first in (0, (n // 2) + 12345, n - w):
        got = dev.download(dy + 4 * first, w, np.float32)
        x = sm.fill_host(w, 0xB0070001, 0, 0, first=first)
        y = sm.fill_host(w, 0xB0070001, 1, 0, first=first)
        assert mismatches(got, oracle_lib.saxpy(y, x, 2.5)) == 0
    dev.free(dx); dev.free(dy)


def test_vadd_at_the_configured_size_2_24(sm, dev, oracle_lib):
    """The benchmark's vector add configuration, whole output compared: N = 2^24,
    a, b ~ U[-1,1) from the seeded stream, bit-exact against the x86-64 build."""
    n = 1 << 24
    x, y = sm.fill_host(n, 0xB0070000, 0, 0), sm.fill_host(n, 0xB0070000, 1, 0)
    dx, dy, dz = dev.upload(x), dev.upload(y), dev.alloc(n * 4)
    dev.vadd(dx, dy, dz, n)
    assert mismatches(dev.download(dz, n, np.float32), oracle_lib.vadd(x, y)) == 0
    for p in (dx, dy, dz):
        dev.free(p)


def test_full_size_vadd_windows_and_sum(sm, dev, oracle_lib):
    """N = 2^28 + 5, the persistent-block geometry with a ragged end: windows at the
    start, an odd middle offset and the end are bit-exact, and over the whole
    output sum(out) = sum(x) + sum(y) within the fp32-sum tolerance (linearity)."""
    n = (1 << 28) + 5
    dx, dy, dz, out = dev.alloc(n * 4), dev.alloc(n * 4), dev.alloc(n * 4), dev.alloc(32)
    dev.fill(dx, 0, n, 0xB0070000, 0, 1)
    dev.fill(dy, 0, n, 0xB0070000, 1, 1)
    dev.vadd(dx, dy, dz, n)
    w = 1 << 20
    for first in (0, (n // 2) + 54321, n - w):
        got = dev.download(dz + 4 * first, w, np.float32)
        x = sm.fill_host(w, 0xB0070000, 0, 1, first=first)
        y = sm.fill_host(w, 0xB0070000, 1, 1, first=first)
        assert mismatches(got, oracle_lib.vadd(x, y)) == 0
    sums = []
    for p in (dx, dy, dz):
        dev.reduce_f32(p, n, out)
        sums.append(float(dev.download(out, 1, np.float64)[0]))
    assert abs(sums[2] - (sums[0] + sums[1])) <= 1e-6 * sums[2]
    for p in (dx, dy, dz, out):
        dev.free(p)


def test_back_to_back_launches_stay_ordered(sm, dev, oracle_lib):
    """The library launches these kernels so that a launch is set up while the one
    before it is still finishing. Each step here reads what the previous step wrote
    (y <- 2.5 x + y sixty times, then out = x + y), at sizes from one block to many
    waves: any launch that started on stale data would show in the bits."""
    for n in (1000, (1 << 16) + 3, 1 << 21):
        x = sm.fill_host(n, 0xB007000C, 0, 0)
        y = sm.fill_host(n, 0xB007000C, 1, 0)
        dx, dy, dz = dev.upload(x), dev.upload(y), dev.alloc(n * 4)
        steps = 60
        for _ in range(steps):
            dev.saxpy(dy, dx, 2.5, n)
        dev.vadd(dx, dy, dz, n)
        dev.saxpy(dz, dy, -1.0, n)                   # and a kernel reading two freshly written vectors
        want = y
        for _ in range(steps):
            want = oracle_lib.saxpy(want, x, 2.5)
        out = oracle_lib.vadd(x, want)
        out = oracle_lib.saxpy(out, want, -1.0)
        assert mismatches(dev.download(dy, n, np.float32), want) == 0
        assert mismatches(dev.download(dz, n, np.float32), out) == 0
        for p in (dx, dy, dz):
            dev.free(p)


def test_host_vector_calls_pipeline_over_chunks(sm, dev, oracle_lib):
    """booth_sm100_saxpy_host / _vadd_host: host vectors longer than two staging
    chunks (16 Mi elements each), pageable and page-locked, bit-exact."""
    n = (1 << 25) + (1 << 22) + 3                     # 2 full chunks + a ragged third
    x = sm.fill_host(n, 31, 0, 0); y = sm.fill_host(n, 31, 1, 0)
    want_s = oracle_lib.saxpy(y, x, 2.5); want_v = oracle_lib.vadd(x, y)
    out = np.empty_like(x)
    dev.vadd_host(x.ctypes.data, y.ctypes.data, out.ctypes.data, n)
    assert mismatches(out, want_v) == 0
    yy = y.copy()
    dev.saxpy_host(yy.ctypes.data, x.ctypes.data, 2.5, n)
    assert mismatches(yy, want_s) == 0
    # page-locked buffers, reused slots on a second call
    hx, hy = dev.hostalloc(n * 4), dev.hostalloc(n * 4)
    import ctypes as C
    C.memmove(hx, x.ctypes.data, n * 4)
    for _ in range(2):
        C.memmove(hy, y.ctypes.data, n * 4)
        dev.saxpy_host(hy, hx, 2.5, n)
        got = np.frombuffer((C.c_float * n).from_address(hy), dtype=np.float32)
        assert mismatches(got.copy(), want_s) == 0
    dev.hostfree(hx); dev.hostfree(hy)
    dev.vadd_host(x.ctypes.data, y.ctypes.data, out.ctypes.data, 0)        # empty input is a no-op


def test_empty_and_maximum_sizes(sm, dev, oracle_lib):
    """n = 0 is a no-op; n = 2^31 - 1 (the largest the kernels' int parameter holds,
    8 GiB per vector) is checked on windows at both ends; n = 2^31 is refused."""
    p = dev.alloc(64)
    dev.vadd(p, p, p, 0)
    dev.saxpy(p, p, 2.5, 0)
    with pytest.raises(sm.Sm100Error) as e:
        dev.saxpy(p, p, 2.5, 1 << 31)
    assert e.value.code == sm.ERR_ARG
    with pytest.raises(sm.Sm100Error):
        dev.vadd(p, p, p, -1)
    dev.free(p)
    n = (1 << 31) - 1
    dx, dy = dev.alloc(n * 4), dev.alloc(n * 4)
    dev.fill(dx, 0, n, 41, 0, 0); dev.fill(dy, 0, n, 41, 1, 0)
    dev.saxpy(dy, dx, 2.5, n)
    w = 1 << 18
    for first in (0, n - w):
        got = dev.download(dy + 4 * first, w, np.float32)
        x = sm.fill_host(w, 41, 0, 0, first=first); y = sm.fill_host(w, 41, 1, 0, first=first)
        assert mismatches(got, oracle_lib.saxpy(y, x, 2.5)) == 0
    dev.free(dx); dev.free(dy)


def test_link_probe_reports_the_host_link(sm, dev):
    """booth_sm100_link_probe: page-locked copies up, down and both at once; rates
    are positive, the two-way rates are not far above the one-way ones (the host is
    shared, so the margin is wide), and bad arguments are refused."""
    up, down, up2, down2 = dev.link_probe(64 << 20, 2)
    assert 1.0 < up < 1000.0 and 1.0 < down < 1000.0
    assert 0.0 < up2 <= 2.0 * up and 0.0 < down2 <= 2.0 * down
    import ctypes as C
    g = (C.c_double * 4)()
    assert sm.lib().booth_sm100_link_probe(dev.handle, 16, 1, g) == sm.ERR_ARG
    assert sm.lib().booth_sm100_link_probe(dev.handle, 1 << 20, 0, g) == sm.ERR_ARG


def test_ieee_special_values_match_the_x86_64_path(sm, dev, oracle_lib):
    """Signed zeros, infinities, subnormals, the largest finite values and products that
    overflow or underflow: the unfused mul and add of the GPU kernels give the bits the
    reference's x86-64 code (mulss, addss; no flush to zero on either side) gives. Where
    the result is a NaN (inf - inf, 0 * inf) both sides must say NaN; the payload of a
    NaN is the one thing the two machines are free to differ in, as the reference's own
    comparison allows (tests/diff/bc_diff.h: two NaNs agree)."""
    tiny, big = np.float32(1e-45), np.finfo(np.float32).max
    pool = np.array([0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, tiny, -tiny, 3e-39, -3e-39, 1.1754944e-38,
                     big, -big, big / 2, 1.5e38, -1.5e38, 0.4, -0.4, 6e-39, 2.5], np.float32)
    x = np.repeat(pool, pool.size)
    y = np.tile(pool, pool.size)
    n = x.size
    dx, dy, dz = dev.upload(x), dev.upload(y), dev.alloc(n * 4)
    dev.vadd(dx, dy, dz, n)
    dev.saxpy(dy, dx, 2.5, n)
    for got, want in ((dev.download(dz, n, np.float32), oracle_lib.vadd(x, y)),
                      (dev.download(dy, n, np.float32), oracle_lib.saxpy(y, x, 2.5))):
        nan = np.isnan(want)
        assert np.array_equal(np.isnan(got), nan)
        assert np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan])
        assert nan.any() and np.isinf(want).any() and (np.abs(want[~nan & (want != 0)]) < 1.2e-38).any()
    for p in (dx, dy, dz):
        dev.free(p)
